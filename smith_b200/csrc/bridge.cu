// bridge.cu -- the C ABI of libsmith_cuda.so (declared in include/smith_cuda_bridge.h).
//
// Mirrors the reference's Metal bridge (native/gpu_bridge.m) function for
// function: context, buffers, a "library" that is the built-in kernel
// registry, pipelines looked up by kernel name, an encoder that records
// pipeline + bound buffers + inline bytes, and sync / async / timed
// submission.  The CUDA-specific part is the memory model: SHARED buffers are
// page-locked host memory that the launchers stage to and from the device
// around each dispatch; PRIVATE, wrapped and resident buffers are read and
// written in place on the device.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/smith_cuda_bridge.h"
#include "kernels.h"

using namespace smith;

namespace {

constexpr uint32_t kCtxMagic = 0x534D4358;  // "SMCX"
constexpr uint32_t kBufMagic = 0x534D4246;  // "SMBF"
constexpr uint32_t kPsoMagic = 0x534D5053;  // "SMPS"
constexpr uint32_t kLibMagic = 0x534D4C42;  // "SMLB"
constexpr int kMaxBind = 8;

thread_local std::string g_err;

int fail(const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_err = buf;
  return 1;
}

#define CU_TRY(expr)                                                              \
  do {                                                                            \
    cudaError_t e_ = (expr);                                                      \
    if (e_ != cudaSuccess) return fail("%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

enum KernelId {
  kMatmulQ4 = 0, kMatmulQ8 = 1, kQuantQ4 = 2, kQuantQ8 = 3,
  // the dense matmul family (shaders/matmul.metal): tiled, simple and batched, f32 and f16 storage
  kMatmulF32, kMatmulF16, kMatmulSimple, kMatmulSimpleF16, kMatmulBatched, kMatmulBatchedF16,
  kNumKernels
};
const char* const kKernelNames[kNumKernels] = {"matmul_q4", "matmul_q8", "quantize_q4", "quantize_q8",
                                               "matmul_f32", "matmul_f16", "matmul_simple", "matmul_simple_f16",
                                               "matmul_batched", "matmul_batched_f16"};

struct Context {
  uint32_t magic = kCtxMagic;
  int device = 0;
  cudaStream_t stream = nullptr;
  cudaEvent_t base = nullptr;
  std::atomic<uint64_t> held{0};  // bytes held by live buffers + arenas
  uint64_t launches = 0;
  void* stage[3] = {nullptr, nullptr, nullptr};
  size_t stage_bytes[3] = {0, 0, 0};
  Workspace ws;
  void* flush = nullptr;
  size_t flush_bytes = 0;
  bool capturing = false;
  char name[256] = {0};
  uint64_t smem_optin = 0;
  uint64_t max_threads = 0;
};

struct Buffer {
  uint32_t magic = kBufMagic;
  Context* ctx = nullptr;
  uint64_t bytes = 0;
  uint32_t mode = SMITH_SHARED;
  void* host = nullptr;   // SHARED: page-locked host memory
  void* dev = nullptr;    // PRIVATE / wrapped / resident SHARED
  bool owns_dev = false;
  bool wrapped = false;
  bool resident = false;
  bool ipc_mapped = false;  // dev is another process's allocation opened through an IPC handle
  std::atomic<int64_t> refs{1};
};

struct Library {
  uint32_t magic = kLibMagic;
};
Library g_library;

struct Pipeline {
  uint32_t magic = kPsoMagic;
  int id = 0;
};
Pipeline g_pipelines[kNumKernels];

struct Graph {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
};

struct Token {
  Context* ctx;
  cudaEvent_t done;
};

Context* as_ctx(void* p) {
  Context* c = static_cast<Context*>(p);
  if (!c || c->magic != kCtxMagic) {
    fail("not a smith context");
    return nullptr;
  }
  cudaSetDevice(c->device);
  g_launch_counter = &c->launches;
  return c;
}

Buffer* as_buf(void* p) {
  Buffer* b = static_cast<Buffer*>(p);
  if (!b || b->magic != kBufMagic) {
    fail("not a smith buffer");
    return nullptr;
  }
  return b;
}

int grow(Context* c, void** ptr, size_t* have, size_t need) {
  if (*have >= need) return 0;
  if (c->capturing) return fail("scratch memory must be sized before graph capture (need %zu bytes)", need);
  size_t want = need + need / 4;
  want = (want + 255) & ~size_t(255);
  if (*ptr) {
    CU_TRY(cudaStreamSynchronize(c->stream));
    CU_TRY(cudaFree(*ptr));
    c->held -= *have;
    *ptr = nullptr;
    *have = 0;
  }
  CU_TRY(cudaMalloc(ptr, want));
  *have = want;
  c->held += want;
  return 0;
}

int env_device() {
  const char* names[2] = {"SMITH_CUDA_DEVICE", "LOCAL_RANK"};
  for (const char* n : names) {
    const char* v = getenv(n);
    if (v && *v) return atoi(v);
  }
  return 0;
}

void* make_context(int device) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
    fail("no CUDA device available");
    return nullptr;
  }
  if (device < 0 || device >= count) {
    fail("device %d out of range (%d visible)", device, count);
    return nullptr;
  }
  if (cudaSetDevice(device) != cudaSuccess) {
    fail("cudaSetDevice(%d) failed", device);
    return nullptr;
  }
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
    fail("cudaGetDeviceProperties failed");
    return nullptr;
  }
  if (prop.major != 10) {
    fail("device %d is sm_%d%d; this library carries sm_100a code only", device, prop.major, prop.minor);
    return nullptr;
  }
  Context* c = new Context();
  c->device = device;
  snprintf(c->name, sizeof c->name, "%s", prop.name);
  c->smem_optin = prop.sharedMemPerBlockOptin;
  c->max_threads = (uint64_t)prop.maxThreadsPerBlock;
  if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreate(&c->base) != cudaSuccess || cudaEventRecord(c->base, c->stream) != cudaSuccess) {
    fail("stream/event creation failed: %s", cudaGetErrorString(cudaGetLastError()));
    delete c;
    return nullptr;
  }
  return c;
}

// Device address a launch should read input `b` from.  SHARED buffers without
// a device copy are uploaded into staging slot `slot` first.
int input_ptr(Context* c, Buffer* b, int slot, size_t need, const void** out) {
  if (b->bytes < need) return fail("buffer at index %d holds %llu bytes, the launch needs %zu", slot,
                                   (unsigned long long)b->bytes, need);
  if (b->dev && (b->mode == SMITH_PRIVATE || b->wrapped || b->resident)) {
    *out = b->dev;
    return 0;
  }
  if (!b->host) return fail("buffer at index %d has neither host nor device memory", slot);
  if (grow(c, &c->stage[slot], &c->stage_bytes[slot], need)) return 1;
  if (need) CU_TRY(cudaMemcpyAsync(c->stage[slot], b->host, need, cudaMemcpyHostToDevice, c->stream));
  *out = c->stage[slot];
  return 0;
}

// Device address a launch should write output `b` to, and whether the result
// has to be copied back to the host view afterwards.
int output_ptr(Context* c, Buffer* b, int slot, size_t need, void** out, bool* copy_back) {
  if (b->bytes < need) return fail("output buffer at index %d holds %llu bytes, the launch needs %zu", slot,
                                   (unsigned long long)b->bytes, need);
  *copy_back = (b->mode == SMITH_SHARED && !b->wrapped && b->host != nullptr);
  if (b->dev && (b->mode == SMITH_PRIVATE || b->wrapped || b->resident)) {
    *out = b->dev;
    return 0;
  }
  if (grow(c, &c->stage[slot], &c->stage_bytes[slot], need)) return 1;
  *out = c->stage[slot];
  return 0;
}

int ensure_workspace(Context* c, size_t need) { return grow(c, &c->ws.ptr, &c->ws.bytes, need); }

int do_qmatmul(Context* c, int kind, const float* A, const uint8_t* B, float* C, uint64_t M, uint64_t N,
               uint64_t K, uint64_t groups, uint32_t path) {
  if (kind != 4 && kind != 8) return fail("kind must be 4 or 8, got %d", kind);
  if (M == 0 || N == 0) return 0;
  int p = (int)path;
  if (p == kAuto) p = resolve_path(kind, (int64_t)M, (int64_t)N, (int64_t)K, (int64_t)groups);
  cudaError_t e;
  switch (p) {
    case kGeneric:
      e = launch_qmatmul_generic(kind, A, B, C, M, N, K, groups, c->stream);
      break;
    case kDecode:
      if (!qdecode_supports(kind, M, N, K, groups))
        return fail("decode kernel does not take M=%llu N=%llu K=%llu groups=%llu", (unsigned long long)M,
                    (unsigned long long)N, (unsigned long long)K, (unsigned long long)groups);
      if (qdecode_workspace_bytes(kind, M, N, K) && ensure_workspace(c, qdecode_workspace_bytes(kind, M, N, K))) return 1;
      e = launch_qdecode(kind, A, B, C, M, N, K, groups, c->ws, c->stream);
      break;
    case kGemv:
      if (!qgemv_supports(kind, M, N, K, groups))
        return fail("GEMV kernel does not take M=%llu N=%llu K=%llu groups=%llu", (unsigned long long)M,
                    (unsigned long long)N, (unsigned long long)K, (unsigned long long)groups);
      e = launch_qgemv(kind, A, B, C, M, N, K, groups, c->stream);
      break;
    case kSkinny:
      if (!qskinny_supports(kind, M, N, K, groups))
        return fail("skinny kernel does not take M=%llu N=%llu K=%llu groups=%llu", (unsigned long long)M,
                    (unsigned long long)N, (unsigned long long)K, (unsigned long long)groups);
      if (ensure_workspace(c, qskinny_workspace_bytes(kind, M, N, K))) return 1;
      e = launch_qskinny(kind, A, B, C, M, N, K, groups, c->ws, c->stream);
      break;
    case kTensor: {
      if (!qgemm_tc_supports(kind, M, N, K, groups))
        return fail("tensor-core kernel does not take M=%llu N=%llu K=%llu groups=%llu", (unsigned long long)M,
                    (unsigned long long)N, (unsigned long long)K, (unsigned long long)groups);
      if (ensure_workspace(c, qgemm_tc_workspace_bytes(kind, M, N, K))) return 1;
      e = launch_qgemm_tc(kind, A, B, C, M, N, K, groups, c->ws, c->stream);
      break;
    }
    default:
      return fail("unknown path %u", path);
  }
  if (e != cudaSuccess) return fail("matmul_q%d launch failed: %s", kind, cudaGetErrorString(e));
  return 0;
}

// The dense matmul, C[b,M,N] = A[b,M,K] @ B[b,K,N].  path 0 follows the reference's own rule
// (src/ops/matmul.js:10,28): the tiled kernel's successor -- the tensor-core kernel -- when M, N and K
// are all at least 64, the any-shape kernel otherwise.
int do_dense(Context* c, int dtype, const void* A, const void* B, void* C, uint64_t M, uint64_t N, uint64_t K,
             uint64_t batch, uint32_t path) {
  if (dtype != kDenseF32 && dtype != kDenseF16) return fail("dtype must be 0 (f32) or 1 (f16), got %d", dtype);
  if (M == 0 || N == 0 || batch == 0) return 0;
  const size_t es = dtype == kDenseF16 ? 2 : 4;
  int p = (int)path;
  if (p == kDenseAuto)
    p = (M >= 64 && N >= 64 && K >= 64 && dense_tc_supports(dtype, (int64_t)M, (int64_t)N, (int64_t)K)) ? kDenseTcExact
                                                                                                       : kDenseGeneric;
  cudaError_t e = cudaSuccess;
  if (p == kDenseGeneric) {
    e = launch_dense_generic(dtype, A, B, C, (int64_t)M, (int64_t)N, (int64_t)K, (int64_t)batch, c->stream);
  } else if (p == kDenseTcExact || p == kDenseTcFast) {
    if (K == 0 || !dense_tc_supports(dtype, (int64_t)M, (int64_t)N, (int64_t)K))
      return fail("tensor-core matmul does not take M=%llu N=%llu K=%llu dtype=%d", (unsigned long long)M,
                  (unsigned long long)N, (unsigned long long)K, dtype);
    if (ensure_workspace(c, dense_tc_workspace_bytes(dtype, p, (int64_t)M, (int64_t)N, (int64_t)K))) return 1;
    for (uint64_t b = 0; b < batch && e == cudaSuccess; b++)
      e = launch_dense_tc(dtype, p, static_cast<const uint8_t*>(A) + b * M * K * es,
                          static_cast<const uint8_t*>(B) + b * K * N * es, static_cast<uint8_t*>(C) + b * M * N * es,
                          (int64_t)M, (int64_t)N, (int64_t)K, c->ws, c->stream);
  } else {
    return fail("unknown dense path %u", path);
  }
  if (e != cudaSuccess) return fail("dense matmul launch failed: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace

struct SmithEncoder {
  Context* ctx = nullptr;
  Pipeline* pso = nullptr;
  Buffer* bufs[kMaxBind] = {nullptr};
  std::vector<uint8_t> bytes[kMaxBind];
  uint64_t grid[3] = {0, 0, 0}, group[3] = {0, 0, 0};
  bool dispatched = false;
};

namespace {

// Stage in, launch, stage out.  Events e0/e1 (optional) bracket the kernels only.
int submit(SmithEncoder* enc, cudaEvent_t e0, cudaEvent_t e1) {
  Context* c = as_ctx(enc->ctx);
  if (!c) return 1;
  if (!enc->pso) return fail("no pipeline set");
  if (!enc->dispatched) return fail("smith_dispatch was not called");
  const int id = enc->pso->id;
  if (id == kMatmulQ4 || id == kMatmulQ8) {
    const int kind = (id == kMatmulQ4) ? 4 : 8;
    const size_t bb = (kind == 4) ? kQ4Bytes : kQ8Bytes;
    if (!enc->bufs[0] || !enc->bufs[1] || !enc->bufs[2]) return fail("matmul_q%d needs buffers 0, 1 and 2", kind);
    if (enc->bytes[3].size() < 16) return fail("matmul_q%d needs 16 bytes {M,N,K,groups} at index 3", kind);
    uint32_t prm[4];
    memcpy(prm, enc->bytes[3].data(), 16);
    const uint64_t M = prm[0], N = prm[1], K = prm[2], G = prm[3];
    const void *a = nullptr, *b = nullptr;
    void* cc = nullptr;
    bool back = false;
    if (input_ptr(c, enc->bufs[0], 0, M * K * 4, &a)) return 1;
    if (input_ptr(c, enc->bufs[1], 1, G * N * bb, &b)) return 1;
    Buffer* ob = enc->bufs[2];
    if (M <= 4 && ob->mode == SMITH_SHARED && !ob->wrapped && !ob->resident && ob->host && ob->bytes >= M * N * 4) {
      // A few rows of output: the kernel stores them straight into the page-locked host buffer (it is
      // mapped into the device's address space), each element once, instead of into a staging buffer
      // that a second copy would then carry over.  One operation less on the stream per call.
      cc = ob->host;
      back = false;
    } else if (output_ptr(c, ob, 2, M * N * 4, &cc, &back)) {
      return 1;
    }
    if (e0) CU_TRY(cudaEventRecord(e0, c->stream));
    if (do_qmatmul(c, kind, (const float*)a, (const uint8_t*)b, (float*)cc, M, N, K, G, kAuto)) return 1;
    if (e1) CU_TRY(cudaEventRecord(e1, c->stream));
    if (back && M * N)
      CU_TRY(cudaMemcpyAsync(enc->bufs[2]->host, cc, M * N * 4, cudaMemcpyDeviceToHost, c->stream));
    return 0;
  }
  if (id >= kMatmulF32 && id <= kMatmulBatchedF16) {
    const char* name = kKernelNames[id];
    const bool batched = (id == kMatmulBatched || id == kMatmulBatchedF16);
    const int dtype = (id == kMatmulF16 || id == kMatmulSimpleF16 || id == kMatmulBatchedF16) ? kDenseF16 : kDenseF32;
    const size_t es = dtype == kDenseF16 ? 2 : 4, need = batched ? 16 : 12;
    if (!enc->bufs[0] || !enc->bufs[1] || !enc->bufs[2]) return fail("%s needs buffers 0, 1 and 2", name);
    if (enc->bytes[3].size() < need)
      return fail("%s needs %zu bytes %s at index 3", name, need, batched ? "{M,N,K,batch}" : "{M,N,K}");
    uint32_t prm[4] = {0, 0, 0, 1};
    memcpy(prm, enc->bytes[3].data(), need);
    const uint64_t M = prm[0], N = prm[1], K = prm[2], batch = prm[3];
    const void *a = nullptr, *b = nullptr;
    void* cc = nullptr;
    bool back = false;
    if (input_ptr(c, enc->bufs[0], 0, batch * M * K * es, &a)) return 1;
    if (input_ptr(c, enc->bufs[1], 1, batch * K * N * es, &b)) return 1;
    if (output_ptr(c, enc->bufs[2], 2, batch * M * N * es, &cc, &back)) return 1;
    // the tiled kernels' successor is the tensor-core kernel; the simple and batched kernels keep
    // their one-thread-per-output order of operations (bit-identical sums)
    const uint32_t path = (id == kMatmulF32 || id == kMatmulF16) ? kDenseAuto : kDenseGeneric;
    if (e0) CU_TRY(cudaEventRecord(e0, c->stream));
    if (do_dense(c, dtype, a, b, cc, M, N, K, batch, path)) return 1;
    if (e1) CU_TRY(cudaEventRecord(e1, c->stream));
    if (back && batch * M * N)
      CU_TRY(cudaMemcpyAsync(enc->bufs[2]->host, cc, batch * M * N * es, cudaMemcpyDeviceToHost, c->stream));
    return 0;
  }
  if (id == kQuantQ4 || id == kQuantQ8) {
    const int kind = (id == kQuantQ4) ? 4 : 8;
    const size_t bb = (kind == 4) ? kQ4Bytes : kQ8Bytes;
    if (!enc->bufs[0] || !enc->bufs[1]) return fail("quantize_q%d needs buffers 0 and 1", kind);
    if (enc->bytes[2].size() < 8) return fail("quantize_q%d needs 8 bytes {K,N} at index 2", kind);
    uint32_t prm[2];
    memcpy(prm, enc->bytes[2].data(), 8);
    const uint64_t K = prm[0], N = prm[1], G = (K + 31) / 32;
    const void* w = nullptr;
    void* o = nullptr;
    bool back = false;
    if (input_ptr(c, enc->bufs[0], 0, K * N * 4, &w)) return 1;
    if (output_ptr(c, enc->bufs[1], 1, G * N * bb, &o, &back)) return 1;
    if (e0) CU_TRY(cudaEventRecord(e0, c->stream));
    cudaError_t e = (kind == 4) ? launch_pack_q4((const float*)w, (uint8_t*)o, K, N, c->stream)
                                : launch_pack_q8((const float*)w, (uint8_t*)o, K, N, c->stream);
    if (e != cudaSuccess) return fail("quantize_q%d launch failed: %s", kind, cudaGetErrorString(e));
    if (e1) CU_TRY(cudaEventRecord(e1, c->stream));
    if (back && G * N)
      CU_TRY(cudaMemcpyAsync(enc->bufs[1]->host, o, G * N * bb, cudaMemcpyDeviceToHost, c->stream));
    return 0;
  }
  return fail("pipeline id %d has no launcher", id);
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------- lifecycle
void* smith_init(void) { return make_context(env_device()); }
void* smith_init_device(int32_t device) { return make_context(device); }

void smith_destroy(void* p) {
  Context* c = as_ctx(p);
  if (!c) return;
  cudaStreamSynchronize(c->stream);
  for (int i = 0; i < 3; i++)
    if (c->stage[i]) cudaFree(c->stage[i]);
  if (c->ws.ptr) cudaFree(c->ws.ptr);
  if (c->flush) cudaFree(c->flush);
  cudaEventDestroy(c->base);
  cudaStreamDestroy(c->stream);
  c->magic = 0;
  if (g_launch_counter == &c->launches) g_launch_counter = nullptr;
  delete c;
}

const char* smith_last_error(void) { return g_err.c_str(); }
void smith_clear_error(void) { g_err.clear(); }

int32_t smith_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

int32_t smith_device_index(void* p) {
  Context* c = as_ctx(p);
  return c ? c->device : -1;
}

void* smith_stream(void* p) {
  Context* c = as_ctx(p);
  return c ? (void*)c->stream : nullptr;
}

int32_t smith_synchronize(void* p) {
  Context* c = as_ctx(p);
  if (!c) return 1;
  CU_TRY(cudaStreamSynchronize(c->stream));
  return 0;
}

// ---------------------------------------------------------------- device info
char* smith_device_name(void* p) {
  Context* c = as_ctx(p);
  const char* s = c ? c->name : "";
  char* out = (char*)malloc(strlen(s) + 1);
  if (out) strcpy(out, s);
  return out;
}

uint64_t smith_max_threadgroup_memory(void* p) {
  Context* c = as_ctx(p);
  return c ? c->smem_optin : 0;
}

uint64_t smith_max_threads_per_threadgroup(void* p) {
  Context* c = as_ctx(p);
  return c ? c->max_threads : 0;
}

// ---------------------------------------------------------------- buffers
void* smith_alloc(void* p, uint64_t bytes, uint32_t mode) {
  Context* c = as_ctx(p);
  if (!c) return nullptr;
  if (mode != SMITH_SHARED && mode != SMITH_PRIVATE) {
    fail("unknown storage mode %u", mode);
    return nullptr;
  }
  Buffer* b = new Buffer();
  b->ctx = c;
  b->bytes = bytes;
  b->mode = mode;
  const size_t n = bytes ? (size_t)bytes : 1;
  cudaError_t e;
  if (mode == SMITH_SHARED) {
    e = cudaHostAlloc(&b->host, n, cudaHostAllocPortable | cudaHostAllocMapped);   // mapped: kernels may store results into it
  } else {
    e = cudaMalloc(&b->dev, n);
    b->owns_dev = true;
  }
  if (e != cudaSuccess) {
    fail("allocation of %llu bytes (mode %u) failed: %s", (unsigned long long)bytes, mode, cudaGetErrorString(e));
    cudaGetLastError();
    delete b;
    return nullptr;
  }
  c->held += bytes;
  return b;
}

void* smith_buffer_contents(void* p) {
  Buffer* b = as_buf(p);
  return b ? b->host : nullptr;
}

uint64_t smith_buffer_length(void* p) {
  Buffer* b = as_buf(p);
  return b ? b->bytes : 0;
}

int64_t smith_buffer_retain_count(void* p) {
  if (!p) return -1;
  Buffer* b = as_buf(p);
  return b ? b->refs.load() : -1;
}

void smith_release_buffer(void* p) {
  if (!p) return;
  Buffer* b = as_buf(p);
  if (!b) return;
  if (--b->refs > 0) return;
  Context* c = b->ctx;
  if (c && c->magic == kCtxMagic) {
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);  // nothing in flight may still touch it
  }
  uint64_t freed = 0;
  if (b->host) {
    cudaFreeHost(b->host);
    freed += b->bytes;
  }
  if (b->dev && b->owns_dev) {
    cudaFree(b->dev);
    freed += b->bytes;
  }
  if (b->dev && b->ipc_mapped) cudaIpcCloseMemHandle(b->dev);
  if (c && c->magic == kCtxMagic) c->held -= freed;
  b->magic = 0;
  delete b;
}

void* smith_buffer_device_ptr(void* p) {
  Buffer* b = as_buf(p);
  return b ? b->dev : nullptr;
}

int32_t smith_buffer_make_resident(void* p) {
  Buffer* b = as_buf(p);
  if (!b) return 1;
  Context* c = as_ctx(b->ctx);
  if (!c) return 1;
  if (b->mode != SMITH_SHARED || b->wrapped) return 0;  // already device memory
  if (!b->dev) {
    CU_TRY(cudaMalloc(&b->dev, b->bytes ? b->bytes : 1));
    b->owns_dev = true;
    c->held += b->bytes;
  }
  if (b->bytes) CU_TRY(cudaMemcpyAsync(b->dev, b->host, b->bytes, cudaMemcpyHostToDevice, c->stream));
  CU_TRY(cudaStreamSynchronize(c->stream));
  b->resident = true;
  return 0;
}

int32_t smith_buffer_evict(void* p) {
  Buffer* b = as_buf(p);
  if (!b) return 1;
  Context* c = as_ctx(b->ctx);
  if (!c) return 1;
  if (b->mode != SMITH_SHARED || b->wrapped || !b->dev) return 0;
  CU_TRY(cudaStreamSynchronize(c->stream));
  CU_TRY(cudaFree(b->dev));
  c->held -= b->bytes;
  b->dev = nullptr;
  b->owns_dev = false;
  b->resident = false;
  return 0;
}

void* smith_wrap_device_memory(void* p, void* device_ptr, uint64_t bytes) {
  Context* c = as_ctx(p);
  if (!c) return nullptr;
  if (!device_ptr && bytes) {
    fail("cannot wrap a null device pointer");
    return nullptr;
  }
  Buffer* b = new Buffer();
  b->ctx = c;
  b->bytes = bytes;
  b->mode = SMITH_PRIVATE;
  b->dev = device_ptr;
  b->wrapped = true;
  return b;
}

int32_t smith_upload(void* p, uint64_t offset, const void* host, uint64_t bytes) {
  Buffer* b = as_buf(p);
  if (!b) return 1;
  Context* c = as_ctx(b->ctx);
  if (!c) return 1;
  if (!b->dev) return fail("buffer has no device side");
  if (offset + bytes > b->bytes) return fail("upload of %llu bytes at %llu overruns a %llu-byte buffer",
                                             (unsigned long long)bytes, (unsigned long long)offset,
                                             (unsigned long long)b->bytes);
  if (bytes) CU_TRY(cudaMemcpyAsync((char*)b->dev + offset, host, bytes, cudaMemcpyHostToDevice, c->stream));
  CU_TRY(cudaStreamSynchronize(c->stream));
  return 0;
}

int32_t smith_download(void* p, uint64_t offset, void* host, uint64_t bytes) {
  Buffer* b = as_buf(p);
  if (!b) return 1;
  Context* c = as_ctx(b->ctx);
  if (!c) return 1;
  if (!b->dev) return fail("buffer has no device side");
  if (offset + bytes > b->bytes) return fail("download of %llu bytes at %llu overruns a %llu-byte buffer",
                                             (unsigned long long)bytes, (unsigned long long)offset,
                                             (unsigned long long)b->bytes);
  if (bytes) CU_TRY(cudaMemcpyAsync(host, (const char*)b->dev + offset, bytes, cudaMemcpyDeviceToHost, c->stream));
  CU_TRY(cudaStreamSynchronize(c->stream));
  return 0;
}

int64_t smith_test_release(void* p) {
  Context* c = as_ctx(p);
  if (!c) return 0;
  void* b = smith_alloc(p, 1048576, SMITH_SHARED);
  if (!b) return 0;
  const uint64_t after_alloc = c->held.load();
  smith_release_buffer(b);
  return (int64_t)(after_alloc - c->held.load());
}

int64_t smith_test_release_after_use(void* p) {
  Context* c = as_ctx(p);
  if (!c) return 0;
  void* b = smith_alloc(p, 1048576, SMITH_PRIVATE);
  if (!b) return 0;
  const uint64_t after_alloc = c->held.load();
  launch_fill_bytes(static_cast<Buffer*>(b)->dev, 1048576, 0u, c->stream);
  cudaStreamSynchronize(c->stream);
  smith_release_buffer(b);
  return (int64_t)(after_alloc - c->held.load());
}

uint64_t smith_allocated_size(void* p) {
  Context* c = as_ctx(p);
  return c ? c->held.load() : 0;
}

// ---------------------------------------------------------------- library / pipelines
void* smith_load_library(void* p, const char* path) {
  (void)path;
  return as_ctx(p) ? &g_library : nullptr;
}

void* smith_compile_source(void* p, const char* source, char** error_out) {
  (void)p;
  (void)source;
  const char* msg = "run-time kernel compilation is not available in the CUDA bridge";
  fail("%s", msg);
  if (error_out) {
    *error_out = (char*)malloc(strlen(msg) + 1);
    if (*error_out) strcpy(*error_out, msg);
  }
  return nullptr;
}

void* smith_create_pipeline(void* p, void* library, const char* fn_name) {
  if (!as_ctx(p)) return nullptr;
  Library* l = static_cast<Library*>(library);
  if (!l || l->magic != kLibMagic) {
    fail("not a smith library handle");
    return nullptr;
  }
  if (!fn_name) {
    fail("kernel name is null");
    return nullptr;
  }
  for (int i = 0; i < kNumKernels; i++)
    if (strcmp(fn_name, kKernelNames[i]) == 0) {
      g_pipelines[i].id = i;
      return &g_pipelines[i];
    }
  fail("kernel '%s' not found", fn_name);
  return nullptr;
}

// ---------------------------------------------------------------- encoder
SmithEncoder* smith_begin(void* p) {
  Context* c = as_ctx(p);
  if (!c) return nullptr;
  SmithEncoder* e = new SmithEncoder();
  e->ctx = c;
  return e;
}

void smith_set_buffer(SmithEncoder* enc, void* buffer, uint32_t index) {
  if (!enc) return;
  if (index >= kMaxBind) {
    fail("buffer index %u out of range", index);
    return;
  }
  enc->bufs[index] = as_buf(buffer);
}

void smith_set_bytes(SmithEncoder* enc, const void* data, uint32_t length, uint32_t index) {
  if (!enc) return;
  if (index >= kMaxBind) {
    fail("bytes index %u out of range", index);
    return;
  }
  const uint8_t* d = static_cast<const uint8_t*>(data);
  enc->bytes[index].assign(d, d + (data ? length : 0));
}

void smith_set_pipeline(SmithEncoder* enc, void* pipeline) {
  if (!enc) return;
  Pipeline* q = static_cast<Pipeline*>(pipeline);
  if (!q || q->magic != kPsoMagic) {
    fail("not a smith pipeline");
    enc->pso = nullptr;
    return;
  }
  enc->pso = q;
}

void smith_set_threadgroup_memory(SmithEncoder* enc, uint64_t length, uint32_t index) {
  (void)enc;
  (void)length;
  (void)index;
}

void smith_dispatch(SmithEncoder* enc, uint64_t gx, uint64_t gy, uint64_t gz, uint64_t tx, uint64_t ty,
                    uint64_t tz) {
  if (!enc) return;
  enc->grid[0] = gx, enc->grid[1] = gy, enc->grid[2] = gz;
  enc->group[0] = tx, enc->group[1] = ty, enc->group[2] = tz;
  enc->dispatched = true;
}

void smith_end_sync(SmithEncoder* enc) {
  if (!enc) return;
  Context* c = enc->ctx;
  if (submit(enc, nullptr, nullptr) == 0) {
    cudaError_t e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) fail("kernel execution failed: %s", cudaGetErrorString(e));
  } else if (c && c->magic == kCtxMagic) {
    cudaStreamSynchronize(c->stream);  // drain any staging copy already queued
  }
  delete enc;
}

void* smith_end_async(SmithEncoder* enc) {
  if (!enc) return nullptr;
  Context* c = enc->ctx;
  Token* t = nullptr;
  if (submit(enc, nullptr, nullptr) == 0) {
    t = new Token{c, nullptr};
    if (cudaEventCreateWithFlags(&t->done, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventRecord(t->done, c->stream) != cudaSuccess) {
      fail("could not record completion event");
      delete t;
      t = nullptr;
      cudaStreamSynchronize(c->stream);
    }
  }
  delete enc;
  return t;
}

void smith_wait(void* token) {
  if (!token) return;
  Token* t = static_cast<Token*>(token);
  cudaSetDevice(t->ctx->device);
  cudaError_t e = cudaEventSynchronize(t->done);
  if (e != cudaSuccess) fail("kernel execution failed: %s", cudaGetErrorString(e));
  cudaEventDestroy(t->done);
  delete t;
}

SmithTiming* smith_end_timed(SmithEncoder* enc) {
  if (!enc) return nullptr;
  Context* c = enc->ctx;
  SmithTiming* out = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (cudaEventCreate(&e0) == cudaSuccess && cudaEventCreate(&e1) == cudaSuccess) {
    if (submit(enc, e0, e1) == 0) {
      cudaError_t e = cudaStreamSynchronize(c->stream);
      float ms = 0.f, since = 0.f;
      if (e == cudaSuccess && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess &&
          cudaEventElapsedTime(&since, c->base, e0) == cudaSuccess) {
        out = (SmithTiming*)calloc(1, sizeof(SmithTiming));
        if (out) {
          out->gpu_start = (double)since * 1e-3;
          out->gpu_end = ((double)since + (double)ms) * 1e-3;
          out->gpu_ms = (double)ms;
        }
      } else {
        fail("timed dispatch failed: %s", cudaGetErrorString(e != cudaSuccess ? e : cudaGetLastError()));
      }
    } else if (c && c->magic == kCtxMagic) {
      cudaStreamSynchronize(c->stream);
    }
  } else {
    fail("could not create timing events");
  }
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  delete enc;
  return out;
}

void smith_dispatch_sync(void* ctx, void* pipeline, void** buffers, uint32_t* indices, uint32_t buffer_count,
                         const void* params, uint32_t params_length, uint32_t params_index, uint64_t gx,
                         uint64_t gy, uint64_t gz, uint64_t tx, uint64_t ty, uint64_t tz) {
  SmithEncoder* enc = smith_begin(ctx);
  if (!enc) return;
  smith_set_pipeline(enc, pipeline);
  for (uint32_t i = 0; i < buffer_count; i++) smith_set_buffer(enc, buffers[i], indices[i]);
  if (params && params_length > 0) smith_set_bytes(enc, params, params_length, params_index);
  smith_dispatch(enc, gx, gy, gz, tx, ty, tz);
  smith_end_sync(enc);
}

// ---------------------------------------------------------------- direct entries
int32_t smith_q4_pack(void* p, void* w, void* out, uint64_t K, uint64_t N) {
  Context* c = as_ctx(p);
  Buffer *bw = as_buf(w), *bo = as_buf(out);
  if (!c || !bw || !bo) return 1;
  if (!bw->dev || !bo->dev) return fail("smith_q4_pack needs buffers with a device side");
  const uint64_t G = (K + 31) / 32;
  if (bw->bytes < K * N * 4 || bo->bytes < G * N * kQ4Bytes) return fail("smith_q4_pack: buffer too small");
  cudaError_t e = launch_pack_q4((const float*)bw->dev, (uint8_t*)bo->dev, K, N, c->stream);
  return e == cudaSuccess ? 0 : fail("pack_q4 launch failed: %s", cudaGetErrorString(e));
}

int32_t smith_q8_pack(void* p, void* w, void* out, uint64_t K, uint64_t N) {
  Context* c = as_ctx(p);
  Buffer *bw = as_buf(w), *bo = as_buf(out);
  if (!c || !bw || !bo) return 1;
  if (!bw->dev || !bo->dev) return fail("smith_q8_pack needs buffers with a device side");
  const uint64_t G = (K + 31) / 32;
  if (bw->bytes < K * N * 4 || bo->bytes < G * N * kQ8Bytes) return fail("smith_q8_pack: buffer too small");
  cudaError_t e = launch_pack_q8((const float*)bw->dev, (uint8_t*)bo->dev, K, N, c->stream);
  return e == cudaSuccess ? 0 : fail("pack_q8 launch failed: %s", cudaGetErrorString(e));
}

int32_t smith_gguf_repack(void* p, uint32_t ggml_type, void* src, void* dst, uint64_t out_dim, uint64_t in_dim) {
  Context* c = as_ctx(p);
  Buffer *bs = as_buf(src), *bd = as_buf(dst);
  if (!c || !bs || !bd) return 1;
  if (ggml_type != 2 && ggml_type != 8)
    return fail("smith_gguf_repack: ggml type %u is not one the quantized kernels read directly (Q4_0 = 2, Q8_0 = 8)", ggml_type);
  if (in_dim == 0 || (in_dim % 32) != 0) return fail("smith_gguf_repack: in_dim = %llu is not a multiple of 32", (unsigned long long)in_dim);
  if (!bs->dev || !bd->dev) return fail("smith_gguf_repack needs buffers with a device side");
  const uint64_t G = in_dim / 32, sb = (ggml_type == 8) ? 34 : 18, db = (ggml_type == 8) ? kQ8Bytes : kQ4Bytes;
  if (bs->bytes < out_dim * G * sb || bd->bytes < out_dim * G * db) return fail("smith_gguf_repack: buffer too small");
  cudaError_t e = launch_gguf_repack((int)ggml_type, (const uint8_t*)bs->dev, (uint8_t*)bd->dev, (int64_t)out_dim, (int64_t)in_dim,
                                     c->stream);
  return e == cudaSuccess ? 0 : fail("gguf repack launch failed: %s", cudaGetErrorString(e));
}

int32_t smith_qmatmul(void* p, uint32_t kind, void* a, void* b, void* cbuf, uint64_t M, uint64_t N, uint64_t K,
                      uint64_t groups, uint32_t path) {
  Context* c = as_ctx(p);
  Buffer *ba = as_buf(a), *bb = as_buf(b), *bc = as_buf(cbuf);
  if (!c || !ba || !bb || !bc) return 1;
  if (!ba->dev || !bb->dev || !bc->dev) return fail("smith_qmatmul needs buffers with a device side");
  const uint64_t blk = (kind == 4) ? kQ4Bytes : kQ8Bytes;
  if (ba->bytes < M * K * 4) return fail("smith_qmatmul: A holds %llu bytes, needs %llu", (unsigned long long)ba->bytes,
                                         (unsigned long long)(M * K * 4));
  if (bb->bytes < groups * N * blk) return fail("smith_qmatmul: B holds %llu bytes, needs %llu",
                                                (unsigned long long)bb->bytes, (unsigned long long)(groups * N * blk));
  if (bc->bytes < M * N * 4) return fail("smith_qmatmul: C holds %llu bytes, needs %llu", (unsigned long long)bc->bytes,
                                         (unsigned long long)(M * N * 4));
  return do_qmatmul(c, (int)kind, (const float*)ba->dev, (const uint8_t*)bb->dev, (float*)bc->dev, M, N, K, groups, path);
}

int32_t smith_matmul(void* p, uint32_t dtype, void* a, void* b, void* cbuf, uint64_t M, uint64_t N, uint64_t K,
                     uint64_t batch, uint32_t path) {
  Context* c = as_ctx(p);
  Buffer *ba = as_buf(a), *bb = as_buf(b), *bc = as_buf(cbuf);
  if (!c || !ba || !bb || !bc) return 1;
  if (!ba->dev || !bb->dev || !bc->dev) return fail("smith_matmul needs buffers with a device side");
  if (dtype != kDenseF32 && dtype != kDenseF16) return fail("dtype must be 0 (f32) or 1 (f16), got %u", dtype);
  const uint64_t es = dtype == kDenseF16 ? 2 : 4;
  if (ba->bytes < batch * M * K * es) return fail("smith_matmul: A holds %llu bytes, needs %llu",
                                                  (unsigned long long)ba->bytes, (unsigned long long)(batch * M * K * es));
  if (bb->bytes < batch * K * N * es) return fail("smith_matmul: B holds %llu bytes, needs %llu",
                                                  (unsigned long long)bb->bytes, (unsigned long long)(batch * K * N * es));
  if (bc->bytes < batch * M * N * es) return fail("smith_matmul: C holds %llu bytes, needs %llu",
                                                  (unsigned long long)bc->bytes, (unsigned long long)(batch * M * N * es));
  return do_dense(c, (int)dtype, ba->dev, bb->dev, bc->dev, M, N, K, batch, path);
}

int32_t smith_qmatmul_multi(void* p, uint32_t kind, void* a, uint32_t count, void* const* b_bufs, void* const* c_bufs,
                            const uint64_t* n_list, uint64_t M, uint64_t K, uint64_t groups) {
  Context* c = as_ctx(p);
  Buffer* ba = as_buf(a);
  if (!c || !ba) return 1;
  if (kind != 4 && kind != 8) return fail("kind must be 4 or 8, got %u", kind);
  if (count < 1 || count > 4) return fail("smith_qmatmul_multi takes 1 to 4 matrices, got %u", count);
  if (!b_bufs || !c_bufs || !n_list) return fail("smith_qmatmul_multi: null lists");
  if (!ba->dev) return fail("smith_qmatmul_multi needs buffers with a device side");
  if (ba->bytes < M * K * 4) return fail("smith_qmatmul_multi: A holds %llu bytes, needs %llu",
                                         (unsigned long long)ba->bytes, (unsigned long long)(M * K * 4));
  const uint64_t blk = (kind == 4) ? kQ4Bytes : kQ8Bytes;
  const uint8_t* Bs[4];
  float* Cs[4];
  int64_t Ns[4];
  for (uint32_t i = 0; i < count; i++) {
    Buffer *bb = as_buf(b_bufs[i]), *bc = as_buf(c_bufs[i]);
    if (!bb || !bc) return 1;
    if (!bb->dev || !bc->dev) return fail("smith_qmatmul_multi needs buffers with a device side");
    if (bb->bytes < groups * n_list[i] * blk || bc->bytes < M * n_list[i] * 4)
      return fail("smith_qmatmul_multi: matrix %u: a buffer is too small for N = %llu", i, (unsigned long long)n_list[i]);
    Bs[i] = (const uint8_t*)bb->dev, Cs[i] = (float*)bc->dev, Ns[i] = (int64_t)n_list[i];
  }
  if (count > 1 && qgemv_supports_multi((int)kind, (int64_t)M, Ns, (int)count, (int64_t)K, (int64_t)groups)) {
    cudaError_t e = launch_qgemv_multi((int)kind, (const float*)ba->dev, (int)count, Bs, Cs, Ns, (int64_t)M, (int64_t)K,
                                       (int64_t)groups, c->stream);
    if (e != cudaSuccess) return fail("multi-matrix GEMV launch failed: %s", cudaGetErrorString(e));
    return 0;
  }
  // Shapes the GEMV kernel does not take: one launch each.  Consecutive launches of the decode kernel
  // share the int8 digits of the activations (made once, kept in the context's scratch memory).
  bool digits_ready = false;
  for (uint32_t i = 0; i < count; i++) {
    const int path = resolve_path((int)kind, (int64_t)M, Ns[i], (int64_t)K, (int64_t)groups);
    if (path == kDecode && qdecode_uses_scratch((int)kind, (int64_t)M, Ns[i], (int64_t)K)) {
      if (ensure_workspace(c, qdecode_workspace_bytes((int)kind, (int64_t)M, Ns[i], (int64_t)K))) return 1;
      const cudaError_t e = launch_qdecode((int)kind, (const float*)ba->dev, Bs[i], Cs[i], (int64_t)M, Ns[i], (int64_t)K,
                                           (int64_t)groups, c->ws, c->stream, digits_ready);
      if (e != cudaSuccess) return fail("matmul_q%u launch failed: %s", kind, cudaGetErrorString(e));
      digits_ready = true;
    } else {
      if (do_qmatmul(c, (int)kind, (const float*)ba->dev, Bs[i], Cs[i], M, (uint64_t)Ns[i], K, groups, kAuto)) return 1;
      digits_ready = false;                 // the other kernels keep their own scratch in the same memory
    }
  }
  return 0;
}

int32_t smith_qmatmul_path(uint32_t kind, uint64_t M, uint64_t N, uint64_t K) {
  return resolve_path((int)kind, (int64_t)M, (int64_t)N, (int64_t)K, (int64_t)((K + 31) / 32));
}

int32_t smith_kernel_status(void* p) {
  Context* c = as_ctx(p);
  if (!c) return -1;
  if (cudaStreamSynchronize(c->stream) != cudaSuccess) return -1;
  return kernel_take_status();
}

uint64_t smith_launch_count(void* p) {
  Context* c = as_ctx(p);
  return c ? c->launches : 0;
}

// ---------------------------------------------------------------- a list of products as one launch
namespace {
struct ListHandle {
  uint32_t magic = 0x534D4C53;  // "SMLS"
  Context* ctx = nullptr;
  ListProgram* prog = nullptr;
  uint32_t count = 0;
};

// Device address of `bytes` bytes at `offset` inside a buffer's device side (nullptr + message on failure).
const uint8_t* list_operand(void* handle, uint64_t offset, uint64_t bytes, uint32_t item, const char* what) {
  Buffer* b = as_buf(handle);
  if (!b) return nullptr;
  if (!b->dev) {
    fail("smith_qmatmul_list_create: item %u: %s has no device side", item, what);
    return nullptr;
  }
  if (offset + bytes > b->bytes) {
    fail("smith_qmatmul_list_create: item %u: %s needs %llu bytes at offset %llu of a %llu-byte buffer", item, what,
         (unsigned long long)bytes, (unsigned long long)offset, (unsigned long long)b->bytes);
    return nullptr;
  }
  return static_cast<const uint8_t*>(b->dev) + offset;
}
}  // namespace

void* smith_qmatmul_list_create(void* p, uint32_t kind, uint64_t M, const SmithListItem* items, uint32_t count) {
  return smith_qmatmul_list_create_gather(p, kind, M, items, nullptr, count, 0, 0);
}

void* smith_qmatmul_list_create_gather(void* p, uint32_t kind, uint64_t M, const SmithListItem* items,
                                       const SmithListGather* gathers, uint32_t count, uint32_t rank, uint32_t flags) {
  Context* c = as_ctx(p);
  if (!c) return nullptr;
  if (!items || count == 0) {
    fail("smith_qmatmul_list_create: empty list");
    return nullptr;
  }
  if (kind != 4 && kind != 8) {
    fail("kind must be 4 or 8, got %u", kind);
    return nullptr;
  }
  if (c->capturing) {
    fail("smith_qmatmul_list_create allocates device memory: create the list before graph capture");
    return nullptr;
  }
  const uint64_t blk = (kind == 4) ? kQ4Bytes : kQ8Bytes;
  std::vector<ListItemDesc> descs(count);
  for (uint32_t i = 0; i < count; i++) {
    const SmithListItem& it = items[i];
    ListItemDesc& d = descs[i];
    if (it.K == 0 || (it.K % 32) != 0) {
      fail("smith_qmatmul_list_create: item %u: K = %llu is not a multiple of 32", i, (unsigned long long)it.K);
      return nullptr;
    }
    const uint64_t wbytes = (it.K / 32) * it.N * blk;
    d.N = (int64_t)it.N, d.K = (int64_t)it.K, d.eps = it.eps;
    d.A = reinterpret_cast<const float*>(list_operand(it.a, it.a_offset, M * it.K * 4, i, "a"));
    d.B = list_operand(it.b, it.b_offset, wbytes, i, "b");
    d.C = reinterpret_cast<float*>(const_cast<uint8_t*>(list_operand(it.c, it.c_offset, M * it.N * 4, i, "c")));
    if (!d.A || !d.B || !d.C) return nullptr;
    d.B2 = nullptr, d.gamma = nullptr, d.residual = nullptr;
    if (it.b2 && !(d.B2 = list_operand(it.b2, it.b2_offset, wbytes, i, "b2"))) return nullptr;
    if (it.gamma && !(d.gamma = reinterpret_cast<const float*>(list_operand(it.gamma, 0, it.K * 4, i, "gamma")))) return nullptr;
    if (it.residual && !(d.residual = reinterpret_cast<const float*>(
                             list_operand(it.residual, it.residual_offset, M * it.N * 4, i, "residual"))))
      return nullptr;
    d.g_world = 0, d.g_n0 = 0, d.g_n_total = 0;
    if (gathers && gathers[i].world) {
      const SmithListGather& g = gathers[i];
      if (g.world > 8) {
        fail("smith_qmatmul_list_create_gather: item %u: world %u out of range", i, g.world);
        return nullptr;
      }
      d.g_world = (int)g.world, d.g_n0 = (int64_t)g.n0, d.g_n_total = (int64_t)g.n_total;
      for (uint32_t r = 0; r < g.world; r++) {
        const uint8_t* row = list_operand(g.rows[r], 0, 2 * M * g.n_total * 8, i, "gather row buffer");
        if (!row) return nullptr;
        d.g_rows[r] = const_cast<uint8_t*>(row);
      }
    }
  }
  const char* why = "";
  ListProgram* prog = qgemv_list_create((int)kind, (int64_t)M, descs.data(), (int)count, (int)rank, flags, &why);
  if (!prog) {
    fail("smith_qmatmul_list_create: %s", why);
    return nullptr;
  }
  c->held += list_device_bytes(prog);
  ListHandle* h = new ListHandle();
  h->ctx = c, h->prog = prog, h->count = count;
  return h;
}

int32_t smith_qmatmul_list_run(void* p, void* list) {
  Context* c = as_ctx(p);
  ListHandle* h = static_cast<ListHandle*>(list);
  if (!c) return 1;
  if (!h || h->magic != 0x534D4C53 || h->ctx != c) return fail("smith_qmatmul_list_run: not a list of this context");
  cudaError_t e = qgemv_list_launch(h->prog, c->stream);
  return e == cudaSuccess ? 0 : fail("list launch failed: %s", cudaGetErrorString(e));
}

void smith_qmatmul_list_destroy(void* list) {
  ListHandle* h = static_cast<ListHandle*>(list);
  if (!h || h->magic != 0x534D4C53) return;
  Context* c = h->ctx;
  if (c && c->magic == kCtxMagic) {
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    c->held -= list_device_bytes(h->prog);
  }
  qgemv_list_destroy(h->prog);
  h->magic = 0;
  delete h;
}

uint32_t smith_qmatmul_list_next_tag(void* list) {
  ListHandle* h = static_cast<ListHandle*>(list);
  if (!h || h->magic != 0x534D4C53) return 0;
  Context* c = as_ctx(h->ctx);
  if (!c) return 0;
  return qgemv_list_next_tag(h->prog);
}

int32_t smith_qmatmul_list_supports(uint32_t kind, uint64_t M, uint64_t N, uint64_t K) {
  return qgemv_list_supports((int)kind, (int64_t)M, (int64_t)N, (int64_t)K) ? 1 : 0;
}

// For callers that must not allocate device memory at the time of the call: code
// running after its memory budget is fixed (a serving process that hands every
// byte to its own arena at start-up), inside a region where cudaMalloc would
// synchronise the device or is forbidden (a latency-critical loop, a host
// callback), or a host runtime that only owns raw device pointers and no
// smith context.  Takes raw device pointers and a stream; always runs the
// tensor-core kernel, with its scratch in a fixed array inside the library.
int32_t smith_qmatmul_static(uint32_t kind, const void* a_dev, const void* b_dev, void* c_dev, uint64_t M,
                             uint64_t N, uint64_t K, uint64_t groups, void* stream) {
  if (kind != 4 && kind != 8) return fail("kind must be 4 or 8, got %u", kind);
  if (!a_dev || !b_dev || !c_dev) return fail("smith_qmatmul_static: null device pointer");
  if (M == 0 || N == 0) return 0;
  const char* why = "";
  cudaError_t e = launch_qgemm_tc_static((int)kind, (const float*)a_dev, (const uint8_t*)b_dev, (float*)c_dev,
                                         (int64_t)M, (int64_t)N, (int64_t)K, (int64_t)groups, (cudaStream_t)stream, &why);
  if (e != cudaSuccess)
    return fail("smith_qmatmul_static: %s%s%s", why, *why ? " -- " : "", cudaGetErrorString(e));
  return 0;
}

// ---------------------------------------------------------------- multi-GPU: peer memory and the fused all-gather
int32_t smith_ipc_export(void* buffer, void* handle_out) {
  Buffer* b = as_buf(buffer);
  if (!b || !handle_out) return fail("smith_ipc_export: bad arguments");
  if (!b->dev || !b->owns_dev) return fail("smith_ipc_export needs a buffer whose device memory this library allocated");
  Context* c = as_ctx(b->ctx);
  if (!c) return 1;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  CU_TRY(cudaIpcGetMemHandle(&h, b->dev));
  memcpy(handle_out, &h, sizeof h);
  return 0;
}

void* smith_ipc_import(void* p, const void* handle, uint64_t bytes) {
  Context* c = as_ctx(p);
  if (!c || !handle) {
    fail("smith_ipc_import: bad arguments");
    return nullptr;
  }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof h);
  void* dev = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&dev, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    fail("cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return nullptr;
  }
  Buffer* b = new Buffer();
  b->ctx = c;
  b->bytes = bytes;
  b->mode = SMITH_PRIVATE;
  b->dev = dev;
  b->wrapped = true;
  b->ipc_mapped = true;
  return b;
}

int32_t smith_qgemv_tiles(uint32_t kind, uint64_t M, uint64_t N, uint64_t K) {
  return qgemv_tiles((int)kind, (int64_t)M, (int64_t)N, (int64_t)K);
}

int32_t smith_qmatmul_allgather(void* p, uint32_t kind, void* a, void* b, uint64_t M, uint64_t n_total, uint64_t n0,
                                uint64_t n_local, uint64_t K, uint64_t groups, uint32_t world, uint32_t rank,
                                void* const* y_bufs, void* const* state_bufs, uint32_t target) {
  return smith_qmatmul_allgather_ex(p, kind, a, b, M, n_total, n0, n_local, K, groups, world, rank, y_bufs, state_bufs,
                                    target, 0);
}

int32_t smith_allgather_wait(void* p, void* state_buf, void* y_buf, uint64_t M, uint64_t n_total) {
  Context* c = as_ctx(p);
  Buffer *bs = as_buf(state_buf), *by = as_buf(y_buf);
  if (!c || !bs || !by) return 1;
  if (M < 1 || M > 4 || (n_total % 8) != 0 || 2 * M * n_total > 0x7FFFFFFFull)
    return fail("smith_allgather_wait: M = %llu, n_total = %llu: rows are read as 16-byte pairs of pairs, so n_total must be a "
                "multiple of 8, M at most 4 and 2 * M * n_total below 2^31", (unsigned long long)M, (unsigned long long)n_total);
  if (!bs->dev || bs->bytes < 16 || !by->dev || by->bytes < 2 * M * n_total * 8)
    return fail("smith_allgather_wait: not the state and row buffers of a deferred all-gather of %llu x %llu",
                (unsigned long long)M, (unsigned long long)n_total);
  cudaError_t e = launch_gather_wait((const unsigned*)bs->dev, by->dev, (int64_t)M, (int64_t)n_total, c->stream);
  return e == cudaSuccess ? 0 : fail("all-gather wait launch failed: %s", cudaGetErrorString(e));
}

int32_t smith_qmatmul_allgather_ex(void* p, uint32_t kind, void* a, void* b, uint64_t M, uint64_t n_total, uint64_t n0,
                                   uint64_t n_local, uint64_t K, uint64_t groups, uint32_t world, uint32_t rank,
                                   void* const* y_bufs, void* const* state_bufs, uint32_t target, uint32_t flags) {
  Context* c = as_ctx(p);
  Buffer *ba = as_buf(a), *bb = as_buf(b);
  if (!c || !ba || !bb) return 1;
  if (kind != 4 && kind != 8) return fail("kind must be 4 or 8, got %u", kind);
  if (world < 1 || world > 8 || rank >= world) return fail("smith_qmatmul_allgather: world %u / rank %u out of range", world, rank);
  if (!y_bufs || !state_bufs) return fail("smith_qmatmul_allgather: null buffer lists");
  // The device code reads and writes the gathered rows with 16-byte accesses and 32-bit element counts.
  if ((n_total % 8) != 0 || (n0 % 8) != 0 || 2 * M * n_total > 0x7FFFFFFFull)
    return fail("smith_qmatmul_allgather: n_total = %llu and n0 = %llu must be multiples of 8 and 2 * M * n_total below 2^31",
                (unsigned long long)n_total, (unsigned long long)n0);
  if (n0 + n_local > n_total) return fail("smith_qmatmul_allgather: slice [%llu, %llu) outside a row of %llu",
                                          (unsigned long long)n0, (unsigned long long)(n0 + n_local),
                                          (unsigned long long)n_total);
  if (!ba->dev || !bb->dev) return fail("smith_qmatmul_allgather needs buffers with a device side");
  const uint64_t blk = (kind == 4) ? kQ4Bytes : kQ8Bytes;
  if (ba->bytes < M * K * 4 || bb->bytes < groups * n_local * blk) return fail("smith_qmatmul_allgather: input buffer too small");
  if (!qgemv_supports((int)kind, M, n_local, K, groups))
    return fail("fused all-gather is built into the GEMV kernel only (M <= 4, N %% 8 == 0, K %% 32 == 0); M=%llu N=%llu K=%llu",
                (unsigned long long)M, (unsigned long long)n_local, (unsigned long long)K);
  GemvGather g{};
  g.world = (int)world, g.rank = (int)rank, g.n0 = (int64_t)n0, g.n_total = (int64_t)n_total, g.target = target;
  g.defer = (flags & 1u) ? 1 : 0;
  g.a_prev = (flags & 2u) ? 1 : 0;
  if (g.a_prev && (!g.defer || K != n_total))
    return fail("smith_qmatmul_allgather_ex: SMITH_GATHER_INPUT_IS_PREVIOUS_ROW needs SMITH_GATHER_DEFER and K == n_total");
  for (uint32_t r = 0; r < world; r++) {
    Buffer *by = as_buf(y_bufs[r]), *bs = as_buf(state_bufs[r]);
    if (!by || !bs || !by->dev || !bs->dev) return fail("smith_qmatmul_allgather: rank %u buffers have no device side", r);
    if (by->bytes < 2 * M * n_total * (g.defer ? 8 : 4) || bs->bytes < 16)
      return fail("smith_qmatmul_allgather: rank %u buffers too small", r);
    g.y[r] = (float*)by->dev;
    g.state[r] = (unsigned*)bs->dev;
  }
  cudaError_t e = launch_qgemv_gather((int)kind, (const float*)ba->dev, (const uint8_t*)bb->dev, nullptr, M, n_local, K,
                                      groups, &g, c->stream);
  return e == cudaSuccess ? 0 : fail("fused GEMV + all-gather launch failed: %s", cudaGetErrorString(e));
}

int32_t smith_qmatmul_allreduce(void* p, uint32_t kind, void* a, void* b, void* out, uint64_t M, uint64_t N,
                                uint64_t k_local, uint64_t groups_local, uint32_t world, uint32_t rank,
                                void* const* partial_bufs, void* const* state_bufs) {
  Context* c = as_ctx(p);
  Buffer *ba = as_buf(a), *bb = as_buf(b), *bo = as_buf(out);
  if (!c || !ba || !bb || !bo) return 1;
  if (kind != 4 && kind != 8) return fail("kind must be 4 or 8, got %u", kind);
  if (world < 1 || world > 8 || rank >= world) return fail("smith_qmatmul_allreduce: world %u / rank %u out of range", world, rank);
  if (!partial_bufs || !state_bufs) return fail("smith_qmatmul_allreduce: null buffer lists");
  if (!ba->dev || !bb->dev || !bo->dev) return fail("smith_qmatmul_allreduce needs buffers with a device side");
  const uint64_t blk = (kind == 4) ? kQ4Bytes : kQ8Bytes;
  if (ba->bytes < M * k_local * 4 || bb->bytes < groups_local * N * blk || bo->bytes < M * N * 4)
    return fail("smith_qmatmul_allreduce: buffer too small");
  if (!qgemv_supports((int)kind, M, N, k_local, groups_local))
    return fail("fused all-reduce is built into the GEMV kernel only (M <= 4, N %% 8 == 0, K %% 32 == 0); M=%llu N=%llu K=%llu",
                (unsigned long long)M, (unsigned long long)N, (unsigned long long)k_local);
  if (2 * (uint64_t)world * M * N > 0x7FFFFFFFull) return fail("smith_qmatmul_allreduce: 2 * world * M * N must stay below 2^31");
  GemvGather g{};
  g.world = (int)world, g.rank = (int)rank, g.n0 = 0, g.n_total = (int64_t)N, g.target = 0, g.reduce = 1;
  for (uint32_t r = 0; r < world; r++) {
    Buffer *by = as_buf(partial_bufs[r]), *bs = as_buf(state_bufs[r]);
    if (!by || !bs || !by->dev || !bs->dev) return fail("smith_qmatmul_allreduce: rank %u buffers have no device side", r);
    if (by->bytes < 2 * (uint64_t)world * M * N * 8 || bs->bytes < smith_qmatmul_allreduce_state_bytes(kind, M, N, k_local))
      return fail("smith_qmatmul_allreduce: rank %u buffers too small", r);
    g.y[r] = (float*)by->dev;
    g.state[r] = (unsigned*)bs->dev;
  }
  cudaError_t e = launch_qgemv_gather((int)kind, (const float*)ba->dev, (const uint8_t*)bb->dev, (float*)bo->dev, M, N,
                                      k_local, groups_local, &g, c->stream);
  return e == cudaSuccess ? 0 : fail("fused GEMV + all-reduce launch failed: %s", cudaGetErrorString(e));
}

uint64_t smith_qmatmul_allreduce_state_bytes(uint32_t kind, uint64_t M, uint64_t N, uint64_t k_local) {
  // 16 bytes (the control words {step, ticket}) for every shape the fused form takes, 0 for the others
  return qgemv_supports((int)kind, (int64_t)M, (int64_t)N, (int64_t)k_local, (int64_t)(k_local / 32)) ? 16 : 0;
}

// ---------------------------------------------------------------- graphs
int32_t smith_graph_begin(void* p) {
  Context* c = as_ctx(p);
  if (!c) return 1;
  if (c->capturing) return fail("a capture is already open on this context");
  CU_TRY(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
  c->capturing = true;
  return 0;
}

void* smith_graph_end(void* p) {
  Context* c = as_ctx(p);
  if (!c) return nullptr;
  if (!c->capturing) {
    fail("no capture is open on this context");
    return nullptr;
  }
  c->capturing = false;
  Graph* g = new Graph();
  cudaError_t e = cudaStreamEndCapture(c->stream, &g->graph);
  if (e == cudaSuccess) e = cudaGraphInstantiate(&g->exec, g->graph, 0);
  if (e != cudaSuccess) {
    fail("graph capture failed: %s", cudaGetErrorString(e));
    cudaGetLastError();
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
    return nullptr;
  }
  return g;
}

int32_t smith_graph_launch(void* p, void* graph) {
  Context* c = as_ctx(p);
  Graph* g = static_cast<Graph*>(graph);
  if (!c || !g || !g->exec) return fail("invalid graph handle");
  CU_TRY(cudaGraphLaunch(g->exec, c->stream));
  return 0;
}

void smith_graph_destroy(void* graph) {
  Graph* g = static_cast<Graph*>(graph);
  if (!g) return;
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  delete g;
}

// ---------------------------------------------------------------- synthetic data / cache flush
int32_t smith_fill_normal(void* p, void* buffer, uint64_t count, uint64_t seed, float std) {
  Context* c = as_ctx(p);
  Buffer* b = as_buf(buffer);
  if (!c || !b) return 1;
  if (!b->dev) return fail("smith_fill_normal needs a buffer with a device side");
  if (b->bytes < count * 4) return fail("smith_fill_normal: buffer too small");
  cudaError_t e = launch_fill_normal((float*)b->dev, count, seed, std, c->stream);
  return e == cudaSuccess ? 0 : fail("fill_normal launch failed: %s", cudaGetErrorString(e));
}

int32_t smith_flush_l2(void* p) {
  Context* c = as_ctx(p);
  if (!c) return 1;
  if (grow(c, &c->flush, &c->flush_bytes, (size_t)256 << 20)) return 1;
  cudaError_t e = launch_fill_bytes(c->flush, c->flush_bytes, 0u, c->stream);
  return e == cudaSuccess ? 0 : fail("flush launch failed: %s", cudaGetErrorString(e));
}

}  // extern "C"
