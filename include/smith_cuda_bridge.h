/*
 * smith_cuda_bridge.h -- flat C ABI of libsmith_cuda.so, the CUDA (sm_100a)
 * replacement for Smith's Metal bridge on the quantized-matmul path.
 *
 * Part 1 keeps, name for name and argument for argument, the functions the
 * reference declares in native/gpu_bridge.h and binds in src/device.js:10-50,
 * so the JS host can dlopen this library instead of libsmith.dylib.  Each
 * declaration cites the reference declaration it replaces.
 *
 * Part 2 is additive: things a CUDA device needs that unified-memory Metal
 * did not (explicit residency, an error channel, device packers, a direct
 * matmul entry, CUDA-graph capture, multi-GPU helpers).
 *
 * No C++ or framework types cross this boundary: pointers, sizes, integers.
 *
 * Memory model.  SMITH_SHARED buffers are page-locked host memory; the pointer
 * from smith_buffer_contents() is a plain host pointer, valid for the life of
 * the buffer, exactly what the JS side wraps in an ArrayBuffer.  A dispatch of
 * a registered kernel copies its SHARED inputs host->device before the launch
 * and its SHARED outputs device->host after it, on the context's stream, so
 * the host view is coherent whenever a synchronous end_* call returns.
 * SMITH_PRIVATE buffers live in device memory only.  A SHARED buffer that holds
 * long-lived data (packed weights) can be pinned on the device with
 * smith_buffer_make_resident(); it is then read from the device copy and is no
 * longer re-uploaded on every dispatch.
 */
#ifndef SMITH_CUDA_BRIDGE_H
#define SMITH_CUDA_BRIDGE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SMITH_SHARED 0  /* host-visible, staged to the device per dispatch (native/gpu_bridge.h:12) */
#define SMITH_PRIVATE 1 /* device memory only                              (native/gpu_bridge.h:13) */

/* ===================== Part 1: the reference's bridge surface ===================== */

/* native/gpu_bridge.h:18.  Creates the context on the device named by the
 * environment (SMITH_CUDA_DEVICE, else LOCAL_RANK, else 0).  NULL on failure. */
void* smith_init(void);
/* native/gpu_bridge.h:21 */
void smith_destroy(void* ctx);

/* native/gpu_bridge.h:26.  malloc'd string, caller frees. */
char* smith_device_name(void* ctx);
/* native/gpu_bridge.h:29.  Largest opt-in dynamic shared memory per block, bytes. */
uint64_t smith_max_threadgroup_memory(void* ctx);
/* native/gpu_bridge.h:32 */
uint64_t smith_max_threads_per_threadgroup(void* ctx);

/* native/gpu_bridge.h:37.  Returns an opaque buffer handle (not the data pointer). */
void* smith_alloc(void* ctx, uint64_t bytes, uint32_t mode);
/* native/gpu_bridge.h:40.  Host pointer for SHARED buffers, NULL for PRIVATE. */
void* smith_buffer_contents(void* buffer);
/* native/gpu_bridge.h:43 */
uint64_t smith_buffer_length(void* buffer);
/* native/gpu_bridge.h:46.  Drops one reference; frees at zero. */
void smith_release_buffer(void* buffer);
/* native/gpu_bridge.h:127.  -1 for NULL. */
int64_t smith_buffer_retain_count(void* buffer);

/* native/gpu_bridge.h:49 and :52.  Allocate 1 MiB, (use it in a launch,) release;
 * return the bytes that came back. */
int64_t smith_test_release(void* ctx);
int64_t smith_test_release_after_use(void* ctx);

/* native/gpu_bridge.h:57.  The kernels are compiled into this library, so the
 * path is not opened; a handle to the built-in registry is returned. */
void* smith_load_library(void* ctx, const char* path);
/* native/gpu_bridge.h:61.  Run-time compilation is not offered: returns NULL and,
 * if error_out is non-NULL, a malloc'd message. */
void* smith_compile_source(void* ctx, const char* source, char** error_out);
/* native/gpu_bridge.h:64.  Known names: "matmul_q4", "matmul_q8" (buffers 0=A
 * f32 [M,K], 1=packed B, 2=C f32 [M,N]; bytes at 3 = uint32 {M,N,K,groups}, as
 * src/ops/quantize.js:80-87 binds them) and the new "quantize_q4",
 * "quantize_q8" (buffers 0=W f32 [K,N], 1=packed out; bytes at 2 = uint32
 * {K,N}); the dense family "matmul_f32", "matmul_f16", "matmul_simple",
 * "matmul_simple_f16" (buffers 0=A [M,K], 1=B [K,N], 2=C [M,N]; bytes at 3 =
 * uint32 {M,N,K}) and "matmul_batched", "matmul_batched_f16" (leading batch
 * dimension on all three; bytes at 3 = uint32 {M,N,K,batch}), as
 * src/ops/matmul.js:26-52,70-79 binds them.  NULL for anything else. */
void* smith_create_pipeline(void* ctx, void* library, const char* fn_name);

typedef struct SmithEncoder SmithEncoder;

/* native/gpu_bridge.h:72 */
SmithEncoder* smith_begin(void* ctx);
/* native/gpu_bridge.h:75 */
void smith_set_buffer(SmithEncoder* enc, void* buffer, uint32_t index);
/* native/gpu_bridge.h:78.  The bytes are copied at call time. */
void smith_set_bytes(SmithEncoder* enc, const void* data, uint32_t length, uint32_t index);
/* native/gpu_bridge.h:81 */
void smith_set_pipeline(SmithEncoder* enc, void* pipeline);
/* native/gpu_bridge.h:85.  Accepted and ignored: the CUDA launchers size their own shared memory. */
void smith_set_threadgroup_memory(SmithEncoder* enc, uint64_t length, uint32_t index);
/* native/gpu_bridge.h:88-90.  The Metal thread grid is recorded but the CUDA
 * launch geometry is derived from the bound parameters. */
void smith_dispatch(SmithEncoder* enc, uint64_t grid_x, uint64_t grid_y, uint64_t grid_z,
                    uint64_t group_x, uint64_t group_y, uint64_t group_z);
/* native/gpu_bridge.h:93.  Stage in, launch, stage out, wait.  Frees enc. */
void smith_end_sync(SmithEncoder* enc);
/* native/gpu_bridge.h:96 and :99.  Submit without waiting; smith_wait(token) waits and frees the token. */
void* smith_end_async(SmithEncoder* enc);
void smith_wait(void* token);

/* native/gpu_bridge.h:104-108 */
void smith_dispatch_sync(void* ctx, void* pipeline, void** buffers, uint32_t* indices,
                         uint32_t buffer_count, const void* params, uint32_t params_length,
                         uint32_t params_index, uint64_t grid_x, uint64_t grid_y, uint64_t grid_z,
                         uint64_t group_x, uint64_t group_y, uint64_t group_z);

/* native/gpu_bridge.h:113-117.  Seconds, seconds, milliseconds; start/end are
 * measured from context creation with CUDA events placed around the kernels. */
typedef struct {
  double gpu_start;
  double gpu_end;
  double gpu_ms;
} SmithTiming;

/* native/gpu_bridge.h:121.  calloc'd, caller frees; NULL on failure. */
SmithTiming* smith_end_timed(SmithEncoder* enc);
/* native/gpu_bridge.h:124.  Device bytes currently held through this context. */
uint64_t smith_allocated_size(void* ctx);

/* ===================== Part 2: additions (no reference counterpart) ===================== */

/* Error channel for the void functions above: message of the most recent
 * failure on the calling thread ("" if none).  Status-returning functions
 * below return 0 on success and non-zero on failure, and also set it. */
const char* smith_last_error(void);
void smith_clear_error(void);

int32_t smith_device_count(void);
void* smith_init_device(int32_t device); /* context on an explicit device */
int32_t smith_device_index(void* ctx);
void* smith_stream(void* ctx);           /* the context's cudaStream_t */
int32_t smith_synchronize(void* ctx);

/* Device address backing a buffer (PRIVATE, wrapped or resident SHARED), else NULL. */
void* smith_buffer_device_ptr(void* buffer);
/* Keep a device copy of a SHARED buffer and read from it in later dispatches
 * (uploads the current host contents now).  smith_buffer_evict drops it. */
int32_t smith_buffer_make_resident(void* buffer);
int32_t smith_buffer_evict(void* buffer);
/* Buffer handle over device memory owned by someone else (not freed on release). */
void* smith_wrap_device_memory(void* ctx, void* device_ptr, uint64_t bytes);
/* Blocking copies between host memory and any buffer's device side. */
int32_t smith_upload(void* buffer, uint64_t offset, const void* host, uint64_t bytes);
int32_t smith_download(void* buffer, uint64_t offset, void* host, uint64_t bytes);

/* Device packers: W f32 [K,N] (device side of w) -> packed blocks (device side
 * of out).  Q4 reproduces src/ops/quantize.js:14-68 bit for bit; Q8 is the
 * build-defined rule documented with the kernel.  Asynchronous on the
 * context's stream. */
int32_t smith_q4_pack(void* ctx, void* w, void* out, uint64_t K, uint64_t N);
int32_t smith_q8_pack(void* ctx, void* w, void* out, uint64_t K, uint64_t N);

/* GGUF blocks straight into the matmul layouts, on the device.  The reference de-quantises a GGUF
 * tensor to f32 on the host (src/gguf.js:187-231, 343-400), transposes it from [out_dim, in_dim] to
 * [in_dim, out_dim] (src/gguf_loader.js:236-252) and multiplies in f32.  src holds the tensor's blocks
 * as they lie in the file (block of row r, group b at (r * in_dim/32 + b) * block bytes); dst receives
 * the packed matrix matmul_q8 / matmul_q4 read, with K = in_dim and N = out_dim:
 *   ggml type 8 (Q8_0, 34-byte blocks): the same 34 bytes, re-tiled to (b * N + r) * 34;
 *   ggml type 2 (Q4_0, 18-byte blocks): the nibble bytes as they are, the f16 scale widened to f32,
 *     zero = 8 -> 24-byte Q4 blocks; scale * (nibble - 8) is the same f32 value either way.
 * Other types are refused (their arithmetic is not the two shaders').  Asynchronous. */
#define SMITH_GGML_Q4_0 2u
#define SMITH_GGML_Q8_0 8u
int32_t smith_gguf_repack(void* ctx, uint32_t ggml_type, void* src, void* dst, uint64_t out_dim, uint64_t in_dim);

/* Direct, asynchronous C[M,N] = A[M,K] * dequant(B) on device-side buffers.
 * kind: 4 or 8.  path: 0 = choose by shape, 1 = any-shape CUDA-core kernel,
 * 2 = decode kernel (M <= 32, integer mma.sync), 3 = tensor-core (tcgen05) kernel,
 * 4 = GEMV kernel (M <= 4, dp4a), 5 = skinny kernel (M <= 64, f16 mma.sync with the weights
 * de-quantised in registers).  A forced path that does not take the shape fails. */
#define SMITH_PATH_AUTO 0
#define SMITH_PATH_GENERIC 1
#define SMITH_PATH_DECODE 2
#define SMITH_PATH_TENSOR 3
#define SMITH_PATH_GEMV 4
#define SMITH_PATH_SKINNY 5
int32_t smith_qmatmul(void* ctx, uint32_t kind, void* a, void* b, void* c, uint64_t M, uint64_t N,
                      uint64_t K, uint64_t groups, uint32_t path);
/* The dense (unquantised) matmul as a direct, asynchronous call on device-side buffers:
 * c[batch,M,N] = a[batch,M,K] @ b[batch,K,N], row-major, dtype 0 = f32, 1 = f16 storage (f32 sums).
 * It stands for the reference's matmul family (src/ops/matmul.js:13-107; shaders/matmul.metal:31-260),
 * which the encoder path reaches under the names matmul_f32, matmul_f16, matmul_simple[_f16] and
 * matmul_batched[_f16] with {M,N,K} or {M,N,K,batch} as uint32 at index 3.
 * path: 0 = the reference's own rule (src/ops/matmul.js:10,28): tensor cores when M, N and K are all
 *           at least 64, the any-shape kernel otherwise;
 *       1 = any-shape CUDA-core kernel: every output the sequential f32 sum of the shaders, bit for bit;
 *       2 = tensor cores (tcgen05), f32 storage split into three bf16 planes and six partial products
 *           (error of the order of f32 rounding), f16 storage as it is;
 *       3 = tensor cores, f32 storage rounded to bf16 once (one product; about 2^-8 relative). */
#define SMITH_DTYPE_F32 0u
#define SMITH_DTYPE_F16 1u
#define SMITH_DENSE_AUTO 0u
#define SMITH_DENSE_GENERIC 1u
#define SMITH_DENSE_TENSOR 2u
#define SMITH_DENSE_TENSOR_FAST 3u
int32_t smith_matmul(void* ctx, uint32_t dtype, void* a, void* b, void* c, uint64_t M, uint64_t N, uint64_t K,
                     uint64_t batch, uint32_t path);
/* No counterpart in the reference, whose callers issue one matmul per weight matrix
 * (src/gguf_cache.js:121-171: wq, wk, wv on the same input; gate and up on the same input).
 * c_bufs[i] [M, n_list[i]] = a [M, K] x dequant(b_bufs[i]) for 1 to 4 packed matrices of the same K
 * and kind.  For M <= 4 they run as ONE launch of the GEMV kernel (its grid covers the tiles of all
 * matrices), which saves the start-up and tail of the launches it replaces; other shapes fall
 * back to one launch per matrix.  Results are those of smith_qmatmul per matrix. */
int32_t smith_qmatmul_multi(void* ctx, uint32_t kind, void* a, uint32_t count, void* const* b_bufs,
                            void* const* c_bufs, const uint64_t* n_list, uint64_t M, uint64_t K, uint64_t groups);
/* Which path 0 would resolve to for a shape (for tests and reports). */
int32_t smith_qmatmul_path(uint32_t kind, uint64_t M, uint64_t N, uint64_t K);
/* No counterpart in the reference, whose decode step issues one matmul per weight matrix and one
 * dispatch per pointwise op between them (src/gguf_cache.js:121-171: rmsnorm, wq/wk/wv, ..., wo, add,
 * rmsnorm, gate, up, swiglu, down, add).  A LIST of GEMV-shaped products (M <= 4, one kind) that run
 * as ONE persistent launch: one CTA per SM walks the list with its ring of weight stages never
 * draining between matrices, so the start-up and tail every separate launch pays (2.7 of 9.0 us at
 * 4096 x 14336) are paid once per list.  Item i computes
 *     x   = gamma ? rmsnorm(a, gamma, eps) : a          (shaders/rmsnorm.metal:15-49; a is f32 [M,K])
 *     p   = x * dequant(b)                              (shaders/matmul_q4.metal:34-65 / matmul_q8.metal:20-57)
 *     p   = b2 ? silu(p) * (x * dequant(b2)) : p        (shaders/swiglu.metal:12-22; b = gate, b2 = up)
 *     c   = residual ? residual + p : p                 (A.add, src/gguf_cache.js:153,165)
 * Operands are buffers with a device side plus byte offsets, so rows of one arena can be chained.
 * Items may read what earlier items write (and overwrite what earlier items read or wrote): such
 * hazards are found when the list is created, from the operands' address ranges, and resolved on the
 * device (the consumer of a hazard waits -- bounded -- for the producer's tiles; weights keep
 * streaming meanwhile).  c must not overlap the item's own a; residual may be c itself.
 * At most four mutually independent earlier items may conflict with one item.
 * Results per item are those of smith_qmatmul on the GEMV path, with the pointwise operations in
 * f32.  smith_qmatmul_list_create allocates device memory (not during capture);
 * smith_qmatmul_list_run is asynchronous on the context's stream, allocates nothing and may be
 * captured in a graph; runs of one list must not overlap on the GPU.  A bounded wait that gives up
 * shows in smith_kernel_status; the list is usable again afterwards. */
typedef struct SmithListItem {
  void* a;          uint64_t a_offset;         /* f32 [M,K] */
  void* b;          uint64_t b_offset;         /* packed [K/32][N][24 or 34 bytes] */
  void* b2;         uint64_t b2_offset;        /* NULL, or the `up` matrix of a gate/up pair (same N, K) */
  void* c;          uint64_t c_offset;         /* f32 [M,N] */
  void* gamma;                                 /* NULL, or f32 [K] */
  void* residual;   uint64_t residual_offset;  /* NULL, or f32 [M,N] */
  uint64_t N, K;
  float eps;                                   /* RMSNorm epsilon (used when gamma is set) */
  uint32_t reserved;
} SmithListItem;
void* smith_qmatmul_list_create(void* ctx, uint32_t kind, uint64_t M, const SmithListItem* items, uint32_t count);
int32_t smith_qmatmul_list_run(void* ctx, void* list);
void smith_qmatmul_list_destroy(void* list);
/* The same list with weights sharded along N over the GPUs of one box (one process per GPU): gathers[i]
 * (world != 0) makes item i end in a fused all-gather.  The item's N columns are then columns
 * [n0, n0 + N) of a row of n_total, and its threads store them, besides c, into EVERY rank's row buffer
 * rows[r] (local, or another process's buffer opened with smith_ipc_import): one 8-byte store
 * {value bits, launch tag} per element and rank, plain stores over NVLink, no fence -- a reader accepts a
 * pair by its tag.  A row buffer holds 2 * M * n_total such pairs (zero-initialised once); launch number
 * t (1, 2, ...; smith_qmatmul_list_next_tag) fills half t % 2, where pair m * n_total + col holds element
 * (m, col) of the gathered row.  Before the launch ends, every rank waits -- bounded, ~0.2 s, reported by
 * smith_kernel_status -- until its own row buffers are whole, unless SMITH_LIST_NO_CLOSING_WAIT is given;
 * that wait also keeps the ranks within one launch of each other, which is what lets the halves
 * alternate.  Every rank must create the same list (its own shards) and run it the same number of times. */
typedef struct SmithListGather {
  uint32_t world;            /* 0: item i is not gathered */
  uint32_t reserved;
  uint64_t n0, n_total;
  void* rows[8];             /* rank r's row buffer (a buffer handle) */
} SmithListGather;
#define SMITH_LIST_NO_CLOSING_WAIT 1u
void* smith_qmatmul_list_create_gather(void* ctx, uint32_t kind, uint64_t M, const SmithListItem* items,
                                       const SmithListGather* gathers, uint32_t count, uint32_t rank, uint32_t flags);
/* Tag the next launch of the list will use (the last finished launch used one less); 0 on error.
 * Synchronises the device. */
uint32_t smith_qmatmul_list_next_tag(void* list);
/* 1 if an item of this shape can be part of a list. */
int32_t smith_qmatmul_list_supports(uint32_t kind, uint64_t M, uint64_t N, uint64_t K);
/* Device-side waits in these kernels (on a shared-memory barrier, a peer's
 * flag) are bounded; one that gives up marks the launch's result invalid.
 * Returns 1 if that happened on this context's device since the last call
 * (and clears the mark), 0 if not, negative on error.  Synchronises the stream. */
int32_t smith_kernel_status(void* ctx);
/* How many kernels this context has launched so far. */
uint64_t smith_launch_count(void* ctx);

/* Multi-GPU, one process per GPU (no counterpart in the reference, which is single-device).
 * smith_ipc_export writes a 64-byte handle for a PRIVATE buffer; another process on
 * the same box turns it into a buffer over the same device memory with smith_ipc_import
 * (reads and writes then travel over NVLink).  Releasing the imported buffer unmaps it. */
int32_t smith_ipc_export(void* buffer, void* handle_out64);
void* smith_ipc_import(void* ctx, const void* handle64, uint64_t bytes);
/* Fused GEMV + all-gather for weights sharded along N (M <= 4).  This rank multiplies its
 * column shard b (n_local columns starting at column n0 of a row of n_total) and stores the
 * result slice into EVERY rank's gathered output through y_bufs[r] (rank r's buffer of
 * 2*M*n_total floats, local or IPC-imported), then adds its tile arrivals to every rank's
 * state_bufs[r] (16 bytes, zero-initialised once).  The launch completes when this rank's
 * own row has received the tiles of all ranks: `target` = sum over ranks of
 * smith_qgemv_tiles(kind, M, n_local_r, K).  The two halves of y are used alternately:
 * the k-th call (k = 0, 1, ...) on a state leaves its row in half k % 2.  The wait is
 * bounded (~0.2 s); if a peer never arrives, smith_kernel_status reports it.
 * Every rank must make the same sequence of calls.  Asynchronous; may be captured in a graph. */
int32_t smith_qmatmul_allgather(void* ctx, uint32_t kind, void* a, void* b, uint64_t M, uint64_t n_total,
                                uint64_t n0, uint64_t n_local, uint64_t K, uint64_t groups, uint32_t world,
                                uint32_t rank, void* const* y_bufs, void* const* state_bufs, uint32_t target);
/* The same with flags.  SMITH_GATHER_DEFER (1): the low-latency form.  A system-scope fence per CTA
 * costs several microseconds per launch, so this form has none: every output travels as one 8-byte
 * store {value bits, step + 1}, y_bufs[r] are then arrays of 2*M*n_total such pairs (zero-initialised
 * once), and a reader accepts a pair only when it carries the tag of the step it expects.  The launch
 * neither signals nor waits; the next smith_qmatmul_allgather_ex call on the same state checks the
 * tags of the previous row -- before it reads its activations if that row is its input (its
 * weights are streaming by then, so the NVLink latency is hidden), otherwise after its main loop
 * and before its own stores (a rank never runs further ahead than that) -- and a chain of such calls is closed by
 * smith_allgather_wait (asynchronous, bounded like the others), after which the last row is whole
 * on this rank: pair i of half (k % 2) after the k-th call holds element i of the row.  `target`
 * is not used in this form. */
#define SMITH_GATHER_DEFER 1u
/* With SMITH_GATHER_DEFER: the activations of this call are the row the previous call on the same
 * state gathered (K == n_total); `a` is then only a placeholder for the very first call of a state. */
#define SMITH_GATHER_INPUT_IS_PREVIOUS_ROW 2u
int32_t smith_qmatmul_allgather_ex(void* ctx, uint32_t kind, void* a, void* b, uint64_t M, uint64_t n_total,
                                   uint64_t n0, uint64_t n_local, uint64_t K, uint64_t groups, uint32_t world,
                                   uint32_t rank, void* const* y_bufs, void* const* state_bufs, uint32_t target,
                                   uint32_t flags);
int32_t smith_allgather_wait(void* ctx, void* state_buf, void* y_buf, uint64_t M, uint64_t n_total);
int32_t smith_qgemv_tiles(uint32_t kind, uint64_t M, uint64_t N, uint64_t K);
/* Fused GEMV + all-reduce for weights sharded along K (M <= 4; the Wo / down projections of a
 * tensor-parallel layer).  This rank multiplies its K-slice: a = [M, k_local] activations, b = its
 * groups_local = k_local / 32 group-rows of all N columns (a contiguous byte range of the packed
 * matrix).  partial_bufs[r] is rank r's slot array: 2 * world * M * N pairs of {value, step tag}
 * (8 bytes each, zero-initialised once; local or IPC-imported).  Every thread pushes its partial sums
 * into this rank's slot on every rank with single 8-byte stores -- no fence: a pair is valid
 * exactly when it carries the step's tag -- then polls (bounded, ~0.2 s) the same elements of all
 * slots in its own memory, adds them in rank order (identical bits on every rank) and writes the sum
 * to out [M, N].  state_bufs[r]: smith_qmatmul_allreduce_state_bytes bytes, zero-initialised once.
 * If a peer never arrives smith_kernel_status reports it.  Every rank must make the same sequence
 * of calls.  Asynchronous; may be captured in a graph. */
int32_t smith_qmatmul_allreduce(void* ctx, uint32_t kind, void* a, void* b, void* out, uint64_t M, uint64_t N,
                                uint64_t k_local, uint64_t groups_local, uint32_t world, uint32_t rank,
                                void* const* partial_bufs, void* const* state_bufs);
uint64_t smith_qmatmul_allreduce_state_bytes(uint32_t kind, uint64_t M, uint64_t N, uint64_t k_local);

/* No counterpart in the reference.  The same product as smith_qmatmul, for
 * callers that cannot allocate device memory when they make the call: a
 * serving process whose memory was all handed to its own arena at start-up, a
 * latency-critical loop or host callback where cudaMalloc (which synchronises
 * the device) is off limits, or a runtime that holds raw device pointers and
 * no smith context.  It takes raw device pointers (a: f32 [M,K], b: packed
 * blocks, c: f32 [M,N], all on the current device, a and b 16-byte aligned) and
 * a cudaStream_t (NULL = default stream), always runs the tensor-core kernel,
 * and keeps that kernel's scratch (a 16-bit copy of the activations) in a
 * fixed 8 MiB array inside the library image instead of allocating it.
 *   - Limit: M*K*2 (rounded up to 256) + 256 + M*4 bytes must fit in 8 MiB
 *     (for example M*K <= 4 Mi elements less a little); larger calls are
 *     refused with an error, as are shapes the tensor-core kernel does not take
 *     (N % 8, K % 32, groups == K/32; Q4 needs K >= 1024).
 *   - Every GPU that loads the library holds the 8 MiB until the process exits.
 *   - The first call on a device looks up the array's device address (and the
 *     first call of each kernel variant sets its shared-memory attribute): make
 *     that first call before any stream capture.
 *   - All calls on a device share the one array and find in it whatever the
 *     previous call left; nothing in it needs to start at zero.  Two calls that
 *     overlap on the GPU (different streams, or graphs replayed concurrently)
 *     race on it: keep calls on one device ordered.
 *   - Calls no cudaMalloc / cudaFree and no allocating library routine.
 * Asynchronous on `stream`.  Returns 0 on success, non-zero with smith_last_error() set. */
int32_t smith_qmatmul_static(uint32_t kind, const void* a_dev, const void* b_dev, void* c_dev, uint64_t M,
                             uint64_t N, uint64_t K, uint64_t groups, void* stream);

/* CUDA-graph capture of a sequence of the asynchronous calls above. */
int32_t smith_graph_begin(void* ctx);
void* smith_graph_end(void* ctx); /* executable graph handle, NULL on failure */
int32_t smith_graph_launch(void* ctx, void* graph);
void smith_graph_destroy(void* graph);

/* Synthetic data on the device: f32 ~ N(0, std) from a counter-based generator
 * keyed by (seed, element index); for benchmarks and large-shape tests. */
int32_t smith_fill_normal(void* ctx, void* buffer, uint64_t count, uint64_t seed, float std);
/* Writes `bytes` of a scratch buffer to push earlier data out of L2. */
int32_t smith_flush_l2(void* ctx);

#ifdef __cplusplus
}
#endif
#endif /* SMITH_CUDA_BRIDGE_H */
