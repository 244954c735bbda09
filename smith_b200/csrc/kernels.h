// kernels.h -- launch entry points shared between the kernel files and the
// C-ABI layer (bridge.cu).  Everything here takes raw device pointers and a
// stream and launches asynchronously.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace smith {

constexpr int kQ4Group = 32;  // elements per Q4 block (src/ops/quantize.js:9)
constexpr int kQ4Bytes = 24;  // 16 nibble bytes + f32 scale + f32 zero (src/ops/quantize.js:10)
constexpr int kQ8Group = 32;  // elements per Q8 block (src/ops/quantize.js:94)
constexpr int kQ8Bytes = 34;  // f16 scale + 32 int8 (src/ops/quantize.js:95)

enum Path : int { kAuto = 0, kGeneric = 1, kDecode = 2, kTensor = 3, kGemv = 4, kSkinny = 5 };

// Scratch memory a matmul launch may use (owned by the caller of the launch).
struct Workspace {
  void* ptr = nullptr;
  size_t bytes = 0;
};

// Counts kernel launches made through these entry points.
extern thread_local uint64_t* g_launch_counter;
inline void count_launch(int n = 1) {
  if (g_launch_counter) *g_launch_counter += (uint64_t)n;
}

// pack.cu
cudaError_t launch_pack_q4(const float* w, uint8_t* out, int64_t K, int64_t N, cudaStream_t s);
cudaError_t launch_pack_q8(const float* w, uint8_t* out, int64_t K, int64_t N, cudaStream_t s);

// gguf_repack.cu : GGUF Q8_0 (ggml type 8) / Q4_0 (type 2) blocks of a [out_dim, in_dim] tensor -> the
// [in_dim/32][out_dim][block] layouts the matmul kernels read (K = in_dim, N = out_dim).
cudaError_t launch_gguf_repack(int ggml_type, const uint8_t* src, uint8_t* dst, int64_t out_dim, int64_t in_dim,
                               cudaStream_t s);

// qmatmul_generic.cu : any shape, CUDA cores, sequential-k f32 accumulation.
cudaError_t launch_qmatmul_generic(int kind, const float* A, const uint8_t* B, float* C, int64_t M,
                                   int64_t N, int64_t K, int64_t groups, cudaStream_t s);

// qdecode.cu : M <= 16, activations as int8 digit pairs in scratch, integer mma.sync against the codes.
bool qdecode_supports(int kind, int64_t M, int64_t N, int64_t K, int64_t groups);
size_t qdecode_workspace_bytes(int kind, int64_t M, int64_t N, int64_t K);
// digits_in_scratch: the launch before this one on the same stream was launch_qdecode with the same
// kind, A, M and K and also kept its digits in `ws` (qdecode_uses_scratch): they are not made again.
bool qdecode_uses_scratch(int kind, int64_t M, int64_t N, int64_t K);
cudaError_t launch_qdecode(int kind, const float* A, const uint8_t* B, float* C, int64_t M,
                           int64_t N, int64_t K, int64_t groups, Workspace ws, cudaStream_t s,
                           bool digits_in_scratch = false);

// qskinny.cu : M <= 64, activations as f16 slabs in scratch, weights de-quantised in registers into
// the B fragments of f16 mma.sync, f32 accumulators through all of K.
bool qskinny_supports(int kind, int64_t M, int64_t N, int64_t K, int64_t groups);
size_t qskinny_workspace_bytes(int kind, int64_t M, int64_t N, int64_t K);
cudaError_t launch_qskinny(int kind, const float* A, const uint8_t* B, float* C, int64_t M,
                           int64_t N, int64_t K, int64_t groups, Workspace ws, cudaStream_t s);

// qgemm_tc.cu : M > 16, dequantise to bf16 tiles in shared memory, tcgen05 MMA, TMEM accumulators.
bool qgemm_tc_supports(int kind, int64_t M, int64_t N, int64_t K, int64_t groups);
size_t qgemm_tc_workspace_bytes(int kind, int64_t M, int64_t N, int64_t K);
cudaError_t launch_qgemm_tc(int kind, const float* A, const uint8_t* B, float* C, int64_t M,
                            int64_t N, int64_t K, int64_t groups, Workspace ws, cudaStream_t s);

// dense_generic.cu / dense_tc.cu : the unquantised matmul, f32 or f16 storage.
enum DenseType : int { kDenseF32 = 0, kDenseF16 = 1 };
enum DensePath : int { kDenseAuto = 0, kDenseGeneric = 1, kDenseTcExact = 2, kDenseTcFast = 3 };
cudaError_t launch_dense_generic(int dtype, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                                 int64_t batch, cudaStream_t s);
bool dense_tc_supports(int dtype, int64_t M, int64_t N, int64_t K);
size_t dense_tc_workspace_bytes(int dtype, int mode, int64_t M, int64_t N, int64_t K);
cudaError_t launch_dense_tc(int dtype, int mode, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                            Workspace ws, cudaStream_t s);

// qgemv.cu : M <= 4, activations as int8 digit pairs, dp4a against the packed codes.
bool qgemv_supports(int kind, int64_t M, int64_t N, int64_t K, int64_t groups);
cudaError_t launch_qgemv(int kind, const float* A, const uint8_t* B, float* C, int64_t M, int64_t N,
                         int64_t K, int64_t groups, cudaStream_t s);
// Same launch ending in a fused all-gather: the N columns computed here are this rank's slice
// [n0, n0 + N) of a row of n_total columns, stored into every rank's gathered buffers.
struct GemvGather {
  float* y[8];          // per rank: gathered output, two buffers [2][M][n_total]
  unsigned* state[8];   // per rank: control words {step, ticket, arrivals[0], arrivals[1]}
  int world, rank;
  int64_t n0, n_total;
  unsigned target;      // CTAs (tiles) arriving per step, summed over ranks
  // reduce != 0: weights are sharded along K instead; y[r] are rank r's slots [2][world][M][N] of
  // {value, step + 1} pairs (one slot per contributing rank) and C receives the sum over ranks
  // (n0 = 0, n_total = N, target unused).
  int reduce;
  // all-gather only, deferred form: y[r] are arrays [2][M][n_total] of 8-byte {value, step + 1}
  // pairs; the launch neither fences nor signals nor waits, and the next launch on the same state
  // (or launch_gather_wait) polls the tags of this step's row (`target` is not used)
  int defer;
  int a_prev;           // deferred form: read the activations from the previous step's gathered row (K == n_total)
};
// Returns when the last deferred all-gather step's row (tagged pairs in y) is whole on this rank
// (bounded wait).
cudaError_t launch_gather_wait(const unsigned* state, const void* y, int64_t M, int64_t n_total, cudaStream_t s);

cudaError_t launch_qgemv_gather(int kind, const float* A, const uint8_t* B, float* C, int64_t M, int64_t N,
                                int64_t K, int64_t groups, const GemvGather* g, cudaStream_t s);
// Up to four weight matrices that share the activations A [M, K], as one launch:
// C_i [M, N_i] = A x dequant(B_i).
bool qgemv_supports_multi(int kind, int64_t M, const int64_t* Ns, int count, int64_t K, int64_t groups);
cudaError_t launch_qgemv_multi(int kind, const float* A, int count, const uint8_t* const* Bs, float* const* Cs,
                               const int64_t* Ns, int64_t M, int64_t K, int64_t groups, cudaStream_t s);
// Grid size the GEMV uses for a shape (-1 if it does not take it).
int qgemv_tiles(int kind, int64_t M, int64_t N, int64_t K);

// qgemv_list.cu : a list of GEMV-shaped products (M <= 4) as one persistent launch, with the
// decode step's pointwise glue folded in.  Raw device pointers; every item of a list has the same
// kind and M.
struct ListItemDesc {
  const float* A;          // activations f32 [M, K]
  const uint8_t* B;        // packed weights [K/32][N][block]
  const uint8_t* B2;       // null, or the `up` matrix of a gate/up pair: C = silu(A x B) * (A x B2)
  float* C;                // output f32 [M, N]
  const float* gamma;      // null, or RMSNorm weights [K]: the product reads rmsnorm(A) * gamma
  const float* residual;   // null, or f32 [M, N] added to the product (may be C)
  int64_t N, K;
  float eps;               // RMSNorm epsilon
  // Fused all-gather of the output over peer memory (g_world == 0: none): this rank's N columns are
  // columns [g_n0, g_n0 + N) of a row of g_n_total; g_rows[r] is rank r's row buffer of
  // 2 * M * g_n_total {value, launch tag} pairs (zero-initialised once, local or peer-mapped).
  int g_world;
  int64_t g_n0, g_n_total;
  void* g_rows[8];
};
// qgemv_list_create flags
constexpr unsigned kListNoClosingWait = 1u;   // do not wait, before the launch ends, for the gathered rows to be whole
struct ListProgram;
bool qgemv_list_supports(int kind, int64_t M, int64_t N, int64_t K);
// Plans the list for the current device and uploads it (allocates device memory).  nullptr with
// *why set on failure.
ListProgram* qgemv_list_create(int kind, int64_t M, const ListItemDesc* items, int count, int rank, unsigned flags,
                               const char** why);
// Tag of the next launch of the list (tags start at 1; reads device memory, synchronises the device).
unsigned qgemv_list_next_tag(const ListProgram* lp);
cudaError_t qgemv_list_launch(const ListProgram* lp, cudaStream_t s);
void qgemv_list_destroy(ListProgram* lp);
size_t list_device_bytes(const ListProgram* lp);
int list_grid(const ListProgram* lp);
uint64_t qgemv_list_weight_bytes(const ListProgram* lp);

// Same computation with the scratch in a fixed array inside the library image (no allocation).
cudaError_t launch_qgemm_tc_static(int kind, const float* A, const uint8_t* B, float* C, int64_t M, int64_t N,
                                   int64_t K, int64_t groups, cudaStream_t s, const char** why);

// util.cu
// Number of SMs of the current device (cached per device; 148 if the query fails).
int device_sm_count();
// Per-device "this kernel's attributes are set" flags: function attributes such as the dynamic
// shared-memory limit belong to a device, so a flag per process would leave the second device of a
// process unconfigured.  Returns the slot for the current device (nullptr on error).
struct PerDeviceFlag {
  bool done[64] = {false};
  bool* here();
};
// 1 if a bounded device-side wait gave up since the last call (then clears it), 0 if not, -1 on error.
int kernel_take_status();
// Device address of that status word on the current device (nullptr on error).
int* kernel_status_ptr();
cudaError_t launch_fill_normal(float* out, uint64_t count, uint64_t seed, float std, cudaStream_t s);
cudaError_t launch_fill_bytes(void* out, size_t bytes, uint32_t value, cudaStream_t s);

// Path resolution for kAuto.
int resolve_path(int kind, int64_t M, int64_t N, int64_t K, int64_t groups);

}  // namespace smith
