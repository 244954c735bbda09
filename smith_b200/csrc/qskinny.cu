// qskinny.cu -- skinny quantized matmul, 5 <= M <= 64 rows of activations, on f16 mma.sync.
//
// C[M,N] = A[M,K] (f32) x dequant(B); B in Smith's Q4 (24-byte) or Q8 (34-byte) block layout,
// block (g, col) at (g*N + col) * block_bytes (shaders/matmul_q4.metal:47-55,
// shaders/matmul_q8.metal:40-48).
//
// In this range the product is still bound by streaming the packed weights once, but the two other
// kernels that take it spend their time on instructions, not on HBM (measured at 4096 x 14336): the
// integer mma.sync kernel applies a scale to every (column, group) sum on the CUDA cores (25 to 40
// warp instructions per 8 x 32 slice: 17 to 37 us), and the tcgen05 kernel de-quantises every weight
// into a shared-memory tile first (7.6 instructions per weight, 59 % of the issue slots: 28 us flat up
// to 128 rows).  Here the weights are de-quantised in REGISTERS, straight into the B fragments of
// mma.sync.m16n8k16 (f16 inputs, f32 accumulators that run through all of K, so nothing is done per
// group but the de-quantisation itself):
//
//  * convert_rows_f16: activations f32 -> f16 in scratch memory, each row multiplied by the power of
//    two that puts its largest magnitude in [2^13, 2^14) (the inverse is applied to the outputs),
//    laid out [group][row][32 values] with the 32 values of a group in the order the B fragments
//    produce their codes, and the four 16-byte chunks of a row XOR-swizzled so that ldmatrix reads
//    eight rows without bank conflicts.  The 64 bytes of a (group, row) make the stage's activation
//    slab one contiguous bulk copy.
//  * main kernel: one CTA owns TN = 8 * NS adjacent columns and all of K; a consumer warp owns up to
//    four 8-column slices and one K-phase and keeps its f32 accumulators for the whole launch.  Per
//    group of 32 and slice, lane (n = lane / 4, j = lane % 4) reads the 8 codes k = 8j .. 8j+7 of
//    column n as one word, turns them into four half2 with one mask-and-magic-number LOP3 each
//    (0x6400 | code = 1024 + code), subtracts the 1024 exactly and applies scale and zero point with
//    one HFMA2: w = code * scale_h + (-zero * scale)_h.  Q8 codes go through a byte permute the same
//    way.  Two MMAs per group, slice and 16-row tile; A fragments come from one ldmatrix.x4 per MMA
//    step and tile and are reused for the warp's slices.
//  * producer warp, bulk-async ring of {weights, activation slab} stages, full/empty mbarriers,
//    bounded waits and the fixed-order phase reduction as in the other streaming kernels.
//
// Accuracy: activations and de-quantised weights are rounded to f16 (2^-11 relative); sums are f32.
// Typical error is about a hundredth of the stated bound (1e-3 * ||a_m|| * ||w_deq[:,n]||) at
// K = 4096; the tests hold every output to the bound.
#include <cuda_fp16.h>

#include "kernels.h"
#include "pipeline.cuh"

namespace smith {
namespace {

constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 220 * 1024;
constexpr int kMaxSlicesPerWarp = 4;

struct Params {
  const uint8_t* B;
  const uint8_t* xh;       // [G][Mp][64 bytes] f16 activations, permuted and swizzled
  const float* row_inv;    // [Mp] inverse of the rows' power-of-two prescale
  float* C;
  int M, Mp, N, K, G;
  int NS, WG, phases;      // 8-column slices per CTA, warp groups (of up to 4 slices), K-phases
  int row_pitch, stage_rows, w_bytes, a_bytes, stage_bytes, stages;
  int* status;
};

__device__ __forceinline__ void hmma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ float2 lds_f32x2(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t x, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(x), "r"(mask), "r"(orv));   // (x & mask) | orv
  return r;
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// Position of packed element k (0..31 inside its group) in the activation slab's order, i.e. the
// order in which the B fragments below present the codes to the two MMA steps of a group.
//   Q4: lane j's word holds codes 8j .. 8j+7 as nibbles 0..7; step s takes {nib 2s, nib 2s+4} as the
//       k-pair (2j, 2j+1) and {nib 2s+1, nib 2s+5} as the pair (2j+8, 2j+9).
//   Q8: lane j's bytes 8j .. 8j+7; step s takes bytes (4s, 4s+1) and (4s+2, 4s+3).
template <int KIND>
__host__ __device__ inline int slab_position(int k) {
  const int j = k >> 3, i = k & 7;
  if (KIND == 4) {
    const int s = (i & 3) >> 1, upper = i & 1, hi = i >> 2;     // i = 2s + upper + 4hi
    return s * 16 + upper * 8 + 2 * j + hi;
  }
  const int s = i >> 2, upper = (i >> 1) & 1, hi = i & 1;       // i = 4s + 2 upper + hi
  return s * 16 + upper * 8 + 2 * j + hi;
}

// ---------------------------------------------------------------- activations -> f16 slabs
// One block of 256 threads per row: the row's largest magnitude, then its values scaled, rounded to
// f16 and scattered to their slab positions.  Rows >= M are written as zeros (fragments never need a
// row check).  An inf or NaN anywhere in a row turns the row's factor into NaN, so every output of the
// row is NaN as the reference's would be.
template <int KIND>
__global__ void __launch_bounds__(256) convert_rows_f16(const float* __restrict__ A, uint8_t* __restrict__ xh,
                                                        float* __restrict__ row_inv, int M, int Mp, int K, int G) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");   // A may be the output of the launch before
  __shared__ float red[8];
  __shared__ int bad_any;
  const int row = blockIdx.x;
  if (threadIdx.x == 0) bad_any = 0;
  __syncthreads();
  float amax = 0.f;
  int bad = 0;
  if (row < M)
    for (int k = threadIdx.x; k < K; k += 256) {
      const float v = fabsf(A[(size_t)row * K + k]);
      bad |= !(v <= 3.4028234e38f);
      amax = fmaxf(amax, v);
    }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  if (bad) bad_any = 1;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; i++) amax = fmaxf(amax, red[i]);
  const int ex = (int)(__float_as_uint(amax) >> 23) & 0xFF;
  int e = (ex == 0) ? 0 : (13 - (ex - 127));            // amax * 2^e in [2^13, 2^14)
  e = max(-126, min(126, e));
  const float up = __uint_as_float((unsigned)(127 + e) << 23);
  if (threadIdx.x == 0)
    row_inv[row] = bad_any ? __int_as_float(0x7FC00000) : __uint_as_float((unsigned)(127 - e) << 23);
  for (int k = threadIdx.x; k < K; k += 256) {
    const float v = (row < M && !bad_any) ? A[(size_t)row * K + k] * up : 0.f;
    const int g = k >> 5, pos = slab_position<KIND>(k & 31);
    const int chunk = (pos >> 3) ^ ((row >> 1) & 3);    // XOR swizzle of the row's four 16-byte chunks
    __half* dst = reinterpret_cast<__half*>(xh + ((size_t)g * Mp + row) * 64) + chunk * 8 + (pos & 7);
    *dst = __float2half_rn(v);
  }
}

// ---------------------------------------------------------------- main kernel
// MT: 16-row tiles of activations (Mp = 16 * MT).
template <int KIND, int MT>
__global__ void __launch_bounds__(MT >= 4 ? 512 : (MT == 2 ? 640 : 800), 1) qskinny_kernel(const Params p) {
  constexpr int BB = (KIND == 4) ? kQ4Bytes : kQ8Bytes;
  constexpr int SL = kMaxSlicesPerWarp;
  extern __shared__ __align__(1024) uint8_t smem[];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + kMaxStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 2 * kMaxStages * 8);
  uint8_t* ring = smem + 1024;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int TN = p.NS * 8;
  const int col0 = blockIdx.x * TN;
  const int tn = min(TN, p.N - col0);
  const int nwarps = p.WG * p.phases;
  const int nst = (p.G + p.stage_rows - 1) / p.stage_rows;
  const uint32_t row_bytes = (uint32_t)tn * BB;

  if (tid == 0) {
    for (int s = 0; s < p.stages; s++) {
      mbar_init(smem_u32(&full[s]), 2);                 // weights armed first, the activation slab once it exists
      mbar_init(smem_u32(&empty[s]), nwarps);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp >= nwarps) {
    // ------------------------------------------------------------ producer warp
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    auto issue_weights = [&](int st, int slot) {
      const int rows = min(p.stage_rows, p.G - st * p.stage_rows);
      const uint32_t bar = smem_u32(&full[slot]);
      if (lane == 0) mbar_expect_tx(bar, (uint32_t)rows * row_bytes);
      __syncwarp();
      const uint32_t dst = smem_u32(ring + (size_t)slot * p.stage_bytes);
      const uint8_t* src = p.B + ((size_t)st * p.stage_rows * p.N + col0) * BB;
      for (int rr = lane; rr < rows; rr += 32)
        bulk_load(dst + rr * p.row_pitch, src + (size_t)rr * p.N * BB, row_bytes, bar, policy);
    };
    auto issue_slab = [&](int st, int slot) {
      const int rows = min(p.stage_rows, p.G - st * p.stage_rows);
      const uint32_t bar = smem_u32(&full[slot]);
      const uint32_t bytes = (uint32_t)rows * p.Mp * 64;
      if (lane == 0) {
        mbar_expect_tx(bar, bytes);
        bulk_load_default(smem_u32(ring + (size_t)slot * p.stage_bytes + p.w_bytes),
                          p.xh + (size_t)st * p.stage_rows * p.Mp * 64, bytes, bar);
      }
      __syncwarp();
    };
    // weights of the first ring-full go out before anything waits on the conversion kernel
    const int first = min(nst, p.stages);
    for (int st = 0; st < first; st++) issue_weights(st, st);
    asm volatile("griddepcontrol.wait;" ::: "memory");   // convert_rows_f16 has finished: the slabs exist
    for (int st = 0; st < first; st++) issue_slab(st, st);
    bool live = true;
    int slot = 0;
    uint32_t par = 1;                                    // second pass over the ring
    for (int st = first; st < nst && live; st++, slot = (slot + 1 == p.stages) ? 0 : slot + 1, par ^= (slot == 0)) {
      int okw = 1;
      if (lane == 0) okw = mbar_wait(smem_u32(&empty[slot]), par ^ 1u, abort_flag, p.status);
      live = __shfl_sync(0xffffffffu, okw, 0) != 0;
      if (!live) break;
      issue_weights(st, slot);
      issue_slab(st, slot);
    }
    return;  // consumers observe every full barrier, so the copies land before the CTA ends
  }

  // -------------------------------------------------------------- consumers
  const int wg = warp % p.WG, phase = warp / p.WG;
  const int s0 = wg * SL;                                // first slice of this warp
  const int r = lane >> 2, j = lane & 3;
  int cnt = min(SL, p.NS - s0);                          // slices this warp owns ...
  cnt = min(cnt, (tn - s0 * 8 + 7) / 8);                 // ... that have columns in this tile
  if (cnt < 0) cnt = 0;
  float acc[MT][SL][4];
#pragma unroll
  for (int t = 0; t < MT; t++)
#pragma unroll
    for (int s = 0; s < SL; s++)
#pragma unroll
      for (int i = 0; i < 4; i++) acc[t][s][i] = 0.f;

  const uint32_t ring_s = smem_u32(ring);
  // this lane's codes: word j (Q4) / bytes 2 + 8j .. (Q8) of the block of column (s0 + s) * 8 + r
  const uint32_t off_w = (uint32_t)(s0 * 8 + r) * BB + (KIND == 4 ? 4u * j : 2u + 8u * j);
  const uint32_t sh8 = (off_w & 3u) * 8;                 // 34-byte blocks: 8 slices further along is 272 bytes, same alignment
  const uint32_t off_q = (uint32_t)(s0 * 8 + r) * BB + (KIND == 4 ? 16u : 0u);   // scale (and zero) of that block
  // ldmatrix: lane l addresses row (l % 8) + 8 * ((l / 8) % 2) of a 16-row tile, chunk 2 * step + l / 16
  const int lrow = (lane & 7) + ((lane >> 3) & 1) * 8;
  const uint32_t off_a = (uint32_t)lrow * 64;
  const uint32_t sw = (uint32_t)((lrow >> 1) & 3);
  const uint32_t a_c0 = (((uint32_t)(lane >> 4)) ^ sw) * 16, a_c1 = (((uint32_t)(2 + (lane >> 4))) ^ sw) * 16;
  const uint32_t w_step = (uint32_t)p.phases * (uint32_t)p.row_pitch;
  const uint32_t a_step = (uint32_t)p.phases * (uint32_t)(p.Mp * 64);

  bool ok = true;
  int slot = 0;
  uint32_t par = 0;
  for (int st = 0; st < nst && ok; st++, slot = (slot + 1 == p.stages) ? 0 : slot + 1, par ^= (slot == 0)) {
    ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&full[slot]), par, abort_flag, p.status));
    if (ok && cnt > 0) {
      const uint32_t stage = ring_s + (uint32_t)slot * (uint32_t)p.stage_bytes;
      const int rows_here = min(p.stage_rows, p.G - st * p.stage_rows);
      uint32_t wrow = stage + (uint32_t)phase * (uint32_t)p.row_pitch;
      uint32_t arow = stage + (uint32_t)p.w_bytes + (uint32_t)phase * (uint32_t)(p.Mp * 64);
#pragma unroll 2
      for (int row = phase; row < rows_here; row += p.phases) {
        // ---- B fragments of both steps for the warp's slices
        uint32_t b[SL][4];                               // [slice][step * 2 + {b0, b1}]
#pragma unroll
        for (int s = 0; s < SL; s++) {
          if (s < cnt) {
            const uint32_t wa = wrow + off_w + (uint32_t)s * (8u * BB);
            if (KIND == 4) {
              const uint32_t w = lds32(wa);
              const float2 sz = lds_f32x2(wrow + off_q + (uint32_t)s * (8u * BB));
              const __half2 sc = __float2half2_rn(sz.x), sc16 = __float2half2_rn(sz.x * 0.0625f);
              const __half2 bias = __float2half2_rn(-sz.y * sz.x);
              const uint32_t w8 = w >> 8;
              // 0x6400 | code = 1024 + code (exact in f16); the high-nibble forms carry 16 * code
              const __half2 k1024 = u32_as_h2(0x64006400u);
              const __half2 n04 = __hsub2(u32_as_h2(lop3_and_or(w, 0x000F000Fu, 0x64006400u)), k1024);
              const __half2 n15 = __hsub2(u32_as_h2(lop3_and_or(w, 0x00F000F0u, 0x64006400u)), k1024);
              const __half2 n26 = __hsub2(u32_as_h2(lop3_and_or(w8, 0x000F000Fu, 0x64006400u)), k1024);
              const __half2 n37 = __hsub2(u32_as_h2(lop3_and_or(w8, 0x00F000F0u, 0x64006400u)), k1024);
              b[s][0] = h2_as_u32(__hfma2(n04, sc, bias));
              b[s][1] = h2_as_u32(__hfma2(n15, sc16, bias));
              b[s][2] = h2_as_u32(__hfma2(n26, sc, bias));
              b[s][3] = h2_as_u32(__hfma2(n37, sc16, bias));
            } else {
              // 34-byte blocks are 2-byte aligned: aligned words around the 8 codes, then funnel shifts
              const uint32_t a = wa & ~3u;
              const uint32_t x0 = lds32(a), x1 = lds32(a + 4), x2 = lds32(a + 8);
              const uint32_t c0 = __funnelshift_r(x0, x1, sh8) ^ 0x80808080u;   // codes + 128 as bytes
              const uint32_t c1 = __funnelshift_r(x1, x2, sh8) ^ 0x80808080u;
              const __half2 sc = __half2half2(__ushort_as_half((unsigned short)lds_u16(wrow + off_q + (uint32_t)s * (8u * BB))));
              const __half2 k1152 = u32_as_h2(0x64806480u);                     // 1024 + 128
              // 0x64 above a byte: 1024 + byte
              const __half2 p01 = __hsub2(u32_as_h2(__byte_perm(c0, 0x64646464u, 0x4140)), k1152);
              const __half2 p23 = __hsub2(u32_as_h2(__byte_perm(c0, 0x64646464u, 0x4342)), k1152);
              const __half2 p45 = __hsub2(u32_as_h2(__byte_perm(c1, 0x64646464u, 0x4140)), k1152);
              const __half2 p67 = __hsub2(u32_as_h2(__byte_perm(c1, 0x64646464u, 0x4342)), k1152);
              b[s][0] = h2_as_u32(__hmul2(p01, sc));
              b[s][1] = h2_as_u32(__hmul2(p23, sc));
              b[s][2] = h2_as_u32(__hmul2(p45, sc));
              b[s][3] = h2_as_u32(__hmul2(p67, sc));
            }
          }
        }
        // ---- A fragments (one ldmatrix.x4 per step and tile), reused for every slice
#pragma unroll
        for (int t = 0; t < MT; t++) {
          uint32_t a0[4], a1[4];
          ldmatrix_x4(a0, arow + (uint32_t)t * 1024u + off_a + a_c0);
          ldmatrix_x4(a1, arow + (uint32_t)t * 1024u + off_a + a_c1);
#pragma unroll
          for (int s = 0; s < SL; s++) {
            if (s < cnt) {
              hmma(acc[t][s], a0, b[s][0], b[s][1]);
              hmma(acc[t][s], a1, b[s][2], b[s][3]);
            }
          }
        }
        wrow += w_step, arow += a_step;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&empty[slot]));
  }

  // ---------------------------------------------- sum the phases, fixed order
  asm volatile("bar.sync 1, %0;" ::"r"(nwarps * 32));  // every consumer is done with the ring
  float* red = reinterpret_cast<float*>(ring);        // [phases][Mp][TN]
#pragma unroll
  for (int t = 0; t < MT; t++)
#pragma unroll
    for (int s = 0; s < SL; s++)
      if (s < cnt) {
        float* dst = red + ((size_t)phase * p.Mp + 16 * t + r) * TN + (s0 + s) * 8 + 2 * j;
        *reinterpret_cast<float2*>(dst) = make_float2(acc[t][s][0], acc[t][s][1]);
        *reinterpret_cast<float2*>(dst + 8 * TN) = make_float2(acc[t][s][2], acc[t][s][3]);
      }
  asm volatile("bar.sync 1, %0;" ::"r"(nwarps * 32));
  if (*abort_flag) return;
  for (int i = tid; i < p.M * tn; i += nwarps * 32) {
    const int m = i / tn, c = i - m * tn;
    float sum = 0.f;
    for (int ph = 0; ph < p.phases; ph++) sum += red[((size_t)ph * p.Mp + m) * TN + c];
    p.C[(size_t)m * p.N + col0 + c] = sum * p.row_inv[m];
  }
}

struct Plan {
  Params p;
  int tiles, MT;
  size_t smem;
  bool ok;
};

constexpr int kMaxRows = 64;

Plan make_plan(int kind, int64_t M, int64_t N, int64_t K) {
  const int BB = (kind == 4) ? kQ4Bytes : kQ8Bytes;
  const int sms = device_sm_count();
  Plan pl{};
  Params& p = pl.p;
  p.M = (int)M, p.N = (int)N, p.K = (int)K, p.G = (int)(K / 32);
  pl.MT = (M <= 16) ? 1 : (M <= 32) ? 2 : 4;
  p.Mp = 16 * pl.MT;
  // Slices per CTA: the fewest that cover N in a whole number of waves, at most 16 (128 columns).
  int NS = 0;
  for (int64_t waves = 1;; waves++) {
    NS = (int)((N + 8 * sms * waves - 1) / (8 * sms * waves));
    if (NS <= 16) break;
  }
  p.NS = NS;
  p.WG = (NS + kMaxSlicesPerWarp - 1) / kMaxSlicesPerWarp;
  const int TN = NS * 8;
  pl.tiles = (int)((N + TN - 1) / TN);
  const int max_warps = (pl.MT >= 4) ? 15 : (pl.MT == 2) ? 19 : 24;   // 128 / 96 / 80 registers per thread
  int phases = max_warps / p.WG;
  if (phases < 1) phases = 1;
  while (phases > 1 && phases * 2 > p.G) phases--;       // short K: do not over-split
  p.phases = phases;
  p.row_pitch = TN * BB;
  // stages of about 48 KB (weights + activation slabs), a multiple of the phases
  const int per_row = p.row_pitch + p.Mp * 64;
  int rows = (48 * 1024) / per_row;
  rows = (rows / phases) * phases;
  if (rows < phases) rows = phases;
  if (rows > p.G) rows = ((p.G + phases - 1) / phases) * phases;
  p.stage_rows = rows;
  p.w_bytes = ((p.stage_rows * p.row_pitch + 16 + 127) / 128) * 128;   // + slack for the Q8 read-ahead
  p.a_bytes = p.stage_rows * p.Mp * 64;
  p.stage_bytes = ((p.w_bytes + p.a_bytes + 1023) / 1024) * 1024;
  int stages = (kSmemBudget - 1024) / p.stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  p.stages = stages;
  const size_t red = (size_t)phases * (size_t)p.Mp * TN * 4;
  const size_t ring = (size_t)(stages > 0 ? stages : 0) * p.stage_bytes;
  pl.smem = 1024 + ((((ring > red ? ring : red)) + 1023) / 1024) * 1024;
  pl.ok = stages >= 2 && pl.smem <= 227 * 1024 && M <= kMaxRows && M >= 1;
  return pl;
}

template <typename... Args>
cudaError_t launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <int KIND, int MT>
cudaError_t launch_main(const Plan& pl, cudaStream_t s) {
  static PerDeviceFlag configured;              // the attribute belongs to a device, not to the process
  bool* set = configured.here();
  if (!set) return cudaErrorInvalidDevice;
  if (!*set) {
    cudaError_t e = cudaFuncSetAttribute(qskinny_kernel<KIND, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    *set = true;
  }
  const int threads = (pl.p.WG * pl.p.phases + 1) * 32;
  const cudaError_t e = launch_pdl(qskinny_kernel<KIND, MT>, dim3((unsigned)pl.tiles), dim3((unsigned)threads), pl.smem, s, pl.p);
  count_launch();
  return e;
}

}  // namespace

bool qskinny_supports(int kind, int64_t M, int64_t N, int64_t K, int64_t groups) {
  if (kind != 4 && kind != 8) return false;
  if (M < 1 || M > kMaxRows) return false;
  if (N < 8 || (N % 8) != 0) return false;       // 16-byte alignment of every group-row span
  if (K < 32 || (K % 32) != 0 || groups != K / 32) return false;
  if (N > (1 << 30) || K > (1 << 22)) return false;
  return make_plan(kind, M, N, K).ok;
}

size_t qskinny_workspace_bytes(int kind, int64_t M, int64_t N, int64_t K) {
  const Plan pl = make_plan(kind, M, N, K);
  const size_t G = (size_t)(K / 32), Mp = (size_t)pl.p.Mp;
  return ((G * Mp * 64 + 255) & ~size_t(255)) + Mp * 4 + 64;
}

cudaError_t launch_qskinny(int kind, const float* A, const uint8_t* B, float* C, int64_t M, int64_t N, int64_t K,
                           int64_t groups, Workspace ws, cudaStream_t s) {
  (void)groups;
  Plan pl = make_plan(kind, M, N, K);
  if (!pl.ok) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(A) & 15)) return cudaErrorMisalignedAddress;
  const size_t need = qskinny_workspace_bytes(kind, M, N, K);
  if (!ws.ptr || ws.bytes < need || (reinterpret_cast<uintptr_t>(ws.ptr) & 255)) return cudaErrorInvalidValue;
  const size_t G = (size_t)(K / 32), Mp = (size_t)pl.p.Mp;
  uint8_t* xh = static_cast<uint8_t*>(ws.ptr);
  float* row_inv = reinterpret_cast<float*>(xh + ((G * Mp * 64 + 255) & ~size_t(255)));
  cudaError_t e;
  if (kind == 4)
    e = launch_pdl(convert_rows_f16<4>, dim3((unsigned)Mp), dim3(256), (size_t)0, s, A, xh, row_inv, (int)M, (int)Mp, (int)K, (int)G);
  else
    e = launch_pdl(convert_rows_f16<8>, dim3((unsigned)Mp), dim3(256), (size_t)0, s, A, xh, row_inv, (int)M, (int)Mp, (int)K, (int)G);
  count_launch();
  if (e != cudaSuccess) return e;
  pl.p.B = B, pl.p.C = C, pl.p.xh = xh, pl.p.row_inv = row_inv;
  pl.p.status = kernel_status_ptr();
  if (!pl.p.status) return cudaErrorUnknown;
#define SMITH_SKINNY_CASE(KD, MTV) \
  if (kind == KD && pl.MT == MTV) return launch_main<KD, MTV>(pl, s);
  SMITH_SKINNY_CASE(4, 1) SMITH_SKINNY_CASE(4, 2) SMITH_SKINNY_CASE(4, 4)
  SMITH_SKINNY_CASE(8, 1) SMITH_SKINNY_CASE(8, 2) SMITH_SKINNY_CASE(8, 4)
#undef SMITH_SKINNY_CASE
  return cudaErrorInvalidValue;
}

}  // namespace smith
