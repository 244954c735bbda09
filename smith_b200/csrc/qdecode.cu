// qdecode.cu -- decode-shaped quantized matmul, M <= 16 rows of activations,
// on the integer tensor-core path (mma.sync m16n8k32, s8 x s8 -> s32).
//
// C[M,N] = A[M,K] (f32) x dequant(B); B in Smith's Q4 (24-byte) or Q8 (34-byte)
// block layout, block (g, col) at (g*N + col) * block_bytes
// (shaders/matmul_q4.metal:47-55, shaders/matmul_q8.metal:40-48).
//
// Like the GEMV kernel this is bound by streaming the packed weights once, and
// like it the activations are first turned into block fixed point: per group of
// 32, a power-of-two scale that moves the largest magnitude under 2^14, an
// integer x_int, and two int8 digits (x_int = hi * 128 + lo).  Here that is
// done once per launch by a small kernel (quantise_rows) into scratch memory,
// laid out [group][row][64 bytes] so that the digits of a pipeline stage are
// one contiguous span that is bulk-copied next to the stage's weights.
//
// When all digits of the launch fit beside the weight ring (short K or few rows) the main
// kernel does the conversion itself, into shared memory, and there is no separate kernel.
// Rows are padded to 8 (M <= 8) or to a multiple of 16 with zero digits, so fragments never
// need a row check.
//
// Main kernel: one CTA owns TN = 8 * NS adjacent columns and all of K.  A
// consumer warp owns one 8-column slice and one K-phase (warp = phase * NS +
// slice), keeps that slice's f32 accumulators in registers for the whole
// launch, and walks the group-rows of its phase.  Per 32-weight group and slice:
//   * B fragment: lane (n = lane/4, j = lane%4) reads the j-th 8 codes of
//     column n's block; Q4 nibbles become bytes with two masks (even codes,
//     odd codes), Q8 codes are bytes already.  No arithmetic on the codes.
//   * A fragment: one 16-byte load of the digit words {hi, lo} x {first four,
//     second four} codes in the same order.  With M <= 8 the MMA's rows 0-7
//     carry the high digits and rows 8-15 the low digits of the same
//     activation rows (one MMA per group); wider M runs tiles of 16 rows, two MMAs each.
//   * The s32 results are exact; dot = 128 * hi + lo is converted to f32 once
//     and scaled:  acc += (scale * 2^-e) * (dot - zero * sum_k x_int)  (Q4),
//     acc += (scale * 2^-e) * dot  (Q8).
// Phases are summed through shared memory in fixed order; every output is
// written once.  Producer warp, bulk-async ring, full/empty mbarriers and
// bounded waits as in the GEMV kernel; both kernels are launched with
// programmatic stream serialisation, and the producer streams weights before
// it waits for the digits of quantise_rows.
#include <cuda_fp16.h>

#include "kernels.h"
#include "pipeline.cuh"

namespace smith {
namespace {

constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 200 * 1024;
constexpr int kMaxConsumerWarps = 28;
constexpr int kStageRows = 16;         // group-rows per pipeline stage (rounded up to a multiple of the phases)

struct Params {
  const uint8_t* B;
  const uint8_t* xdig;     // [G][M][64] digit words
  const float2* xsc;       // [G][M] {2^-e, float(sum_k x_int)}
  float* C;
  const float* A;          // activations, read directly when the digits are resident
  int M, Mp, N, K, G;      // Mp: rows padded to 8 or a multiple of 16
  int res_off;             // resident digits: byte offset in shared memory (0 = streamed from scratch)
  int NS, phases;          // slices per CTA (TN = 8 * NS), K-phases; consumer warps = NS * phases
  int row_pitch, stage_rows, w_bytes, d_bytes, s_bytes, stage_bytes, stages;
  int* status;
};

__device__ __forceinline__ void imma(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Shared-memory loads by 32-bit address (keeps the hot loop's address arithmetic to single adds).
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ float2 lds_f32x2(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ uint4 lds_u32x4(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}

// ---------------------------------------------------------------- activations -> digits (global scratch)
// Eight threads per (group, row), four consecutive k each.  Digit layout of a (group, row): 16 words.
//   Q4: word j*4 + {0,1,2,3} = {even-k hi, even-k lo, odd-k hi, odd-k lo} of k = 8j .. 8j+7
//       (byte b of an even word is k = 8j + 2b) -- the order in which two masks pull the codes out of a word.
//   Q8: word j*4 + {0,1,2,3} = {hi, lo of k = 8j .. 8j+3, hi, lo of k = 8j+4 .. 8j+7}.
// One (group, padded row): 8 lanes (lane8 = 0..7), four consecutive k each.  Rows >= M get zero digits.
template <int KIND>
__device__ __forceinline__ void quantise_pair(const float* __restrict__ A, int M, int K, int g, int m, int lane8,
                                              uint8_t* d, float2* sc_out) {
  float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (m < M) v4 = __ldg(reinterpret_cast<const float4*>(A + (size_t)m * K + (size_t)g * 32) + lane8);
  const float v[4] = {v4.x, v4.y, v4.z, v4.w};
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  int bad = 0;
#pragma unroll
  for (int i = 0; i < 4; i++) bad |= !(fabsf(v[i]) <= 3.4028234e38f);
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    bad |= __shfl_xor_sync(0xffffffffu, bad, o);
  }
  const int ex = (int)(__float_as_uint(amax) >> 23) & 0xFF;
  int e = (ex == 0) ? 0 : (13 - (ex - 127));
  e = max(-126, min(126, e));
  const float up = __uint_as_float((unsigned)(127 + e) << 23);
  float down = __uint_as_float((unsigned)(127 - e) << 23);
  if (bad) down = __int_as_float(0x7FC00000);  // inf / NaN activations reach every output of the row
  int q[4], sum = 0;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    q[i] = max(-16383, min(16383, __float2int_rn(v[i] * up)));
    sum += q[i];
  }
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (d == nullptr) return;
  if (KIND == 4) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int word = lane8 >> 1, byte = ((lane8 & 1) << 1) | (i >> 1), odd = i & 1;
      uint8_t* w = d + word * 16 + odd * 8 + byte;
      w[0] = (uint8_t)(q[i] >> 7);
      w[4] = (uint8_t)(q[i] & 127);
    }
  } else {
    uint32_t hi = 0, lo = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      hi |= (uint32_t)((q[i] >> 7) & 0xFF) << (8 * i);
      lo |= (uint32_t)(q[i] & 127) << (8 * i);
    }
    reinterpret_cast<uint2*>(d)[lane8] = make_uint2(hi, lo);
  }
  if (lane8 == 0) *sc_out = make_float2(down, (float)sum);
}

template <int KIND>
__global__ void __launch_bounds__(256) quantise_rows(const float* __restrict__ A, uint8_t* __restrict__ xdig,
                                                     float2* __restrict__ xsc, int M, int Mp, int K, int G) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // A may be the output of the launch before
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  int pair = t >> 3;                       // (group, padded row)
  const bool live = pair < Mp * G;
  if (!live) pair = Mp * G - 1;            // keep whole warps in the shuffles
  const int g = pair / Mp, m = pair - g * Mp;
  quantise_pair<KIND>(A, M, K, g, m, t & 7, live ? xdig + (size_t)pair * 64 : nullptr, xsc + pair);
}

// ---------------------------------------------------------------- main kernel
// NT = 0: M <= 8, one MMA per group (high digits in MMA rows 0-7, low digits in rows 8-15).
// NT >= 1: NT tiles of 16 activation rows, two MMAs (high, low digits) per tile and group.
template <int KIND, int NT>
__global__ void __launch_bounds__((kMaxConsumerWarps + 1) * 32, 1) qdecode_kernel(const Params p) {
  constexpr int BB = (KIND == 4) ? kQ4Bytes : kQ8Bytes;
  constexpr int NACC = (NT == 0) ? 2 : 4 * NT;
  const bool resident = p.res_off != 0;
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
  const int nwarps = p.NS * p.phases;
  const int nst = (p.G + p.stage_rows - 1) / p.stage_rows;
  const uint32_t row_bytes = (uint32_t)tn * BB;

  if (tid == 0) {
    for (int s = 0; s < p.stages; s++) {
      mbar_init(smem_u32(&full[s]), resident ? 1 : 2);   // weights armed first, streamed digits once they exist
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
    auto issue_digits = [&](int st, int slot) {
      const int rows = min(p.stage_rows, p.G - st * p.stage_rows);
      const uint32_t bar = smem_u32(&full[slot]);
      // bulk copies move multiples of 16 bytes: the scale span is rounded up (the scratch has slack)
      const uint32_t db = (uint32_t)rows * p.Mp * 64, sb = (((uint32_t)rows * p.Mp * 8) + 15u) & ~15u;
      if (lane == 0) {
        mbar_expect_tx(bar, db + sb);
        uint8_t* base = ring + (size_t)slot * p.stage_bytes + p.w_bytes;
        bulk_load_default(smem_u32(base), p.xdig + (size_t)st * p.stage_rows * p.Mp * 64, db, bar);
        bulk_load_default(smem_u32(base + p.d_bytes), p.xsc + (size_t)st * p.stage_rows * p.Mp, sb, bar);
      }
      __syncwarp();
    };
    // weights of the first ring-full go out before anything waits on the previous launch
    const int first = min(nst, p.stages);
    for (int st = 0; st < first; st++) issue_weights(st, st);      // first <= stages: slot == st
    if (!resident) {
      asm volatile("griddepcontrol.wait;" ::: "memory");   // quantise_rows has finished: the digits exist
      for (int st = 0; st < first; st++) issue_digits(st, st);
    }
    bool live = true;
    // slot and parity are carried along (no division by the run-time ring depth in the loop)
    int slot = 0;
    uint32_t par = 1;                               // second pass over the ring
    for (int st = first; st < nst && live; st++, slot = (slot + 1 == p.stages) ? 0 : slot + 1, par ^= (slot == 0)) {
      int okw = 1;
      if (lane == 0) okw = mbar_wait(smem_u32(&empty[slot]), par ^ 1u, abort_flag, p.status);
      live = __shfl_sync(0xffffffffu, okw, 0) != 0;
      if (!live) break;
      issue_weights(st, slot);
      if (!resident) issue_digits(st, slot);
    }
    return;  // consumers observe every full barrier, so the copies land before the CTA ends
  }

  // -------------------------------------------------------------- consumers
  const int slice = warp % p.NS, phase = warp / p.NS;
  const bool has_cols = slice * 8 < tn;
  const int r = lane >> 2, j = lane & 3;
  uint8_t* res_dig = smem + p.res_off;                                   // [G][Mp][64]
  float2* res_sc = reinterpret_cast<float2*>(res_dig + (size_t)p.G * p.Mp * 64);  // [G][Mp]
  if (resident) {
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the activations may belong to the launch before
    const int pairs = p.G * p.Mp;
    for (int i = tid; i < ((pairs * 8 + 31) & ~31); i += nwarps * 32) {
      const int pair = min(i >> 3, pairs - 1);           // duplicates rewrite equal bytes; keeps warps whole
      const int g = pair / p.Mp, m = pair - g * p.Mp;
      quantise_pair<KIND>(p.A, p.M, p.K, g, m, i & 7, res_dig + (size_t)pair * 64, res_sc + pair);
    }
    asm volatile("bar.sync 1, %0;" ::"r"(nwarps * 32));
  }
  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; i++) acc[i] = 0.f;
  const uint32_t ring_s = smem_u32(ring);
  // Q4: word j of the block of column slice*8 + r.  Q8: its codes 8j .. 8j+7 start at byte 2 + 8j.
  const uint32_t off_w = (uint32_t)(slice * 8 + r) * BB + (KIND == 4 ? 4u * j : 2u + 8u * j);
  const uint32_t sh8 = (off_w & 3u) * 8;
  const uint32_t off_q = (uint32_t)(slice * 8 + 2 * j) * BB + (KIND == 4 ? 16u : 0u);   // scale (and zero)
  const uint32_t off_d = (uint32_t)r * 64 + 16u * j;   // digit words of row r of a tile (+512 for row r + 8)
  const uint32_t off_x = (uint32_t)r * 8;              // its {2^-e, sum} pair (+64 for row r + 8)
  const uint32_t w_step = (uint32_t)p.phases * (uint32_t)p.row_pitch;
  const uint32_t d_step = (uint32_t)p.phases * (uint32_t)(p.Mp * 64), s_step = (uint32_t)p.phases * (uint32_t)(p.Mp * 8);
  const uint32_t res_dig_s = smem_u32(res_dig), res_sc_s = smem_u32(res_sc);

  bool ok = true;
  int slot = 0;
  uint32_t par = 0;
  for (int st = 0; st < nst && ok; st++, slot = (slot + 1 == p.stages) ? 0 : slot + 1, par ^= (slot == 0)) {
    ok = mbar_wait(smem_u32(&full[slot]), par, abort_flag, p.status);
    if (ok && has_cols) {
      // 32-bit shared addresses: a per-thread constant part plus a per-row base that advances by a stride
      const uint32_t stage = ring_s + (uint32_t)slot * (uint32_t)p.stage_bytes;
      const int rows_here = min(p.stage_rows, p.G - st * p.stage_rows);
      uint32_t wrow = stage + (uint32_t)phase * (uint32_t)p.row_pitch;
      const uint32_t first_row = (uint32_t)(st * p.stage_rows + phase);   // group index of this phase's first row
      uint32_t drow = resident ? res_dig_s + first_row * (uint32_t)(p.Mp * 64)
                               : stage + (uint32_t)p.w_bytes + (uint32_t)phase * (uint32_t)(p.Mp * 64);
      uint32_t srow = resident ? res_sc_s + first_row * (uint32_t)(p.Mp * 8)
                               : stage + (uint32_t)(p.w_bytes + p.d_bytes) + (uint32_t)phase * (uint32_t)(p.Mp * 8);
#pragma unroll 4
      for (int row = phase; row < rows_here; row += p.phases) {   // this phase's group-rows inside the stage
        // ---- B fragment: the j-th eight codes of column slice*8 + r
        uint32_t b0, b1;
        float sc0, sc1, z0 = 0.f, z1 = 0.f;
        if (KIND == 4) {
          const uint32_t w = lds_u32(wrow + off_w);
          b0 = w & 0x0F0F0F0Fu;          // codes of k = 8j + 0, 2, 4, 6
          b1 = (w >> 4) & 0x0F0F0F0Fu;   // codes of k = 8j + 1, 3, 5, 7
          const float2 q0 = lds_f32x2(wrow + off_q);
          const float2 q1 = lds_f32x2(wrow + off_q + BB);
          sc0 = q0.x, z0 = q0.y, sc1 = q1.x, z1 = q1.y;
        } else {
          // 34-byte blocks are 2-byte aligned: aligned words around the codes, then a funnel shift.
          // Stage bases and row pitches are multiples of 16, so the constant part decides the shift.
          const uint32_t a = wrow + (off_w & ~3u);
          const uint32_t w0 = lds_u32(a), w1 = lds_u32(a + 4), w2 = lds_u32(a + 8);
          b0 = __funnelshift_r(w0, w1, sh8);   // codes of k = 8j .. 8j+3
          b1 = __funnelshift_r(w1, w2, sh8);   // codes of k = 8j+4 .. 8j+7
          sc0 = __half2float(__ushort_as_half((unsigned short)lds_u16(wrow + off_q)));
          sc1 = __half2float(__ushort_as_half((unsigned short)lds_u16(wrow + off_q + BB)));
        }
        // ---- A fragment(s) and the scaled accumulation
        if (NT == 0) {
          // rows 0-7: high digits, rows 8-15: low digits of the same activation rows
          const uint4 d0 = lds_u32x4(drow + off_d);
          const float2 x0 = lds_f32x2(srow + off_x);
          const uint32_t a4[4] = {d0.x, d0.y, d0.z, d0.w};
          int c[4] = {0, 0, 0, 0};
          imma(c, a4, b0, b1);
          const float f0 = (float)(c[0] * 128 + c[2]), f1 = (float)(c[1] * 128 + c[3]);
          if (KIND == 4) {
            acc[0] = fmaf(sc0 * x0.x, fmaf(-z0, x0.y, f0), acc[0]);
            acc[1] = fmaf(sc1 * x0.x, fmaf(-z1, x0.y, f1), acc[1]);
          } else {
            acc[0] = fmaf(sc0 * x0.x, f0, acc[0]);
            acc[1] = fmaf(sc1 * x0.x, f1, acc[1]);
          }
        } else {
#pragma unroll
          for (int t = 0; t < (NT == 0 ? 1 : NT); t++) {
            const uint4 d0 = lds_u32x4(drow + off_d + (uint32_t)t * 1024u);
            const uint4 d1 = lds_u32x4(drow + off_d + (uint32_t)t * 1024u + 512u);
            const float2 x0 = lds_f32x2(srow + off_x + (uint32_t)t * 128u);
            const float2 x1 = lds_f32x2(srow + off_x + (uint32_t)t * 128u + 64u);
            const uint32_t ah[4] = {d0.x, d1.x, d0.z, d1.z};   // high digits of rows r, r + 8 of the tile
            const uint32_t al4[4] = {d0.y, d1.y, d0.w, d1.w};  // low digits
            int ch[4] = {0, 0, 0, 0}, cl[4] = {0, 0, 0, 0};
            imma(ch, ah, b0, b1);
            imma(cl, al4, b0, b1);
            const float f00 = (float)(ch[0] * 128 + cl[0]), f01 = (float)(ch[1] * 128 + cl[1]);
            const float f10 = (float)(ch[2] * 128 + cl[2]), f11 = (float)(ch[3] * 128 + cl[3]);
            float* a = acc + 4 * t;
            if (KIND == 4) {
              a[0] = fmaf(sc0 * x0.x, fmaf(-z0, x0.y, f00), a[0]);
              a[1] = fmaf(sc1 * x0.x, fmaf(-z1, x0.y, f01), a[1]);
              a[2] = fmaf(sc0 * x1.x, fmaf(-z0, x1.y, f10), a[2]);
              a[3] = fmaf(sc1 * x1.x, fmaf(-z1, x1.y, f11), a[3]);
            } else {
              a[0] = fmaf(sc0 * x0.x, f00, a[0]);
              a[1] = fmaf(sc1 * x0.x, f01, a[1]);
              a[2] = fmaf(sc0 * x1.x, f10, a[2]);
              a[3] = fmaf(sc1 * x1.x, f11, a[3]);
            }
          }
        }
        wrow += w_step, drow += d_step, srow += s_step;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&empty[slot]));
  }

  // ---------------------------------------------- sum the phases, fixed order
  asm volatile("bar.sync 1, %0;" ::"r"(nwarps * 32));  // every consumer is done with the ring
  constexpr int ROWS = (NT == 0) ? 8 : 16 * NT;
  float* red = reinterpret_cast<float*>(ring);        // [phases][ROWS][TN]
  if (NT == 0) {
    float* dst = red + ((size_t)phase * ROWS + r) * TN + slice * 8 + 2 * j;
    *reinterpret_cast<float2*>(dst) = make_float2(acc[0], acc[1]);
  } else {
#pragma unroll
    for (int t = 0; t < (NT == 0 ? 1 : NT); t++) {
      float* dst = red + ((size_t)phase * ROWS + 16 * t + r) * TN + slice * 8 + 2 * j;
      *reinterpret_cast<float2*>(dst) = make_float2(acc[4 * t], acc[4 * t + 1]);
      *reinterpret_cast<float2*>(dst + 8 * TN) = make_float2(acc[4 * t + 2], acc[4 * t + 3]);
    }
  }
  asm volatile("bar.sync 1, %0;" ::"r"(nwarps * 32));
  if (*abort_flag) return;
  for (int i = tid; i < p.M * tn; i += nwarps * 32) {
    const int m = i / tn, c = i - m * tn;
    float sum = 0.f;
    for (int ph = 0; ph < p.phases; ph++) sum += red[((size_t)ph * ROWS + m) * TN + c];
    p.C[(size_t)m * p.N + col0 + c] = sum;
  }
}

struct Plan {
  Params p;
  int tiles, NT;
  size_t smem;
  bool ok;
};

constexpr int kMaxRows = 32;   // rows beyond this go to the tensor-core kernel

Plan make_plan(int kind, int64_t M, int64_t N, int64_t K) {
  const int BB = (kind == 4) ? kQ4Bytes : kQ8Bytes;
  const int sms = device_sm_count();
  Plan pl{};
  Params& p = pl.p;
  p.M = (int)M, p.N = (int)N, p.K = (int)K, p.G = (int)(K / 32);
  pl.NT = (M <= 8) ? 0 : (int)((M + 15) / 16);
  p.Mp = (M <= 8) ? 8 : 16 * pl.NT;
  // Slices per CTA: the fewest that cover N in a whole number of waves, at most 16 (128 columns).
  int NS = 0;
  for (int64_t waves = 1;; waves++) {
    NS = (int)((N + 8 * sms * waves - 1) / (8 * sms * waves));
    if (NS <= 16) break;
  }
  p.NS = NS;
  const int TN = NS * 8;
  pl.tiles = (int)((N + TN - 1) / TN);
  int phases = kMaxConsumerWarps / NS;
  if (phases < 1) phases = 1;
  while (phases > 1 && phases * 4 > p.G) phases--;   // short K: do not over-split
  p.phases = phases;
  p.row_pitch = TN * BB;
  // Digits resident in shared memory (converted by the kernel itself) only for short reductions, where a
  // second launch would cost more than every CTA redoing the conversion; measured at K = 4096, M = 8 the
  // streamed form is faster (17.4 us against 21.8 us).
  const size_t res_bytes = (size_t)p.G * p.Mp * 72;
  const bool resident = res_bytes <= 24 * 1024;
  const int target_rows = (p.Mp >= 32 && !resident) ? 8 : kStageRows;
  p.stage_rows = phases * ((target_rows + phases - 1) / phases);
  p.w_bytes = ((p.stage_rows * p.row_pitch + 16 + 127) / 128) * 128;   // + slack for the Q8 read-ahead
  p.d_bytes = resident ? 0 : p.stage_rows * p.Mp * 64;
  p.s_bytes = resident ? 0 : ((p.stage_rows * p.Mp * 8 + 127) / 128) * 128;
  p.stage_bytes = ((p.w_bytes + p.d_bytes + p.s_bytes + 1023) / 1024) * 1024;
  const int res_room = resident ? (int)((res_bytes + 1023) / 1024) * 1024 : 0;
  int stages = (kSmemBudget + 20 * 1024 - 1024 - res_room) / p.stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  p.stages = stages;
  const size_t red = (size_t)phases * (size_t)p.Mp * TN * 4;
  const size_t ring = (size_t)(stages > 0 ? stages : 0) * p.stage_bytes;
  const size_t ring_room = (((ring > red ? ring : red) + 1023) / 1024) * 1024;
  p.res_off = resident ? (int)(1024 + ring_room) : 0;
  pl.smem = 1024 + ring_room + res_room;
  pl.ok = stages >= 2 && pl.smem <= 227 * 1024 && M <= kMaxRows;
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

template <int KIND, int NT>
cudaError_t launch_main(const Plan& pl, cudaStream_t s) {
  static PerDeviceFlag configured;              // the attribute belongs to a device, not to the process
  bool* set = configured.here();
  if (!set) return cudaErrorInvalidDevice;
  if (!*set) {
    cudaError_t e = cudaFuncSetAttribute(qdecode_kernel<KIND, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         227 * 1024);
    if (e != cudaSuccess) return e;
    *set = true;
  }
  const int threads = (pl.p.NS * pl.p.phases + 1) * 32;
  const cudaError_t e = launch_pdl(qdecode_kernel<KIND, NT>, dim3((unsigned)pl.tiles), dim3((unsigned)threads),
                                   pl.smem, s, pl.p);
  count_launch();
  return e;
}

}  // namespace

bool qdecode_supports(int kind, int64_t M, int64_t N, int64_t K, int64_t groups) {
  if (kind != 4 && kind != 8) return false;
  if (M < 1 || M > kMaxRows) return false;
  if (N < 8 || (N % 8) != 0) return false;       // 16-byte alignment of every group-row span
  if (K < 32 || (K % 32) != 0 || groups != K / 32) return false;
  if (N > (1 << 30) || K > (1 << 22)) return false;
  return make_plan(kind, M, N, K).ok;
}

size_t qdecode_workspace_bytes(int kind, int64_t M, int64_t N, int64_t K) {
  const Plan pl = make_plan(kind, M, N, K);
  if (pl.p.res_off != 0) return 0;               // digits live in shared memory
  const size_t G = (size_t)(K / 32), Mp = (size_t)pl.p.Mp;
  return ((G * Mp * 64 + 255) & ~size_t(255)) + G * Mp * 8 + 64;
}

bool qdecode_uses_scratch(int kind, int64_t M, int64_t N, int64_t K) {
  const Plan pl = make_plan(kind, M, N, K);
  return pl.ok && pl.p.res_off == 0;
}

cudaError_t launch_qdecode(int kind, const float* A, const uint8_t* B, float* C, int64_t M, int64_t N, int64_t K,
                           int64_t groups, Workspace ws, cudaStream_t s, bool digits_in_scratch) {
  (void)groups;
  Plan pl = make_plan(kind, M, N, K);
  if (!pl.ok) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(A) & 15)) return cudaErrorMisalignedAddress;
  pl.p.A = A, pl.p.B = B, pl.p.C = C, pl.p.xdig = nullptr, pl.p.xsc = nullptr;
  if (pl.p.res_off == 0) {
    const size_t need = qdecode_workspace_bytes(kind, M, N, K);
    if (!ws.ptr || ws.bytes < need || (reinterpret_cast<uintptr_t>(ws.ptr) & 255)) return cudaErrorInvalidValue;
    const size_t G = (size_t)(K / 32), Mp = (size_t)pl.p.Mp;
    uint8_t* xdig = static_cast<uint8_t*>(ws.ptr);
    float2* xsc = reinterpret_cast<float2*>(xdig + ((G * Mp * 64 + 255) & ~size_t(255)));
    const int qthreads = (int)(Mp * G * 8);
    cudaError_t e = cudaSuccess;
    if (digits_in_scratch)
      ;   // the launch before this one left the digits of the same activations there
    else if (kind == 4)
      e = launch_pdl(quantise_rows<4>, dim3((unsigned)((qthreads + 255) / 256)), dim3(256), (size_t)0, s, A, xdig,
                     xsc, (int)M, (int)Mp, (int)K, (int)G);
    else
      e = launch_pdl(quantise_rows<8>, dim3((unsigned)((qthreads + 255) / 256)), dim3(256), (size_t)0, s, A, xdig,
                     xsc, (int)M, (int)Mp, (int)K, (int)G);
    if (!digits_in_scratch) count_launch();
    if (e != cudaSuccess) return e;
    pl.p.xdig = xdig, pl.p.xsc = xsc;
  }
  pl.p.status = kernel_status_ptr();
  if (!pl.p.status) return cudaErrorUnknown;
#define SMITH_DECODE_CASE(KD, NTV) \
  if (kind == KD && pl.NT == NTV) return launch_main<KD, NTV>(pl, s);
  SMITH_DECODE_CASE(4, 0) SMITH_DECODE_CASE(4, 1) SMITH_DECODE_CASE(4, 2)
  SMITH_DECODE_CASE(8, 0) SMITH_DECODE_CASE(8, 1) SMITH_DECODE_CASE(8, 2)
#undef SMITH_DECODE_CASE
  return cudaErrorInvalidValue;
}

}  // namespace smith
