// qdecode.cu -- decode-shaped quantized matmul, M <= 16 rows of activations.
//
// C[M,N] = A[M,K] (f32) x dequant(B); B in Smith's Q4 (24-byte) or Q8 (34-byte)
// block layout, block (g, col) at (g*N + col) * block_bytes
// (shaders/matmul_q4.metal:47-55, shaders/matmul_q8.metal:40-48).
//
// The work is bound by reading the packed weights from HBM exactly once, so
// the kernel is organised around that stream:
//
//  * One CTA owns a tile of TN adjacent output columns and the whole K range.
//    For one group g the TN blocks of the tile are contiguous in memory
//    (TN * block_bytes, a multiple of 16 bytes because TN % 8 == 0), so a
//    single thread moves them with one 1-D bulk async copy
//    (cp.async.bulk.shared::cluster.global, no multicast) per group-row into
//    a ring of shared-memory stages guarded by full/empty mbarriers.  One
//    stage holds kWarps group-rows; up to kMaxStages stages are in flight.
//  * kWarps consumer warps each take one group-row of a stage and sweep the
//    tile's columns eight at a time with warp-level mma.sync m16n8k16.  The
//    B fragment is built in registers straight from the packed codes
//    (exact small integers in bf16 / f16, via an exponent-bias trick), the A
//    fragment is the activations split into a high and a low 16-bit part
//    (bf16 for Q4; f16 of the row-prescaled activation for Q8) so that
//    activations keep ~16-17 bits of mantissa, and accumulation is f32.
//    With M <= 8 the high parts sit in MMA rows 0-7 and the low parts in rows
//    8-15 of the same instruction; with 8 < M <= 16 two instructions are used.
//  * The per-group scale (and Q4 zero point) is applied to the group's f32
//    partial sum in registers:
//        Q4: acc += scale * (sum_k x_k (128 + q_k)  -  (128 + zero) * sum_k x_k)
//        Q8: acc += scale * sum_k x_k q_k
//    (128 is the exponent bias that makes 0x4300 | q a valid bf16 number).
//  * Each consumer warp covers a different subset of the groups; the kWarps
//    partial tiles are summed through shared memory at the end and written
//    once.  No atomics, no scratch in global memory; summation order is fixed,
//    so results are reproducible run to run.
//
// Every mbarrier wait is bounded by wall-clock time; a wait that gives up
// raises a flag in shared and global memory, the CTA stops consuming, and the
// host reads the flag (qdecode_take_status).  The result is then invalid.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.h"
#include "pipeline.cuh"

namespace smith {
namespace {

constexpr int kWarps = 16;                       // consumer warps = group-rows per stage
constexpr int kThreads = (kWarps + 1) * 32;      // + one producer warp
constexpr int kMaxSlices = 16;                   // TN <= 128 columns
constexpr int kMaxStages = 6;
constexpr int kRingBudget = 196 * 1024;          // bytes of shared memory for the ring
constexpr int kHeaderBytes = 1024;               // barriers + per-row scales

struct Params {
  const float* A;
  const uint8_t* B;
  float* C;
  int M, N, K, G;
  int TN;          // columns per CTA (multiple of 8)
  int row_pitch;   // bytes between group-rows inside a stage
  int stages;      // ring depth
  int stage_bytes;
  int* status;     // device-wide "a wait gave up" word
};

// Plain shared-memory loads: the compiler may schedule them freely among
// themselves, but not above the barrier wait (whose asm clobbers memory).
__device__ __forceinline__ uint32_t lds32(const uint8_t* p) { return *reinterpret_cast<const uint32_t*>(p); }
__device__ __forceinline__ uint32_t lds16(const uint8_t* p) { return *reinterpret_cast<const uint16_t*>(p); }
__device__ __forceinline__ float2 lds_f2(const uint8_t* p) { return *reinterpret_cast<const float2*>(p); }

// {upper 16 bits = cvt(hi_slot), lower 16 bits = cvt(lo_slot)}
__device__ __forceinline__ uint32_t pack_bf16(float lo_slot, float hi_slot) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi_slot), "f"(lo_slot));
  return d;
}
__device__ __forceinline__ uint32_t pack_f16(float lo_slot, float hi_slot) {
  uint32_t d;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi_slot), "f"(lo_slot));
  return d;
}

template <int KIND>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (KIND == 4) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// Split a (possibly prescaled) activation pair into 16-bit high and low parts.
// hi = round16(x); lo = round16(x - hi).  `sum` accumulates hi + lo as the MMA sees them.
template <int KIND>
__device__ __forceinline__ void split_pair(float xa, float xb, uint32_t& hi, uint32_t& lo, float& sum) {
  if (KIND == 4) {
    hi = pack_bf16(xa, xb);
    const float ha = __uint_as_float(hi << 16), hb = __uint_as_float(hi & 0xFFFF0000u);
    const float la = xa - ha, lb = xb - hb;
    lo = pack_bf16(la, lb);
    sum += (ha + __uint_as_float(lo << 16)) + (hb + __uint_as_float(lo & 0xFFFF0000u));
  } else {
    hi = pack_f16(xa, xb);
    const __half2 h2 = *reinterpret_cast<const __half2*>(&hi);
    const float ha = __low2float(h2), hb = __high2float(h2);
    lo = pack_f16(xa - ha, xb - hb);
  }
}

// Activations of one group for this thread: 8 consecutive k (k = 8j .. 8j+7) of
// row `r` (and r + 8 when WIDE).  Rows >= M read as zero.
template <bool WIDE>
struct XRegs {
  float4 v[WIDE ? 4 : 2];
};

template <bool WIDE>
__device__ __forceinline__ void load_x(XRegs<WIDE>& x, const float* __restrict__ A, int M, int K, int g, int r,
                                       int j) {
  const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4* p0 = reinterpret_cast<const float4*>(A + (size_t)r * K + g * 32 + j * 8);
  x.v[0] = (r < M) ? __ldg(p0) : z;
  x.v[1] = (r < M) ? __ldg(p0 + 1) : z;
  if (WIDE) {
    const float4* p1 = reinterpret_cast<const float4*>(A + (size_t)(r + 8) * K + g * 32 + j * 8);
    x.v[2] = (r + 8 < M) ? __ldg(p1) : z;
    x.v[3] = (r + 8 < M) ? __ldg(p1 + 1) : z;
  }
}

// A fragments of the two MMAs that cover one 32-element group.
//   !WIDE: f[m] = {hi(row r; pair a), lo(row r; pair a), hi(row r; pair b), lo(row r; pair b)}
//    WIDE: hi[m] = {hi(r;a), hi(r+8;a), hi(r;b), hi(r+8;b)}, lo[m] likewise
// Pair layout (which of the thread's 8 k values share a register) follows the
// code unpacking: Q4 pairs nibble i with nibble i+4, Q8 pairs adjacent bytes.
template <int KIND, bool WIDE>
struct AFrag {
  uint32_t hi[2][4];
  uint32_t lo[2][4];  // only used when WIDE
  float sx0, sx1;     // sum_k (hi + lo) of row r / row r + 8 over the whole group (Q4 only)
};

template <int KIND, bool WIDE>
__device__ __forceinline__ void build_a(AFrag<KIND, WIDE>& f, const XRegs<WIDE>& x, float rs0, float rs1) {
  float e[8], o[8];
  e[0] = x.v[0].x, e[1] = x.v[0].y, e[2] = x.v[0].z, e[3] = x.v[0].w;
  e[4] = x.v[1].x, e[5] = x.v[1].y, e[6] = x.v[1].z, e[7] = x.v[1].w;
  if (KIND == 8) {
#pragma unroll
    for (int i = 0; i < 8; i++) e[i] *= rs0;
  }
  // index pairs: [mma][a|b] -> (first, second)
  constexpr int P4[2][2][2] = {{{0, 4}, {1, 5}}, {{2, 6}, {3, 7}}};
  constexpr int P8[2][2][2] = {{{0, 1}, {2, 3}}, {{4, 5}, {6, 7}}};
  float s0 = 0.f, s1 = 0.f;
  if (!WIDE) {
#pragma unroll
    for (int m = 0; m < 2; m++)
#pragma unroll
      for (int ab = 0; ab < 2; ab++) {
        const int i0 = (KIND == 4) ? P4[m][ab][0] : P8[m][ab][0];
        const int i1 = (KIND == 4) ? P4[m][ab][1] : P8[m][ab][1];
        split_pair<KIND>(e[i0], e[i1], f.hi[m][2 * ab], f.hi[m][2 * ab + 1], s0);
      }
  } else {
    o[0] = x.v[2].x, o[1] = x.v[2].y, o[2] = x.v[2].z, o[3] = x.v[2].w;
    o[4] = x.v[3].x, o[5] = x.v[3].y, o[6] = x.v[3].z, o[7] = x.v[3].w;
    if (KIND == 8) {
#pragma unroll
      for (int i = 0; i < 8; i++) o[i] *= rs1;
    }
#pragma unroll
    for (int m = 0; m < 2; m++)
#pragma unroll
      for (int ab = 0; ab < 2; ab++) {
        const int i0 = (KIND == 4) ? P4[m][ab][0] : P8[m][ab][0];
        const int i1 = (KIND == 4) ? P4[m][ab][1] : P8[m][ab][1];
        split_pair<KIND>(e[i0], e[i1], f.hi[m][2 * ab], f.lo[m][2 * ab], s0);
        split_pair<KIND>(o[i0], o[i1], f.hi[m][2 * ab + 1], f.lo[m][2 * ab + 1], s1);
      }
  }
  if (KIND == 4) {  // the four threads of a quad hold the four quarters of the group
    s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
    s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
    if (WIDE) {
      s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
      s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    }
  }
  f.sx0 = s0;
  f.sx1 = s1;
}

template <int KIND, bool WIDE>
__global__ void __launch_bounds__(kThreads, 1) qdecode_kernel(const Params p) {
  constexpr int BB = (KIND == 4) ? kQ4Bytes : kQ8Bytes;
  constexpr int NACC = WIDE ? 4 : 2;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);            // [kMaxStages]
  uint64_t* empty = full + kMaxStages;                            // [kMaxStages]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 128);
  float* row_scale = reinterpret_cast<float*>(smem + 256);        // [16] Q8 prescale 2^e
  float* row_inv = row_scale + 16;                                // [16] 2^-e
  unsigned* row_max = reinterpret_cast<unsigned*>(row_inv + 16);  // [16] bits of max |x|
  uint8_t* ring = smem + kHeaderBytes;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int col0 = blockIdx.x * p.TN;
  const int tn = min(p.TN, p.N - col0);
  const int ns = tn >> 3;
  const int nst = (p.G + kWarps - 1) / kWarps;
  const uint32_t row_bytes = (uint32_t)tn * BB;

  if (tid == 0) {
    for (int s = 0; s < p.stages; s++) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), kWarps);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid < 16) row_max[tid] = 0u;
  __syncthreads();

  if (warp == kWarps) {
    // ------------------------------------------------------------ producer
    // One lane per group-row: the rows of a stage are issued by the warp in
    // parallel (a single thread issuing them one by one is too slow to keep
    // the stream busy).  Lane 0 arms the barrier before any copy can complete.
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    bool live = true;
    for (int st = 0; st < nst && live; st++) {
      const int slot = st % p.stages;
      if (st >= p.stages) {
        int okw = 1;
        if (lane == 0) okw = mbar_wait(smem_u32(&empty[slot]), ((st / p.stages) - 1) & 1, abort_flag, p.status);
        live = __shfl_sync(0xffffffffu, okw, 0) != 0;
        if (!live) break;
      }
      const int rows = min(kWarps, p.G - st * kWarps);
      const uint32_t bar = smem_u32(&full[slot]);
      if (lane == 0) mbar_expect_tx(bar, (uint32_t)rows * row_bytes);
      __syncwarp();
      const uint32_t dst = smem_u32(ring + (size_t)slot * p.stage_bytes);
      const uint8_t* src = p.B + ((size_t)(st * kWarps) * p.N + col0) * BB;
      if (lane < rows) bulk_load(dst + lane * p.row_pitch, src + (size_t)lane * p.N * BB, row_bytes, bar, policy);
    }
    return;  // consumers observe every full barrier, so the copies land before the CTA ends
  }

  // -------------------------------------------------------------- consumers
  const int r = lane >> 2, j = lane & 3;
  float rs0 = 1.f, rs1 = 1.f;
  if (KIND == 8) {
    // Per-row power-of-two prescale so that f16 can carry the activations:
    // max |x_row| is moved into [2^13, 2^14).
    for (int row = 0; row < p.M; row++) {
      float m = 0.f;
      for (int k = tid; k < p.K; k += kWarps * 32) m = fmaxf(m, fabsf(__ldg(p.A + (size_t)row * p.K + k)));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      if (lane == 0) atomicMax(&row_max[row], __float_as_uint(m));
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32));
    if (tid < 16) {
      const unsigned bits = row_max[tid];
      int e = 0;
      const int ex = (int)(bits >> 23);
      if (ex > 0 && ex < 255) e = 13 - (ex - 127);
      e = max(-100, min(100, e));
      row_scale[tid] = __uint_as_float((unsigned)(127 + e) << 23);
      row_inv[tid] = __uint_as_float((unsigned)(127 - e) << 23);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32));
    rs0 = row_scale[r];
    rs1 = row_scale[r + 8];
  }

  float acc[kMaxSlices][NACC];
#pragma unroll
  for (int s = 0; s < kMaxSlices; s++)
#pragma unroll
    for (int i = 0; i < NACC; i++) acc[s][i] = 0.f;

  XRegs<WIDE> xr;
  if (warp < p.G) load_x<WIDE>(xr, p.A, p.M, p.K, warp, r, j);
  bool ok = true;

  for (int st = 0; st < nst && ok; st++) {
    const int slot = st % p.stages;
    const int g = st * kWarps + warp;
    AFrag<KIND, WIDE> af;
    if (g < p.G) {
      build_a<KIND, WIDE>(af, xr, rs0, rs1);
      if (g + kWarps < p.G) load_x<WIDE>(xr, p.A, p.M, p.K, g + kWarps, r, j);
    }
    ok = mbar_wait(smem_u32(&full[slot]), (st / p.stages) & 1, abort_flag, p.status);
    if (ok && g < p.G) {
      const uint8_t* row_base = ring + (size_t)slot * p.stage_bytes + (size_t)warp * p.row_pitch;
#pragma unroll
      for (int s = 0; s < kMaxSlices; s++) {
        if (s < ns) {
          uint32_t b[4];
          float sc0, sc1, zz0 = 0.f, zz1 = 0.f;
          if (KIND == 4) {
            const uint32_t w = lds32(row_base + (uint32_t)(s * 8 + r) * BB + 4 * j);
            const float2 q0 = lds_f2(row_base + (uint32_t)(s * 8 + 2 * j) * BB + 16);
            const float2 q1 = lds_f2(row_base + (uint32_t)(s * 8 + 2 * j + 1) * BB + 16);
            sc0 = q0.x, sc1 = q1.x;
            zz0 = 128.f + q0.y, zz1 = 128.f + q1.y;
            // nibble i in the low half, nibble i+4 in the high half, each OR-ed into bf16 128.0
            b[0] = (w & 0x000F000Fu) | 0x43004300u;
            b[1] = ((w >> 4) & 0x000F000Fu) | 0x43004300u;
            b[2] = ((w >> 8) & 0x000F000Fu) | 0x43004300u;
            b[3] = ((w >> 12) & 0x000F000Fu) | 0x43004300u;
          } else {
            // the stage base is 1024-byte aligned and row pitches are multiples of 16,
            // so the byte offset inside the stage decides the word alignment
            const uint32_t off = (uint32_t)(s * 8 + r) * BB + 2 + 8 * j;
            const uint8_t* al = row_base + (off & ~3u);
            const uint32_t sh = (off & 3u) * 8;
            const uint32_t w0 = lds32(al), w1 = lds32(al + 4), w2 = lds32(al + 8);
            const uint32_t lo = __funnelshift_r(w0, w1, sh) ^ 0x80808080u;
            const uint32_t hi = __funnelshift_r(w1, w2, sh) ^ 0x80808080u;
            const uint32_t h0 = lds16(row_base + (uint32_t)(s * 8 + 2 * j) * BB);
            const uint32_t h1 = lds16(row_base + (uint32_t)(s * 8 + 2 * j + 1) * BB);
            sc0 = __half2float(__ushort_as_half((unsigned short)h0));
            sc1 = __half2float(__ushort_as_half((unsigned short)h1));
            // bytes u = q + 128 become f16 (1024 + u); subtracting 1152 leaves q exactly
            const uint32_t k1152 = 0x64806480u;
            uint32_t t;
            t = __byte_perm(lo, 0x64646464u, 0x4140);
            asm("sub.f16x2 %0, %1, %2;" : "=r"(b[0]) : "r"(t), "r"(k1152));
            t = __byte_perm(lo, 0x64646464u, 0x4342);
            asm("sub.f16x2 %0, %1, %2;" : "=r"(b[1]) : "r"(t), "r"(k1152));
            t = __byte_perm(hi, 0x64646464u, 0x4140);
            asm("sub.f16x2 %0, %1, %2;" : "=r"(b[2]) : "r"(t), "r"(k1152));
            t = __byte_perm(hi, 0x64646464u, 0x4342);
            asm("sub.f16x2 %0, %1, %2;" : "=r"(b[3]) : "r"(t), "r"(k1152));
          }
          float c[4] = {0.f, 0.f, 0.f, 0.f};
          mma16816<KIND>(c, af.hi[0], b[0], b[1]);
          mma16816<KIND>(c, af.hi[1], b[2], b[3]);
          if (WIDE) {
            mma16816<KIND>(c, af.lo[0], b[0], b[1]);
            mma16816<KIND>(c, af.lo[1], b[2], b[3]);
          }
          if (!WIDE) {
            // rows 0-7 carry the high parts, rows 8-15 the low parts of the same activations
            const float t0 = c[0] + c[2], t1 = c[1] + c[3];
            if (KIND == 4) {
              acc[s][0] = fmaf(sc0, fmaf(-zz0, af.sx0, t0), acc[s][0]);
              acc[s][1] = fmaf(sc1, fmaf(-zz1, af.sx0, t1), acc[s][1]);
            } else {
              acc[s][0] = fmaf(sc0, t0, acc[s][0]);
              acc[s][1] = fmaf(sc1, t1, acc[s][1]);
            }
          } else {
            if (KIND == 4) {
              acc[s][0] = fmaf(sc0, fmaf(-zz0, af.sx0, c[0]), acc[s][0]);
              acc[s][1] = fmaf(sc1, fmaf(-zz1, af.sx0, c[1]), acc[s][1]);
              acc[s][2] = fmaf(sc0, fmaf(-zz0, af.sx1, c[2]), acc[s][2]);
              acc[s][3] = fmaf(sc1, fmaf(-zz1, af.sx1, c[3]), acc[s][3]);
            } else {
              acc[s][0] = fmaf(sc0, c[0], acc[s][0]);
              acc[s][1] = fmaf(sc1, c[1], acc[s][1]);
              acc[s][2] = fmaf(sc0, c[2], acc[s][2]);
              acc[s][3] = fmaf(sc1, c[3], acc[s][3]);
            }
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&empty[slot]));
  }

  // ---------------------------------------------- cross-warp sum, fixed order
  asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32));  // every consumer is done with the ring
  constexpr int ROWS = WIDE ? 16 : 8;
  float* red = reinterpret_cast<float*>(ring);  // [kWarps][ROWS][TN]
  const int TNp = p.TN;
#pragma unroll
  for (int s = 0; s < kMaxSlices; s++) {
    if (s < ns) {
      float* dst = red + ((size_t)warp * ROWS + r) * TNp + s * 8 + 2 * j;
      *reinterpret_cast<float2*>(dst) = make_float2(acc[s][0], acc[s][1]);
      if (WIDE) *reinterpret_cast<float2*>(dst + 8 * TNp) = make_float2(acc[s][2], acc[s][3]);
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32));
  if (*abort_flag) return;
  for (int idx = tid; idx < p.M * tn; idx += kWarps * 32) {
    const int row = idx / tn, col = idx - row * tn;
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; w++) sum += red[((size_t)w * ROWS + row) * TNp + col];
    if (KIND == 8) sum *= row_inv[row];
    p.C[(size_t)row * p.N + col0 + col] = sum;
  }
}

struct Plan {
  int TN, tiles, row_pitch, stage_bytes, stages;
  size_t smem;
};

Plan make_plan(int kind, int64_t M, int64_t N) {
  const int BB = (kind == 4) ? kQ4Bytes : kQ8Bytes;
  const int sms = 148;
  // Smallest multiple-of-8 tile width that covers N with a whole number of
  // waves of CTAs, capped at kMaxSlices * 8 columns.
  int64_t waves = 1;
  int TN;
  for (;; waves++) {
    TN = (int)(8 * ((N + 8 * sms * waves - 1) / (8 * sms * waves)));
    if (TN <= kMaxSlices * 8) break;
  }
  Plan pl;
  pl.TN = TN;
  pl.tiles = (int)((N + TN - 1) / TN);
  pl.row_pitch = TN * BB;  // multiple of 16 since TN % 8 == 0
  pl.stage_bytes = ((kWarps * pl.row_pitch + 1023) / 1024) * 1024;
  pl.stages = kRingBudget / pl.stage_bytes;
  if (pl.stages > kMaxStages) pl.stages = kMaxStages;
  if (pl.stages < 2) pl.stages = 2;
  const size_t ring = (size_t)pl.stages * pl.stage_bytes + 16;
  const size_t red = (size_t)kWarps * (M > 8 ? 16 : 8) * TN * 4;
  pl.smem = kHeaderBytes + (ring > red ? ring : red);
  return pl;
}

template <int KIND, bool WIDE>
cudaError_t launch_one(const Params& p, const Plan& pl, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(qdecode_kernel<KIND, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         227 * 1024);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  qdecode_kernel<KIND, WIDE><<<pl.tiles, kThreads, pl.smem, s>>>(p);
  count_launch();
  return cudaGetLastError();
}

}  // namespace

bool qdecode_supports(int kind, int64_t M, int64_t N, int64_t K, int64_t groups) {
  if (kind != 4 && kind != 8) return false;
  if (M < 1 || M > 16) return false;
  if (N < 8 || (N % 8) != 0) return false;       // 16-byte alignment of every group-row span
  if (K < 32 || (K % 32) != 0 || groups != K / 32) return false;
  if (N > (1 << 30) || K > (1 << 24)) return false;
  return true;
}

cudaError_t launch_qdecode(int kind, const float* A, const uint8_t* B, float* C, int64_t M, int64_t N,
                           int64_t K, int64_t groups, cudaStream_t s) {
  if ((reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(A) & 15)) return cudaErrorMisalignedAddress;
  const Plan pl = make_plan(kind, M, N);
  Params p;
  p.A = A, p.B = B, p.C = C;
  p.M = (int)M, p.N = (int)N, p.K = (int)K, p.G = (int)groups;
  p.status = kernel_status_ptr();
  if (!p.status) return cudaErrorUnknown;
  p.TN = pl.TN, p.row_pitch = pl.row_pitch, p.stages = pl.stages, p.stage_bytes = pl.stage_bytes;
  if (kind == 4) return (M > 8) ? launch_one<4, true>(p, pl, s) : launch_one<4, false>(p, pl, s);
  return (M > 8) ? launch_one<8, true>(p, pl, s) : launch_one<8, false>(p, pl, s);
}

}  // namespace smith
