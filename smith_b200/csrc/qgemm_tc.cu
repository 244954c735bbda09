// qgemm_tc.cu -- prefill-shaped quantized matmul, M > 16, on the 5th-generation
// tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// C[M,N] = A[M,K] (f32) x dequant(B); B in Smith's Q4 (24-byte) or Q8 (34-byte)
// block layout, block (g, col) at (g*N + col) * block_bytes
// (shaders/matmul_q4.metal:47-55, shaders/matmul_q8.metal:40-48).
//
// Two launches:
//  1. convert_activations: A f32 -> 16-bit [M,K] in scratch memory.  Q4 uses
//     bf16 (same exponent range as f32).  Q8 uses f16 -- its block scale is an
//     f16 number by format, so scale * code is formed exactly in f16 -- with
//     each activation row pre-multiplied by a power of two that moves its
//     largest magnitude into [2^13, 2^14); the inverse is applied in the epilogue.
//  2. qgemm_tc_kernel: one CTA computes MT x 128 rows by BN columns, 64 k at a
//     time, through two shared-memory rings: a deep one of packed group-rows
//     (a few KB per k-block, loaded from HBM far ahead) and a shallow one of
//     {activation tile, dequantised B tile} slots.
//     warp 0     activation producer: lane t TMA-loads row tile t's 128 x 64
//                tile (128-byte swizzle) of each k-block into a tile slot.
//     warps 4,8  MMA issuers, one per row tile (warp 4 also allocates tensor
//                memory): per k-block four tcgen05.mma (128 x BN x 16), A and B
//                from shared memory through K-major 128-byte-swizzle
//                descriptors, D = f32 in TMEM; tcgen05.commit frees the slot.
//     warp 12    weight producer: lanes 0-1 bulk-copy the k-block's two packed
//                group-rows of the tile's BN columns into a packed-ring slot.
//     the 24 warps that are not multiples of four dequantise, in `groups` teams that own
//                alternate k-blocks (team t works on k-blocks t, t + groups, ...): each
//                thread takes half of a (column, group) block (16 weights),
//                forms scale * (code - zero) (Q4,
//                packed bf16: exact code - round(zero), then one fused
//                multiply-add with the scale and the zero point's fraction) or
//                code * scale (Q8, packed f16, exact product of two f16-exact
//                numbers rounded once), and stores 16-byte chunks into the
//                K-major swizzled B tile, then fence.proxy.async + mbarrier arrive.
//                Q4 emits each 8 codes in the order 0,4,1,5,2,6,3,7 (how the
//                nibbles pair up in a 32-bit word); convert_activations stores
//                the activations' k in the same order, so the dot products
//                are unchanged and no byte shuffles are needed.
//     warps 1-3, 16 and 5-7, 20  epilogue (even and odd chunks): tcgen05.ld their 32-lane quarter of each
//                accumulator, 32 columns at a time, and store C rows.
//   Weights of a tile are dequantised once and feed MT row tiles, so for
//   M >= 256 the CUDA-core dequantisation stays below the tensor time.
//
// No multicast, no clusters.  Every mbarrier wait is time-bounded
// (pipeline.cuh); on a give-up the CTA skips to the end, frees its TMEM and
// leaves the status word set.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.h"
#include "pipeline.cuh"
#include "tcgen05.cuh"

namespace smith {
namespace {

constexpr int kBM = 128;            // rows per MMA / per accumulator
constexpr int kBK = 64;             // k per stage: one 128-byte swizzle row of 16-bit values
// Warp roles.  The four single-thread roles sit on the warps that are multiples of four, which
// share one of the SM's four warp schedulers; the dequant warps are all the others.  A lone thread
// on a scheduler that also hosts seven always-ready dequant warps gets about an eighth of its
// issue slots, and these threads' instruction chains are the k-loop's critical path.
constexpr int kWarps = 32;
constexpr int kThreads = kWarps * 32;
constexpr int kDequantWarps = 28;          // the 24 warps with warp % 4 != 0 first, then warps 16, 20, 24, 28
constexpr int kMaxItems = 3;               // most blocks per dequant thread and k-block that a plan may ask for
constexpr int kActProducerWarp = 0;
constexpr int kMmaWarp0 = 4;               // row tile 0 (also allocates tensor memory); row tile 1: warp 8
constexpr int kWeightProducerWarp = 12;
constexpr int kEpilogueWarp0 = 16;         // reads TMEM lanes 0-31 in the epilogue; warps 1-3 read the rest
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 227 * 1024;

struct Params {
  const uint8_t* B;
  float* C;
  const float* row_inv;   // Q8: per-row inverse prescale, else nullptr
  int M, N, K, G;
  int BN;                 // columns per CTA, multiple of 16, <= 256
  int stages;             // tile ring depth
  int pk_stages;          // packed ring depth
  int sb;                 // 64-wide k-blocks per slot and hand-off (1 or 2): a "step" is sb k-blocks
  int groups;             // dequant teams; team t owns steps t, t + groups, ...
  int team_warps;         // warps per team; groups * team_warps <= kDequantWarps
  int a_bytes, pk_pitch, pk_bytes, b_bytes, stage_bytes;  // stage_bytes = a_bytes + b_bytes: one tile slot
  int tmem_cols;
  int* status;
};

// Instruction descriptor of tcgen05.mma kind::f16: f32 accumulate, A and B both
// K-major, 16-bit format `fmt` (0 = f16, 1 = bf16), M = 128, N = n.
//   [4,6) D format: 1 = f32   [7,10) A format   [10,13) B format
//   [15] A major (0 = K)  [16] B major (0 = K)  [17,23) N >> 3   [24,29) M >> 4
__host__ __device__ constexpr uint32_t instr_desc(int fmt, int n) {
  return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(kBM >> 4) << 24);
}

// ---------------------------------------------------------------- activations -> 16 bit
template <int KIND>
__global__ void __launch_bounds__(256) convert_activations(const float* __restrict__ A, uint16_t* __restrict__ out,
                                                            float* __restrict__ row_inv, int M, int K) {
  __shared__ float red[8];
  // the main kernel may start now: everything in it but the activation loads (and the Q8 row
  // scales) is independent of this kernel and waits for it explicitly
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int row = blockIdx.x;
  const float* src = A + (size_t)row * K;
  float up = 1.f;
  if (KIND == 8) {
    float m = 0.f;
    for (int k = threadIdx.x; k < K; k += 256) m = fmaxf(m, fabsf(src[k]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int i = 1; i < 8; i++) m = fmaxf(m, red[i]);
    const int ex = (int)(__float_as_uint(m) >> 23) & 0xFF;
    int e = (ex == 0 || ex == 255) ? 0 : (13 - (ex - 127));
    e = max(-100, min(100, e));
    up = __uint_as_float((unsigned)(127 + e) << 23);
    if (threadIdx.x == 0) row_inv[row] = __uint_as_float((unsigned)(127 - e) << 23);
  }
  uint16_t* dst = out + (size_t)row * K;
  if (KIND == 4) {
    // bf16, and within every 8 consecutive k the order 0,4,1,5,2,6,3,7 that the Q4 dequantiser emits
    for (int k = threadIdx.x * 8; k < K; k += 256 * 8) {
      const float4 a = *reinterpret_cast<const float4*>(src + k);
      const float4 b = *reinterpret_cast<const float4*>(src + k + 4);
      uint4 o;
      asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o.x) : "f"(b.x), "f"(a.x));
      asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o.y) : "f"(b.y), "f"(a.y));
      asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o.z) : "f"(b.z), "f"(a.z));
      asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o.w) : "f"(b.w), "f"(a.w));
      *reinterpret_cast<uint4*>(dst + k) = o;
    }
  } else {
    for (int k = threadIdx.x * 2; k < K; k += 512) {
      const float2 v = *reinterpret_cast<const float2*>(src + k);
      uint32_t packed;
      asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(v.y * up), "f"(v.x * up));
      *reinterpret_cast<uint32_t*>(dst + k) = packed;
    }
  }
}

// ---------------------------------------------------------------- dequantise one (column, group) block
// Writes the 32 values of one group of B-tile row `col` (K-major, 128-byte swizzle: 16-byte
// chunk c of row n sits at chunk position c ^ (n & 7)).  `blk` is the packed block in shared
// memory, `blk_off` its byte offset inside the 16-byte-aligned packed slot (Q8 needs the
// alignment), `dst` the position of the group's first chunk in the tile (row offset plus swizzled
// chunk position); chunk i of the group then lies at dst ^ (i << 4) in offset terms.
template <int KIND>
__device__ __forceinline__ void dequant_block(const uint8_t* __restrict__ blk, uint32_t blk_off,
                                              uint8_t* __restrict__ tile, uint32_t dst, bool zero_fill) {
  if (zero_fill) {
#pragma unroll
    for (int i = 0; i < 4; i++) *reinterpret_cast<uint4*>(tile + (dst ^ (uint32_t)(i << 4))) = make_uint4(0, 0, 0, 0);
    return;
  }
  if (KIND == 4) {
    const uint2 n01 = *reinterpret_cast<const uint2*>(blk);
    const uint2 n23 = *reinterpret_cast<const uint2*>(blk + 8);
    const float2 sz = *reinterpret_cast<const float2*>(blk + 16);
    // scale * (code - zero) = scale * (code - zi) + (-scale * zf), zi = round(zero): code - zi is an exact
    // small integer in bf16; the multiply-add rounds once.
    // zi is kept within +-120 so that 128 + zi and code - zi stay exact bf16 integers; a zero point
    // beyond that leaves a large zf, whose rounding is then relative to the weight itself.
    const float zi = fminf(fmaxf(rintf(sz.y), -120.f), 120.f);
    const float zf = sz.y - zi;
    uint32_t s2, c2, z2;
    asm("cvt.rn.bf16x2.f32 %0, %1, %1;" : "=r"(s2) : "f"(sz.x));
    asm("cvt.rn.bf16x2.f32 %0, %1, %1;" : "=r"(c2) : "f"(-sz.x * zf));
    asm("cvt.rn.bf16x2.f32 %0, %1, %1;" : "=r"(z2) : "f"(128.f + zi));
    const uint32_t w[4] = {n01.x, n01.y, n23.x, n23.y};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const uint32_t r = ((w[i] >> (4 * j)) & 0x000F000Fu) | 0x43004300u;  // bf16 (128 + q_j, 128 + q_{j+4})
        uint32_t d;
        asm("sub.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(r), "r"(z2));
        asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(o[j]) : "r"(d), "r"(s2), "r"(c2));
      }
      *reinterpret_cast<uint4*>(tile + (dst ^ (uint32_t)(i << 4))) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  } else {
    // 34-byte blocks are 2-byte aligned: read the aligned words around the 32 codes and shift
    const uint32_t mis = (blk_off + 2) & 3u;
    const uint32_t sh = mis * 8;
    const uint32_t* al = reinterpret_cast<const uint32_t*>(blk + 2 - mis);
    uint32_t raw[9];
#pragma unroll
    for (int i = 0; i < 9; i++) raw[i] = al[i];
    const uint32_t h = *reinterpret_cast<const unsigned short*>(blk);
    const uint32_t s2 = h | (h << 16);
    const uint32_t k1152 = 0x64806480u;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 2; j++) {
        const uint32_t u = __funnelshift_r(raw[2 * i + j], raw[2 * i + j + 1], sh) ^ 0x80808080u;
        uint32_t p0 = __byte_perm(u, 0x64646464u, 0x4140);   // f16 (1024 + u0, 1024 + u1)
        uint32_t p1 = __byte_perm(u, 0x64646464u, 0x4342);
        asm("sub.f16x2 %0, %0, %1;" : "+r"(p0) : "r"(k1152));  // exact codes
        asm("sub.f16x2 %0, %0, %1;" : "+r"(p1) : "r"(k1152));
        asm("mul.f16x2 %0, %1, %2;" : "=r"(o[2 * j]) : "r"(p0), "r"(s2));
        asm("mul.f16x2 %0, %1, %2;" : "=r"(o[2 * j + 1]) : "r"(p1), "r"(s2));
      }
      *reinterpret_cast<uint4*>(tile + (dst ^ (uint32_t)(i << 4))) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// ---------------------------------------------------------------- main kernel
// Two rings in shared memory, so that each resource is only as deep as its latency needs:
//   packed ring   `pk_stages` slots of two packed group-rows (the k-block's weights as they lie in
//                 HBM, a few KB): deep, because these loads come from HBM;
//   tile ring     `stages` slots of {activation tile (TMA), dequantised B tile}: the large ones.
// A k-block's critical cycle is then  B slot free -> dequantise -> MMAs -> B slot free ;
// the weight loads run far ahead of it and the activation load overlaps the dequantisation.
template <int KIND, int MT>
__global__ void __launch_bounds__(kThreads, 1) qgemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                               const Params p) {
  constexpr int BB = (KIND == 4) ? kQ4Bytes : kQ8Bytes;
  extern __shared__ __align__(1024) uint8_t smem[];
  // header (first 1024 bytes): barriers, TMEM base, abort flag
  uint64_t* pk_full = reinterpret_cast<uint64_t*>(smem);          // [kMaxStages] packed group-rows landed
  uint64_t* pk_empty = pk_full + kMaxStages;                       // [kMaxStages] ... and read by their team
  uint64_t* a_full = pk_empty + kMaxStages;                        // [kMaxStages] activation tile landed
  uint64_t* b_ready = a_full + kMaxStages;                         // [kMaxStages] B tile written
  uint64_t* empty = b_ready + kMaxStages;                          // [kMaxStages] MMAs of the tile slot done
  uint64_t* acc_ready = empty + kMaxStages;                        // [1]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  uint8_t* tiles = smem + 1024;                                    // [stages][a_bytes + b_bytes]
  uint8_t* packed = tiles + (size_t)p.stages * p.stage_bytes;      // [pk_stages][pk_bytes]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // row tiles vary fastest, so the CTAs that share a weight tile run at the same time
  const int col0 = blockIdx.y * p.BN;
  const int row0 = blockIdx.x * (MT * kBM);
  const int tn = min(p.BN, p.N - col0);
  const int nkb = (p.K + p.sb * kBK - 1) / (p.sb * kBK);   // steps of sb k-blocks
  const int team_warps = p.team_warps;

  if (tid == 0) {
    for (int s = 0; s < kMaxStages; s++) {
      mbar_init(smem_u32(&pk_full[s]), 1);
      mbar_init(smem_u32(&pk_empty[s]), team_warps);   // the team that owns the slot's k-block
      mbar_init(smem_u32(&a_full[s]), 1);
      mbar_init(smem_u32(&b_ready[s]), team_warps);
      mbar_init(smem_u32(&empty[s]), MT);              // one commit per MMA issuer
    }
    mbar_init(smem_u32(acc_ready), MT);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp0) {
    tmem_alloc(smem_u32(tmem_base_slot), (uint32_t)p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  // The loops of the single-thread roles carry slot index and parity along: an integer division
  // by a run-time ring depth costs a lone thread hundreds of cycles per k-block.
  const int wq = warp & 3;
  bool ok = true;
  if (warp == kActProducerWarp) {
    // ------------------------------------------------------------ activation producer (lane t: row tile t)
    if (lane < MT * p.sb) {                 // lane = sub * MT + t: k-block `sub` of the step, row tile t
      int s = 0;
      uint32_t par = 0;
      const int sub = lane / MT, t = lane - sub * MT;
      const uint32_t dst0 = smem_u32(tiles) + lane * (kBM * kBK * 2);
      uint32_t dst = dst0;
      asm volatile("griddepcontrol.wait;" ::: "memory");   // the 16-bit activations are written by the launch before
      for (int kb = 0; kb < nkb; kb++) {
        if (kb >= p.stages) {
          if (!mbar_wait(smem_u32(&empty[s]), par ^ 1u, abort_flag, p.status)) break;
        }
        const uint32_t bar = smem_u32(&a_full[s]);
        // a box beyond K is filled with zeros and still counts its bytes
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)(p.sb * MT * kBM * kBK * 2));
        tma_load_2d(dst, &tmap_a, (kb * p.sb + sub) * kBK, row0 + t * kBM, bar);
        dst += p.stage_bytes;
        if (++s == p.stages) s = 0, par ^= 1u, dst = dst0;
      }
    }
  } else if (warp == kWeightProducerWarp) {
    // ------------------------------------------------------------ weight producer (lane g: group-row g of the k-block)
    if (lane < 2 * p.sb) {                  // lane: group-row of the step
      int s = 0;
      uint32_t par = 0;
      const size_t brow = (size_t)p.N * BB;
      const uint8_t* src = p.B + (size_t)col0 * BB + lane * brow;
      const uint32_t b_tx = (uint32_t)tn * BB;
      const int per = 2 * p.sb;
      const uint32_t dst0 = smem_u32(packed) + lane * p.pk_pitch;
      uint32_t dst = dst0;
      for (int kb = 0; kb < nkb; kb++) {
        if (kb >= p.pk_stages) {
          if (!mbar_wait(smem_u32(&pk_empty[s]), par ^ 1u, abort_flag, p.status)) break;
        }
        const uint32_t bar = smem_u32(&pk_full[s]);
        const int ngr = min(per, p.G - kb * per);
        // the copy's complete_tx may reach the barrier before lane 0's expect_tx: the phase cannot
        // complete before that arrival, and the transaction count may run negative meanwhile
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)ngr * b_tx);
        if (lane < ngr) bulk_load_plain(dst, src, b_tx, bar);
        src += per * brow;
        dst += p.pk_bytes;
        if (++s == p.pk_stages) s = 0, par ^= 1u, dst = dst0;
      }
    }
  } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 4) {
    // ------------------------------------------------------------ MMA issuers, one per row tile
    const int t = (warp - kMmaWarp0) >> 2;
    if (lane == 0 && t < MT) {
      const uint32_t idesc = instr_desc(KIND == 4 ? 1 : 0, p.BN);
      int s = 0;
      uint32_t par = 0;
      // descriptors differ between slots and k-steps only in the start-address field
      // (bytes >> 4, the low 14 bits): add, do not rebuild
      const uint64_t a_desc0 = smem_desc_sw128(smem_u32(tiles + t * (kBM * kBK * 2)));
      const uint64_t b_desc0 = smem_desc_sw128(smem_u32(tiles + p.a_bytes));
      const uint32_t a_sub = (uint32_t)(MT * kBM * kBK * 2) >> 4, b_sub = (uint32_t)(p.BN * kBK * 2) >> 4;
      const uint32_t a_lo0 = (uint32_t)a_desc0, b_lo0 = (uint32_t)b_desc0, desc_hi = (uint32_t)(a_desc0 >> 32);
      const uint32_t slot_step = (uint32_t)p.stage_bytes >> 4;
      const uint32_t d_tmem = tmem_base + (uint32_t)(t * p.BN);
      uint32_t soff = 0;
      static_assert(kBK == 64, "umma_f16_kblock issues the four k-steps of a 64-wide k-block");
      for (int kb = 0; kb < nkb; kb++) {
        // b_ready covers the activation tile too: the team's first warp waits for it before arriving
        ok = mbar_wait(smem_u32(&b_ready[s]), par, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        umma_f16_kblock(d_tmem, a_lo0 + soff, b_lo0 + soff, desc_hi, idesc, kb > 0 ? 1u : 0u);
        if (p.sb == 2) umma_f16_kblock(d_tmem, a_lo0 + soff + a_sub, b_lo0 + soff + b_sub, desc_hi, idesc, 1u);
        umma_commit(smem_u32(&empty[s]));
        soff += slot_step;
        if (++s == p.stages) s = 0, par ^= 1u, soff = 0;
      }
      if (ok) umma_commit(smem_u32(acc_ready));
    }
  } else if (wq != 0 || warp >= kEpilogueWarp0) {
    // ------------------------------------------------------------ dequantise
    // dequant warp index: the other three scheduler partitions first, the role partition's spare warps last
    const int dw = wq ? (warp >> 2) * 3 + wq - 1 : 24 + ((warp - kEpilogueWarp0) >> 2);
    if (dw < p.groups * team_warps) {
    const int team = dw % p.groups;                      // this warp's team
    const int team_threads = team_warps * 32;
    const int dt = (dw / p.groups) * 32 + lane;          // thread index inside the team
    int s = team, sp = team;                             // groups <= stages, pk_stages
    uint32_t par = 0, parp = 0;
    // This thread's (column, group) blocks are the same in every step: index them once.
    // item = group * BN + col over the step's 2 * sb * BN blocks, dealt round-robin to the team.
    // it_dst: tile-slot offset of the block's first chunk (bits 0-19), group of the step (bits 28-30),
    // pad column (bit 31).
    uint32_t it_src[kMaxItems], it_dst[kMaxItems];
    const int per = 2 * p.sb;
#pragma unroll
    for (int i = 0; i < kMaxItems; i++) {
      const int it = dt + i * team_threads;
      int gl = 0, col = it;
      while (gl < per - 1 && col >= p.BN) col -= p.BN, gl++;
      it_src[i] = (uint32_t)(gl * p.pk_pitch + col * BB);
      it_dst[i] = (it < per * p.BN)
                      ? ((uint32_t)((gl >> 1) * (p.BN * kBK * 2) + (col >> 3) * 1024 + (col & 7) * 128 +
                                    (((gl & 1) * 64) ^ ((col & 7) << 4))) |
                         (col >= tn ? 0x80000000u : 0u) | ((uint32_t)gl << 28))
                      : 0xffffffffu;                                              // no such item
    }
    for (int kb = team; kb < nkb; kb += p.groups) {
      ok = mbar_wait(smem_u32(&pk_full[sp]), parp, abort_flag, p.status);
      if (ok && kb >= p.stages) {
        ok = mbar_wait(smem_u32(&empty[s]), par ^ 1u, abort_flag, p.status);   // the slot's last MMAs have read it
        tc_fence_after();
      }
      if (!ok) break;
      const uint8_t* pk = packed + (size_t)sp * p.pk_bytes;
      uint8_t* bt = tiles + (size_t)s * p.stage_bytes + p.a_bytes;
      const int left = p.G - kb * per;               // groups of this step that lie inside K
#pragma unroll
      for (int i = 0; i < kMaxItems; i++) {
        const uint32_t d = it_dst[i];
        if (d != 0xffffffffu) {
          const bool zero = (d & 0x80000000u) || (int)((d >> 28) & 7u) >= left;
          dequant_block<KIND>(pk + it_src[i], it_src[i], bt, d & 0x000fffffu, zero);
        }
      }
      fence_async_smem();       // make the generic-proxy stores visible to the tensor core's reads
      if (dw < p.groups) ok = mbar_wait(smem_u32(&a_full[s]), par, abort_flag, p.status);   // the team's first warp
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&b_ready[s]));
        mbar_arrive(smem_u32(&pk_empty[sp]));
      }
      if (!ok) break;
      s += p.groups;
      if (s >= p.stages) s -= p.stages, par ^= 1u;
      sp += p.groups;
      if (sp >= p.pk_stages) sp -= p.pk_stages, parp ^= 1u;
    }
    }
  }
  // ---------------------------------------------------------------- epilogue
  // Two warps per TMEM lane quarter (a warp may read the quarter warp % 4): warps 1-3 and 16 take
  // the even 32-column chunks, warps 5-7 and 20 the odd ones, each after its dequant work.
  const int eset = (warp == kEpilogueWarp0 || (warp >= 1 && warp <= 3)) ? 0
                   : (warp == kEpilogueWarp0 + 4 || (warp >= 5 && warp <= 7)) ? 1 : -1;
  if (eset >= 0) {
    // warp-uniform: the TMEM loads below are warp-collective
    const bool got = __all_sync(0xffffffffu, ok && mbar_wait(smem_u32(acc_ready), 0, abort_flag, p.status));
    tc_fence_after();
    if (KIND == 8) asm volatile("griddepcontrol.wait;" ::: "memory");   // row_inv comes from the launch before
    if (got) {
      const int q = warp & 3;                          // TMEM lane quarter this warp may read
      // tcgen05.ld hands lane l the 32 columns of accumulator row 32 * q + l.  Storing those straight to
      // C would touch 32 rows per instruction (32 wavefronts of the L1 data pipe each); instead the warp
      // turns the 32 x 32 chunk around in shared memory (the tile ring is idle by now) and stores
      // four whole 128-byte row segments per instruction.
      constexpr int kPitch = 36;                       // floats per staged row: 16-byte aligned, conflict-free
      float* stage = reinterpret_cast<float*>(tiles) + (eset * 4 + q) * (32 * kPitch);
      const int sr = lane >> 3, sc = (lane & 7) * 4;   // this lane's row (of each 4) and column in the read-back
#pragma unroll 1
      for (int t = 0; t < MT; t++) {
        const int rbase = row0 + t * kBM + q * 32;
        const float inv = (KIND == 8 && rbase + lane < p.M) ? p.row_inv[rbase + lane] : 1.f;
#pragma unroll 1
        for (int c = eset * 32; c < p.BN; c += 64) {
          uint32_t r[32];
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(t * p.BN + c), r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float4 v = make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                                   __uint_as_float(r[i + 3]));
            if (KIND == 8) v.x *= inv, v.y *= inv, v.z *= inv, v.w *= inv;
            *reinterpret_cast<float4*>(stage + lane * kPitch + i) = v;
          }
          __syncwarp();
          const int cc = c + sc;                        // first of this lane's four columns within the tile
          float* dcol = p.C + col0 + cc;
          const bool vec = (cc + 4 <= tn) && ((reinterpret_cast<uintptr_t>(dcol) & 15) == 0);   // N % 8 == 0: same for all rows
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const int rr = 4 * i + sr;
            const int row = rbase + rr;
            if (row < p.M) {
              const float4 v = *reinterpret_cast<const float4*>(stage + rr * kPitch + sc);
              float* dst = dcol + (size_t)row * p.N;
              if (vec) {
                *reinterpret_cast<float4*>(dst) = v;
              } else {
                if (cc < tn) dst[0] = v.x;
                if (cc + 1 < tn) dst[1] = v.y;
                if (cc + 2 < tn) dst[2] = v.z;
                if (cc + 3 < tn) dst[3] = v.w;
              }
            }
          }
          __syncwarp();
        }
      }
    }
  }
  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

struct Plan {
  int MT, BN, sb, stages, pk_stages, tmem_cols, groups, team_warps;
  int a_bytes, pk_pitch, pk_bytes, b_bytes, stage_bytes;
  size_t smem;
  dim3 grid;
};

Plan make_plan(int kind, int64_t M, int64_t N) {
  const int BB = (kind == 4) ? kQ4Bytes : kQ8Bytes;
  Plan pl{};
  pl.MT = (M > kBM) ? 2 : 1;
  const int64_t mtiles = (M + pl.MT * kBM - 1) / (pl.MT * kBM);
  // Column tile: the multiple of 16 in [16, 256] that wastes the least of the
  // machine (partial last tile x partial last wave); wider wins ties.
  const int64_t sms = device_sm_count();
  double best = -1.0;
  int bestBN = 128;
  for (int bn = 256; bn >= 16; bn -= 16) {
    const int64_t nt = (N + bn - 1) / bn;
    if (nt > 65535) continue;                                  // grid.y
    const int64_t ctas = nt * mtiles;
    const int64_t waves = (ctas + sms - 1) / sms;
    // useful fraction of the tiles x fill of the last wave x a mild preference for wide MMAs
    // (narrow tiles re-read the activations more often and amortise the dequantised tile less)
    const double eff = ((double)N / (double)(nt * bn)) * ((double)ctas / (double)(waves * sms)) *
                       ((double)bn / (double)(bn + 48));
    if (eff > best + 1e-9) best = eff, bestBN = bn;
  }
  pl.BN = bestBN;
  // Steps of two k-blocks halve the hand-offs between the roles; they pay when there is a single row
  // tile (little tensor time per k-block to hide the hand-offs behind) and three slots still fit.
  const int budget = kSmemBudget - 1024;
  for (pl.sb = (pl.MT == 1 ? 2 : 1); pl.sb >= 1; pl.sb--) {
    pl.a_bytes = pl.sb * pl.MT * kBM * kBK * 2;
    pl.pk_pitch = ((pl.BN * BB + 15) / 16) * 16;
    pl.pk_bytes = ((2 * pl.sb * pl.pk_pitch + 16 + 1023) / 1024) * 1024;   // + slack for the Q8 read-ahead
    pl.b_bytes = pl.sb * pl.BN * kBK * 2;
    pl.stage_bytes = pl.a_bytes + pl.b_bytes;                      // one tile slot; every part a multiple of 1024
    // tile ring as deep as fits beside four packed slots, the packed ring takes what is left
    pl.stages = (budget - 4 * pl.pk_bytes) / pl.stage_bytes;
    if (pl.stages >= 3 || pl.sb == 1) break;
  }
  if (pl.stages > kMaxStages) pl.stages = kMaxStages;
  pl.pk_stages = (budget - pl.stages * pl.stage_bytes) / pl.pk_bytes;
  if (pl.pk_stages > kMaxStages) pl.pk_stages = kMaxStages;
  // Dequant teams: g teams work on g k-blocks side by side (each needs a tile slot beside the one
  // being multiplied), every thread taking ceil(blocks / team threads) of the k-block's 2 * BN
  // blocks.  Pick the g with the least passes per k-block; ties go to fewer passes (shorter latency).
  const int blocks = 2 * pl.sb * pl.BN;
  pl.groups = 1, pl.team_warps = kDequantWarps;
  double best_cost = 1e9;
  int best_passes = 1 << 30;
  for (int g = 1; g <= 4 && (g == 1 || g < pl.stages); g++) {
    for (int pool = 24; pool <= kDequantWarps; pool += kDequantWarps - 24) {
      int tw = pool / g;
      if (tw > (blocks + 31) / 32) tw = (blocks + 31) / 32;      // no more warps than a single pass needs
      const int passes = (blocks + tw * 32 - 1) / (tw * 32);
      if (passes > kMaxItems) continue;
      // warps beyond the first 24 share the single-thread roles' scheduler and slow them down
      const double cost = (double)passes / g * (g * tw > 24 ? 1.4 : 1.0);
      if (cost < best_cost - 1e-9 || (cost < best_cost + 1e-9 && passes < best_passes))
        best_cost = cost, best_passes = passes, pl.groups = g, pl.team_warps = tw;
    }
  }
  // the epilogue reads the accumulators 32 columns at a time, so the last tile is rounded up
  const int need = (pl.MT - 1) * pl.BN + ((pl.BN + 31) / 32) * 32;
  int cols = 32;
  while (cols < need) cols <<= 1;
  pl.tmem_cols = cols;
  pl.smem = 1024 + (size_t)pl.stages * pl.stage_bytes + (size_t)pl.pk_stages * pl.pk_bytes;
  pl.grid = dim3((unsigned)mtiles, (unsigned)((N + pl.BN - 1) / pl.BN));
  return pl;
}

template <int KIND, int MT>
cudaError_t launch_main(const CUtensorMap& map, const Params& p, const Plan& pl, cudaStream_t s) {
  static PerDeviceFlag configured;              // the attribute belongs to a device, not to the process
  bool* set = configured.here();
  if (!set) return cudaErrorInvalidDevice;
  if (!*set) {
    cudaError_t e = cudaFuncSetAttribute(qgemm_tc_kernel<KIND, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         227 * 1024);
    if (e != cudaSuccess) return e;
    *set = true;
  }
  // Programmatic dependent launch: CTAs start as SMs come free while the activation conversion is
  // still running; their weight pipeline fills meanwhile.
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = pl.grid, cfg.blockDim = dim3(kThreads), cfg.dynamicSmemBytes = pl.smem, cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, qgemm_tc_kernel<KIND, MT>, map, p);
  count_launch();
  return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace

bool qgemm_tc_supports(int kind, int64_t M, int64_t N, int64_t K, int64_t groups) {
  if (kind != 4 && kind != 8) return false;
  if (M < 1 || M > (1 << 24)) return false;
  if (N < 8 || (N % 8) != 0) return false;              // 16-byte alignment of group-row spans
  if (K < 32 || (K % 32) != 0 || groups != K / 32) return false;
  // Q4 runs in bf16: its 2^-9 rounding of every weight averages out over K, and the stated tolerance
  // (1e-3 of the row/column norms) needs K of about a thousand for a comfortable margin.  Shorter
  // reductions go to the any-shape kernel.  Q8 runs in f16 (2^-12) and has no such limit.
  if (kind == 4 && K < 1024) return false;
  if (N > (1 << 30) || K > (1 << 24)) return false;
  if ((N + 255) / 256 > 65535) return false;
  return encode_fn() != nullptr;
}

size_t qgemm_tc_workspace_bytes(int kind, int64_t M, int64_t N, int64_t K) {
  (void)kind;
  (void)N;
  return (size_t)M * K * 2 + 256 + (size_t)M * 4;
}

cudaError_t launch_qgemm_tc(int kind, const float* A, const uint8_t* B, float* C, int64_t M, int64_t N, int64_t K,
                            int64_t groups, Workspace ws, cudaStream_t s) {
  if (ws.bytes < qgemm_tc_workspace_bytes(kind, M, N, K) || !ws.ptr) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(ws.ptr) & 255))
    return cudaErrorMisalignedAddress;
  EncodeTiledFn enc = encode_fn();
  if (!enc) return cudaErrorNotSupported;
  uint16_t* a16 = static_cast<uint16_t*>(ws.ptr);
  const size_t a16_bytes = ((size_t)M * K * 2 + 255) & ~size_t(255);
  float* row_inv = reinterpret_cast<float*>(static_cast<uint8_t*>(ws.ptr) + a16_bytes);

  if (kind == 4)
    convert_activations<4><<<(unsigned)M, 256, 0, s>>>(A, a16, row_inv, (int)M, (int)K);
  else
    convert_activations<8><<<(unsigned)M, 256, 0, s>>>(A, a16, row_inv, (int)M, (int)K);
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;

  const Plan pl = make_plan(kind, M, N);
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)kBM};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(&map, kind == 4 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a16,
                         dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;

  Params p{};
  p.B = B, p.C = C, p.row_inv = (kind == 8) ? row_inv : nullptr;
  p.M = (int)M, p.N = (int)N, p.K = (int)K, p.G = (int)groups;
  p.BN = pl.BN, p.stages = pl.stages, p.pk_stages = pl.pk_stages, p.groups = pl.groups, p.team_warps = pl.team_warps, p.sb = pl.sb;
  p.a_bytes = pl.a_bytes, p.pk_pitch = pl.pk_pitch, p.pk_bytes = pl.pk_bytes, p.b_bytes = pl.b_bytes;
  p.stage_bytes = pl.stage_bytes, p.tmem_cols = pl.tmem_cols;
  p.status = kernel_status_ptr();
  if (!p.status) return cudaErrorUnknown;
  if (kind == 4) return pl.MT == 2 ? launch_main<4, 2>(map, p, pl, s) : launch_main<4, 1>(map, p, pl, s);
  return pl.MT == 2 ? launch_main<8, 2>(map, p, pl, s) : launch_main<8, 1>(map, p, pl, s);
}

// ---------------------------------------------------------------- entry point that allocates nothing
// Scratch for smith_qmatmul_static: the 16-bit copy of the activations
// (M * K * 2 bytes, rounded up to 256) followed by one f32 per row.  It is part
// of the library image, so every GPU that loads the library holds these bytes
// until the process exits.  In host code the name below is only a stand-in for
// the symbol; the device address comes from cudaGetSymbolAddress.
constexpr size_t kStaticScratchBytes = (size_t)8 << 20;  // 8 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
// Device address of g_static_scratch per device, looked up once per device with that device current.
void* g_static_scratch_ptr[64] = {nullptr};
}  // namespace

cudaError_t launch_qgemm_tc_static(int kind, const float* A, const uint8_t* B, float* C, int64_t M, int64_t N,
                                   int64_t K, int64_t groups, cudaStream_t s, const char** why) {
  *why = "";
  if (!qgemm_tc_supports(kind, M, N, K, groups)) {
    *why = "shape not taken by the tensor-core kernel (needs N % 8 == 0, K % 32 == 0, groups == K / 32; Q4 needs K >= 1024)";
    return cudaErrorInvalidValue;
  }
  const size_t need = qgemm_tc_workspace_bytes(kind, M, N, K);
  if (need > kStaticScratchBytes) {
    *why = "M * K exceeds the built-in scratch (8 MiB: M * K * 2 + 256 + M * 4 bytes must fit)";
    return cudaErrorInvalidValue;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) {
    *why = "device index out of range";
    return cudaErrorInvalidDevice;
  }
  if (!g_static_scratch_ptr[dev]) {  // set-up, once per device, with that device current
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) {
      *why = "cudaGetSymbolAddress failed for the built-in scratch";
      return e != cudaSuccess ? e : cudaErrorUnknown;
    }
    g_static_scratch_ptr[dev] = p;
  }
  Workspace ws;
  ws.ptr = g_static_scratch_ptr[dev];
  ws.bytes = kStaticScratchBytes;
  // Nothing in the scratch has to start at zero: convert_activations rewrites every element the
  // main kernel reads (all M * K values and, for Q8, all M row factors) before it is read.
  return launch_qgemm_tc(kind, A, B, C, M, N, K, groups, ws, s);
}

}  // namespace smith
