// dense_tc.cu -- dense matmul C[M,N] = A[M,K] @ B[K,N] on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory); the unquantised sibling of qgemm_tc.cu.
//
// What it replaces: the reference's tiled kernels matmul_f32 / matmul_f16 (shaders/matmul.metal:31-112,
// 172-231; chosen by src/ops/matmul.js:28 when M, N and K are all at least 64), which form every
// output as an f32 sum over k of f32 products.
//
// The tensor cores multiply 16-bit numbers.  f16 storage goes in as it is.  f32 storage is split into
// three bf16 planes, x = h + m + l with h = bf16(x), m = bf16(x - h), l = bf16(x - h - m): 3 x 8 = 24
// significand bits, so the three planes hold x exactly (bf16 has f32's exponent range, so no scaling
// is needed).  The product a * b is then accumulated as the six partial products
//     ah*bh + ah*bm + am*bh + ah*bl + al*bh + am*bm
// in tensor memory; the three left out (am*bl, al*bm, al*bl) are below 2^-23 of |a*b|, the size of
// one f32 rounding.  The tensor core truncates each f32 accumulation, so ah*bh has an accumulator of
// its own and the five small products share a second one (added in the epilogue): the error is then
// that of the K/16 truncated accumulations of the leading product, about 1e-7 * ||a_m|| * ||b_n||
// at K = 2048 and growing in proportion to K.  Six MMAs at the bf16 rate are the cost of three at the tf32 rate, with
// 6 instead of 8 bytes per element staged through shared memory.  A `fast` mode keeps only ah*bh
// (one plane each, 2^-9 relative per factor) for callers that accept bf16 inputs.
//
// Launches:
//  1. split kernels: A -> planes [P][Mp][Kp] (row-major as A is), B -> planes [P][Np][Kp]
//     TRANSPOSED, so that both operands are K-major for the MMA and rows start on 16 bytes.  For f16
//     storage A is read in place and only B is transposed.
//  2. dense_tc_kernel: one CTA computes MT x 128 rows by BN columns, 64 k at a time, through a ring
//     of stages {A planes' tiles, B planes' tiles}.
//       warp 0  producer: one thread issues the stage's tensor-map loads (128-byte swizzle)
//       warp 1  allocates tensor memory; one thread issues, per stage and row tile, the 4 MMAs
//               (128 x BN x 16) of each plane pair, then tcgen05.commit frees the stage
//       warps 2-5  epilogue: tcgen05.ld their 32-lane quarter of the accumulators, turn 32 x 32
//               chunks around in shared memory and store whole 128-byte row segments of C
// No multicast; clusters of two CTAs in the pair form only.  Every mbarrier wait is time-bounded (pipeline.cuh); on a give-up the
// CTA skips to the end, frees its tensor memory and leaves the status word set.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdlib.h>

#include "kernels.h"
#include "pipeline.cuh"
#include "qgemv_common.cuh"
#include "tcgen05.cuh"

namespace smith {
namespace {

constexpr int kBM = 128, kBK = 64;
constexpr int kATile = kBM * kBK * 2;       // 16 KB: one plane's 128 x 64 tile
constexpr int kMaxStages = 8;
constexpr int kMaxPairs = 6;
constexpr int kThreads = 7 * 32;
constexpr int kSecondIssuerWarp = 6;     // on another warp scheduler than warp 1 (warp % 4 picks the scheduler)

struct Params {
  void* C;
  int M, N, K;
  int out_f16;
  int MT, BN;
  int planes;              // 1 or 3 per operand
  int npairs;
  int issuers;             // threads that issue MMAs: 2 in the single-CTA three-plane form (pairs 0-2 / 3-5), else 1
  uint32_t pair_a, pair_b;  // plane index of pair q in bits [4q, 4q+4)
  int a_plane_rows, b_plane_rows;   // row distance between planes in the stacked tensor maps
  int a_bytes, b_tile, stage_bytes, stages, tmem_cols;
  uint32_t idesc;
  int* status;
};

// ---------------------------------------------------------------- f32 -> bf16 planes
// x = h + m + l, each part a bf16.  Non-finite x: h carries it, m = l = 0.  A finite x that rounds
// up to infinity in bf16 takes the truncated h instead.
__device__ __forceinline__ void split3(float x, __nv_bfloat16& h, __nv_bfloat16& m, __nv_bfloat16& l) {
  h = __float2bfloat16_rn(x);
  float hf = __bfloat162float(h);
  const bool finite = fabsf(x) <= 3.4028234e38f;
  if (finite && !(fabsf(hf) <= 3.4028234e38f)) h = __float2bfloat16_rz(x), hf = __bfloat162float(h);
  const float r1 = finite ? x - hf : 0.f;
  m = __float2bfloat16_rn(r1);
  const float r2 = r1 - __bfloat162float(m);
  l = __float2bfloat16_rn(r2);
}

// A [M,K] f32 -> planes [P][Mp][Kp] bf16 (same orientation); one thread per pair of k.
template <int P>
__global__ void __launch_bounds__(256) split_rows_kernel(const float* __restrict__ A, __nv_bfloat16* __restrict__ out,
                                                         int M, int K, int Mp, int Kp) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int row = blockIdx.x;
  const size_t plane = (size_t)Mp * Kp;
  for (int k = (blockIdx.y * 256 + threadIdx.x) * 2; k < Kp; k += gridDim.y * 512) {
    const float x0 = (k < K) ? A[(size_t)row * K + k] : 0.f;
    const float x1 = (k + 1 < K) ? A[(size_t)row * K + k + 1] : 0.f;
    __nv_bfloat16 h0, m0, l0, h1, m1, l1;
    split3(x0, h0, m0, l0);
    split3(x1, h1, m1, l1);
    __nv_bfloat16* dst = out + (size_t)row * Kp + k;
    *reinterpret_cast<__nv_bfloat162*>(dst) = __halves2bfloat162(h0, h1);
    if (P == 3) {
      *reinterpret_cast<__nv_bfloat162*>(dst + plane) = __halves2bfloat162(m0, m1);
      *reinterpret_cast<__nv_bfloat162*>(dst + 2 * plane) = __halves2bfloat162(l0, l1);
    }
  }
}

// B [K,N] -> planes [P][Np][Kp] TRANSPOSED.  A block turns a 64 (k) x 32 (n) tile around in shared
// memory: reads run along n, writes along k (two k per thread, 128 bytes per warp).
// IN = float: split into P bf16 planes; IN = __half: P = 1, copied as it is.
template <typename IN, int P>
__global__ void __launch_bounds__(256) split_transpose_kernel(const IN* __restrict__ B, uint16_t* __restrict__ out,
                                                              int K, int N, int Np, int Kp) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __shared__ float tile[64][33];
  const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 64;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int k = k0 + ty + 8 * i, n = n0 + tx;
    float v = 0.f;
    if (k < K && n < N) {
      if (sizeof(IN) == 4) v = reinterpret_cast<const float*>(B)[(size_t)k * N + n];
      else v = __half2float(reinterpret_cast<const __half*>(B)[(size_t)k * N + n]);
    }
    tile[ty + 8 * i][tx] = v;
  }
  __syncthreads();
  const size_t plane = (size_t)Np * Kp;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int n = n0 + ty + 8 * i, k = k0 + 2 * tx;
    if (n >= Np || k >= Kp) continue;
    const float x0 = tile[2 * tx][ty + 8 * i], x1 = tile[2 * tx + 1][ty + 8 * i];
    uint16_t* dst = out + (size_t)n * Kp + k;
    if (sizeof(IN) == 2) {
      const __half2 h = __floats2half2_rn(x0, x1);       // exact: the values came from halves
      *reinterpret_cast<__half2*>(dst) = h;
    } else {
      __nv_bfloat16 h0, m0, l0, h1, m1, l1;
      split3(x0, h0, m0, l0);
      split3(x1, h1, m1, l1);
      *reinterpret_cast<__nv_bfloat162*>(dst) = __halves2bfloat162(h0, h1);
      if (P == 3) {
        *reinterpret_cast<__nv_bfloat162*>(dst + plane) = __halves2bfloat162(m0, m1);
        *reinterpret_cast<__nv_bfloat162*>(dst + 2 * plane) = __halves2bfloat162(l0, l1);
      }
    }
  }
}

// ---------------------------------------------------------------- main kernel
// PAIR: two CTAs of a cluster work as one MMA unit (cta_group::2) on 2 x MT x 128 rows by BN columns;
// each stages its own rows of A and its own half of the BN columns of B, so a stage carries half the B
// bytes per MMA: what binds the single-CTA form is the bytes per clock an SM receives from L2.
template <bool PAIR>
__global__ void __launch_bounds__(kThreads, 1) dense_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                               const __grid_constant__ CUtensorMap tmap_b,
                                                               const Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);             // [kMaxStages] the stage's tiles landed
  uint64_t* empty = full + kMaxStages;                             // [kMaxStages] its MMAs are done
  uint64_t* acc_ready = empty + kMaxStages;                        // [1]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  uint8_t* tiles = smem + 1024;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // row tiles vary fastest, so the CTAs that share a B tile run at the same time
  const int row0 = blockIdx.x * (p.MT * kBM);
  const int col0 = blockIdx.y * p.BN;
  const int tn = min(p.BN, p.N - col0);
  const int nkb = (p.K + kBK - 1) / kBK;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;   // 0: the CTA that issues the pair's MMAs

  if (tid == 0) {
    for (int s = 0; s < kMaxStages; s++) {
      mbar_init(smem_u32(&full[s]), PAIR ? 2 : 1);      // pair: one arrival per CTA's producer, on the leader's barrier
      mbar_init(smem_u32(&empty[s]), p.issuers);         // one commit per issuing thread
    }
    mbar_init(smem_u32(acc_ready), p.issuers);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(tmem_base_slot), (uint32_t)p.tmem_cols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_base_slot), (uint32_t)p.tmem_cols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();                        // both CTAs' barriers exist before either signals the other's
  tc_fence_after();
  const uint32_t own_tmem = *tmem_base_slot;           // what this CTA's allocation returned (freed at the end)
  // the accumulators' address is the leader's: its thread issues the MMAs for both CTAs
  const uint32_t tmem_base = PAIR ? ld_cluster_u32(mapa_u32(smem_u32(tmem_base_slot), 0)) : own_tmem;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  bool ok = true;
  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      asm volatile("griddepcontrol.wait;" ::: "memory");   // the planes are written by the launches before
      int s = 0;
      uint32_t par = 0;
      const uint32_t tx_bytes = (uint32_t)(p.planes * p.MT * kATile + p.planes * p.b_tile);
      for (int kb = 0; kb < nkb; kb++) {
        if (kb >= p.stages) {
          if (!mbar_wait(smem_u32(&empty[s]), par ^ 1u, abort_flag, p.status)) break;
        }
        // a box beyond K or beyond the last row is filled with zeros and still counts its bytes
        uint32_t dst = smem_u32(tiles) + (uint32_t)s * (uint32_t)p.stage_bytes;
        if (PAIR) {
          // both CTAs' bytes are counted on the LEADER's barrier, the one its MMA thread waits on
          const uint32_t bar = mapa_u32(smem_u32(&full[s]), 0);
          mbar_expect_tx_cluster(bar, tx_bytes);
          for (int pl = 0; pl < p.planes; pl++)
            for (int t = 0; t < p.MT; t++, dst += kATile)
              tma_load_2d_pair(dst, &tmap_a, kb * kBK, pl * p.a_plane_rows + row0 + t * kBM, bar);
          for (int pl = 0; pl < p.planes; pl++, dst += p.b_tile)     // this CTA's half of the BN columns
            tma_load_2d_pair(dst, &tmap_b, kb * kBK, pl * p.b_plane_rows + col0 + (int)rank * (p.BN / 2), bar);
        } else {
          const uint32_t bar = smem_u32(&full[s]);
          mbar_expect_tx(bar, tx_bytes);
          for (int pl = 0; pl < p.planes; pl++)
            for (int t = 0; t < p.MT; t++, dst += kATile)
              tma_load_2d(dst, &tmap_a, kb * kBK, pl * p.a_plane_rows + row0 + t * kBM, bar);
          for (int pl = 0; pl < p.planes; pl++, dst += p.b_tile)
            tma_load_2d(dst, &tmap_b, kb * kBK, pl * p.b_plane_rows + col0, bar);
        }
        if (++s == p.stages) s = 0, par ^= 1u;
      }
    }
  } else if (warp == 1 || (warp == kSecondIssuerWarp && p.issuers == 2)) {
    // ------------------------------------------------------------ MMA issuer(s) (pair: the leader's only)
    // The single-CTA three-plane form has TWO issuing threads: 24 MMAs per stage with their address
    // arithmetic and descriptor packing are more than one thread gets through in the stage's tensor
    // time.  Thread 0 (warp 1) sends pairs 3-5 (two small products into its own accumulator, then the
    // leading product), thread 1 sends pairs 0-2 (three small products into a third accumulator); the
    // epilogue adds the accumulators.
    const int who = (warp == 1) ? 0 : 1;
    const int q_lo = (p.issuers == 2) ? (who == 0 ? 3 : 0) : 0, q_hi = (p.issuers == 2) ? (who == 0 ? 6 : 3) : p.npairs;
    if (lane == 0 && rank == 0) {
      int s = 0;
      uint32_t par = 0;
      const uint64_t desc0 = smem_desc_sw128(smem_u32(tiles));
      const uint32_t lo0 = (uint32_t)desc0, desc_hi = (uint32_t)(desc0 >> 32);
      const uint32_t slot_step = (uint32_t)p.stage_bytes >> 4;
      const uint32_t a_tile_step = (uint32_t)kATile >> 4, b_off = (uint32_t)p.a_bytes >> 4;
      const uint32_t b_tile_step = (uint32_t)p.b_tile >> 4;
      uint32_t soff = 0;
      for (int kb = 0; kb < nkb; kb++) {
        ok = mbar_wait(smem_u32(&full[s]), par, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
        for (int t = 0; t < p.MT; t++) {
          // With three planes the leading product ah*bh has an accumulator of its own and the five
          // small ones share a second: the tensor core truncates every f32 accumulation, so small
          // terms added to the large sum would each cost an ulp of the LARGE sum.
          const uint32_t d_main = tmem_base + (uint32_t)(t * p.BN);
          const uint32_t d_corr = tmem_base + (uint32_t)(((1 + who) * p.MT + t) * p.BN);   // this thread's own
          for (int q = q_lo; q < q_hi; q++) {
            const uint32_t pa = (p.pair_a >> (4 * q)) & 15u, pb = (p.pair_b >> (4 * q)) & 15u;
            const uint32_t a_lo = lo0 + soff + (uint32_t)((int)pa * p.MT + t) * a_tile_step;
            const uint32_t b_lo = lo0 + soff + b_off + pb * b_tile_step;
            const bool lead = (pa | pb) == 0u;
            const uint32_t first = (kb > 0 || (!lead && q > q_lo)) ? 1u : 0u;
            if (PAIR) umma_f16_kblock_pair(lead ? d_main : d_corr, a_lo, b_lo, desc_hi, p.idesc, first);
            else umma_f16_kblock(lead ? d_main : d_corr, a_lo, b_lo, desc_hi, p.idesc, first);
          }
        }
        if (PAIR) {                                    // the stage is free in both CTAs
          umma_commit_pair(smem_u32(&empty[s]));
          umma_commit_pair(mapa_u32(smem_u32(&empty[s]), 1));
        } else {
          umma_commit(smem_u32(&empty[s]));
        }
        soff += slot_step;
        if (++s == p.stages) s = 0, par ^= 1u, soff = 0;
      }
      if (ok) {
        if (PAIR) {
          umma_commit_pair(smem_u32(acc_ready));
          umma_commit_pair(mapa_u32(smem_u32(acc_ready), 1));
        } else {
          umma_commit(smem_u32(acc_ready));
        }
      }
    }
  } else if (warp >= 2 && warp <= 5) {
    // ------------------------------------------------------------ epilogue (warps 2-5)
    const bool got = __all_sync(0xffffffffu, mbar_wait(smem_u32(acc_ready), 0, abort_flag, p.status));
    tc_fence_after();
    if (got) {
      const int q = warp & 3;                          // TMEM lane quarter this warp may read
      // tcgen05.ld hands lane l the 32 columns of accumulator row 32 * q + l; the warp turns the
      // 32 x 32 chunk around in shared memory (the ring is idle by now) and stores whole row segments.
      constexpr int kPitch = 36;                       // floats per staged row: 16-byte aligned, conflict-free
      float* stage = reinterpret_cast<float*>(tiles) + q * (32 * kPitch);
      const int sr = lane >> 3, sc = (lane & 7) * 4;
#pragma unroll 1
      for (int t = 0; t < p.MT; t++) {
        const int rbase = row0 + t * kBM + q * 32;
        if (rbase >= p.M) break;
#pragma unroll 1
        for (int c = 0; c < tn; c += 32) {
          uint32_t r[32];
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(t * p.BN + c), r);
          tmem_ld_wait();
          for (int extra = 1; extra <= (p.npairs > 1 ? p.issuers : 0); extra++) {   // the small products' accumulator(s)
            uint32_t r2[32];
            tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)((extra * p.MT + t) * p.BN + c), r2);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(r2[i]));
          }
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(stage + lane * kPitch + i) =
                make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                            __uint_as_float(r[i + 3]));
          __syncwarp();
          const int cc = c + sc;                       // first of this lane's four columns within the tile
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const int rr = 4 * i + sr;
            const int row = rbase + rr;
            if (row >= p.M || cc >= tn) continue;
            const float4 v = *reinterpret_cast<const float4*>(stage + rr * kPitch + sc);
            const float vv[4] = {v.x, v.y, v.z, v.w};
            const size_t at = (size_t)row * p.N + col0 + cc;
            if (p.out_f16) {
              __half* dst = static_cast<__half*>(p.C) + at;
              if (cc + 4 <= tn && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
                const __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
                uint2 pk;
                pk.x = *reinterpret_cast<const uint32_t*>(&h0), pk.y = *reinterpret_cast<const uint32_t*>(&h1);
                *reinterpret_cast<uint2*>(dst) = pk;
              } else {
#pragma unroll
                for (int j = 0; j < 4; j++)
                  if (cc + j < tn) dst[j] = __float2half_rn(vv[j]);
              }
            } else {
              float* dst = static_cast<float*>(p.C) + at;
              if (cc + 4 <= tn && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                *reinterpret_cast<float4*>(dst) = v;
              } else {
#pragma unroll
                for (int j = 0; j < 4; j++)
                  if (cc + j < tn) dst[j] = vv[j];
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
  if (PAIR) cluster_sync_all();     // the peer's MMAs read this CTA's shared memory and signal its barriers until here
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(own_tmem, (uint32_t)p.tmem_cols);
    else tmem_dealloc(own_tmem, (uint32_t)p.tmem_cols);
  }
}

// ---------------------------------------------------------------- host side
struct Plan {
  bool pair;
  int MT, BN, planes, npairs, issuers, stages, tmem_cols;
  int a_bytes, b_tile, stage_bytes;
  int64_t Mp, Np, Kp;
  size_t smem;
  dim3 grid;
};

// Set when a cluster launch was refused on this process's device (a partition without cluster support):
// plans then stay on single CTAs.
bool g_pairs_refused = false;

Plan make_plan(int dtype, int mode, int64_t M, int64_t N, int64_t K) {
  Plan pl{};
  const bool exact = (dtype == kDenseF32 && mode != kDenseTcFast);
  pl.planes = exact ? 3 : 1;
  pl.npairs = exact ? 6 : 1;
  const int sms = device_sm_count();
  const int n16 = (int)((N + 15) / 16 * 16), n32 = (int)((N + 31) / 32 * 32);
  static const bool no_pair = getenv("SMITH_DENSE_NO_PAIR") != nullptr;   // for A/B measurements
  auto waves = [](int64_t tiles, int64_t units) { return (double)((tiles + units - 1) / units); };
  if (exact) {
    // One CTA: 128 x 128 tiles (six 16 KB plane tiles per stage, two stages).  A CTA pair: 256 x 256
    // tiles, each CTA staging 48 KB of A and its 48 KB half of B per stage; the MMA thread then issues
    // the same 24 instructions per stage for twice the tensor time and each SM receives half the B
    // bytes per MMA (measured: 84 % of the tensor pipe busy against 62 to 66 % for single CTAs, whose
    // stages need 61 bytes per clock from L2 at the full MMA rate).
    // The pair's tile is four times as large, so it is taken where the waves it leaves cost less.
    pl.MT = 1, pl.BN = (n16 < 128) ? n16 : 128;
    const int bn2 = (n32 < 256) ? n32 : 256;
    const double t1 = waves((M + 127) / 128 * ((N + 127) / 128), sms) / 0.66;
    const double t2 = waves((M + 255) / 256 * ((N + bn2 - 1) / bn2), sms / 2) * 2.0 * (bn2 / 128.0) / 2.0 / 0.85;
    pl.pair = !no_pair && !g_pairs_refused && M > kBM && N > 128 && t2 < t1;
    if (pl.pair) pl.BN = bn2;
  } else {
    // one plane per operand: 256 x 256 tiles on one CTA.  (512 x 256 tiles on a CTA pair, 48 KB instead
    // of 64 KB staged per 256 x 256 x 64 of MMA work, measured SLOWER: 179 against 138 us at f16 4096^3.)
    pl.MT = (M > 128) ? 2 : 1;
    pl.BN = (n16 < 256) ? n16 : 256;
    pl.pair = false;
  }
  pl.a_bytes = pl.planes * pl.MT * kATile;
  pl.b_tile = (pl.pair ? pl.BN / 2 : pl.BN) * kBK * 2;
  pl.b_tile = (pl.b_tile + 1023) / 1024 * 1024;  // every tile starts on 1024 bytes (the swizzle pattern's period)
  pl.stage_bytes = pl.a_bytes + pl.planes * pl.b_tile;
  int stages = (226 * 1024 - 1024) / pl.stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  pl.stages = stages;
  int cols = 32;                                 // the epilogue reads whole 32-column chunks
  pl.issuers = (exact && !pl.pair) ? 2 : 1;
  const int accs = pl.MT * (exact ? 1 + pl.issuers : 1);   // three planes: one more accumulator per issuing thread for the small products
  while (cols < (accs - 1) * pl.BN + (pl.BN + 31) / 32 * 32) cols <<= 1;
  pl.tmem_cols = cols;
  pl.smem = 1024 + (size_t)stages * pl.stage_bytes;
  pl.Kp = (K + 7) / 8 * 8;
  pl.Mp = (M + 511) / 512 * 512;                 // whole row tiles of a pair, so a plane's boxes stay inside the plane
  pl.Np = (N + 31) / 32 * 32;
  unsigned gx = (unsigned)((M + pl.MT * kBM - 1) / (pl.MT * kBM));
  if (pl.pair) gx = (gx + 1) & ~1u;              // an odd last row tile gets a partner that stores nothing
  pl.grid = dim3(gx, (unsigned)((N + pl.BN - 1) / pl.BN));
  return pl;
}

template <typename... Args>
cudaError_t launch_pdl_cluster(void (*kernel)(Args...), int cluster_x, dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                               Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cluster_x > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)cluster_x, attr[1].val.clusterDim.y = 1, attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args...);
  count_launch();
  return e;
}

template <typename... Args>
cudaError_t launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  return launch_pdl_cluster(kernel, 1, grid, block, smem, s, args...);
}

bool encode_2d(CUtensorMap* map, bool f16, const void* base, int64_t inner, int64_t rows, int64_t pitch_elems, int box_rows) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)pitch_elems * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return enc(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
             dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool dense_tc_supports(int dtype, int64_t M, int64_t N, int64_t K) {
  if (dtype != kDenseF32 && dtype != kDenseF16) return false;
  if (M < 1 || N < 1 || K < 1) return false;
  if (M > (1 << 24) || N > (1 << 24) || K > (1 << 24)) return false;
  if (dtype == kDenseF16 && (K % 8) != 0) return false;          // A is read in place: rows must start on 16 bytes
  if ((M + 127) / 128 > 65535 * 2 || (N + 127) / 128 > 65535) return false;
  return encode_fn() != nullptr;
}

size_t dense_tc_workspace_bytes(int dtype, int mode, int64_t M, int64_t N, int64_t K) {
  const Plan pl = make_plan(dtype, mode, M, N, K);
  const size_t a = (dtype == kDenseF32) ? (size_t)pl.planes * pl.Mp * pl.Kp * 2 : 0;
  const size_t b = (size_t)pl.planes * pl.Np * pl.Kp * 2;
  return ((a + 1023) & ~size_t(1023)) + ((b + 1023) & ~size_t(1023)) + 1024;
}

namespace {
cudaError_t launch_dense_tc_once(int dtype, int mode, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                                 Workspace ws, cudaStream_t s, bool* was_pair);
}

cudaError_t launch_dense_tc(int dtype, int mode, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                            Workspace ws, cudaStream_t s) {
  bool was_pair = false;
  cudaError_t e = launch_dense_tc_once(dtype, mode, A, B, C, M, N, K, ws, s, &was_pair);
  if (e != cudaSuccess && was_pair && !g_pairs_refused) {
    // the cluster launch itself was refused: run this and every later product on single CTAs
    cudaGetLastError();
    g_pairs_refused = true;
    e = launch_dense_tc_once(dtype, mode, A, B, C, M, N, K, ws, s, &was_pair);
  }
  return e;
}

namespace {
cudaError_t launch_dense_tc_once(int dtype, int mode, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                                 Workspace ws, cudaStream_t s, bool* was_pair) {
  if (!dense_tc_supports(dtype, M, N, K)) return cudaErrorInvalidValue;
  const Plan pl = make_plan(dtype, mode, M, N, K);
  *was_pair = false;
  if (pl.stages < 2 || pl.smem > 227 * 1024) return cudaErrorInvalidValue;
  if (!ws.ptr || ws.bytes < dense_tc_workspace_bytes(dtype, mode, M, N, K) || (reinterpret_cast<uintptr_t>(ws.ptr) & 255))
    return cudaErrorInvalidValue;
  const bool f16 = dtype == kDenseF16;
  if (f16 && (reinterpret_cast<uintptr_t>(A) & 15)) return cudaErrorMisalignedAddress;
  const size_t a_bytes = f16 ? 0 : (((size_t)pl.planes * pl.Mp * pl.Kp * 2 + 1023) & ~size_t(1023));
  uint8_t* base = static_cast<uint8_t*>(ws.ptr);
  uint16_t* a_planes = reinterpret_cast<uint16_t*>(base);
  uint16_t* b_planes = reinterpret_cast<uint16_t*>(base + a_bytes);
  cudaError_t e;
  const dim3 tgrid((unsigned)(pl.Np / 32), (unsigned)((pl.Kp + 63) / 64));
  if (tgrid.y > 65535) return cudaErrorInvalidValue;
  if (f16) {
    e = launch_pdl(split_transpose_kernel<__half, 1>, tgrid, dim3(256), (size_t)0, s, (const __half*)B, b_planes, (int)K,
                   (int)N, (int)pl.Np, (int)pl.Kp);
  } else {
    const dim3 agrid((unsigned)M, (unsigned)((pl.Kp / 2 + 255) / 256 > 64 ? 64 : (pl.Kp / 2 + 255) / 256));
    if (pl.planes == 3) {
      e = launch_pdl(split_rows_kernel<3>, agrid, dim3(256), (size_t)0, s, (const float*)A,
                     reinterpret_cast<__nv_bfloat16*>(a_planes), (int)M, (int)K, (int)pl.Mp, (int)pl.Kp);
      if (e == cudaSuccess)
        e = launch_pdl(split_transpose_kernel<float, 3>, tgrid, dim3(256), (size_t)0, s, (const float*)B, b_planes, (int)K,
                       (int)N, (int)pl.Np, (int)pl.Kp);
    } else {
      e = launch_pdl(split_rows_kernel<1>, agrid, dim3(256), (size_t)0, s, (const float*)A,
                     reinterpret_cast<__nv_bfloat16*>(a_planes), (int)M, (int)K, (int)pl.Mp, (int)pl.Kp);
      if (e == cudaSuccess)
        e = launch_pdl(split_transpose_kernel<float, 1>, tgrid, dim3(256), (size_t)0, s, (const float*)B, b_planes, (int)K,
                       (int)N, (int)pl.Np, (int)pl.Kp);
    }
  }
  if (e != cudaSuccess) return e;

  CUtensorMap map_a, map_b;
  if (f16) {
    if (!encode_2d(&map_a, true, A, K, M, K, kBM)) return cudaErrorInvalidValue;
  } else {
    if (!encode_2d(&map_a, false, a_planes, K, (int64_t)pl.planes * pl.Mp, pl.Kp, kBM)) return cudaErrorInvalidValue;
  }
  if (!encode_2d(&map_b, f16, b_planes, K, (int64_t)pl.planes * pl.Np, pl.Kp, pl.pair ? pl.BN / 2 : pl.BN)) return cudaErrorInvalidValue;

  Params p{};
  p.C = C, p.M = (int)M, p.N = (int)N, p.K = (int)K, p.out_f16 = f16 ? 1 : 0;
  p.MT = pl.MT, p.BN = pl.BN, p.planes = pl.planes, p.npairs = pl.npairs, p.issuers = pl.issuers;
  // the five small products (smallest first), then the leading one
  static const int pa[kMaxPairs] = {1, 2, 0, 1, 0, 0}, pb[kMaxPairs] = {1, 0, 2, 0, 1, 0};
  p.pair_a = p.pair_b = 0;
  if (pl.npairs == 6)
    for (int i = 0; i < kMaxPairs; i++) p.pair_a |= (uint32_t)pa[i] << (4 * i), p.pair_b |= (uint32_t)pb[i] << (4 * i);
  p.a_plane_rows = (int)pl.Mp, p.b_plane_rows = (int)pl.Np;
  p.a_bytes = pl.a_bytes, p.b_tile = pl.b_tile, p.stage_bytes = pl.stage_bytes, p.stages = pl.stages, p.tmem_cols = pl.tmem_cols;
  // tcgen05.mma kind::f16 instruction descriptor: [4,6) D = f32; [7,10) A format, [10,13) B format
  // (0 = f16, 1 = bf16); both operands K-major; [17,23) N >> 3; [24,29) M >> 4
  const uint32_t fmt = f16 ? 0u : 1u;
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(pl.BN >> 3) << 17) |
            ((uint32_t)((pl.pair ? 2 * kBM : kBM) >> 4) << 24);
  p.status = kernel_status_ptr();
  if (!p.status) return cudaErrorUnknown;

  static PerDeviceFlag configured;
  bool* set = configured.here();
  if (!set) return cudaErrorInvalidDevice;
  if (!*set) {
    e = cudaFuncSetAttribute(dense_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(dense_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    *set = true;
  }
  if (pl.pair) {
    e = launch_pdl_cluster(dense_tc_kernel<true>, 2, pl.grid, dim3(kThreads), pl.smem, s, map_a, map_b, p);
    *was_pair = (e != cudaSuccess);      // only a refused LAUNCH is retried; earlier errors are reported as they are
  } else {
    e = launch_pdl(dense_tc_kernel<false>, pl.grid, dim3(kThreads), pl.smem, s, map_a, map_b, p);
  }
  return e != cudaSuccess ? e : cudaGetLastError();
}
}  // namespace

}  // namespace smith
