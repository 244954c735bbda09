// qgemv_common.cuh -- device helpers shared by the GEMV kernels (qgemv.cu: one matrix or a few per
// launch; qgemv_list.cu: a whole list of matrices per persistent launch): activations to block
// fixed point, the dp4a dot product of one packed block, and the 2-D tensor-map box copy.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "kernels.h"

namespace smith {

__device__ __forceinline__ int dp4a_ss(int a, int b, int c) {
  int d;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_su(int a, unsigned b, int c) {  // a signed bytes, b unsigned bytes
  int d;
  asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// Quantise the activations of one (row, group) to digit words; eight threads
// per group, four consecutive k each (lane8 = position inside the group).
//   digits: 64 bytes.  Q4: word i*4 + {0,1,2,3} = {even-k hi, even-k lo, odd-k hi, odd-k lo}
//                          of k = 8i .. 8i+7 (byte b of an even word is k = 8i + 2b).
//                      Q8: word i*2 + {0,1} = {hi, lo} of k = 4i .. 4i+3.
//   sc: {2^-e, float(sum_k x_int)}.
template <int KIND>
__device__ __forceinline__ void quantise_quarter(const float4 t, int lane8, uint8_t* digits, float2* sc) {
  const float v[4] = {t.x, t.y, t.z, t.w};
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  int bad = 0;
#pragma unroll
  for (int i = 0; i < 4; i++) bad |= !(fabsf(v[i]) <= 3.4028234e38f);  // inf or NaN
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    bad |= __shfl_xor_sync(0xffffffffu, bad, o);
  }
  const int ex = (int)(__float_as_uint(amax) >> 23) & 0xFF;
  int e = (ex == 0) ? 0 : (13 - (ex - 127));  // amax * 2^e in [2^13, 2^14)
  e = max(-126, min(126, e));
  const float up = __uint_as_float((unsigned)(127 + e) << 23);
  float down = __uint_as_float((unsigned)(127 - e) << 23);
  if (bad) down = __int_as_float(0x7FC00000);  // let inf / NaN reach the outputs of every column
  int q[4], sum = 0;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    q[i] = max(-16383, min(16383, __float2int_rn(v[i] * up)));
    sum += q[i];
  }
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (KIND == 4) {
    // k = 4*lane8 + i lives in code word (lane8 >> 1); even k -> bytes {0,1} or {2,3} of the even words
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int word = lane8 >> 1, byte = ((lane8 & 1) << 1) | (i >> 1), odd = i & 1;
      uint8_t* w = digits + word * 16 + odd * 8 + byte;
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
    reinterpret_cast<uint2*>(digits)[lane8] = make_uint2(hi, lo);
  }
  if (lane8 == 0) *sc = make_float2(down, (float)sum);
}

// One 32-weight block against MR activation rows.
template <int KIND, int MR>
__device__ __forceinline__ void block_dot(const uint8_t* __restrict__ blk, uint32_t off_in_stage,
                                          const uint4* __restrict__ xd, const float2* __restrict__ xs, int G,
                                          float (&acc)[MR]) {
  if (KIND == 4) {
    const uint2 n0 = *reinterpret_cast<const uint2*>(blk);
    const uint2 n1 = *reinterpret_cast<const uint2*>(blk + 8);
    const float2 sz = *reinterpret_cast<const float2*>(blk + 16);
    const uint32_t w[4] = {n0.x, n0.y, n1.x, n1.y};
    uint32_t be[4], bo[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      be[i] = w[i] & 0x0F0F0F0Fu;   // codes of even k
      bo[i] = w[i] & 0xF0F0F0F0u;   // 16 * codes of odd k
    }
#pragma unroll
    for (int m = 0; m < MR; m++) {
      int eh = 0, el = 0, oh = 0, ol = 0;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const uint4 d = xd[(size_t)m * G * 4 + i];
        eh = dp4a_su((int)d.x, be[i], eh);
        el = dp4a_su((int)d.y, be[i], el);
        oh = dp4a_su((int)d.z, bo[i], oh);
        ol = dp4a_su((int)d.w, bo[i], ol);
      }
      const int dot = (eh * 128 + el) + ((oh * 128 + ol) >> 4);  // odd part is an exact multiple of 16
      const float2 s = xs[(size_t)m * G];
      acc[m] = fmaf(sz.x * s.x, fmaf(-sz.y, s.y, (float)dot), acc[m]);
    }
  } else {
    // 34-byte blocks are only 2-byte aligned: read the aligned words around the
    // 32 code bytes and shift.  Stage base and row pitch are multiples of 16, so
    // the offset inside the stage gives the alignment.
    const uint32_t off = off_in_stage + 2;
    const uint32_t sh = (off & 3u) * 8;
    const uint32_t* al = reinterpret_cast<const uint32_t*>(blk + 2 - (off & 3u));
    uint32_t raw[9];
#pragma unroll
    for (int i = 0; i < 9; i++) raw[i] = al[i];
    uint32_t cw[8];
#pragma unroll
    for (int i = 0; i < 8; i++) cw[i] = __funnelshift_r(raw[i], raw[i + 1], sh);
    const float scale = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(blk)));
#pragma unroll
    for (int m = 0; m < MR; m++) {
      int dh = 0, dl = 0;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const uint4 d = xd[(size_t)m * G * 4 + i];
        dh = dp4a_ss((int)d.x, (int)cw[2 * i], dh);
        dl = dp4a_ss((int)d.y, (int)cw[2 * i], dl);
        dh = dp4a_ss((int)d.z, (int)cw[2 * i + 1], dh);
        dl = dp4a_ss((int)d.w, (int)cw[2 * i + 1], dl);
      }
      const float2 s = xs[(size_t)m * G];
      acc[m] = fmaf(scale * s.x, (float)(dh * 128 + dl), acc[m]);
    }
  }
}

// ---- the same block product on 32-bit shared-memory addresses (explicit ld.shared)
__device__ __forceinline__ uint2 lds_b64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ uint4 lds_b128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_b32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_b16(uint32_t a) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
  return v;
}

// blk: shared address of the packed block; xd: shared address of the group's four digit words of row 0
// (row m lies m * G * 64 bytes further); xs: shared address of its {scale, sum} pair (row m: + m * G * 8).
template <int KIND, int MR>
__device__ __forceinline__ void block_dot_s(uint32_t blk, uint32_t xd, uint32_t xs, int G, float (&acc)[MR]) {
  if (KIND == 4) {
    const uint2 n0 = lds_b64(blk), n1 = lds_b64(blk + 8), szb = lds_b64(blk + 16);
    const float sc = __uint_as_float(szb.x), zp = __uint_as_float(szb.y);
    const uint32_t w[4] = {n0.x, n0.y, n1.x, n1.y};
    uint32_t be[4], bo[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      be[i] = w[i] & 0x0F0F0F0Fu;   // codes of even k
      bo[i] = w[i] & 0xF0F0F0F0u;   // 16 * codes of odd k
    }
#pragma unroll
    for (int m = 0; m < MR; m++) {
      int eh = 0, el = 0, oh = 0, ol = 0;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const uint4 d = lds_b128(xd + (uint32_t)(m * G * 64 + i * 16));
        eh = dp4a_su((int)d.x, be[i], eh);
        el = dp4a_su((int)d.y, be[i], el);
        oh = dp4a_su((int)d.z, bo[i], oh);
        ol = dp4a_su((int)d.w, bo[i], ol);
      }
      const int dot = (eh * 128 + el) + ((oh * 128 + ol) >> 4);  // odd part is an exact multiple of 16
      const uint2 sb = lds_b64(xs + (uint32_t)(m * G * 8));
      acc[m] = fmaf(sc * __uint_as_float(sb.x), fmaf(-zp, __uint_as_float(sb.y), (float)dot), acc[m]);
    }
  } else {
    // 34-byte blocks are only 2-byte aligned: read the aligned words around the 32 code bytes and shift
    const uint32_t off = blk + 2;
    const uint32_t sh = (off & 3u) * 8;
    const uint32_t al = off & ~3u;
    uint32_t raw[9];
#pragma unroll
    for (int i = 0; i < 9; i++) raw[i] = lds_b32(al + 4u * i);
    uint32_t cw[8];
#pragma unroll
    for (int i = 0; i < 8; i++) cw[i] = __funnelshift_r(raw[i], raw[i + 1], sh);
    const float scale = __half2float(__ushort_as_half((unsigned short)lds_b16(blk)));
#pragma unroll
    for (int m = 0; m < MR; m++) {
      int dh = 0, dl = 0;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const uint4 d = lds_b128(xd + (uint32_t)(m * G * 64 + i * 16));
        dh = dp4a_ss((int)d.x, (int)cw[2 * i], dh);
        dl = dp4a_ss((int)d.y, (int)cw[2 * i], dl);
        dh = dp4a_ss((int)d.z, (int)cw[2 * i + 1], dh);
        dl = dp4a_ss((int)d.w, (int)cw[2 * i + 1], dl);
      }
      const uint2 sb = lds_b64(xs + (uint32_t)(m * G * 8));
      acc[m] = fmaf(scale * __uint_as_float(sb.x), (float)(dh * 128 + dl), acc[m]);
    }
  }
}

__device__ __forceinline__ void tma_box_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar,
                                           uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar), "l"(policy)
      : "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime (the library does not link libcuda); nullptr if the driver lacks it.
inline EncodeTiledFn encode_fn() {
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

}  // namespace smith
