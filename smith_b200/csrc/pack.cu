// pack.cu -- device packers for Smith's 32-element block formats.
//
// pack_q4 reproduces the reference's host packer quantizeQ4
// (src/ops/quantize.js:14-68) bit for bit: the reference computes in JavaScript
// Numbers, i.e. IEEE f64, so the min/max scan, range, scale, zero point and
// every code are evaluated here in f64 with explicitly rounded (never fused)
// operations, Math.round is restated as "floor, then +1 if the fraction >= 0.5",
// and scale/zero are rounded to f32 only when stored (quantize.js:55-58).
// Quirks kept: a constant group gets scale 1 / zero 8; min == +0 stores zero
// as -0.0; NaN inputs never win a comparison and encode as code 0; the tail
// group takes min/max over its valid rows only and pads codes with v = 0.
//
// pack_q8 has no reference counterpart (the reference never produces the
// layout its matmul_q8 shader reads, shaders/matmul_q8.metal:40-52).  The rule:
// amax = max|v| over valid rows; d = amax/127 (f64); h = the reference's own
// truncating f16 encoder applied to d (src/dtype.js:29-58); dq = decode(h)
// (src/dtype.js:60-79); code = dq > 0 ? clamp(round_half_up(v/dq), -127, 127) : 0.
// Block bytes: [f16 scale, little endian][32 x int8].
//
// Speed: 32 f64 divisions per block would make the packers divide-bound (measured 1.84 TB/s of
// read + write traffic, 0.28 of the HBM copy peak).  A code only depends on which side of a
// half-integer the quotient falls, so each element first takes v * (1 / scale), which is within a few
// ulps of the correctly rounded quotient, and only when the result lies closer to a half-integer than
// that error can reach (about once in 10^13 elements for ordinary data) is the reference's own
// expression, division included, evaluated.  The codes are the same bit for bit either way.
//
// Layout of both outputs: block (g, col) at byte (g*N + col) * block_bytes, so
// for one g the N blocks are contiguous.  One thread packs one block; a CTA
// packs 256 adjacent columns of one group, reads W coalesced (adjacent threads
// read adjacent floats of a row) and writes its blocks through shared memory
// so the global stores are contiguous.
#include "kernels.h"

namespace smith {

namespace {

constexpr int kPackThreads = 256;

__device__ __forceinline__ double js_round(double x) {
  double f = floor(x);
  return (__dsub_rn(x, f) >= 0.5) ? f + 1.0 : f;
}

// src/dtype.js:29-58 (bit-level restatement, including the subnormal branch
// that ends up returning a signed zero).
__device__ __forceinline__ uint32_t js_to_float16(double val) {
  float f = __double2float_rn(val);
  uint32_t bits = __float_as_uint(f);
  uint32_t sign = (bits >> 31) & 1u;
  int e = (int)((bits >> 23) & 0xFFu);
  uint32_t frac = bits & 0x7FFFFFu;
  if (e == 0xFF) return (sign << 15) | 0x7C00u | (frac ? 0x200u : 0u);
  e -= 127;
  if (e > 15) return (sign << 15) | 0x7C00u;
  if (e < -14) {
    if (e < -24) return sign << 15;
    frac |= 0x800000u;
    frac >>= (-1 - e);
    return (sign << 15) | (frac >> 13);
  }
  return (sign << 15) | ((uint32_t)(e + 15) << 10) | (frac >> 13);
}

// src/dtype.js:60-79, exact in f64.
__device__ __forceinline__ double js_from_float16(uint32_t h) {
  uint32_t sign = (h >> 15) & 1u;
  int e = (int)((h >> 10) & 0x1Fu);
  uint32_t frac = h & 0x3FFu;
  double v;
  if (e == 0) {
    v = (double)frac * 5.9604644775390625e-08;  // frac/1024 * 2^-14 = frac * 2^-24
  } else if (e == 31) {
    v = frac ? __longlong_as_double(0x7FF8000000000000LL) : __longlong_as_double(0x7FF0000000000000LL);
  } else {
    long long bits = ((long long)(e - 15 + 1023) << 52) | ((long long)frac << 42);
    v = __longlong_as_double(bits);
  }
  return sign ? -v : v;
}

__global__ void __launch_bounds__(kPackThreads)
pack_q4_kernel(const float* __restrict__ w, uint8_t* __restrict__ out, int64_t K, int64_t N) {
  __shared__ __align__(16) uint2 stage[kPackThreads * 3];
  const int64_t g = blockIdx.y;
  const int64_t col0 = (int64_t)blockIdx.x * kPackThreads;
  const int64_t col = col0 + threadIdx.x;
  const int64_t k0 = g * kQ4Group;
  const int valid = (int)((K - k0 < kQ4Group) ? (K - k0) : kQ4Group);

  if (col < N) {
    float v[kQ4Group];
    const float* src = w + k0 * N + col;
#pragma unroll
    for (int k = 0; k < kQ4Group; k++) v[k] = (k < valid) ? src[(int64_t)k * N] : 0.0f;

    // quantize.js:26-31 -- in-order compares so NaN and signed zeros behave as in JS.
    float mn = __int_as_float(0x7F800000), mx = __int_as_float(0xFF800000);
#pragma unroll
    for (int k = 0; k < kQ4Group; k++) {
      if (k < valid) {
        if (v[k] < mn) mn = v[k];
        if (v[k] > mx) mx = v[k];
      }
    }
    const double range = __dsub_rn((double)mx, (double)mn);
    const bool pos = range > 0.0;
    const double scale = pos ? __ddiv_rn(range, 15.0) : 1.0;
    const double zero = pos ? __ddiv_rn(-(double)mn, scale) : 8.0;

    const double rcp = __ddiv_rn(1.0, scale);
    uint32_t words[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int k = 0; k < kQ4Group; k++) {
      // Fast: a = v * (1/scale) differs from RN(v / scale) by at most 3 * 2^-53 * |a|, and the sum with
      // `zero` adds one more rounding of a number below 16 + |a| + |zero|.
      const double a = __dmul_rn((double)v[k], rcp);
      double t = __dadd_rn(a, zero);
      double m = (t > 0.0) ? t : 0.0;
      m = (m < 15.0) ? m : 15.0;
      double f = floor(m);
      double fr = __dsub_rn(m, f);
      if (!(fabs(__dsub_rn(fr, 0.5)) > 2e-15 * (fabs(a) + fabs(zero) + 16.0))) {
        // too close to a rounding boundary to call (or not a number): the reference's expression itself
        t = __dadd_rn(__ddiv_rn((double)v[k], scale), zero);  // quantize.js:45
        // Math.max(0, t) then Math.min(15, t); a NaN ends as code 0 like the typed-array store.
        m = (t > 0.0) ? t : 0.0;
        m = (m < 15.0) ? m : 15.0;
        f = floor(m);
        fr = __dsub_rn(m, f);
      }
      const uint32_t q = (uint32_t)((fr >= 0.5) ? f + 1.0 : f);     // Math.round: ties toward +infinity
      words[k >> 3] |= q << ((k & 7) * 4);  // element k: byte k>>1, low nibble if k even
    }
    const uint32_t sbits = __float_as_uint(__double2float_rn(scale));
    const uint32_t zbits = __float_as_uint(__double2float_rn(zero));
    uint2* mine = stage + threadIdx.x * 3;
    mine[0] = make_uint2(words[0], words[1]);
    mine[1] = make_uint2(words[2], words[3]);
    mine[2] = make_uint2(sbits, zbits);
  }
  __syncthreads();
  const int64_t ncols = (N - col0 < kPackThreads) ? (N - col0) : kPackThreads;
  uint2* dst = reinterpret_cast<uint2*>(out + (g * N + col0) * kQ4Bytes);  // 24*i is 8-byte aligned
  for (int i = threadIdx.x; i < ncols * 3; i += kPackThreads) dst[i] = stage[i];
}

__global__ void __launch_bounds__(kPackThreads)
pack_q8_kernel(const float* __restrict__ w, uint8_t* __restrict__ out, int64_t K, int64_t N) {
  __shared__ __align__(16) uint16_t stage[kPackThreads * 17];
  const int64_t g = blockIdx.y;
  const int64_t col0 = (int64_t)blockIdx.x * kPackThreads;
  const int64_t col = col0 + threadIdx.x;
  const int64_t k0 = g * kQ8Group;
  const int valid = (int)((K - k0 < kQ8Group) ? (K - k0) : kQ8Group);

  if (col < N) {
    float v[kQ8Group];
    const float* src = w + k0 * N + col;
#pragma unroll
    for (int k = 0; k < kQ8Group; k++) v[k] = (k < valid) ? src[(int64_t)k * N] : 0.0f;
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < kQ8Group; k++) {
      float a = fabsf(v[k]);
      if (k < valid && a > amax) amax = a;  // NaN never wins
    }
    const double d = __ddiv_rn((double)amax, 127.0);
    const uint32_t h = js_to_float16(d);
    const double dq = js_from_float16(h);
    const double rcp = (dq > 0.0) ? __ddiv_rn(1.0, dq) : 0.0;
    uint16_t* mine = stage + threadIdx.x * 17;
    mine[0] = (uint16_t)h;
#pragma unroll
    for (int k = 0; k < kQ8Group; k += 2) {
      int q[2];
#pragma unroll
      for (int i = 0; i < 2; i++) {
        int c = 0;
        if (k + i < valid && dq > 0.0) {
          // fast quotient first; the exact one only next to a rounding boundary (see the file comment)
          const double a = __dmul_rn((double)v[k + i], rcp);
          double f = floor(a);
          double t;
          if (fabs(__dsub_rn(__dsub_rn(a, f), 0.5)) > 2e-15 * (fabs(a) + 1.0))
            t = (__dsub_rn(a, f) >= 0.5) ? f + 1.0 : f;
          else
            t = js_round(__ddiv_rn((double)v[k + i], dq));
          if (t == t) {
            t = (t > 127.0) ? 127.0 : t;
            t = (t < -127.0) ? -127.0 : t;
            c = (int)t;
          }
        }
        q[i] = c & 0xFF;
      }
      mine[1 + (k >> 1)] = (uint16_t)(q[0] | (q[1] << 8));
    }
  }
  __syncthreads();
  const int64_t ncols = (N - col0 < kPackThreads) ? (N - col0) : kPackThreads;
  uint8_t* dstb = out + (g * N + col0) * kQ8Bytes;  // always 2-byte aligned
  const int64_t nhalf = ncols * 17;
  if ((reinterpret_cast<uintptr_t>(dstb) & 15) == 0 && (nhalf & 7) == 0) {
    uint4* dst = reinterpret_cast<uint4*>(dstb);
    const uint4* s4 = reinterpret_cast<const uint4*>(stage);
    for (int i = threadIdx.x; i < nhalf / 8; i += kPackThreads) dst[i] = s4[i];
  } else {
    uint16_t* dst = reinterpret_cast<uint16_t*>(dstb);
    for (int i = threadIdx.x; i < nhalf; i += kPackThreads) dst[i] = stage[i];
  }
}

}  // namespace

cudaError_t launch_pack_q4(const float* w, uint8_t* out, int64_t K, int64_t N, cudaStream_t s) {
  if (K <= 0 || N <= 0) return cudaSuccess;
  const int64_t groups = (K + kQ4Group - 1) / kQ4Group;
  if (groups > 65535) return cudaErrorInvalidValue;
  dim3 grid((unsigned)((N + kPackThreads - 1) / kPackThreads), (unsigned)groups);
  pack_q4_kernel<<<grid, kPackThreads, 0, s>>>(w, out, K, N);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_pack_q8(const float* w, uint8_t* out, int64_t K, int64_t N, cudaStream_t s) {
  if (K <= 0 || N <= 0) return cudaSuccess;
  const int64_t groups = (K + kQ8Group - 1) / kQ8Group;
  if (groups > 65535) return cudaErrorInvalidValue;
  dim3 grid((unsigned)((N + kPackThreads - 1) / kPackThreads), (unsigned)groups);
  pack_q8_kernel<<<grid, kPackThreads, 0, s>>>(w, out, K, N);
  count_launch();
  return cudaGetLastError();
}

}  // namespace smith
