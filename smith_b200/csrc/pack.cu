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
// Speed: evaluated per element in f64 the packers were bound by instruction issue (an ncu capture
// counted 48 instructions per weight: 0.28 to 0.37 of the HBM copy peak).  A code only depends on which
// side of a half-integer the f64 value falls, so a full block is first SCREENED in f32, branch-free:
// fma(v, 1/scale, zero) in f32 is within 2.5e-7 * (|v/scale| + |zero| + 16) of the f64 value, and
// unless some element of the block lies closer than that to a half-integer (a block in a few hundred
// for ordinary data) the nearest integers ARE the reference's codes.  Only the remaining blocks, tail
// groups and blocks with an extraordinary scale go through the reference's own expressions, division
// included (q4_block_exact / q8_block_exact).  Scale and zero point are always computed in f64.  The
// bytes are the same either way.
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

constexpr float kMagic = 12582912.f;   // 1.5 * 2^23: x + kMagic rounds x to the nearest integer (|x| < 2^22),
                                       // which then sits in the low mantissa bits

// One block by the reference's own expressions, evaluated element by element in f64 (division
// included), reading the values again from global memory.  The slow lane: tail groups, blocks whose
// scale is far from ordinary, and blocks with an element the f32 screen could not call.
__device__ __noinline__ void q4_block_exact(const float* __restrict__ src, int64_t N, int valid, uint32_t* words,
                                            uint32_t* sbits, uint32_t* zbits) {
  // quantize.js:26-31 -- in-order compares so NaN and signed zeros behave as in JS.
  float mn = __int_as_float(0x7F800000), mx = __int_as_float(0xFF800000);
#pragma unroll 1
  for (int k = 0; k < valid; k++) {
    const float x = src[(int64_t)k * N];
    if (x < mn) mn = x;
    if (x > mx) mx = x;
  }
  const double range = __dsub_rn((double)mx, (double)mn);
  const bool pos = range > 0.0;
  const double scale = pos ? __ddiv_rn(range, 15.0) : 1.0;
  const double zero = pos ? __ddiv_rn(-(double)mn, scale) : 8.0;
  words[0] = words[1] = words[2] = words[3] = 0u;
#pragma unroll 1
  for (int k = 0; k < kQ4Group; k++) {
    const double x = (k < valid) ? (double)src[(int64_t)k * N] : 0.0;
    const double t = __dadd_rn(__ddiv_rn(x, scale), zero);  // quantize.js:45
    // Math.max(0, t) then Math.min(15, t); a NaN ends as code 0 like the typed-array store.
    double m = (t > 0.0) ? t : 0.0;
    m = (m < 15.0) ? m : 15.0;
    const double f = floor(m);
    const uint32_t q = (uint32_t)((__dsub_rn(m, f) >= 0.5) ? f + 1.0 : f);   // Math.round: ties toward +infinity
    words[k >> 3] |= q << ((k & 7) * 4);  // element k: byte k>>1, low nibble if k even
  }
  *sbits = __float_as_uint(__double2float_rn(scale));
  *zbits = __float_as_uint(__double2float_rn(zero));
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
    const float* src = w + k0 * N + col;
    uint32_t words[4], sbits = 0, zbits = 0;
    bool done = false;
    if (valid == kQ4Group) {
      float v[kQ4Group];
#pragma unroll
      for (int k = 0; k < kQ4Group; k++) v[k] = src[(int64_t)k * N];
      // min / max.  fminf / fmaxf skip NaNs as the reference's compares do; where they differ is the
      // SIGN of a zero minimum (the reference keeps the first zero it meets), restored below.
      float mn = __int_as_float(0x7F800000), mx = __int_as_float(0xFF800000);
#pragma unroll
      for (int k = 0; k < kQ4Group; k++) mn = fminf(mn, v[k]), mx = fmaxf(mx, v[k]);
      if (mn == 0.f) {
#pragma unroll
        for (int k = kQ4Group - 1; k >= 0; k--)
          if (v[k] == 0.f) mn = v[k];
      }
      const double range = __dsub_rn((double)mx, (double)mn);
      const bool pos = range > 0.0;
      const double scale = pos ? __ddiv_rn(range, 15.0) : 1.0;
      const double zero = pos ? __ddiv_rn(-(double)mn, scale) : 8.0;
      // f32 screen (see the file comment).  rcp32 is within 2 * 2^-24 of 1/scale, zero32 within 2^-24 of
      // zero, the fused multiply-add rounds once: t32 is within 2^-24 * (2|a| + |zero| + |t|) of the f64
      // value, inside bound = 2.5e-7 * (|a| + |zero| + 16).
      if (pos && scale > 1e-30 && scale < 1e30) {
        const float rcp32 = __frcp_rn(__double2float_rn(scale));
        const float zero32 = __double2float_rn(zero);
        const float slope = 2.5e-7f * fabsf(rcp32);                       // bound = slope * |v| + bound0
        const float thr0 = 0.5f - 2.5e-7f * (fabsf(zero32) + 16.f);       // may go negative: then nothing passes
        bool ok = true;
        float acc[8];
#pragma unroll
        for (int k = 0; k < kQ4Group; k++) {
          const float t32 = fmaf(v[k], rcp32, zero32);
          const float m32 = fminf(fmaxf(t32, 0.f), 15.f);                 // a NaN becomes 0, as in the reference
          const float r = (m32 + kMagic) - kMagic;                        // nearest integer
          ok = ok && (fabsf(m32 - r) < fmaf(-slope, fabsf(v[k]), thr0));  // false for NaN and near a half-integer
          // four codes per accumulator, weights 1, 16, 256, 4096: exact in f32 (sum < 2^16)
          const float wgt = (float)(1 << (4 * (k & 3)));
          acc[k >> 2] = (k & 3) ? fmaf(r, wgt, acc[k >> 2]) : r;
        }
        if (ok) {
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const uint32_t lo = __float_as_uint(acc[2 * i] + kMagic), hi = __float_as_uint(acc[2 * i + 1] + kMagic);
            words[i] = __byte_perm(lo, hi, 0x5410);                       // low 16 bits of each
          }
          sbits = __float_as_uint(__double2float_rn(scale));
          zbits = __float_as_uint(__double2float_rn(zero));
          done = true;
        }
      }
    }
    if (!done) q4_block_exact(src, N, valid, words, &sbits, &zbits);
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

// One Q8 block by the rule's own expressions in f64 (see q4_block_exact).
__device__ __noinline__ void q8_block_exact(const float* __restrict__ src, int64_t N, int valid, uint16_t* mine) {
  float amax = 0.0f;
#pragma unroll 1
  for (int k = 0; k < valid; k++) {
    const float a = fabsf(src[(int64_t)k * N]);
    if (a > amax) amax = a;  // NaN never wins
  }
  const double d = __ddiv_rn((double)amax, 127.0);
  const uint32_t h = js_to_float16(d);
  const double dq = js_from_float16(h);
  mine[0] = (uint16_t)h;
#pragma unroll 1
  for (int k = 0; k < kQ8Group; k += 2) {
    int q[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
      int c = 0;
      if (k + i < valid && dq > 0.0) {
        double t = js_round(__ddiv_rn((double)src[(int64_t)(k + i) * N], dq));
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

__global__ void __launch_bounds__(kPackThreads)
pack_q8_kernel(const float* __restrict__ w, uint8_t* __restrict__ out, int64_t K, int64_t N) {
  __shared__ __align__(16) uint16_t stage[kPackThreads * 17];
  const int64_t g = blockIdx.y;
  const int64_t col0 = (int64_t)blockIdx.x * kPackThreads;
  const int64_t col = col0 + threadIdx.x;
  const int64_t k0 = g * kQ8Group;
  const int valid = (int)((K - k0 < kQ8Group) ? (K - k0) : kQ8Group);

  if (col < N) {
    const float* src = w + k0 * N + col;
    uint16_t* mine = stage + threadIdx.x * 17;
    bool done = false;
    if (valid == kQ8Group) {
      float v[kQ8Group];
#pragma unroll
      for (int k = 0; k < kQ8Group; k++) v[k] = src[(int64_t)k * N];
      float amax = 0.0f;
#pragma unroll
      for (int k = 0; k < kQ8Group; k++) amax = fmaxf(amax, fabsf(v[k]));   // NaN never wins
      const double d = __ddiv_rn((double)amax, 127.0);
      const uint32_t h = js_to_float16(d);
      const double dq = js_from_float16(h);
      if (dq > 1e-30 && dq < 1e30) {
        // dq is a half, so exact in f32; rcp32 within 2^-24 of 1/dq; a32 = v * rcp32 within
        // 2 * 2^-24 * |a| of v / dq, inside bound = 2.5e-7 * (|a| + 1).  |v| <= amax keeps |a| below 128.
        const float rcp32 = __frcp_rn(__double2float_rn(dq));
        bool ok = true;
        uint32_t ub[kQ8Group];
#pragma unroll
        for (int k = 0; k < kQ8Group; k++) {
          const float a32 = v[k] * rcp32;
          const float c32 = fminf(fmaxf(a32, -127.f), 127.f);             // clamping before or after rounding is the same
          const float u = c32 + kMagic;
          const float r = u - kMagic;
          ok = ok && (fabsf(a32) < 200.f) && (fabsf(c32 - r) < fmaf(-2.5e-7f, fabsf(a32), 0.5f - 2.5e-7f));
          ub[k] = __float_as_uint(u);                                     // low byte = the code in two's complement
        }
        if (ok) {
          mine[0] = (uint16_t)h;
#pragma unroll
          for (int k = 0; k < kQ8Group; k += 2) mine[1 + (k >> 1)] = (uint16_t)__byte_perm(ub[k], ub[k + 1], 0x0040);
          done = true;
        }
      } else if (!(dq > 0.0) && amax == amax) {
        // the scale underflowed to zero: every code is 0
        mine[0] = (uint16_t)h;
#pragma unroll
        for (int k = 0; k < kQ8Group; k += 2) mine[1 + (k >> 1)] = 0;
        done = true;
      }
    }
    if (!done) q8_block_exact(src, N, valid, mine);
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
