/*
 * smith_oracle.c -- CPU restatement of Smith's quantized-matmul hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
 * compared against; it is never linked into, imported by, or called from the
 * shipped library.  Only the test-suite, the smoke check and the benchmark's
 * CPU-baseline leg may load it.
 *
 * What is restated, and from where (paths are inside the reference project):
 *   oracle_quantize_q4   src/ops/quantize.js:14-68   (JS Number = IEEE f64)
 *   oracle_to_float16    src/dtype.js:29-58          (truncating encoder)
 *   oracle_from_float16  src/dtype.js:60-79
 *   oracle_matmul_q4     shaders/matmul_q4.metal:24-28,34-65
 *   oracle_matmul_q8     shaders/matmul_q8.metal:20-57
 *   oracle_rmsnorm       shaders/rmsnorm.metal:15-49, src/ops/rmsnorm.js:19-38
 *   oracle_dense_f32/f16 shaders/matmul.metal:31-165 (f32), 172-260 (f16): the dense matmul family
 *   oracle_swiglu        shaders/swiglu.metal:12-22
 *   oracle_gguf_dequant  src/gguf.js:187-197 (Q4_0), 221-231 (Q8_0)
 *   oracle_quantize_q8   NO reference counterpart ("parity unpinned"): the
 *                        reference has no producer for the layout that
 *                        matmul_q8 consumes.  The rule frozen here is written
 *                        in the idiom of quantizeQ4 and of the reference's own
 *                        f16 encoder; only the byte layout it emits is pinned
 *                        (by shaders/matmul_q8.metal:40-52).
 *
 * Parity status of the packer: the reference's JavaScript cannot run on a
 * machine without a JS engine, so the Q4 packer is pinned by the assertions of
 * the reference's own test (tests/inference.test.js:94-135), by hand-worked
 * known answers, and by a round trip through the reference's shader source
 * compiled as C++ (oracle/_ref).  The two matmul functions are pinned
 * bit-for-bit against that compiled shader source.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see oracle/Makefile).
 * -ffp-contract=off keeps every multiply and add separately rounded, which is
 * the canonical sequential-f32 reading of the shader loops.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define Q4_GROUP 32
#define Q4_BYTES 24
#define Q8_GROUP 32
#define Q8_BYTES 34

/* JS Math.round: nearest integer, ties toward +infinity (also for negatives).
 * floor(x + 0.5) is wrong at 0.49999999999999994, so compare the fraction. */
static double js_round(double x) {
  double f = floor(x);
  return (x - f >= 0.5) ? f + 1.0 : f;
}

/* Math.max(0, t) / Math.min(15, t) with JS NaN propagation. */
static double js_clamp(double t, double lo, double hi) {
  if (t != t) return t;
  double m = (t > lo) ? t : lo; /* Math.max(lo, -0) = +0 when lo = +0 */
  return (m < hi) ? m : hi;
}

/* ---- quantizeQ4: src/ops/quantize.js:14-68 ---------------------------- */
/* w: f32 [K,N] row-major.  out: ceil(K/32)*N*24 bytes.  Returns groups. */
int64_t oracle_quantize_q4(const float *w, int64_t K, int64_t N, uint8_t *out) {
  int64_t groups = (K + Q4_GROUP - 1) / Q4_GROUP;
  memset(out, 0, (size_t)(groups * N * Q4_BYTES)); /* new Uint8Array(...) is zero-filled (:18) */
  for (int64_t g = 0; g < groups; g++) {
    int64_t k0 = g * Q4_GROUP;
    int64_t k1 = (k0 + Q4_GROUP < K) ? k0 + Q4_GROUP : K;
    for (int64_t col = 0; col < N; col++) {
      double mn = INFINITY, mx = -INFINITY;          /* :26 */
      for (int64_t k = k0; k < k1; k++) {
        double v = (double)w[k * N + col];
        if (v < mn) mn = v;                          /* NaN: both compares false */
        if (v > mx) mx = v;
      }
      double range = mx - mn;                        /* :34 */
      double scale = (range > 0) ? range / 15.0 : 1.0;
      double zero = (range > 0) ? (-mn) / scale : 8.0; /* min == +0 gives -0.0 */
      uint8_t *blk = out + (g * N + col) * Q4_BYTES;
      int64_t valid = k1 - k0;
      for (int k = 0; k < Q4_GROUP; k++) {
        double v = (k < valid) ? (double)w[(k0 + k) * N + col] : 0.0; /* :44 */
        double t = js_round(js_clamp(v / scale + zero, 0.0, 15.0));   /* :45 */
        unsigned q = (t != t) ? 0u : (unsigned)t;    /* ToInt32 / ToUint8 of NaN = 0 */
        if (k & 1) blk[k >> 1] |= (uint8_t)(q << 4);
        else blk[k >> 1] = (uint8_t)q;
      }
      float fs = (float)scale, fz = (float)zero;     /* Float32Array store: RNE (:55-58) */
      memcpy(blk + 16, &fs, 4);
      memcpy(blk + 20, &fz, 4);
    }
  }
  return groups;
}

/* ---- f16 codec: src/dtype.js:29-79 ------------------------------------ */
uint16_t oracle_to_float16(double val) {
  float f = (float)val; /* _f32[0] = val */
  uint32_t bits;
  memcpy(&bits, &f, 4);
  uint32_t sign = (bits >> 31) & 1u;
  int32_t e = (int32_t)((bits >> 23) & 0xFFu);
  uint32_t frac = bits & 0x7FFFFFu;
  if (e == 0xFF) return (uint16_t)((sign << 15) | 0x7C00u | (frac ? 0x200u : 0u));
  e -= 127;
  if (e > 15) return (uint16_t)((sign << 15) | 0x7C00u);
  if (e < -14) {
    if (e < -24) return (uint16_t)(sign << 15);
    frac |= 0x800000u;
    int shift = -1 - e;      /* 14..23 */
    frac >>= shift;
    return (uint16_t)((sign << 15) | (frac >> 13)); /* as written upstream: always 0 here */
  }
  return (uint16_t)((sign << 15) | ((uint32_t)(e + 15) << 10) | (frac >> 13));
}

double oracle_from_float16(uint16_t h) {
  int sign = (h >> 15) & 1;
  int e = (h >> 10) & 0x1F;
  int frac = h & 0x3FF;
  double v;
  if (e == 0) {
    if (frac == 0) return sign ? -0.0 : 0.0;
    v = ldexp(1.0, -14) * ((double)frac / 1024.0);
  } else if (e == 31) {
    if (frac) return NAN;
    v = INFINITY;
  } else {
    v = ldexp(1.0, e - 15) * (1.0 + (double)frac / 1024.0);
  }
  return sign ? -v : v;
}

/* ---- quantizeQ8: build-defined (no reference producer) ----------------- */
/* Block (g,col) at (g*N+col)*34: [f16 scale, little endian][32 x int8].
 * amax over the valid k; d = amax/127 in f64; h = to_float16(d);
 * dq = from_float16(h); code = dq > 0 ? clamp(js_round(v/dq), -127, 127) : 0;
 * NaN codes store 0; padding k >= K stores 0. */
int64_t oracle_quantize_q8(const float *w, int64_t K, int64_t N, uint8_t *out) {
  int64_t groups = (K + Q8_GROUP - 1) / Q8_GROUP;
  memset(out, 0, (size_t)(groups * N * Q8_BYTES));
  for (int64_t g = 0; g < groups; g++) {
    int64_t k0 = g * Q8_GROUP;
    int64_t k1 = (k0 + Q8_GROUP < K) ? k0 + Q8_GROUP : K;
    for (int64_t col = 0; col < N; col++) {
      double amax = 0.0;
      for (int64_t k = k0; k < k1; k++) {
        double a = fabs((double)w[k * N + col]);
        if (a > amax) amax = a;
      }
      double d = amax / 127.0;
      uint16_t h = oracle_to_float16(d);
      double dq = oracle_from_float16(h);
      uint8_t *blk = out + (g * N + col) * Q8_BYTES;
      blk[0] = (uint8_t)(h & 0xFF);
      blk[1] = (uint8_t)(h >> 8);
      int64_t valid = k1 - k0;
      for (int k = 0; k < Q8_GROUP; k++) {
        int q = 0;
        if (k < valid && dq > 0) {
          double t = js_round((double)w[(k0 + k) * N + col] / dq);
          if (t == t) {
            if (t > 127.0) t = 127.0;
            if (t < -127.0) t = -127.0;
            q = (int)t;
          }
        }
        blk[2 + k] = (uint8_t)(int8_t)q;
      }
    }
  }
  return groups;
}

/* ---- de-quantised weights (f32), used only to form tolerance norms ----- */
/* Same expression as the shaders: scale*(float(nibble)-zero) / scale*float(i8). */
void oracle_dequant_q4(const uint8_t *B, int64_t K, int64_t N, float *w) {
  int64_t groups = (K + Q4_GROUP - 1) / Q4_GROUP;
  for (int64_t g = 0; g < groups; g++)
    for (int64_t col = 0; col < N; col++) {
      const uint8_t *blk = B + (g * N + col) * Q4_BYTES;
      float s, z;
      memcpy(&s, blk + 16, 4);
      memcpy(&z, blk + 20, 4);
      for (int k = 0; k < Q4_GROUP && g * Q4_GROUP + k < K; k++) {
        uint8_t byte = blk[k >> 1];
        uint8_t nib = (k & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0x0F);
        w[(g * Q4_GROUP + k) * N + col] = s * ((float)nib - z);
      }
    }
}

static float half_bits_to_float(uint16_t h) { return (float)oracle_from_float16(h); }

void oracle_dequant_q8(const uint8_t *B, int64_t K, int64_t N, float *w) {
  int64_t groups = (K + Q8_GROUP - 1) / Q8_GROUP;
  for (int64_t g = 0; g < groups; g++)
    for (int64_t col = 0; col < N; col++) {
      const uint8_t *blk = B + (g * N + col) * Q8_BYTES;
      float s = half_bits_to_float((uint16_t)(blk[0] | (blk[1] << 8)));
      for (int k = 0; k < Q8_GROUP && g * Q8_GROUP + k < K; k++)
        w[(g * Q8_GROUP + k) * N + col] = s * (float)(int8_t)blk[2 + k];
    }
}

/* ---- matmul_q4: shaders/matmul_q4.metal:34-65 -------------------------- */
/* Per output: acc = 0f; for g, for k: acc += A[row,k] * (scale*(float(nib)-zero)),
 * strictly in that order, every operation rounded to f32.  The loop nest here
 * is interchanged (columns innermost) for cache behaviour; each output's own
 * sequence of operations is unchanged.  col0/col1 select a column range so a
 * sampled subset of a large matrix can be checked; C keeps its full [M,N]
 * indexing.  threads <= 1 runs serially. */
void oracle_matmul_q4(const float *A, const uint8_t *B, float *C, int64_t M, int64_t N,
                      int64_t K, int64_t groups, int64_t col0, int64_t col1, int threads) {
  (void)threads;
#pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1) collapse(2)
  for (int64_t row = 0; row < M; row++) {
    for (int64_t cb = col0; cb < col1; cb += 256) {
      int64_t ce = cb + 256 < col1 ? cb + 256 : col1;
      float acc[256];
      for (int64_t c = cb; c < ce; c++) acc[c - cb] = 0.0f;
      for (int64_t g = 0; g < groups; g++) {
        const float *a = A + row * K + g * Q4_GROUP;
        int kn = (int)((g * Q4_GROUP + Q4_GROUP <= K) ? Q4_GROUP : (K - g * Q4_GROUP));
        if (kn < 0) kn = 0;
        for (int64_t c = cb; c < ce; c++) {
          const uint8_t *blk = B + (g * N + c) * Q4_BYTES;
          float s, z, t = acc[c - cb];
          memcpy(&s, blk + 16, 4);
          memcpy(&z, blk + 20, 4);
          for (int k = 0; k < kn; k++) {
            uint8_t byte = blk[k >> 1];
            uint8_t nib = (k & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0x0F);
            float b = s * ((float)nib - z);
            t += a[k] * b;
          }
          acc[c - cb] = t;
        }
      }
      for (int64_t c = cb; c < ce; c++) C[row * N + c] = acc[c - cb];
    }
  }
}

/* ---- matmul_q8: shaders/matmul_q8.metal:20-57 -------------------------- */
void oracle_matmul_q8(const float *A, const uint8_t *B, float *C, int64_t M, int64_t N,
                      int64_t K, int64_t groups, int64_t col0, int64_t col1, int threads) {
  (void)threads;
#pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1) collapse(2)
  for (int64_t row = 0; row < M; row++) {
    for (int64_t cb = col0; cb < col1; cb += 256) {
      int64_t ce = cb + 256 < col1 ? cb + 256 : col1;
      float acc[256];
      for (int64_t c = cb; c < ce; c++) acc[c - cb] = 0.0f;
      for (int64_t g = 0; g < groups; g++) {
        const float *a = A + row * K + g * Q8_GROUP;
        int kn = (int)((g * Q8_GROUP + Q8_GROUP <= K) ? Q8_GROUP : (K - g * Q8_GROUP));
        if (kn < 0) kn = 0;
        for (int64_t c = cb; c < ce; c++) {
          const uint8_t *blk = B + (g * N + c) * Q8_BYTES;
          float s = half_bits_to_float((uint16_t)(blk[0] | (blk[1] << 8)));
          float t = acc[c - cb];
          for (int k = 0; k < kn; k++) {
            float b = s * (float)(int8_t)blk[2 + k];
            t += a[k] * b;
          }
          acc[c - cb] = t;
        }
      }
      for (int64_t c = cb; c < ce; c++) C[row * N + c] = acc[c - cb];
    }
  }
}

/* ---- rmsnorm_forward: shaders/rmsnorm.metal:15-49 ------------------------ */
/* One threadgroup of tpg threads per row (tpg = the power of two >= min(cols, 256),
 * at least 2: src/ops/rmsnorm.js:26).  Thread tid sums x[i]^2 over i = tid, tid + tpg, ...;
 * the partials are added pairwise by the halving tree of the shader (stride tpg/2, tpg/4, ... 1);
 * rms = 1/sqrt(sum / cols + eps); out[i] = x[i] * rms * gamma[i].  Every operation is rounded to
 * f32, in the shader's order (the GPU's own rsqrt is an approximation; 1/sqrtf stands in for it). */
void oracle_rmsnorm(const float *x, const float *gamma, float *out, int64_t rows, int64_t cols, float eps) {
  int64_t lim = cols < 256 ? cols : 256;
  if (lim < 2) lim = 2;
  int64_t tpg = 1;
  while (tpg < lim) tpg <<= 1;
  for (int64_t r = 0; r < rows; r++) {
    const float *xr = x + r * cols;
    float part[256];
    for (int64_t t = 0; t < tpg; t++) {
      float ss = 0.0f;
      for (int64_t i = t; i < cols; i += tpg) ss += xr[i] * xr[i];
      part[t] = ss;
    }
    for (int64_t s = tpg / 2; s > 0; s >>= 1)
      for (int64_t t = 0; t < s; t++) part[t] += part[t + s];
    float rms = 1.0f / sqrtf(part[0] / (float)cols + eps);
    for (int64_t i = 0; i < cols; i++) out[r * cols + i] = xr[i] * rms * gamma[i];
  }
}

/* ---- swiglu_forward: shaders/swiglu.metal:12-22 -------------------------- */
void oracle_swiglu(const float *gate, const float *up, float *out, int64_t n) {
  for (int64_t i = 0; i < n; i++) {
    float g = gate[i];
    float silu = g / (1.0f + expf(-g));
    out[i] = silu * up[i];
  }
}

/* ---- dense matmul: shaders/matmul.metal ------------------------------------------------------
 * matmul_simple (:116-132) and matmul_batched (:145-165): sum = 0; for k: sum += A[row,k] * B[k,col],
 * every product and sum rounded to f32.  The tiled matmul_f32 (:31-112) keeps one accumulator per
 * output and walks its k-tiles in order, so it forms the same sum (its zero padding of the last
 * k-tile adds +0 terms, which can only turn a -0 result into +0).  C[b,M,N] = A[b,M,K] @ B[b,K,N]. */
void oracle_dense_f32(const float *a, const float *b, float *c, int64_t M, int64_t N, int64_t K, int64_t batch) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bi = 0; bi < batch; bi++)
    for (int64_t m = 0; m < M; m++) {
      const float *ar = a + (bi * M + m) * K;
      const float *bm = b + bi * K * N;
      float *cr = c + (bi * M + m) * N;
      for (int64_t n = 0; n < N; n++) {
        float sum = 0.0f;
        for (int64_t k = 0; k < K; k++) sum += ar[k] * bm[k * N + n];
        cr[n] = sum;
      }
    }
}

/* The f16 variants (:172-260): halves widened to f32, f32 products and sums, the sum rounded to
 * half once (round to nearest even).  Operands and result are IEEE binary16 bit patterns. */
void oracle_dense_f16(const uint16_t *a, const uint16_t *b, uint16_t *c, int64_t M, int64_t N, int64_t K,
                      int64_t batch) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bi = 0; bi < batch; bi++)
    for (int64_t m = 0; m < M; m++) {
      const uint16_t *ar = a + (bi * M + m) * K;
      const uint16_t *bm = b + bi * K * N;
      uint16_t *cr = c + (bi * M + m) * N;
      for (int64_t n = 0; n < N; n++) {
        float sum = 0.0f;
        for (int64_t k = 0; k < K; k++) {
          _Float16 x, y;
          memcpy(&x, ar + k, 2);
          memcpy(&y, bm + k * N + n, 2);
          sum += (float)x * (float)y;
        }
        _Float16 h = (_Float16)sum;
        memcpy(cr + n, &h, 2);
      }
    }
}

/* ---- GGUF block decoders: src/gguf.js:187-197 (Q4_0) and 221-231 (Q8_0) ------------- */
/* blocks: `nblocks` consecutive blocks as they lie in the file; out: 32 f32 per block.
 * Q4_0 (type 2): 18 bytes, value = scale * (nibble - 8), element i in byte i >> 1, low nibble if i is
 * even (the reference's reading).  Q8_0 (type 8): 34 bytes, value = scale * int8.  The scale goes
 * through the reference's fromFloat16; the product is rounded to f32 by the Float32Array store. */
int oracle_gguf_dequant(int ggml_type, const uint8_t *blocks, int64_t nblocks, float *out) {
  if (ggml_type != 2 && ggml_type != 8) return 1;
  const int bytes = ggml_type == 2 ? 18 : 34;
  for (int64_t b = 0; b < nblocks; b++) {
    const uint8_t *blk = blocks + b * bytes;
    const double scale = oracle_from_float16((uint16_t)(blk[0] | (blk[1] << 8)));
    for (int i = 0; i < 32; i++) {
      if (ggml_type == 2) {
        const uint8_t byte = blk[2 + (i >> 1)];
        const int nib = (i & 1) ? (byte >> 4) : (byte & 0x0F);
        out[b * 32 + i] = (float)(scale * (double)(nib - 8));
      } else {
        out[b * 32 + i] = (float)(scale * (double)(int8_t)blk[2 + i]);
      }
    }
  }
  return 0;
}

int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
