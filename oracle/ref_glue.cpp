// ref_glue.cpp -- runs the reference's own rmsnorm_forward, swiglu_forward and dense matmul shader
// functions on the CPU.  TEST INFRASTRUCTURE ONLY.
//
// As in ref_driver.cpp the shader text is #included from the reference checkout at build time and
// never copied.  rmsnorm_forward is a threadgroup kernel (shaders/rmsnorm.metal:15-49): its tpg
// threads are played by an OpenMP team of tpg threads that all call the kernel function with their
// own tid; the shim turns its `threadgroup float shared[256]` into one static array and its
// threadgroup_barrier() into a barrier of that team.  Dispatch geometry as in
// src/ops/rmsnorm.js:26-33 (one threadgroup per row, tpg = power of two >= min(cols, 256)).
// The tiled matmul_f32 / matmul_f16 (shaders/matmul.metal:31-112, 172-231) run the same way with
// teams of 64, one team per 32 x 32 tile of the output (src/ops/matmul.js:28-45); matmul_simple
// and matmul_batched are one call per output element.
#include <stdint.h>
#include <omp.h>

#define SMITH_SHIM_THREADGROUP
#include <metal_stdlib>

namespace shader_rmsnorm {
#include "rmsnorm.metal"
}
namespace shader_swiglu {
#include "swiglu.metal"
}
namespace shader_matmul {
#include "matmul.metal"
}
#undef kernel
#undef device
#undef thread
#undef threadgroup
#undef constant

extern "C" {

void ref_rmsnorm(const float* x, const float* gamma, float* out, int64_t rows, int64_t cols, float eps) {
  int64_t lim = cols < 256 ? cols : 256;
  if (lim < 2) lim = 2;
  int tpg = 1;
  while (tpg < lim) tpg <<= 1;
  shader_rmsnorm::RMSNormParams p{(uint)rows, (uint)cols, eps};
  omp_set_dynamic(0);
  for (int64_t row = 0; row < rows; row++) {
    int got = 0;
#pragma omp parallel num_threads(tpg)
    {
#pragma omp single
      got = omp_get_num_threads();
      if (omp_get_num_threads() == tpg)
        shader_rmsnorm::rmsnorm_forward(x, gamma, out, p, (uint)row, (uint)omp_get_thread_num(), (uint)tpg);
    }
    if (got != tpg) {  // the team could not be formed: leave a mark the caller cannot miss
      for (int64_t i = 0; i < cols; i++) out[row * cols + i] = __builtin_nanf("");
    }
  }
}

void ref_swiglu(const float* gate, const float* up, float* out, int64_t n) {
  for (int64_t i = 0; i < n; i++) shader_swiglu::swiglu_forward(gate, up, out, (uint)i);
}

// which: 0 = matmul_simple, 1 = matmul_f32 (tiled), 2 = matmul_batched; f16 != 0 selects the half variants
// (operands are then IEEE binary16 bit patterns).  Returns 0, or 1 if a team of 64 could not be formed.
int ref_dense(int which, int f16, const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K, int64_t batch) {
  namespace sm = shader_matmul;
  const float *af = (const float*)a, *bf = (const float*)b;
  float* cf = (float*)c;
  const half *ah = (const half*)a, *bh = (const half*)b;
  half* ch = (half*)c;
  if (which == 0) {
    sm::MatmulParams p{(uint)M, (uint)N, (uint)K};
    for (uint row = 0; row < (uint)M; row++)
      for (uint col = 0; col < (uint)N; col++) {
        if (f16) sm::matmul_simple_f16(ah, bh, ch, p, uint2{col, row});
        else sm::matmul_simple(af, bf, cf, p, uint2{col, row});
      }
    return 0;
  }
  if (which == 2) {
    sm::BatchMatmulParams p{(uint)M, (uint)N, (uint)K, (uint)batch};
    for (uint bi = 0; bi < (uint)batch; bi++)
      for (uint row = 0; row < (uint)M; row++)
        for (uint col = 0; col < (uint)N; col++) {
          if (f16) sm::matmul_batched_f16(ah, bh, ch, p, uint3{col, row, bi});
          else sm::matmul_batched(af, bf, cf, p, uint3{col, row, bi});
        }
    return 0;
  }
  sm::MatmulParams p{(uint)M, (uint)N, (uint)K};
  const uint gx = (uint)((N + 31) / 32), gy = (uint)((M + 31) / 32);
  omp_set_dynamic(0);
  int bad = 0;
  for (uint y = 0; y < gy; y++)
    for (uint x = 0; x < gx; x++) {
      int got = 0;
#pragma omp parallel num_threads(64)
      {
#pragma omp single
        got = omp_get_num_threads();
        if (omp_get_num_threads() == 64) {
          if (f16) sm::matmul_f16(ah, bh, ch, p, uint2{x, y}, (uint)omp_get_thread_num());
          else sm::matmul_f32(af, bf, cf, p, uint2{x, y}, (uint)omp_get_thread_num());
        }
      }
      if (got != 64) bad = 1;
    }
  return bad;
}
}
