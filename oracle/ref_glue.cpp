// ref_glue.cpp -- runs the reference's own rmsnorm_forward and swiglu_forward shader functions on
// the CPU.  TEST INFRASTRUCTURE ONLY.
//
// As in ref_driver.cpp the shader text is #included from the reference checkout at build time and
// never copied.  rmsnorm_forward is a threadgroup kernel (shaders/rmsnorm.metal:15-49): its tpg
// threads are played by an OpenMP team of tpg threads that all call the kernel function with their
// own tid; the shim turns its `threadgroup float shared[256]` into one static array and its
// threadgroup_barrier() into a barrier of that team.  Dispatch geometry as in
// src/ops/rmsnorm.js:26-33 (one threadgroup per row, tpg = power of two >= min(cols, 256)).
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
}
