// ref_driver.cpp -- runs the reference's own matmul_q4 / matmul_q8 shader
// functions on the CPU.  TEST INFRASTRUCTURE ONLY.
//
// The shader text is NOT copied into this repository: the two files are
// #included from the reference checkout at build time (the Makefile passes its
// location with -I), each inside its own namespace, through the small
// <metal_stdlib> stand-in in oracle/ref_shim.  Each (row, col) "thread" of the
// reference dispatch (src/ops/quantize.js:82-87: grid = N x M threads) becomes
// one call of the kernel function with gid = {col, row}.
#include <stdint.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#include <metal_stdlib>  // the stand-in, at global scope so both namespaces see its types

namespace ref_q4 {
#include "matmul_q4.metal"
}
namespace ref_q8 {
#include "matmul_q8.metal"
}
// The address-space macros must not leak into the driver code below.
#undef kernel
#undef device
#undef thread
#undef threadgroup
#undef constant

extern "C" {

// Columns [col0, col1) of every row; C keeps its full [M,N] indexing.
void ref_matmul_q4(const float* A, const unsigned char* B, float* C, int64_t M, int64_t N,
                   int64_t K, int64_t groups, int64_t col0, int64_t col1, int threads) {
  ref_q4::Q4MatmulParams p{(uint)M, (uint)N, (uint)K, (uint)groups};
#pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1) collapse(2)
  for (int64_t row = 0; row < M; row++)
    for (int64_t col = col0; col < col1; col++)
      ref_q4::matmul_q4(A, B, C, p, uint2{(uint)col, (uint)row});
}

void ref_matmul_q8(const float* A, const unsigned char* B, float* C, int64_t M, int64_t N,
                   int64_t K, int64_t groups, int64_t col0, int64_t col1, int threads) {
  ref_q8::Q8MatmulParams p{(uint)M, (uint)N, (uint)K, (uint)groups};
#pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1) collapse(2)
  for (int64_t row = 0; row < M; row++)
    for (int64_t col = col0; col < col1; col++)
      ref_q8::matmul_q8(A, B, C, p, uint2{(uint)col, (uint)row});
}

int ref_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
}
