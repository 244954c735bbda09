// qmatmul_generic.cu -- any-shape quantized matmul on CUDA cores.
//
// C[M,N] = A[M,K] (f32) x dequant(B), B in the Q4 (24-byte) or Q8 (34-byte)
// block layout with block (g, col) at (g*N + col) * block_bytes
// (shaders/matmul_q4.metal:47-55, shaders/matmul_q8.metal:40-48).
//
// This kernel serves the shapes the streaming kernels do not take (odd N, tiny
// problems, K that is not a multiple of 32) and doubles as the on-device
// statement of the reference arithmetic: every output is accumulated in f32,
// strictly in k order, with separately rounded multiply and add
// (acc += a * (scale * (float(code) - zero))), which is the canonical reading
// of the reference shader loops.  It is therefore bit-identical to a CPU run of
// those loops, which the faster kernels are only within tolerance of.
//
// Mapping: one thread per output column, kRows rows of A per CTA.  Adjacent
// threads read adjacent blocks, so a warp's loads cover one contiguous span.
// The A rows of the CTA are staged through shared memory one 256-element
// chunk at a time and read as broadcasts.
#include <cuda_fp16.h>

#include "kernels.h"

namespace smith {
namespace {

constexpr int kCols = 128;   // threads per CTA = columns per CTA
constexpr int kRows = 8;     // rows of A per CTA
constexpr int kChunkG = 8;   // groups per shared-memory chunk of A

template <int KIND>
__global__ void __launch_bounds__(kCols)
qmatmul_generic_kernel(const float* __restrict__ A, const uint8_t* __restrict__ B,
                       float* __restrict__ C, int64_t M, int64_t N, int64_t K, int64_t groups) {
  constexpr int BB = (KIND == 4) ? kQ4Bytes : kQ8Bytes;
  __shared__ float xs[kRows][kChunkG * 32];
  const int64_t col = (int64_t)blockIdx.x * kCols + threadIdx.x;
  const int64_t row0 = (int64_t)blockIdx.y * kRows;
  const int rows = (int)((M - row0 < kRows) ? (M - row0) : kRows);
  float acc[kRows];
#pragma unroll
  for (int r = 0; r < kRows; r++) acc[r] = 0.0f;

  for (int64_t g0 = 0; g0 < groups; g0 += kChunkG) {
    __syncthreads();
    for (int i = threadIdx.x; i < kRows * kChunkG * 32; i += kCols) {
      const int r = i / (kChunkG * 32), kk = i % (kChunkG * 32);
      const int64_t k = g0 * 32 + kk;
      xs[r][kk] = (r < rows && k < K) ? A[(row0 + r) * K + k] : 0.0f;
    }
    __syncthreads();
    if (col >= N) continue;
    const int gend = (int)((groups - g0 < kChunkG) ? (groups - g0) : kChunkG);
    for (int gl = 0; gl < gend; gl++) {
      const int64_t g = g0 + gl;
      const uint8_t* blk = B + (g * N + col) * BB;
      int kn = (int)((g * 32 + 32 <= K) ? 32 : (K - g * 32));
      if (kn < 0) kn = 0;
      if (KIND == 4) {
        const uint2* p = reinterpret_cast<const uint2*>(blk);  // 24*i: 8-byte aligned
        const uint2 n0 = __ldg(p), n1 = __ldg(p + 1), sz = __ldg(p + 2);
        const uint32_t w[4] = {n0.x, n0.y, n1.x, n1.y};
        const float s = __uint_as_float(sz.x), z = __uint_as_float(sz.y);
#pragma unroll
        for (int k = 0; k < 32; k++) {
          if (k < kn) {
            const float nib = (float)((w[k >> 3] >> ((k & 7) * 4)) & 0xFu);
            const float b = __fmul_rn(s, __fsub_rn(nib, z));
#pragma unroll
            for (int r = 0; r < kRows; r++)
              acc[r] = __fadd_rn(acc[r], __fmul_rn(xs[r][gl * 32 + k], b));
          }
        }
      } else {
        const uint16_t* p = reinterpret_cast<const uint16_t*>(blk);  // 34*i: 2-byte aligned
        const float s = __half2float(__ushort_as_half(__ldg(p)));
#pragma unroll
        for (int k2 = 0; k2 < 16; k2++) {
          const uint32_t two = __ldg(p + 1 + k2);
#pragma unroll
          for (int i = 0; i < 2; i++) {
            const int k = 2 * k2 + i;
            if (k < kn) {
              const float q = (float)(int)(int8_t)((two >> (8 * i)) & 0xFFu);
              const float b = __fmul_rn(s, q);
#pragma unroll
              for (int r = 0; r < kRows; r++)
                acc[r] = __fadd_rn(acc[r], __fmul_rn(xs[r][gl * 32 + k], b));
            }
          }
        }
      }
    }
  }
  if (col < N) {
#pragma unroll
    for (int r = 0; r < kRows; r++)
      if (r < rows) C[(row0 + r) * N + col] = acc[r];
  }
}

}  // namespace

cudaError_t launch_qmatmul_generic(int kind, const float* A, const uint8_t* B, float* C, int64_t M,
                                   int64_t N, int64_t K, int64_t groups, cudaStream_t s) {
  if (M <= 0 || N <= 0) return cudaSuccess;
  const int64_t gy = (M + kRows - 1) / kRows;
  if (gy > 65535) return cudaErrorInvalidValue;
  dim3 grid((unsigned)((N + kCols - 1) / kCols), (unsigned)gy);
  if (kind == 4)
    qmatmul_generic_kernel<4><<<grid, kCols, 0, s>>>(A, B, C, M, N, K, groups);
  else
    qmatmul_generic_kernel<8><<<grid, kCols, 0, s>>>(A, B, C, M, N, K, groups);
  count_launch();
  return cudaGetLastError();
}

}  // namespace smith
