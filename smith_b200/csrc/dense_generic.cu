// dense_generic.cu -- dense matmul of any shape on the CUDA cores, f32 or f16 storage.
//
// C[b,M,N] = A[b,M,K] @ B[b,K,N], every output the sequential sum
//     sum = 0; for k in 0..K-1: sum = sum + a[m,k] * b[k,n]      (f32 multiply, then f32 add)
// which is what all three of the reference's kernels compute: matmul_simple and matmul_batched
// directly (shaders/matmul.metal:116-132, 145-165) and the tiled matmul_f32 by walking its k-tiles
// in order with one accumulator per output (shaders/matmul.metal:59-98).  The f16 variants read
// halves, accumulate in f32 and round the sum to half once (shaders/matmul.metal:172-260).
// Results are bit-identical to that order: products and sums are kept apart (no fused
// multiply-add) and every output's k runs in sequence, whatever the tiling.
//
// 64 x 64 outputs per CTA, 256 threads, 4 x 4 outputs per thread, 16 k per shared-memory tile.
// This is the kernel for what the tensor-core kernel declines: matrices under 64 on a side (the
// reference's own threshold for its simple kernel, src/ops/matmul.js:10,28), odd strides, batches
// of small heads.
#include <cuda_fp16.h>

#include "kernels.h"

namespace smith {
namespace {

constexpr int kTile = 64, kTileK = 16;

__device__ __forceinline__ float load_as_f32(const float* p) { return *p; }
__device__ __forceinline__ float load_as_f32(const __half* p) { return __half2float(*p); }
__device__ __forceinline__ void store_from_f32(float* p, float v) { *p = v; }
__device__ __forceinline__ void store_from_f32(__half* p, float v) { *p = __float2half_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256) dense_generic_kernel(const T* __restrict__ A, const T* __restrict__ B,
                                                            T* __restrict__ C, int M, int N, int K) {
  __shared__ float As[kTileK][kTile + 4];   // [k][row]
  __shared__ float Bs[kTileK][kTile + 4];   // [k][col]
  const size_t b = blockIdx.z;
  A += b * (size_t)M * K, B += b * (size_t)K * N, C += b * (size_t)M * N;
  const int row0 = blockIdx.y * kTile, col0 = blockIdx.x * kTile;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += kTileK) {
    // A tile: 64 rows x 16 k, this thread's k = threadIdx.x % 16 (adjacent threads read adjacent k)
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int r = (threadIdx.x >> 4) + 16 * i, k = threadIdx.x & 15;
      const int gr = row0 + r, gk = k0 + k;
      As[k][r] = (gr < M && gk < K) ? load_as_f32(A + (size_t)gr * K + gk) : 0.f;
    }
    // B tile: 16 k x 64 columns
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int k = (threadIdx.x >> 6) + 4 * i, c = threadIdx.x & 63;
      const int gk = k0 + k, gc = col0 + c;
      Bs[k][c] = (gk < K && gc < N) ? load_as_f32(B + (size_t)gk * N + gc) : 0.f;
    }
    __syncthreads();
    const int kn = min(kTileK, K - k0);   // a padded k would add 0 * 0 = +0, which may flip a -0 sum
    for (int k = 0; k < kn; k++) {
      const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 bb = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int gr = row0 + ty * 4 + i;
    if (gr >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int gc = col0 + tx * 4 + j;
      if (gc < N) store_from_f32(C + (size_t)gr * N + gc, acc[i][j]);
    }
  }
}

}  // namespace

cudaError_t launch_dense_generic(int dtype, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                                 int64_t batch, cudaStream_t s) {
  if (M <= 0 || N <= 0 || batch <= 0) return cudaSuccess;
  if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30) || batch > 65535) return cudaErrorInvalidValue;
  const dim3 grid((unsigned)((N + kTile - 1) / kTile), (unsigned)((M + kTile - 1) / kTile), (unsigned)batch);
  if (grid.y > 65535) return cudaErrorInvalidValue;
  if (dtype == kDenseF16)
    dense_generic_kernel<__half><<<grid, 256, 0, s>>>((const __half*)A, (const __half*)B, (__half*)C, (int)M, (int)N, (int)K);
  else if (dtype == kDenseF32)
    dense_generic_kernel<float><<<grid, 256, 0, s>>>((const float*)A, (const float*)B, (float*)C, (int)M, (int)N, (int)K);
  else
    return cudaErrorInvalidValue;
  count_launch();
  return cudaGetLastError();
}

}  // namespace smith
