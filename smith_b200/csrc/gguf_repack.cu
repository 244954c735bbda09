// gguf_repack.cu -- GGUF block formats straight into the layouts the quantized matmul kernels read.
//
// The reference loads a GGUF checkpoint by de-quantising every tensor to f32 on the host
// (src/gguf.js:187-231 per block, src/gguf.js:343-400 per tensor) and transposing weight matrices
// from GGUF's [outDim, inDim] to its own [inDim, outDim] (src/gguf_loader.js:236-252); the f32
// weights then run through the f32 matmul.  Two of GGUF's formats need no de-quantisation to run on
// the quantized path:
//
//   Q8_0 (type 8): 34-byte blocks [f16 scale, little endian][32 x int8] of 32 consecutive inDim
//     elements of one output row -- byte for byte the block shaders/matmul_q8.metal:40-52 reads.
//     GGUF block (row r, group b) at (r * G + b) * 34 becomes block (g = b, col = r) at (b * N + r) * 34.
//   Q4_0 (type 2): 18-byte blocks [f16 scale][16 nibble bytes], element i in byte i >> 1, low nibble
//     for even i as the reference reads them (src/gguf.js:187-197), value = scale * (nibble - 8).
//     That is the 24-byte Q4 block of shaders/matmul_q4.metal:24-28 with the same nibble bytes, scale
//     widened to f32 (exact) and zero = 8: scale * (float(nibble) - 8.0f) is the same f32 product.
//
// One thread moves one block; adjacent threads take adjacent output rows of one group, so the
// stores of a warp are contiguous.  A load-time operation: the source blocks are touched once.
#include <cuda_fp16.h>

#include "kernels.h"

namespace smith {
namespace {

__global__ void __launch_bounds__(256) repack_q8_0_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                          int64_t N, int64_t G) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // output row = column of the matmul layout
  const int64_t b = blockIdx.y;                                       // group along inDim
  if (r >= N) return;
  const uint16_t* s = reinterpret_cast<const uint16_t*>(src + (r * G + b) * kQ8Bytes);   // 34-byte blocks are 2-byte aligned
  uint16_t* d = reinterpret_cast<uint16_t*>(dst + (b * N + r) * kQ8Bytes);
#pragma unroll
  for (int i = 0; i < kQ8Bytes / 2; i++) d[i] = s[i];
}

__global__ void __launch_bounds__(256) repack_q4_0_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                          int64_t N, int64_t G) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t b = blockIdx.y;
  if (r >= N) return;
  const uint16_t* s = reinterpret_cast<const uint16_t*>(src + (r * G + b) * 18);          // 18-byte blocks are 2-byte aligned
  uint32_t* d = reinterpret_cast<uint32_t*>(dst + (b * N + r) * kQ4Bytes);                // 24-byte blocks are 8-byte aligned
  const float scale = __half2float(__ushort_as_half(s[0]));                              // exact: every f16 is an f32
#pragma unroll
  for (int i = 0; i < 4; i++) d[i] = (uint32_t)s[1 + 2 * i] | ((uint32_t)s[2 + 2 * i] << 16);
  d[4] = __float_as_uint(scale);
  d[5] = __float_as_uint(8.0f);
}

}  // namespace

cudaError_t launch_gguf_repack(int ggml_type, const uint8_t* src, uint8_t* dst, int64_t out_dim, int64_t in_dim,
                               cudaStream_t s) {
  if (out_dim <= 0 || in_dim <= 0) return cudaSuccess;
  if ((in_dim % 32) != 0) return cudaErrorInvalidValue;
  const int64_t G = in_dim / 32;
  if (G > 65535) return cudaErrorInvalidValue;
  dim3 grid((unsigned)((out_dim + 255) / 256), (unsigned)G);
  if (ggml_type == 8)
    repack_q8_0_kernel<<<grid, 256, 0, s>>>(src, dst, out_dim, G);
  else if (ggml_type == 2)
    repack_q4_0_kernel<<<grid, 256, 0, s>>>(src, dst, out_dim, G);
  else
    return cudaErrorInvalidValue;
  count_launch();
  return cudaGetLastError();
}

}  // namespace smith
