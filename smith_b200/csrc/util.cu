// util.cu -- small device utilities of the bridge: synthetic normal data for
// benchmarks and large-shape tests, and a byte fill used to flush L2.
#include "kernels.h"
#include "pipeline.cuh"

namespace smith {

thread_local uint64_t* g_launch_counter = nullptr;

__device__ int g_kernel_status = 0;

// Device address of the status word on the current device (one lookup per device).
int* kernel_status_ptr() {
  static int* ptrs[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ptrs[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_kernel_status) != cudaSuccess) return nullptr;
    ptrs[dev] = static_cast<int*>(p);
  }
  return ptrs[dev];
}

int device_sm_count() {
  static int sms[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!sms[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) {
      cudaGetLastError();
      return 148;
    }
    sms[dev] = n;
  }
  return sms[dev];
}

bool* PerDeviceFlag::here() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  return &done[dev];
}

// Reads and clears the "a bounded device-side wait gave up" word of the current device.
int kernel_take_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_kernel_status, sizeof v) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_kernel_status, &zero, sizeof zero);
  return v;
}

namespace {

__device__ __forceinline__ uint64_t mix64(uint64_t x) {  // splitmix64 finaliser
  x += 0x9E3779B97F4A7C15ULL;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ULL;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBULL;
  return x ^ (x >> 31);
}

// Element pair (2i, 2i+1) = Box-Muller of two uniforms hashed from (seed, i).
__global__ void fill_normal_kernel(float* __restrict__ out, uint64_t count, uint64_t seed, float std) {
  const uint64_t pairs = (count + 1) / 2;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs;
       i += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t h = mix64(seed * 0xD1342543DE82EF95ULL + i);
    const uint32_t a = (uint32_t)(h >> 32), b = (uint32_t)h;
    const float u1 = ((float)(a >> 8) + 1.0f) * (1.0f / 16777216.0f);  // (0, 1]
    const float u2 = (float)(b >> 8) * (1.0f / 16777216.0f);           // [0, 1)
    const float r = sqrtf(-2.0f * __logf(u1)) * std;
    float sn, cs;
    __sincosf(6.283185307179586f * u2, &sn, &cs);
    out[2 * i] = r * cs;
    if (2 * i + 1 < count) out[2 * i + 1] = r * sn;
  }
}

__global__ void fill_bytes_kernel(uint4* __restrict__ out, size_t n16, uint32_t value) {
  const uint4 v = make_uint4(value, value, value, value);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16;
       i += (size_t)gridDim.x * blockDim.x)
    out[i] = v;
}

}  // namespace

cudaError_t launch_fill_normal(float* out, uint64_t count, uint64_t seed, float std, cudaStream_t s) {
  if (count == 0) return cudaSuccess;
  fill_normal_kernel<<<device_sm_count() * 8, 256, 0, s>>>(out, count, seed, std);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_fill_bytes(void* out, size_t bytes, uint32_t value, cudaStream_t s) {
  if (bytes < 16) return cudaSuccess;
  fill_bytes_kernel<<<device_sm_count() * 4, 256, 0, s>>>(reinterpret_cast<uint4*>(out), bytes / 16, value);
  count_launch();
  return cudaGetLastError();
}

}  // namespace smith
