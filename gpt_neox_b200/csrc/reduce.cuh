// Warp / block reductions used by the memory-bound kernels.
#pragma once
#include <cuda_runtime.h>

namespace nx {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum of two values at once; `sh` must hold 2 * 32 floats. All threads get the result.
__device__ __forceinline__ float2 block_sum2(float a, float b, float* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  a = warp_sum(a);
  b = warp_sum(b);
  __syncthreads();  // protect sh from a previous use
  if (lane == 0) {
    sh[warp] = a;
    sh[32 + warp] = b;
  }
  __syncthreads();
  float ra = lane < nw ? sh[lane] : 0.f;
  float rb = lane < nw ? sh[32 + lane] : 0.f;
  ra = warp_sum(ra);
  rb = warp_sum(rb);
  return make_float2(ra, rb);
}
// Block-wide maximum of two non-negative values at once; `sh` must hold 2 * 32 floats. All threads get the result.
__device__ __forceinline__ float2 block_max2(float a, float b, float* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  a = warp_max(a);
  b = warp_max(b);
  __syncthreads();
  if (lane == 0) {
    sh[warp] = a;
    sh[32 + warp] = b;
  }
  __syncthreads();
  float ra = lane < nw ? sh[lane] : 0.f;
  float rb = lane < nw ? sh[32 + lane] : 0.f;
  return make_float2(warp_max(ra), warp_max(rb));
}
__device__ __forceinline__ float block_sum(float a, float* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  a = warp_sum(a);
  __syncthreads();
  if (lane == 0) sh[warp] = a;
  __syncthreads();
  float ra = lane < nw ? sh[lane] : 0.f;
  return warp_sum(ra);
}
__device__ __forceinline__ float block_max(float a, float* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  a = warp_max(a);
  __syncthreads();
  if (lane == 0) sh[warp] = a;
  __syncthreads();
  float ra = lane < nw ? sh[lane] : -INFINITY;
  return warp_max(ra);
}

}  // namespace nx
