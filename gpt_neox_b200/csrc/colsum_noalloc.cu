// Column sums without a caller-provided workspace: see no_alloc.h for the contract.
#include "no_alloc.h"

#include <mutex>

#include "common.h"
#include "ptx.cuh"

// Scratch for the per-slab partial sums.  In host code this name is only a stand-in for the device
// symbol, never a device address: the address is looked up once per device below.
static __device__ __align__(256) float g_colsum_scratch[NX_COLSUM_NOALLOC_MAX_FLOATS];

namespace {

constexpr int COLS = 64;  // columns per block

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const float2 a = nx::unpack_h16x2(u.x), b = nx::unpack_h16x2(u.y), c = nx::unpack_h16x2(u.z),
               d = nx::unpack_h16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

// Stage 1: block (column group, slab) sums its slab of rows for 64 columns into ws[slab, c].
__global__ void partial_sums(const __nv_bfloat16* __restrict__ x, float* __restrict__ ws,
                             long long rows, int N, long long ld, int slabs) {
  __shared__ float sh[8][COLS];
  const int c0 = blockIdx.x * COLS;
  const int slab = blockIdx.y;
  const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
  const long long per = (rows + slabs - 1) / slabs;
  const long long r0 = slab * per, r1 = min(rows, r0 + per);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int c = c0 + tx * 8;
  if (c < N) {
    for (long long r = r0 + ty; r < r1; r += 32) {
      float v[8];
      load8(x + r * ld + c, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 8);
    acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 16);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane < 8) {
#pragma unroll
    for (int j = 0; j < 8; ++j) sh[warp][lane * 8 + j] = acc[j];
  }
  __syncthreads();
  if (threadIdx.x < COLS && c0 + threadIdx.x < N) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += sh[w][threadIdx.x];
    ws[static_cast<long long>(slab) * N + c0 + threadIdx.x] = s;  // every (slab, column) is written
  }
}

// Stage 2: out[c] (+)= sum over slabs.
__global__ void final_sums(const float* __restrict__ ws, float* __restrict__ out, int N, int slabs,
                           int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= N) return;
  float s = 0.f;
  for (int i = 0; i < slabs; ++i) s += ws[static_cast<long long>(i) * N + c];
  out[c] = accumulate ? out[c] + s : s;
}

// Device address of the scratch array, resolved once per device with that device current.
// The small cache is filled under a lock, so first calls from several host threads are safe.  It is
// not refreshed after cudaDeviceReset: a process that resets a device must not call in again.
float* scratch_for_current_device(int* status) {
  static float* ptrs[64] = {nullptr};
  static std::mutex mu;
  std::lock_guard<std::mutex> guard(mu);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    nx::set_last_error("colsum_noalloc: cudaGetDevice failed or device index out of range (%d): %s", dev,
                       cudaGetErrorString(e));
    *status = NX_ERR_CUDA;
    return nullptr;
  }
  if (ptrs[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_colsum_scratch);
    if (e != cudaSuccess || p == nullptr) {
      nx::set_last_error("colsum_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                         cudaGetErrorString(e));
      *status = NX_ERR_CUDA;
      return nullptr;
    }
    ptrs[dev] = p;
  }
  *status = NX_OK;
  return ptrs[dev];
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int nx_colsum_bf16_noalloc(
    const void* x, void* out_f32, long long rows, int N, long long ld, int accumulate, void* stream_) {
  // an empty input (rows == 0) may come with a null pointer: the sums are then all zero
  NX_REQUIRE((x != nullptr || rows == 0) && out_f32 != nullptr, "colsum_noalloc: null input or output");
  NX_REQUIRE(rows >= 0 && N >= 0, "colsum_noalloc: negative size");
  NX_REQUIRE(N % 8 == 0 && ld % 8 == 0 && ld >= N, "colsum_noalloc: N and ld must be multiples of 8, ld >= N");
  NX_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0, "colsum_noalloc: x must be 16-byte aligned");
  if (N == 0) return NX_OK;
  long long slabs = rows / 256;
  if (slabs < 1) slabs = 1;
  if (slabs > 64) slabs = 64;
  NX_REQUIRE(slabs * N <= NX_COLSUM_NOALLOC_MAX_FLOATS,
             "colsum_noalloc: %lld slabs x %d columns = %lld floats exceeds the built-in scratch of %d floats "
             "(use nx_colsum_bf16 with a caller workspace for this size)",
             slabs, N, slabs * N, NX_COLSUM_NOALLOC_MAX_FLOATS);
  int st = NX_OK;
  float* ws = scratch_for_current_device(&st);
  if (ws == nullptr) return st;
  auto stream = static_cast<cudaStream_t>(stream_);
  dim3 grid((N + COLS - 1) / COLS, static_cast<unsigned>(slabs));
  partial_sums<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), ws, rows, N, ld,
                                         static_cast<int>(slabs));
  NX_LAUNCH_CHECK();
  final_sums<<<(N + 127) / 128, 128, 0, stream>>>(ws, static_cast<float*>(out_f32), N,
                                                  static_cast<int>(slabs), accumulate);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
