// Scaled + masked softmax, forward and backward, for the non-flash ("global") attention path.
//
// API-parity counterparts of the reference's fused kernels
// (megatron/fused_kernels/scaled_upper_triang_masked_softmax.h:143-361 and
//  megatron/fused_kernels/scaled_masked_softmax.h:117-335), without their 2048-column cap:
// rows of any length are handled by one warp (<= 1024 columns, values kept in registers) or one
// block (longer rows, values re-read through L2).
//   causal : x[attn_batches, sq, sk]; row i of each [sq, sk] matrix sees columns 0..i+(sk-sq);
//            masked positions are written as 0.
//   masked : x[b, np, sq, sk], mask[b or 1, 1, sq, sk] uint8 (1 = masked -> -10000 before softmax).
#include "common.h"
#include "ptx.cuh"
#include "reduce.cuh"

namespace nx {

// One block per row; generic in row length.
template <bool CAUSAL>
__global__ void softmax_fwd_kernel(const h16* __restrict__ x,
                                   h16* __restrict__ y, const uint8_t* __restrict__ mask,
                                   int sq, int sk, int np, int mask_batch_stride_is_zero,
                                   float scale) {
  __shared__ float sh[64];
  const long long row = blockIdx.x;  // over attn_batches * sq
  const int qi = static_cast<int>(row % sq);
  const h16* xr = x + row * sk;
  h16* yr = y + row * sk;
  const int limit = CAUSAL ? min(sk, qi + 1 + (sk - sq)) : sk;
  const uint8_t* mr = nullptr;
  if (!CAUSAL && mask != nullptr) {
    const long long b = row / (static_cast<long long>(np) * sq);
    mr = mask + ((mask_batch_stride_is_zero ? 0 : b) * sq + qi) * static_cast<long long>(sk);
  }
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < limit; c += blockDim.x) {
    float v = h16_to_float(xr[c]) * scale;
    if (mr != nullptr && mr[c]) v = -10000.f;
    mx = fmaxf(mx, v);
  }
  mx = block_max(mx, sh);
  float sum = 0.f;
  for (int c = threadIdx.x; c < limit; c += blockDim.x) {
    float v = h16_to_float(xr[c]) * scale;
    if (mr != nullptr && mr[c]) v = -10000.f;
    sum += __expf(v - mx);
  }
  sum = block_sum(sum, sh);
  const float inv = sum > 0.f ? 1.f / sum : 0.f;
  for (int c = threadIdx.x; c < sk; c += blockDim.x) {
    float o = 0.f;
    if (c < limit) {
      float v = h16_to_float(xr[c]) * scale;
      if (mr != nullptr && mr[c]) v = -10000.f;
      o = __expf(v - mx) * inv;
    }
    yr[c] = float_to_h16(o);
  }
}

// dx = scale * y * (dy - sum(dy * y))
__global__ void softmax_bwd_kernel(const h16* __restrict__ dy,
                                   const h16* __restrict__ y,
                                   h16* __restrict__ dx, int sk, float scale) {
  __shared__ float sh[64];
  const long long row = blockIdx.x;
  const h16* dyr = dy + row * sk;
  const h16* yr = y + row * sk;
  float s = 0.f;
  for (int c = threadIdx.x; c < sk; c += blockDim.x)
    s += h16_to_float(dyr[c]) * h16_to_float(yr[c]);
  s = block_sum(s, sh);
  for (int c = threadIdx.x; c < sk; c += blockDim.x) {
    const float yv = h16_to_float(yr[c]);
    dx[row * sk + c] = float_to_h16(scale * yv * (h16_to_float(dyr[c]) - s));
  }
}

static int softmax_threads(int sk) { return sk <= 256 ? 64 : (sk <= 1024 ? 128 : 256); }

}  // namespace nx

using bf = h16;

NX_API int NX_SYM(nx_softmax_causal_fwd)(const void* x, void* y, long long attn_batches, int sq, int sk,
                                 float scale, void* stream_) {
  using namespace nx;
  const long long rows = attn_batches * sq;
  if (rows == 0) return NX_OK;
  NX_REQUIRE(rows < (1ll << 31), "softmax: too many rows");
  softmax_fwd_kernel<true><<<(unsigned)rows, softmax_threads(sk), 0, (cudaStream_t)stream_>>>(
      (const bf*)x, (bf*)y, nullptr, sq, sk, 1, 1, scale);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
NX_API int NX_SYM(nx_softmax_masked_fwd)(const void* x, const void* mask, void* y, int b, int np, int sq,
                                 int sk, int mask_batch, float scale, void* stream_) {
  using namespace nx;
  const long long rows = static_cast<long long>(b) * np * sq;
  if (rows == 0) return NX_OK;
  NX_REQUIRE(rows < (1ll << 31), "softmax: too many rows");
  NX_REQUIRE(mask_batch == 1 || mask_batch == b, "softmax: mask batch must be 1 or b");
  softmax_fwd_kernel<false><<<(unsigned)rows, softmax_threads(sk), 0, (cudaStream_t)stream_>>>(
      (const bf*)x, (bf*)y, (const uint8_t*)mask, sq, sk, np, mask_batch == 1 ? 1 : 0, scale);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
NX_API int NX_SYM(nx_softmax_bwd)(const void* dy, const void* y, void* dx, long long rows, int sk, float scale,
                          void* stream_) {
  using namespace nx;
  if (rows == 0) return NX_OK;
  NX_REQUIRE(rows < (1ll << 31), "softmax: too many rows");
  softmax_bwd_kernel<<<(unsigned)rows, softmax_threads(sk), 0, (cudaStream_t)stream_>>>(
      (const bf*)dy, (const bf*)y, (bf*)dx, sk, scale);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
// Parity with the reference's scaled_masked_softmax_cuda.get_batch_per_block
// (megatron/fused_kernels/scaled_masked_softmax.h:338-352): rows one 128-thread block of the
// warp-per-row scheme would cover. Only used by callers that size their launches from it.
NX_API int NX_SYM(nx_softmax_batch_per_block)(int sq, int sk, int b, int np) {
  int p2 = 1;
  while (p2 < sk) p2 <<= 1;
  const int warp_size = p2 < 32 ? p2 : 32;
  const int batches_per_warp = p2 <= 128 ? 2 : 1;
  const int warps_per_block = 128 / warp_size;
  (void)sq; (void)b; (void)np;
  return warps_per_block * batches_per_warp;
}
