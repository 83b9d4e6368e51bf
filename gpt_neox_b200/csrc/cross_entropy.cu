// (Vocab-parallel) softmax cross-entropy, forward statistics and in-place gradient.
//
// Counterpart of megatron/mpu/cross_entropy.py:27-112 and the fp32 up-cast in
// megatron/model/gpt2_model.py:60-78.  The reference materialises fp32 logits, runs three
// all-reduces (max, target logit, sum-exp) and keeps the full softmax for backward.  Here one
// pass over the bf16 logits of this rank's vocabulary shard yields (max, sum-exp relative to
// that max, target logit if it lives in the shard) per row; ranks combine those three floats
// (one small collective) and the backward recomputes exp(logit - lse) while writing the
// gradient over the logits buffer.
#include "common.h"
#include "ptx.cuh"
#include "reduce.cuh"

namespace nx {

__device__ __forceinline__ void online_add(float& m, float& s, float v) {
  if (v > m) {
    s = s * __expf(m - v) + 1.f;
    m = v;
  } else {
    s += __expf(v - m);
  }
}

template <typename T>
__device__ __forceinline__ float ldf(const T* p);
template <>
__device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ldf<h16>(const h16* p) {
  return h16_to_float(*p);
}

template <typename T>
__global__ void ce_fwd_kernel(const T* __restrict__ logits, const long long* __restrict__ labels,
                              float* __restrict__ stats, int V, long long ld, int vocab_start) {
  __shared__ float shm[32], shs[32];
  const long long row = blockIdx.x;
  const T* lr = logits + row * ld;
  float m = -INFINITY, s = 0.f;
  if (sizeof(T) == 2 && (V % 8) == 0 && (ld % 8) == 0) {
    const uint4* lv = reinterpret_cast<const uint4*>(lr);
    for (int i = threadIdx.x; i < V / 8; i += blockDim.x) {
      const uint4 u = lv[i];
      const float2 a = unpack_h16x2(u.x), b = unpack_h16x2(u.y), c = unpack_h16x2(u.z),
                   d = unpack_h16x2(u.w);
      const float mx8 = fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(b.x, b.y)),
                              fmaxf(fmaxf(c.x, c.y), fmaxf(d.x, d.y)));
      if (mx8 > m) {
        s *= __expf(m - mx8);
        m = mx8;
      }
      s += __expf(a.x - m) + __expf(a.y - m) + __expf(b.x - m) + __expf(b.y - m) +
           __expf(c.x - m) + __expf(c.y - m) + __expf(d.x - m) + __expf(d.y - m);
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) online_add(m, s, ldf<T>(lr + i));
  }
  // combine (m, s) pairs across the block
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const float mm = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * __expf(m - mm)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mm));
    m = mm;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) {
    shm[warp] = m;
    shs[warp] = s;
  }
  __syncthreads();
  if (warp == 0) {
    m = lane < nw ? shm[lane] : -INFINITY;
    s = lane < nw ? shs[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
      const float mm = fmaxf(m, m2);
      s = (m == -INFINITY ? 0.f : s * __expf(m - mm)) +
          (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mm));
      m = mm;
    }
    if (lane == 0) {
      const long long lab = labels[row] - vocab_start;
      const float t = (lab >= 0 && lab < V) ? ldf<T>(lr + lab) : 0.f;
      stats[row * 3 + 0] = m;
      stats[row * 3 + 1] = s;
      stats[row * 3 + 2] = t;
    }
  }
}

// dlogits[r, c] = (exp(logit - lse[r]) - [c == label]) * gscale[r]      (bf16 out, may alias in)
template <typename T>
__global__ void ce_bwd_kernel(const T* __restrict__ logits, const long long* __restrict__ labels,
                              const float* __restrict__ lse, const float* __restrict__ gscale,
                              h16* __restrict__ dlogits, int V, long long ld,
                              long long ld_out, int vocab_start) {
  const long long row = blockIdx.x;
  const T* lr = logits + row * ld;
  h16* dr = dlogits + row * ld_out;
  const float l = lse[row], g = gscale[row];
  const long long lab = labels[row] - vocab_start;
  if (sizeof(T) == 2 && (V % 8) == 0 && (ld % 8) == 0 && (ld_out % 8) == 0) {
    const uint4* lv = reinterpret_cast<const uint4*>(lr);
    uint4* dv = reinterpret_cast<uint4*>(dr);
    for (int i = threadIdx.x; i < V / 8; i += blockDim.x) {
      const uint4 u = lv[i];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
      uint32_t o[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 a = unpack_h16x2(w[q]);
        const int c = i * 8 + q * 2;
        const float p0 = (__expf(a.x - l) - (c == lab ? 1.f : 0.f)) * g;
        const float p1 = (__expf(a.y - l) - (c + 1 == lab ? 1.f : 0.f)) * g;
        o[q] = pack_h16x2(p0, p1);
      }
      dv[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float p = (__expf(ldf<T>(lr + i) - l) - (i == lab ? 1.f : 0.f)) * g;
      dr[i] = float_to_h16(p);
    }
  }
}

}  // namespace nx

// dtype: 0 = bf16 logits, 1 = fp32 logits.  stats: float[rows, 3] = (max, sumexp, target logit).
NX_API int NX_SYM(nx_ce_fwd)(const void* logits, const void* labels, void* stats, long long rows, int V,
                     long long ld, int vocab_start, int dtype, void* stream_) {
  using namespace nx;
  if (rows == 0) return NX_OK;
  NX_REQUIRE(rows < (1ll << 31), "ce: too many rows");
  auto s = (cudaStream_t)stream_;
  if (dtype == 0)
    ce_fwd_kernel<h16><<<(unsigned)rows, 256, 0, s>>>(
        (const h16*)logits, (const long long*)labels, (float*)stats, V, ld, vocab_start);
  else
    ce_fwd_kernel<float><<<(unsigned)rows, 256, 0, s>>>((const float*)logits,
                                                        (const long long*)labels, (float*)stats, V,
                                                        ld, vocab_start);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
NX_API int NX_SYM(nx_ce_bwd)(const void* logits, const void* labels, const void* lse, const void* gscale,
                     void* dlogits, long long rows, int V, long long ld, long long ld_out,
                     int vocab_start, int dtype, void* stream_) {
  using namespace nx;
  if (rows == 0) return NX_OK;
  NX_REQUIRE(rows < (1ll << 31), "ce: too many rows");
  auto s = (cudaStream_t)stream_;
  if (dtype == 0)
    ce_bwd_kernel<h16><<<(unsigned)rows, 256, 0, s>>>(
        (const h16*)logits, (const long long*)labels, (const float*)lse,
        (const float*)gscale, (h16*)dlogits, V, ld, ld_out, vocab_start);
  else
    ce_bwd_kernel<float><<<(unsigned)rows, 256, 0, s>>>(
        (const float*)logits, (const long long*)labels, (const float*)lse, (const float*)gscale,
        (h16*)dlogits, V, ld, ld_out, vocab_start);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
