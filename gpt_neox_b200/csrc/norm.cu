// LayerNorm / RMSNorm forward and backward (bf16 in/out, fp32 statistics).
//
// Replaces apex's FusedLayerNorm / FusedRMSNorm used by the reference
// (megatron/model/fused_layer_norm.py:34-262) and the unfused modules in
// megatron/model/norms.py:62-99.  Two fusions the reference does not have:
//   * "dual" forward: the GPT-J parallel-residual block applies two different norms to the
//     same input (megatron/model/transformer.py:1083); both outputs are produced from one
//     read of x and one set of statistics.
//   * backward can add an incoming residual-stream gradient (dx = dx_in + ...), so the sum of
//     the residual path and the norm paths needs no extra pass.
// Memory-bound: one block per row in forward, persistent blocks in backward (row-strided) so
// that dgamma / dbeta accumulate in registers and are reduced across blocks by a second tiny
// kernel through a caller-provided fp32 workspace [blocks, 2, H].
#include "common.h"
#include "ptx.cuh"
#include "reduce.cuh"

namespace nx {

constexpr int MAXV = 4;  // 16-byte vectors cached per thread

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z),
               d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

template <bool RMS>
__global__ void norm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                const __nv_bfloat16* __restrict__ g1,
                                const __nv_bfloat16* __restrict__ b1, __nv_bfloat16* __restrict__ y1,
                                const __nv_bfloat16* __restrict__ g2,
                                const __nv_bfloat16* __restrict__ b2, __nv_bfloat16* __restrict__ y2,
                                float* __restrict__ mean_out, float* __restrict__ rstd_out, int H,
                                float eps) {
  __shared__ float sh[64];
  const long long row = blockIdx.x;
  const int nv = H >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  float xv[MAXV][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nv) {
      unpack8(xr[idx], xv[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += RMS ? xv[i][j] * xv[i][j] : xv[i][j];
    }
  }
  float mean = 0.f, rstd;
  if (RMS) {
    const float ms = block_sum(s, sh) / H;
    rstd = rsqrtf(ms + eps);
  } else {
    mean = block_sum(s, sh) / H;
    float v = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      if (idx < nv) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = xv[i][j] - mean;
          v += d * d;
        }
      }
    }
    const float var = block_sum(v, sh) / H;
    rstd = rsqrtf(var + eps);
  }
  if (threadIdx.x == 0) {
    if (mean_out != nullptr) mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nv) {
      float g[8], b[8], o[8];
      unpack8(reinterpret_cast<const uint4*>(g1)[idx], g);
      if (b1 != nullptr) unpack8(reinterpret_cast<const uint4*>(b1)[idx], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = (xv[i][j] - mean) * rstd;
        o[j] = xh * g[j] + (b1 != nullptr ? b[j] : 0.f);
      }
      reinterpret_cast<uint4*>(y1 + row * H)[idx] = pack8(o);
      if (g2 != nullptr) {
        unpack8(reinterpret_cast<const uint4*>(g2)[idx], g);
        if (b2 != nullptr) unpack8(reinterpret_cast<const uint4*>(b2)[idx], b);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[i][j] - mean) * rstd;
          o[j] = xh * g[j] + (b2 != nullptr ? b[j] : 0.f);
        }
        reinterpret_cast<uint4*>(y2 + row * H)[idx] = pack8(o);
      }
    }
  }
}

template <bool RMS>
__global__ void norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                const __nv_bfloat16* __restrict__ x,
                                const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                                const __nv_bfloat16* __restrict__ gamma,
                                const __nv_bfloat16* __restrict__ dx_in,
                                __nv_bfloat16* __restrict__ dx, float* __restrict__ ws,
                                long long rows, int H) {
  __shared__ float sh[64];
  const int nv = H >> 3;
  float dg[MAXV][8], db[MAXV][8], g[MAXV][8];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
#pragma unroll
    for (int j = 0; j < 8; ++j) dg[i][j] = db[i][j] = 0.f;
    if (idx < nv) unpack8(reinterpret_cast<const uint4*>(gamma)[idx], g[i]);
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mean = RMS ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float xh[MAXV][8], wdy[MAXV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      if (idx < nv) {
        float xv[8], dv[8];
        unpack8(reinterpret_cast<const uint4*>(x + row * H)[idx], xv);
        unpack8(reinterpret_cast<const uint4*>(dy + row * H)[idx], dv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xv[j] - mean) * rstd;
          wdy[i][j] = dv[j] * g[i][j];
          s1 += wdy[i][j] * xh[i][j];
          s2 += wdy[i][j];
          dg[i][j] += dv[j] * xh[i][j];
          db[i][j] += dv[j];
        }
      }
    }
    const float2 r = block_sum2(s1, s2, sh);
    const float c1 = r.x / H, c2 = RMS ? 0.f : r.y / H;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      if (idx < nv) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (wdy[i][j] - c2 - xh[i][j] * c1);
        if (dx_in != nullptr) {
          float a[8];
          unpack8(reinterpret_cast<const uint4*>(dx_in + row * H)[idx], a);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += a[j];
        }
        reinterpret_cast<uint4*>(dx + row * H)[idx] = pack8(o);
      }
    }
  }
  float* wg = ws + static_cast<long long>(blockIdx.x) * 2 * H;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nv) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        wg[idx * 8 + j] = dg[i][j];
        wg[H + idx * 8 + j] = db[i][j];
      }
    }
  }
}

// out[c] (+)= sum_b ws[b, which, c].  Block = 128 columns x 8 row groups: each thread sums every 8th
// partial row (eight independent load chains per column instead of one long one), then the groups are
// combined through shared memory.
__global__ void __launch_bounds__(1024)
norm_param_grad_reduce(const float* __restrict__ ws, int nblocks, int H, float* __restrict__ dgamma,
                       float* __restrict__ dbeta, int accumulate) {
  __shared__ float sa[8][128], sb[8][128];
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int g = threadIdx.y;
  float a = 0.f, b = 0.f;
  if (c < H) {
    for (int i = g; i < nblocks; i += 8) {
      a += ws[static_cast<long long>(i) * 2 * H + c];
      if (dbeta != nullptr) b += ws[static_cast<long long>(i) * 2 * H + H + c];
    }
  }
  sa[g][threadIdx.x] = a;
  sb[g][threadIdx.x] = b;
  __syncthreads();
  if (g == 0 && c < H) {
#pragma unroll
    for (int k = 1; k < 8; ++k) {
      a += sa[k][threadIdx.x];
      b += sb[k][threadIdx.x];
    }
    if (accumulate) {
      dgamma[c] += a;
      if (dbeta != nullptr) dbeta[c] += b;
    } else {
      dgamma[c] = a;
      if (dbeta != nullptr) dbeta[c] = b;
    }
  }
}

static int threads_for(int H) {
  const int nv = H / 8;
  int t = (nv + MAXV - 1) / MAXV;
  t = ((t + 31) / 32) * 32;
  if (t < 64) t = 64;
  return t;
}

}  // namespace nx

// kind: 0 = LayerNorm, 1 = RMSNorm.  g2/b2/y2 null -> single output.  beta pointers may be null.
NX_API int nx_norm_fwd(int kind, const void* x, const void* g1, const void* b1, void* y1,
                       const void* g2, const void* b2, void* y2, void* mean, void* rstd,
                       long long rows, int H, float eps, void* stream_) {
  using namespace nx;
  if (rows <= 0) return NX_OK;
  NX_REQUIRE(H % 8 == 0 && H <= 8 * MAXV * 1024, "norm: H=%d must be a multiple of 8 and <= %d", H,
             8 * MAXV * 1024);
  NX_REQUIRE(rows < (1ll << 31), "norm: too many rows");
  auto s = static_cast<cudaStream_t>(stream_);
  const int t = threads_for(H);
  using bf = __nv_bfloat16;
  if (kind == 0)
    norm_fwd_kernel<false><<<(unsigned)rows, t, 0, s>>>((const bf*)x, (const bf*)g1, (const bf*)b1,
                                                         (bf*)y1, (const bf*)g2, (const bf*)b2,
                                                         (bf*)y2, (float*)mean, (float*)rstd, H, eps);
  else
    norm_fwd_kernel<true><<<(unsigned)rows, t, 0, s>>>((const bf*)x, (const bf*)g1, (const bf*)b1,
                                                        (bf*)y1, (const bf*)g2, (const bf*)b2,
                                                        (bf*)y2, (float*)mean, (float*)rstd, H, eps);
  NX_LAUNCH_CHECK();
  return NX_OK;
}

// Number of persistent blocks the backward uses == rows of the fp32 workspace [blocks, 2, H].
NX_API int nx_norm_bwd_blocks(long long rows) {
  const long long cap = static_cast<long long>(nx::sm_count()) * 4;
  return static_cast<int>(rows < cap ? rows : cap);
}

// dx = dx_in (optional) + norm backward; dgamma/dbeta fp32 (dbeta may be null; accumulate != 0
// adds into them).  ws: fp32 workspace of nx_norm_bwd_blocks(rows) * 2 * H floats.
NX_API int nx_norm_bwd(int kind, const void* dy, const void* x, const void* mean, const void* rstd,
                       const void* gamma, const void* dx_in, void* dx, void* dgamma, void* dbeta,
                       void* ws, long long rows, int H, int accumulate, void* stream_) {
  using namespace nx;
  if (rows <= 0) return NX_OK;
  NX_REQUIRE(H % 8 == 0 && H <= 8 * MAXV * 1024, "norm: H=%d unsupported", H);
  NX_REQUIRE(ws != nullptr, "norm_bwd: workspace is null");
  auto s = static_cast<cudaStream_t>(stream_);
  const int t = threads_for(H);
  const int blocks = nx_norm_bwd_blocks(rows);
  using bf = __nv_bfloat16;
  if (kind == 0)
    norm_bwd_kernel<false><<<blocks, t, 0, s>>>((const bf*)dy, (const bf*)x, (const float*)mean,
                                                 (const float*)rstd, (const bf*)gamma,
                                                 (const bf*)dx_in, (bf*)dx, (float*)ws, rows, H);
  else
    norm_bwd_kernel<true><<<blocks, t, 0, s>>>((const bf*)dy, (const bf*)x, (const float*)mean,
                                                (const float*)rstd, (const bf*)gamma,
                                                (const bf*)dx_in, (bf*)dx, (float*)ws, rows, H);
  NX_LAUNCH_CHECK();
  norm_param_grad_reduce<<<(H + 127) / 128, dim3(128, 8), 0, s>>>((const float*)ws, blocks, H,
                                                         (float*)dgamma, (float*)dbeta, accumulate);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
