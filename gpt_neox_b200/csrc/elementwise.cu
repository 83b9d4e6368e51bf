// Stand-alone element-wise kernels (used where the op is not folded into a GEMM epilogue):
// bias + activation fwd/bwd, gated activations (SwiGLU / GeGLU / ReGLU), bias + dropout +
// residual, column sums (bias gradients) and dtype casts.
//
// Counterparts in the reference: torch.jit bias_gelu / bias_gelu_back
// (megatron/model/activations.py:78-112), Gated_Activation (megatron/model/transformer.py:182-198),
// bias_dropout_add (megatron/model/fused_bias_dropout.py:28-55).
#include <curand_kernel.h>

#include "common.h"
#include "ptx.cuh"
#include "reduce.cuh"

namespace nx {

enum Act : int { ACT_GELU_ERF = 0, ACT_GELU_TANH = 1, ACT_RELU = 2, ACT_SILU = 3, ACT_IDENTITY = 4,
                 ACT_SIGMOID = 5, ACT_RELU2 = 6 };

__device__ __forceinline__ float act_fwd(int a, float x) {
  switch (a) {
    case ACT_GELU_ERF: return gelu_erf(x);
    case ACT_GELU_TANH: return gelu_tanh(x);
    case ACT_RELU: return fmaxf(x, 0.f);
    case ACT_SILU: return silu(x);
    case ACT_SIGMOID: return 1.f / (1.f + __expf(-x));
    case ACT_RELU2: { const float r = fmaxf(x, 0.f); return r * r; }
    default: return x;
  }
}
__device__ __forceinline__ float act_grad(int a, float x) {
  switch (a) {
    case ACT_GELU_ERF: return gelu_erf_grad(x);
    case ACT_GELU_TANH: return gelu_tanh_grad(x);
    case ACT_RELU: return x > 0.f ? 1.f : 0.f;
    case ACT_SILU: return silu_grad(x);
    case ACT_SIGMOID: { const float s = 1.f / (1.f + __expf(-x)); return s * (1.f - s); }
    case ACT_RELU2: return x > 0.f ? 2.f * x : 0.f;
    default: return 1.f;
  }
}

__device__ __forceinline__ void ld8(const h16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_h16x2(u.x), b = unpack_h16x2(u.y), c = unpack_h16x2(u.z),
               d = unpack_h16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void st8(h16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_h16x2(f[0], f[1]);
  u.y = pack_h16x2(f[2], f[3]);
  u.z = pack_h16x2(f[4], f[5]);
  u.w = pack_h16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// y[r, c] = act(x[r, c] + bias[c])
__global__ void bias_act_fwd_kernel(const h16* __restrict__ x,
                                    const h16* __restrict__ bias,
                                    h16* __restrict__ y, long long nvec, int ncols8,
                                    int act) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float v[8], b[8];
    ld8(x + i * 8, v);
    if (bias != nullptr) {
      ld8(bias + (i % ncols8) * 8, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += b[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = act_fwd(act, v[j]);
    st8(y + i * 8, v);
  }
}

// dx[r, c] = dy[r, c] * act'(x[r, c] + bias[c])
__global__ void bias_act_bwd_kernel(const h16* __restrict__ dy,
                                    const h16* __restrict__ x,
                                    const h16* __restrict__ bias,
                                    h16* __restrict__ dx, long long nvec, int ncols8,
                                    int act) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float v[8], b[8], g[8];
    ld8(x + i * 8, v);
    ld8(dy + i * 8, g);
    if (bias != nullptr) {
      ld8(bias + (i % ncols8) * 8, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += b[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= act_grad(act, v[j]);
    st8(dx + i * 8, g);
  }
}

// x: [rows, 2F] = [value | gate];  y[r, f] = value * act(gate)
__global__ void gated_act_fwd_kernel(const h16* __restrict__ x,
                                     h16* __restrict__ y, long long rows, int F, int act) {
  const int f8 = F >> 3;
  const long long nvec = rows * f8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / f8;
    const int c = static_cast<int>(i - r * f8) * 8;
    float v[8], g[8];
    ld8(x + r * 2 * F + c, v);
    ld8(x + r * 2 * F + F + c, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= act_fwd(act, g[j]);
    st8(y + r * F + c, v);
  }
}
// dx[:, :F] = dy * act(gate);  dx[:, F:] = dy * value * act'(gate)
__global__ void gated_act_bwd_kernel(const h16* __restrict__ dy,
                                     const h16* __restrict__ x,
                                     h16* __restrict__ dx, long long rows, int F, int act) {
  const int f8 = F >> 3;
  const long long nvec = rows * f8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / f8;
    const int c = static_cast<int>(i - r * f8) * 8;
    float v[8], g[8], d[8], dv[8], dg[8];
    ld8(x + r * 2 * F + c, v);
    ld8(x + r * 2 * F + F + c, g);
    ld8(dy + r * F + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dv[j] = d[j] * act_fwd(act, g[j]);
      dg[j] = d[j] * v[j] * act_grad(act, g[j]);
    }
    st8(dx + r * 2 * F + c, dv);
    st8(dx + r * 2 * F + F + c, dg);
  }
}

// out = residual + dropout(x + bias, p) ; mask (uint8, optional) records kept elements.
__global__ void bias_dropout_add_kernel(const h16* __restrict__ x,
                                        const h16* __restrict__ bias,
                                        const h16* __restrict__ residual,
                                        h16* __restrict__ out,
                                        uint8_t* __restrict__ mask, long long nvec, int ncols8,
                                        float p, unsigned long long seed,
                                        unsigned long long offset) {
  const float keep_scale = p > 0.f ? 1.f / (1.f - p) : 1.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float v[8], b[8];
    ld8(x + i * 8, v);
    if (bias != nullptr) {
      ld8(bias + (i % ncols8) * 8, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += b[j];
    }
    if (p > 0.f) {
      curandStatePhilox4_32_10_t st;
      curand_init(seed, static_cast<unsigned long long>(i), offset, &st);
      const float4 r0 = curand_uniform4(&st), r1 = curand_uniform4(&st);
      const float r[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
      uint8_t m = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool keep = r[j] > p;
        v[j] = keep ? v[j] * keep_scale : 0.f;
        m |= static_cast<uint8_t>(keep) << j;
      }
      if (mask != nullptr) mask[i] = m;
    }
    if (residual != nullptr) {
      ld8(residual + i * 8, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += b[j];
    }
    st8(out + i * 8, v);
  }
}
// dx = dy * mask * 1/(1-p)   (mask bit-packed, one byte per 8 elements)
__global__ void dropout_bwd_kernel(const h16* __restrict__ dy,
                                   const uint8_t* __restrict__ mask, h16* __restrict__ dx,
                                   long long nvec, float p) {
  const float keep_scale = 1.f / (1.f - p);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float g[8];
    ld8(dy + i * 8, g);
    const uint8_t m = mask[i];
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] = ((m >> j) & 1) ? g[j] * keep_scale : 0.f;
    st8(dx + i * 8, g);
  }
}

// out[c] (+)= sum_r x[r, c]   (bf16 in, fp32 out).  Stage 1: each block reduces a row slab for
// 64 columns into ws[slab, c]; stage 2 sums the slabs.
constexpr int CS_COLS = 64;
__global__ void colsum_stage1(const h16* __restrict__ x, float* __restrict__ ws,
                              long long rows, int N, long long ld, int slabs) {
  __shared__ float sh[8][CS_COLS];
  const int c0 = blockIdx.x * CS_COLS;
  const int slab = blockIdx.y;
  const int tx = threadIdx.x & 7;   // 8 vectors of 8 columns
  const int ty = threadIdx.x >> 3;  // 32 row lanes
  const long long rows_per = (rows + slabs - 1) / slabs;
  const long long r0 = slab * rows_per, r1 = min(rows, r0 + rows_per);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int c = c0 + tx * 8;
  if (c < N) {
    for (long long r = r0 + ty; r < r1; r += 32) {
      float v[8];
      ld8(x + r * ld + c, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
  }
  // reduce over ty (32 lanes spread over 8 warps: thread = ty*8+tx -> warp = ty/4)
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
  if (threadIdx.x < CS_COLS) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += sh[w][threadIdx.x];
    if (c0 + threadIdx.x < N) ws[static_cast<long long>(slab) * N + c0 + threadIdx.x] = s;
  }
}
__global__ void colsum_stage2(const float* __restrict__ ws, float* __restrict__ out_f32,
                              h16* __restrict__ out_bf16, int N, int slabs,
                              int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= N) return;
  float s = 0.f;
  for (int i = 0; i < slabs; ++i) s += ws[static_cast<long long>(i) * N + c];
  if (out_f32 != nullptr) out_f32[c] = accumulate ? out_f32[c] + s : s;
  if (out_bf16 != nullptr) out_bf16[c] = float_to_h16(s);
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ x, h16* __restrict__ y,
                                        long long n, float scale) {
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < n;
       i += (long long)gridDim.x * blockDim.x * 4) {
    if (i + 4 <= n) {
      const float4 v = *reinterpret_cast<const float4*>(x + i);
      uint2 o;
      o.x = pack_h16x2(v.x * scale, v.y * scale);
      o.y = pack_h16x2(v.z * scale, v.w * scale);
      *reinterpret_cast<uint2*>(y + i) = o;
    } else {
      for (long long j = i; j < n; ++j) y[j] = float_to_h16(x[j] * scale);
    }
  }
}

static inline int grid_for(long long nvec, int threads) {
  long long g = (nvec + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  return static_cast<int>(g < cap ? (g > 0 ? g : 1) : cap);
}

}  // namespace nx

using bf = h16;

NX_API int NX_SYM(nx_bias_act_fwd)(const void* x, const void* bias, void* y, long long rows, int cols,
                           int act, void* stream_) {
  using namespace nx;
  NX_REQUIRE(cols % 8 == 0, "bias_act: cols %% 8 != 0");
  const long long nvec = rows * (cols / 8);
  if (nvec == 0) return NX_OK;
  bias_act_fwd_kernel<<<grid_for(nvec, 256), 256, 0, (cudaStream_t)stream_>>>(
      (const bf*)x, (const bf*)bias, (bf*)y, nvec, cols / 8, act);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
NX_API int NX_SYM(nx_bias_act_bwd)(const void* dy, const void* x, const void* bias, void* dx, long long rows,
                           int cols, int act, void* stream_) {
  using namespace nx;
  NX_REQUIRE(cols % 8 == 0, "bias_act: cols %% 8 != 0");
  const long long nvec = rows * (cols / 8);
  if (nvec == 0) return NX_OK;
  bias_act_bwd_kernel<<<grid_for(nvec, 256), 256, 0, (cudaStream_t)stream_>>>(
      (const bf*)dy, (const bf*)x, (const bf*)bias, (bf*)dx, nvec, cols / 8, act);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
NX_API int NX_SYM(nx_gated_act_fwd)(const void* x, void* y, long long rows, int F, int act, void* stream_) {
  using namespace nx;
  NX_REQUIRE(F % 8 == 0, "gated_act: F %% 8 != 0");
  const long long nvec = rows * (F / 8);
  if (nvec == 0) return NX_OK;
  gated_act_fwd_kernel<<<grid_for(nvec, 256), 256, 0, (cudaStream_t)stream_>>>((const bf*)x, (bf*)y,
                                                                              rows, F, act);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
NX_API int NX_SYM(nx_gated_act_bwd)(const void* dy, const void* x, void* dx, long long rows, int F, int act,
                            void* stream_) {
  using namespace nx;
  NX_REQUIRE(F % 8 == 0, "gated_act: F %% 8 != 0");
  const long long nvec = rows * (F / 8);
  if (nvec == 0) return NX_OK;
  gated_act_bwd_kernel<<<grid_for(nvec, 256), 256, 0, (cudaStream_t)stream_>>>(
      (const bf*)dy, (const bf*)x, (bf*)dx, rows, F, act);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
NX_API int NX_SYM(nx_bias_dropout_add)(const void* x, const void* bias, const void* residual, void* out,
                               void* mask, long long rows, int cols, float p,
                               unsigned long long seed, unsigned long long offset, void* stream_) {
  using namespace nx;
  NX_REQUIRE(cols % 8 == 0, "bias_dropout_add: cols %% 8 != 0");
  NX_REQUIRE(p >= 0.f && p < 1.f, "bias_dropout_add: p out of range");
  const long long nvec = rows * (cols / 8);
  if (nvec == 0) return NX_OK;
  bias_dropout_add_kernel<<<grid_for(nvec, 256), 256, 0, (cudaStream_t)stream_>>>(
      (const bf*)x, (const bf*)bias, (const bf*)residual, (bf*)out, (uint8_t*)mask, nvec, cols / 8, p,
      seed, offset);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
NX_API int NX_SYM(nx_dropout_bwd)(const void* dy, const void* mask, void* dx, long long n, float p,
                          void* stream_) {
  using namespace nx;
  NX_REQUIRE(n % 8 == 0, "dropout_bwd: n %% 8 != 0");
  if (n == 0) return NX_OK;
  dropout_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream_>>>(
      (const bf*)dy, (const uint8_t*)mask, (bf*)dx, n / 8, p);
  NX_LAUNCH_CHECK();
  return NX_OK;
}

// Slabs of the column-sum workspace: ws holds nx_colsum_slabs(rows) * N floats.
NX_API int NX_SYM(nx_colsum_slabs)(long long rows) {
  long long s = rows / 256;
  if (s < 1) s = 1;
  if (s > 64) s = 64;
  return static_cast<int>(s);
}
NX_API int NX_SYM(nx_colsum_bf16)(const void* x, void* out_f32, void* out_bf16, void* ws, long long rows,
                          int N, long long ld, int accumulate, void* stream_) {
  using namespace nx;
  NX_REQUIRE(N % 8 == 0 && ld % 8 == 0, "colsum: N and ld must be multiples of 8");
  NX_REQUIRE(ws != nullptr, "colsum: workspace is null");
  if (N == 0) return NX_OK;
  const int slabs = NX_SYM(nx_colsum_slabs)(rows);
  dim3 grid((N + CS_COLS - 1) / CS_COLS, slabs);
  colsum_stage1<<<grid, 256, 0, (cudaStream_t)stream_>>>((const bf*)x, (float*)ws, rows, N, ld,
                                                         slabs);
  NX_LAUNCH_CHECK();
  colsum_stage2<<<(N + 127) / 128, 128, 0, (cudaStream_t)stream_>>>(
      (const float*)ws, (float*)out_f32, (bf*)out_bf16, N, slabs, accumulate);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
NX_API int NX_SYM(nx_cast_f32_to_bf16)(const void* x, void* y, long long n, float scale, void* stream_) {
  using namespace nx;
  if (n == 0) return NX_OK;
  cast_f32_to_bf16_kernel<<<grid_for((n + 3) / 4, 256), 256, 0, (cudaStream_t)stream_>>>(
      (const float*)x, (bf*)y, n, scale);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
