// Fused optimizer kernels over flat (ZeRO-partitioned) buffers.
//
// Counterpart of apex / DeepSpeed FusedAdam (megatron/training.py:1069-1083) and of the
// DeepSpeed engine's clip / unscale / overflow logic the reference delegates to
// (megatron/training.py:1357,1380).  One launch updates a whole flat shard:
// fp32 master weights + Adam moments, gradient read as bf16 or fp32, multiplied by a scale that
// lives in device memory (loss-scale reciprocal x clip coefficient, so no host sync is needed
// between the norm reduction and the update), new bf16 model weights written in the same pass.
// If the device-side "skip" word is non-zero (non-finite gradients) nothing is modified.
#include "common.h"
#include "ptx.cuh"
#include "reduce.cuh"

namespace nx {

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2;
  int adam_w_mode;  // 1 = decoupled weight decay (AdamW), 0 = L2 added to the gradient
};

template <typename G>
__device__ __forceinline__ float4 load_grad4(const G* g, long long i);
template <>
__device__ __forceinline__ float4 load_grad4<float>(const float* g, long long i) {
  return *reinterpret_cast<const float4*>(g + i);
}
template <>
__device__ __forceinline__ float4 load_grad4<h16>(const h16* g, long long i) {
  const uint2 u = *reinterpret_cast<const uint2*>(g + i);
  const float2 a = unpack_h16x2(u.x), b = unpack_h16x2(u.y);
  return make_float4(a.x, a.y, b.x, b.y);
}

template <typename G>
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                             const G* __restrict__ g, h16* __restrict__ p_bf16,
                             long long n, AdamArgs a, const float* __restrict__ grad_scale,
                             const int* __restrict__ skip) {
  if (skip != nullptr && *skip != 0) return;
  const float gs = grad_scale != nullptr ? *grad_scale : 1.f;
  const float step = a.lr / a.bias_corr1;
  const float inv_bc2_sqrt = rsqrtf(a.bias_corr2);
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < n;
       i += (long long)gridDim.x * blockDim.x * 4) {
    if (i + 4 <= n) {
      float4 pv = *reinterpret_cast<float4*>(p + i);
      float4 mv = *reinterpret_cast<float4*>(m + i);
      float4 vv = *reinterpret_cast<float4*>(v + i);
      const float4 gv = load_grad4<G>(g, i);
      float pp[4] = {pv.x, pv.y, pv.z, pv.w}, mm[4] = {mv.x, mv.y, mv.z, mv.w},
            vvv[4] = {vv.x, vv.y, vv.z, vv.w}, gg[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float gr = gg[j] * gs;
        if (!a.adam_w_mode) gr += a.weight_decay * pp[j];
        mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gr;
        vvv[j] = a.beta2 * vvv[j] + (1.f - a.beta2) * gr * gr;
        const float denom = sqrtf(vvv[j]) * inv_bc2_sqrt + a.eps;
        float upd = mm[j] / denom;
        if (a.adam_w_mode) pp[j] -= a.lr * a.weight_decay * pp[j];
        pp[j] -= step * upd;
      }
      *reinterpret_cast<float4*>(p + i) = make_float4(pp[0], pp[1], pp[2], pp[3]);
      *reinterpret_cast<float4*>(m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(v + i) = make_float4(vvv[0], vvv[1], vvv[2], vvv[3]);
      if (p_bf16 != nullptr) {
        uint2 o;
        o.x = pack_h16x2(pp[0], pp[1]);
        o.y = pack_h16x2(pp[2], pp[3]);
        *reinterpret_cast<uint2*>(p_bf16 + i) = o;
      }
    } else {
      for (long long j = i; j < n; ++j) {
        float gr;
        if (sizeof(G) == 2) gr = h16_to_float(reinterpret_cast<const h16*>(g)[j]);
        else gr = reinterpret_cast<const float*>(g)[j];
        gr *= gs;
        float pj = p[j];
        if (!a.adam_w_mode) gr += a.weight_decay * pj;
        const float mj = a.beta1 * m[j] + (1.f - a.beta1) * gr;
        const float vj = a.beta2 * v[j] + (1.f - a.beta2) * gr * gr;
        const float denom = sqrtf(vj) * inv_bc2_sqrt + a.eps;
        if (a.adam_w_mode) pj -= a.lr * a.weight_decay * pj;
        pj -= step * (mj / denom);
        p[j] = pj; m[j] = mj; v[j] = vj;
        if (p_bf16 != nullptr) p_bf16[j] = float_to_h16(pj);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// AdamW with 8-bit block-wise optimizer state (what `use_bnb_optimizer` selects in the reference through
// bitsandbytes' Adam8bit, megatron/training.py:1058-1067): the two moments are stored as one byte per element
// plus one fp32 scale (the block's largest magnitude) per 2048 elements, 2 bytes of state per parameter instead
// of 8.  The byte is a logarithmic code relative to the block scale:
//   first moment  (signed):  bit 7 = sign, c = low 7 bits: 0 -> 0,  c -> scale * 2^((c - 127) * 14 / 126)
//   second moment (>= 0)  :  c = 0 -> 0,                         c -> scale * 2^((c - 255) * 28 / 254)
// (steps of 8 % and 8 % in value, i.e. at most about 4 % rounding error, over 2^-14 and 2^-28 of the scale).
// One CUDA block owns one quantisation block: it decodes, applies the update in fp32, finds the new scales
// with a block reduction and re-encodes, so the state is read and written exactly once.
// ------------------------------------------------------------------------------------------------
constexpr int Q8_BLOCK = 2048;
constexpr float Q8_M_STEP = 14.f / 126.f, Q8_V_STEP = 28.f / 254.f;

__device__ __forceinline__ float q8_decode_m(uint32_t b, float scale) {
  const uint32_t c = b & 127u;
  const float mag = c == 0u ? 0.f : scale * exp2f((static_cast<float>(c) - 127.f) * Q8_M_STEP);
  return (b & 128u) ? -mag : mag;
}
__device__ __forceinline__ float q8_decode_v(uint32_t c, float scale) {
  return c == 0u ? 0.f : scale * exp2f((static_cast<float>(c) - 255.f) * Q8_V_STEP);
}
__device__ __forceinline__ uint32_t q8_encode_m(float x, float inv_scale) {
  const float r = fabsf(x) * inv_scale;          // in [0, 1]
  float c = r > 0.f ? rintf(127.f + log2f(r) * (1.f / Q8_M_STEP)) : 0.f;
  c = fminf(fmaxf(c, 0.f), 127.f);
  return static_cast<uint32_t>(c) | (x < 0.f ? 128u : 0u);
}
__device__ __forceinline__ uint32_t q8_encode_v(float x, float inv_scale) {
  const float r = x * inv_scale;
  float c = r > 0.f ? rintf(255.f + log2f(r) * (1.f / Q8_V_STEP)) : 0.f;
  return static_cast<uint32_t>(fminf(fmaxf(c, 0.f), 255.f));
}

template <typename G>
__global__ void __launch_bounds__(256) adam8_kernel(float* __restrict__ p, uint8_t* __restrict__ m8,
                                                    uint8_t* __restrict__ v8, float* __restrict__ scale_m,
                                                    float* __restrict__ scale_v, const G* __restrict__ g,
                                                    h16* __restrict__ p_lp, long long n, AdamArgs a,
                                                    const float* __restrict__ grad_scale, const int* __restrict__ skip) {
  if (skip != nullptr && *skip != 0) return;
  __shared__ float sh[64];
  const float gs = grad_scale != nullptr ? *grad_scale : 1.f;
  const float step = a.lr / a.bias_corr1;
  const float inv_bc2_sqrt = rsqrtf(a.bias_corr2);
  const long long blk = blockIdx.x;
  const long long i0 = blk * Q8_BLOCK + threadIdx.x * 8;       // n is a multiple of 8: a thread's 8 elements are all in or all out
  const bool live = i0 < n;
  const float sm = scale_m[blk], sv = scale_v[blk];
  float mm[8], vv[8], pp[8];
  float max_m = 0.f, max_v = 0.f;
  if (live) {
    const uint2 mb = *reinterpret_cast<const uint2*>(m8 + i0);
    const uint2 vb = *reinterpret_cast<const uint2*>(v8 + i0);
    const float4 p0 = *reinterpret_cast<const float4*>(p + i0), p1 = *reinterpret_cast<const float4*>(p + i0 + 4);
    const float4 g0 = load_grad4<G>(g, i0), g1 = load_grad4<G>(g, i0 + 4);
    const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    pp[0] = p0.x; pp[1] = p0.y; pp[2] = p0.z; pp[3] = p0.w; pp[4] = p1.x; pp[5] = p1.y; pp[6] = p1.z; pp[7] = p1.w;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t bm = ((j < 4 ? mb.x : mb.y) >> ((j & 3) * 8)) & 255u;
      const uint32_t bv = ((j < 4 ? vb.x : vb.y) >> ((j & 3) * 8)) & 255u;
      float gr = gg[j] * gs;
      if (!a.adam_w_mode) gr += a.weight_decay * pp[j];
      mm[j] = a.beta1 * q8_decode_m(bm, sm) + (1.f - a.beta1) * gr;
      vv[j] = a.beta2 * q8_decode_v(bv, sv) + (1.f - a.beta2) * gr * gr;
      const float denom = sqrtf(vv[j]) * inv_bc2_sqrt + a.eps;
      if (a.adam_w_mode) pp[j] -= a.lr * a.weight_decay * pp[j];
      pp[j] -= step * (mm[j] / denom);
      max_m = fmaxf(max_m, fabsf(mm[j]));
      max_v = fmaxf(max_v, vv[j]);
    }
  }
  const float2 mx = block_max2(max_m, max_v, sh);
  if (live) {
    const float inv_m = mx.x > 0.f ? 1.f / mx.x : 0.f, inv_v = mx.y > 0.f ? 1.f / mx.y : 0.f;
    uint2 mb = make_uint2(0u, 0u), vb = make_uint2(0u, 0u);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t cm = q8_encode_m(mm[j], inv_m) << ((j & 3) * 8), cv = q8_encode_v(vv[j], inv_v) << ((j & 3) * 8);
      if (j < 4) { mb.x |= cm; vb.x |= cv; } else { mb.y |= cm; vb.y |= cv; }
    }
    *reinterpret_cast<uint2*>(m8 + i0) = mb;
    *reinterpret_cast<uint2*>(v8 + i0) = vb;
    *reinterpret_cast<float4*>(p + i0) = make_float4(pp[0], pp[1], pp[2], pp[3]);
    *reinterpret_cast<float4*>(p + i0 + 4) = make_float4(pp[4], pp[5], pp[6], pp[7]);
    if (p_lp != nullptr) {
      uint4 o;
      o.x = pack_h16x2(pp[0], pp[1]); o.y = pack_h16x2(pp[2], pp[3]);
      o.z = pack_h16x2(pp[4], pp[5]); o.w = pack_h16x2(pp[6], pp[7]);
      *reinterpret_cast<uint4*>(p_lp + i0) = o;
    }
  }
  if (threadIdx.x == 0) {
    scale_m[blk] = mx.x;
    scale_v[blk] = mx.y;
  }
}

// acc[0] += sum(x^2) ; acc[1] = max(acc[1], any non-finite ? 1 : 0)   (acc: float[2])
template <typename G>
__global__ void sumsq_kernel(const G* __restrict__ x, long long n, float* __restrict__ acc) {
  __shared__ float sh[64];
  float s = 0.f;
  float bad = 0.f;
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < n;
       i += (long long)gridDim.x * blockDim.x * 4) {
    if (i + 4 <= n) {
      const float4 v = load_grad4<G>(x, i);
      s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    } else {
      for (long long j = i; j < n; ++j) {
        float f;
        if (sizeof(G) == 2) f = h16_to_float(reinterpret_cast<const h16*>(x)[j]);
        else f = reinterpret_cast<const float*>(x)[j];
        s += f * f;
      }
    }
  }
  if (!isfinite(s)) bad = 1.f;
  const float2 r = block_sum2(s, bad, sh);
  if (threadIdx.x == 0) {
    atomicAdd(acc, r.x);
    if (r.y > 0.f || !isfinite(r.x)) atomicExch(acc + 1, 1.f);
  }
}

// out[0] = min(1, max_norm / (sqrt(acc[0]) * inv_scale + 1e-6)) * inv_scale ; skip = acc[1] != 0
// (the gradient multiplier for the update), out[1] = unscaled global norm.
__global__ void clip_coef_kernel(const float* __restrict__ acc, float max_norm, float inv_scale,
                                 float* __restrict__ out, int* __restrict__ skip) {
  const float norm = sqrtf(acc[0]) * inv_scale;
  float coef = 1.f;
  if (max_norm > 0.f) coef = fminf(1.f, max_norm / (norm + 1e-6f));
  out[0] = coef * inv_scale;
  out[1] = norm;
  if (skip != nullptr) *skip = (acc[1] != 0.f || !isfinite(norm)) ? 1 : 0;
}

}  // namespace nx

// grad_dtype: 0 = bf16, 1 = fp32.  grad_scale (device float*, nullable) multiplies every gradient;
// skip (device int*, nullable) non-zero turns the launch into a no-op.
NX_API int NX_SYM(nx_adamw_step)(void* p, void* m, void* v, const void* g, void* p_bf16, long long n,
                         float lr, float beta1, float beta2, float eps, float weight_decay,
                         float bias_corr1, float bias_corr2, int adam_w_mode,
                         const void* grad_scale, const void* skip, int grad_dtype, void* stream_) {
  using namespace nx;
  if (n == 0) return NX_OK;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, adam_w_mode};
  const long long nvec = (n + 3) / 4;
  long long g_ = (nvec + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  const int grid = static_cast<int>(g_ < cap ? g_ : cap);
  auto s = (cudaStream_t)stream_;
  if (grad_dtype == 0)
    adamw_kernel<h16><<<grid, 256, 0, s>>>((float*)p, (float*)m, (float*)v,
                                                     (const h16*)g, (h16*)p_bf16,
                                                     n, a, (const float*)grad_scale, (const int*)skip);
  else
    adamw_kernel<float><<<grid, 256, 0, s>>>((float*)p, (float*)m, (float*)v, (const float*)g,
                                             (h16*)p_bf16, n, a, (const float*)grad_scale,
                                             (const int*)skip);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
// AdamW with 8-bit block-wise state: m8 / v8 one byte per element, scale_m / scale_v one float per 2048 elements
// (ceil(n / 2048) each; all-zero state = all moments zero).  n % 8 == 0; p, g, p_lp 16-byte aligned, m8 / v8 8-byte.
NX_API int NX_SYM(nx_adamw8bit_step)(void* p, void* m8, void* v8, void* scale_m, void* scale_v, const void* g,
                                     void* p_lp, long long n, float lr, float beta1, float beta2, float eps,
                                     float weight_decay, float bias_corr1, float bias_corr2, int adam_w_mode,
                                     const void* grad_scale, const void* skip, int grad_dtype, void* stream_) {
  using namespace nx;
  if (n == 0) return NX_OK;
  NX_REQUIRE(n % 8 == 0, "adamw8bit: n (%lld) must be a multiple of 8", n);
  NX_REQUIRE(((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(p_lp)) & 15) == 0 &&
                 ((reinterpret_cast<uintptr_t>(m8) | reinterpret_cast<uintptr_t>(v8)) & 7) == 0,
             "adamw8bit: misaligned buffer");
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, adam_w_mode};
  const long long blocks = (n + Q8_BLOCK - 1) / Q8_BLOCK;
  NX_REQUIRE(blocks < (1ll << 31), "adamw8bit: too many blocks");
  auto s = (cudaStream_t)stream_;
  if (grad_dtype == 0)
    adam8_kernel<h16><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        (float*)p, (uint8_t*)m8, (uint8_t*)v8, (float*)scale_m, (float*)scale_v, (const h16*)g, (h16*)p_lp, n, a,
        (const float*)grad_scale, (const int*)skip);
  else
    adam8_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        (float*)p, (uint8_t*)m8, (uint8_t*)v8, (float*)scale_m, (float*)scale_v, (const float*)g, (h16*)p_lp, n, a,
        (const float*)grad_scale, (const int*)skip);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
NX_API int NX_SYM(nx_sumsq)(const void* x, long long n, void* acc, int dtype, void* stream_) {
  using namespace nx;
  if (n == 0) return NX_OK;
  const long long nvec = (n + 3) / 4;
  long long g_ = (nvec + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  const int grid = static_cast<int>(g_ < cap ? g_ : cap);
  auto s = (cudaStream_t)stream_;
  if (dtype == 0) sumsq_kernel<h16><<<grid, 256, 0, s>>>((const h16*)x, n, (float*)acc);
  else sumsq_kernel<float><<<grid, 256, 0, s>>>((const float*)x, n, (float*)acc);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
NX_API int NX_SYM(nx_clip_coef)(const void* acc, float max_norm, float inv_scale, void* out, void* skip,
                        void* stream_) {
  nx::clip_coef_kernel<<<1, 1, 0, (cudaStream_t)stream_>>>((const float*)acc, max_norm, inv_scale,
                                                           (float*)out, (int*)skip);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
