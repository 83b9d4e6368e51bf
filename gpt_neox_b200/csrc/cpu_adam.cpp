// AdamW on the host for optimizer-state offload ("type": "CPUAdam" / ZeRO offload_optimizer in the reference,
// which takes DeepSpeedCPUAdam from DeepSpeed's native ops, megatron/training.py:1002-1012).
//
// The fp32 master weights and both moments live in pinned host memory; each step the device sends its gradient
// shard down, this routine updates the shard with all host cores, and writes the 16-bit (bf16 or fp16) copy of
// the new weights that travels back up.  Vector code comes from the compiler: the inner loop is a straight-line
// `omp simd` body, built once per instruction set (AVX-512 / AVX2 / baseline) with the choice made at load time,
// so the library built on one host runs on another.
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <thread>
#include <vector>

namespace {

inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);   // NaN stays NaN
  u += 0x7fffu + ((u >> 16) & 1u);                                                          // round to nearest even
  return static_cast<uint16_t>(u >> 16);
}
inline float bf16_to_f32(uint16_t h) {
  const uint32_t u = static_cast<uint32_t>(h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f32_to_f16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  x &= 0x7fffffffu;
  if (x >= 0x7f800000u) return static_cast<uint16_t>(sign | 0x7c00u | (x > 0x7f800000u ? 0x200u : 0u));
  if (x >= 0x477ff000u) return static_cast<uint16_t>(sign | 0x7c00u);                      // overflow -> inf
  if (x < 0x33000001u) return static_cast<uint16_t>(sign);                                  // underflow -> 0
  if (x < 0x38800000u) {                                                                    // subnormal half
    const int shift = 126 - static_cast<int>(x >> 23);
    uint32_t mant = (x & 0x7fffffu) | 0x800000u;
    const uint32_t rest = mant & ((1u << shift) - 1u), half = 1u << (shift - 1);
    mant >>= shift;
    if (rest > half || (rest == half && (mant & 1u))) ++mant;
    return static_cast<uint16_t>(sign | mant);
  }
  uint32_t r = x - 0x38000000u;                                                             // rebias the exponent
  r += 0xfffu + ((r >> 13) & 1u);
  return static_cast<uint16_t>(sign | (r >> 13));
}
inline float f16_to_f32(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 31u, m = h & 1023u, u;
  if (e == 0) {
    if (m == 0) {
      u = sign;
    } else {
      e = 113;
      while (!(m & 1024u)) { m <<= 1; --e; }
      u = sign | (e << 23) | ((m & 1023u) << 13);
    }
  } else if (e == 31) {
    u = sign | 0x7f800000u | (m << 13);
  } else {
    u = sign | ((e + 112u) << 23) | (m << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

struct Args {
  float *p, *m, *v;
  const void* g;
  uint16_t* lp;
  int g_kind, lp_kind;     // 0 = bf16, 1 = fp32 (gradient only), 2 = fp16
  float lr, b1, b2, eps, wd, step, inv_bc2_sqrt, gscale;
  int adamw;
};

__attribute__((target_clones("avx512f", "avx2", "default"))) void adam_range(const Args& a, long long lo, long long hi) {
  constexpr long long T = 1024;
  float gbuf[T];
  for (long long t0 = lo; t0 < hi; t0 += T) {
    const long long n = std::min(T, hi - t0);
    if (a.g_kind == 1) {
      const float* g = static_cast<const float*>(a.g) + t0;
      for (long long i = 0; i < n; ++i) gbuf[i] = g[i] * a.gscale;
    } else {
      const uint16_t* g = static_cast<const uint16_t*>(a.g) + t0;
      if (a.g_kind == 0) for (long long i = 0; i < n; ++i) gbuf[i] = bf16_to_f32(g[i]) * a.gscale;
      else for (long long i = 0; i < n; ++i) gbuf[i] = f16_to_f32(g[i]) * a.gscale;
    }
    float* __restrict__ p = a.p + t0;
    float* __restrict__ m = a.m + t0;
    float* __restrict__ v = a.v + t0;
#pragma omp simd
    for (long long i = 0; i < n; ++i) {
      float g = gbuf[i];
      float pi = p[i];
      if (!a.adamw) g += a.wd * pi;
      const float mi = a.b1 * m[i] + (1.f - a.b1) * g;
      const float vi = a.b2 * v[i] + (1.f - a.b2) * g * g;
      const float denom = sqrtf(vi) * a.inv_bc2_sqrt + a.eps;
      if (a.adamw) pi -= a.lr * a.wd * pi;
      pi -= a.step * (mi / denom);
      p[i] = pi; m[i] = mi; v[i] = vi;
    }
    if (a.lp != nullptr) {
      uint16_t* lp = a.lp + t0;
      if (a.lp_kind == 2) for (long long i = 0; i < n; ++i) lp[i] = f32_to_f16(p[i]);
      else for (long long i = 0; i < n; ++i) lp[i] = f32_to_bf16(p[i]);
    }
  }
}

}  // namespace

// p / m / v: fp32 [n] on the host, updated in place.  g: gradients (g_kind 0 = bf16, 1 = fp32, 2 = fp16), multiplied
// by grad_scale.  lp (nullable): receives the new weights in 16 bits (lp_kind 0 = bf16, 2 = fp16).
// threads <= 0: one per hardware thread, at most 64.  Returns 0.
extern "C" __attribute__((visibility("default"))) int nx_cpu_adamw(
    float* p, float* m, float* v, const void* g, int g_kind, uint16_t* lp, int lp_kind, long long n, float lr,
    float beta1, float beta2, float eps, float weight_decay, float bias_corr1, float bias_corr2, int adam_w_mode,
    float grad_scale, int threads) {
  if (n <= 0) return 0;
  Args a{p, m, v, g, lp, g_kind, lp_kind, lr, beta1, beta2, eps, weight_decay, lr / bias_corr1,
         1.f / sqrtf(bias_corr2), grad_scale, adam_w_mode};
  int nt = threads > 0 ? threads : static_cast<int>(std::thread::hardware_concurrency());
  nt = std::max(1, std::min(nt, 64));
  const long long per = ((n + nt - 1) / nt + 1023) / 1024 * 1024;      // whole 1024-element tiles per thread
  if (nt == 1 || n <= 65536) {
    adam_range(a, 0, n);
    return 0;
  }
  std::vector<std::thread> pool;
  for (int t = 0; t < nt; ++t) {
    const long long lo = t * per, hi = std::min(n, lo + per);
    if (lo >= hi) break;
    pool.emplace_back([&a, lo, hi] { adam_range(a, lo, hi); });
  }
  for (auto& th : pool) th.join();
  return 0;
}
