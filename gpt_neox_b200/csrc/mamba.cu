// Mamba-1 kernels: causal depthwise conv1d (width <= 4) + SiLU, and the S6 selective scan, forward
// and backward, on token-major activations addressed by (batch stride, time stride) so the
// [seq, batch, channel] tensors the projections produce are consumed without a transpose.
//
// Counterparts in the reference: causal_conv1d_fn and selective_scan_fn / selective_scan_ref from
// the external causal_conv1d / mamba_ssm packages, called at megatron/model/mamba/mamba.py:220-247
// and :264-320 (which run on [batch, channel, seq] and need two rearranges per block).
//
// Scan parallelisation: the sequence is cut into chunks of 128 steps; a thread owns 4 of the 16
// states of one channel (a quad of lanes per channel), 64 channels per CTA.
//   forward : pass 1 runs every chunk from a zero state and records the chunk's end state and its
//             sum of delta (the chunk's decay is exp(A * sum delta)); pass 2 folds the earlier
//             chunks into the chunk's initial state and produces the output.
//   backward: the same trick for the reverse recurrence of dL/dh, then one pass per chunk that
//             recomputes h in 16-step sub-chunks (history in registers) and walks them in reverse.
// dB and dC (sums over channels) leave the kernel as per-CTA partials and are summed by the caller.
#include "common.h"
#include "ptx.cuh"

namespace nx {

// ---------------------------------------------------------------------------------------------
// causal depthwise conv1d + SiLU
// ---------------------------------------------------------------------------------------------
constexpr int CONV_TILE = 64;   // timesteps per thread

__device__ __forceinline__ float ldbf(const h16* p) { return h16_to_float(*p); }

// y[b,t,d] = silu(bias[d] + sum_k w[d,k] * x[b, t-(W-1)+k, d])
__global__ void __launch_bounds__(128)
conv1d_silu_fwd_kernel(const h16* __restrict__ x, long long xsb, long long xst,
                       const h16* __restrict__ w, const h16* __restrict__ bias,
                       h16* __restrict__ y, long long ysb, long long yst, int L, int D, int W) {
  const int d = blockIdx.x * 128 + threadIdx.x;
  if (d >= D) return;
  const int t0 = blockIdx.y * CONV_TILE;
  const int b = blockIdx.z;
  float wk[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k = 0; k < W; ++k) wk[4 - W + k] = ldbf(w + (long long)d * W + k);
  const float bv = bias ? ldbf(bias + d) : 0.f;
  const h16* xp = x + b * xsb + d;
  float win[4];
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    const int t = t0 - 3 + k;
    win[k + 1] = t >= 0 ? ldbf(xp + t * xst) : 0.f;
  }
  const int t1 = min(t0 + CONV_TILE, L);
  for (int t = t0; t < t1; ++t) {
    win[0] = win[1]; win[1] = win[2]; win[2] = win[3];
    win[3] = ldbf(xp + t * xst);
    const float pre = bv + wk[0] * win[0] + wk[1] * win[1] + wk[2] * win[2] + wk[3] * win[3];
    y[b * ysb + t * yst + d] = float_to_h16(silu(pre));
  }
}

// dx[t] = sum_k w[k] * dpre[t + (3-k)];  dw[k] += dpre[t] * x[t-3+k];  dbias += dpre[t]
__global__ void __launch_bounds__(128)
conv1d_silu_bwd_kernel(const h16* __restrict__ x, long long xsb, long long xst,
                       const h16* __restrict__ w, const h16* __restrict__ bias,
                       const h16* __restrict__ dy, long long dsb, long long dst,
                       h16* __restrict__ dx, long long gsb, long long gst,
                       float* __restrict__ dw, float* __restrict__ dbias, int L, int D, int W) {
  const int d = blockIdx.x * 128 + threadIdx.x;
  if (d >= D) return;
  const int t0 = blockIdx.y * CONV_TILE;
  const int b = blockIdx.z;
  float wk[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k = 0; k < W; ++k) wk[4 - W + k] = ldbf(w + (long long)d * W + k);
  const float bv = bias ? ldbf(bias + d) : 0.f;
  const h16* xp = x + b * xsb + d;
  const h16* gp = dy + b * dsb + d;
  float win[4], dp[4] = {0.f, 0.f, 0.f, 0.f};
  float aw[4] = {0.f, 0.f, 0.f, 0.f}, ab = 0.f;
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    const int t = t0 - 3 + k;
    win[k + 1] = t >= 0 ? ldbf(xp + t * xst) : 0.f;
  }
  const int t_own = min(t0 + CONV_TILE, L);
  const int t_end = min(t0 + CONV_TILE + 3, L + 3);
  for (int t = t0; t < t_end; ++t) {
    win[0] = win[1]; win[1] = win[2]; win[2] = win[3];
    win[3] = t < L ? ldbf(xp + t * xst) : 0.f;
    float dpre = 0.f;
    if (t < L) {
      const float pre = bv + wk[0] * win[0] + wk[1] * win[1] + wk[2] * win[2] + wk[3] * win[3];
      dpre = ldbf(gp + t * dst) * silu_grad(pre);
    }
    if (t < t_own) {
      aw[0] += dpre * win[0]; aw[1] += dpre * win[1]; aw[2] += dpre * win[2]; aw[3] += dpre * win[3];
      ab += dpre;
    }
    dp[0] = dp[1]; dp[1] = dp[2]; dp[2] = dp[3]; dp[3] = dpre;   // dp[j] = dpre[t-3+j]
    const int to = t - 3;
    if (to >= t0 && to < t_own)
      dx[b * gsb + to * gst + d] =
          float_to_h16(wk[3] * dp[0] + wk[2] * dp[1] + wk[1] * dp[2] + wk[0] * dp[3]);
  }
  for (int k = 0; k < W; ++k) atomicAdd(dw + (long long)d * W + k, aw[4 - W + k]);
  if (dbias) atomicAdd(dbias + d, ab);
}

NX_API int NX_SYM(nx_conv1d_silu_fwd)(const void* x, long long xsb, long long xst, const void* w, const void* bias,
                              void* y, long long ysb, long long yst, int B, int L, int D, int W,
                              cudaStream_t stream) {
  NX_REQUIRE(W >= 1 && W <= 4, "conv1d: kernel width %d not in [1, 4]", W);
  dim3 grid((D + 127) / 128, (L + CONV_TILE - 1) / CONV_TILE, B);
  conv1d_silu_fwd_kernel<<<grid, 128, 0, stream>>>((const h16*)x, xsb, xst, (const h16*)w,
                                                   (const h16*)bias, (h16*)y, ysb, yst, L, D, W);
  NX_LAUNCH_CHECK();
  return NX_OK;
}

// dw [D, W] and dbias [D] are fp32 and must be zeroed by the caller.
NX_API int NX_SYM(nx_conv1d_silu_bwd)(const void* x, long long xsb, long long xst, const void* w, const void* bias,
                              const void* dy, long long dsb, long long dst, void* dx, long long gsb,
                              long long gst, void* dw, void* dbias, int B, int L, int D, int W,
                              cudaStream_t stream) {
  NX_REQUIRE(W >= 1 && W <= 4, "conv1d: kernel width %d not in [1, 4]", W);
  dim3 grid((D + 127) / 128, (L + CONV_TILE - 1) / CONV_TILE, B);
  conv1d_silu_bwd_kernel<<<grid, 128, 0, stream>>>(
      (const h16*)x, xsb, xst, (const h16*)w, (const h16*)bias,
      (const h16*)dy, dsb, dst, (h16*)dx, gsb, gst, (float*)dw, (float*)dbias, L, D, W);
  NX_LAUNCH_CHECK();
  return NX_OK;
}


// ---------------------------------------------------------------------------------------------
// selective scan
// ---------------------------------------------------------------------------------------------
constexpr int SC_CH = 64;      // channels per CTA
constexpr int SC_CHUNK = 128;  // timesteps per CTA
constexpr int SC_SUB = 16;     // timesteps staged in shared memory at a time
constexpr int SC_NSUB = SC_CHUNK / SC_SUB;
constexpr int SC_THREADS = SC_CH * 4;

struct ScanParams {
  const h16 *x, *dt, *z, *Bm, *Cm, *dout;
  long long xsb, xst, dsb, dst, zsb, zst, bsb, bst, csb, cst, gsb, gst;
  const float *A, *Dv, *dt_bias;
  h16 *out, *dx, *ddt, *dz;       // [.., D] with strides osb / ost
  long long osb, ost;
  float *chunk_state, *chunk_sumdt, *chunk_h0, *chunk_E;   // [B, NC, D, 16] / [B, NC, D]
  float *partBC;                                           // [ceil(D/64), B, L, 32]
  float *dA, *dD, *dbias;
  int B, L, D, NC;
};

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(__expf(v)); }
__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + __expf(-v)); }
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

struct ScanStage {
  float xs[SC_SUB][SC_CH], dl[SC_SUB][SC_CH], Bs[SC_SUB][16], Cs[SC_SUB][16];
};

// Stages x, delta = softplus(dt + bias), B and C of timesteps [t0, t0 + SC_SUB) (zero beyond t_end).
__device__ __forceinline__ void stage_fwd(const ScanParams& p, ScanStage& s, int b, int d0, int t0, int t_end) {
  for (int i = threadIdx.x; i < SC_SUB * SC_CH; i += SC_THREADS) {
    const int t = i / SC_CH, c = i % SC_CH, tt = t0 + t, d = d0 + c;
    float xv = 0.f, dv = 0.f;
    if (tt < t_end && d < p.D) {
      xv = ldbf(p.x + b * p.xsb + tt * p.xst + d);
      dv = softplus_f(ldbf(p.dt + b * p.dsb + tt * p.dst + d) + p.dt_bias[d]);
    }
    s.xs[t][c] = xv;
    s.dl[t][c] = dv;
  }
  for (int i = threadIdx.x; i < SC_SUB * 16; i += SC_THREADS) {
    const int t = i / 16, n = i % 16, tt = t0 + t;
    const bool ok = tt < t_end;
    s.Bs[t][n] = ok ? ldbf(p.Bm + b * p.bsb + tt * p.bst + n) : 0.f;
    s.Cs[t][n] = ok ? ldbf(p.Cm + b * p.csb + tt * p.cst + n) : 0.f;
  }
}

template <bool FINAL>
__global__ void __launch_bounds__(SC_THREADS)
scan_fwd_kernel(const ScanParams p) {
  __shared__ ScanStage s;
  __shared__ float ys[SC_SUB][SC_CH];
  const int ch = threadIdx.x >> 2, q = threadIdx.x & 3;
  const int d0 = blockIdx.x * SC_CH, d = d0 + ch;
  const int c = blockIdx.y, b = blockIdx.z;
  const bool dv_ok = d < p.D;
  const int dd = dv_ok ? d : 0;
  float A[4], h[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 4; ++j) A[j] = p.A[dd * 16 + q * 4 + j];
  const float Dv = p.Dv ? p.Dv[dd] : 0.f;
  if (FINAL) {
    for (int cp = 0; cp < c; ++cp) {
      const long long o = ((long long)b * p.NC + cp) * p.D + dd;
      const float sd = p.chunk_sumdt[o];
#pragma unroll
      for (int j = 0; j < 4; ++j) h[j] = h[j] * __expf(A[j] * sd) + p.chunk_state[o * 16 + q * 4 + j];
    }
    if (dv_ok) {
      const long long o = ((long long)b * p.NC + c) * p.D + d;
#pragma unroll
      for (int j = 0; j < 4; ++j) p.chunk_h0[o * 16 + q * 4 + j] = h[j];
    }
  }
  const int tc0 = c * SC_CHUNK, t_end = min(tc0 + SC_CHUNK, p.L);
  float sdt = 0.f;
  for (int sub = 0; sub < SC_NSUB; ++sub) {
    const int t0 = tc0 + sub * SC_SUB;
    if (t0 >= t_end) break;
    __syncthreads();
    stage_fwd(p, s, b, d0, t0, t_end);
    __syncthreads();
#pragma unroll
    for (int t = 0; t < SC_SUB; ++t) {
      const float xv = s.xs[t][ch], dl = s.dl[t][ch];
      float yp = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        h[j] = __expf(dl * A[j]) * h[j] + dl * s.Bs[t][q * 4 + j] * xv;
        yp += h[j] * s.Cs[t][q * 4 + j];
      }
      sdt += dl;
      if (FINAL) {
        yp = quad_sum(yp);
        if (q == 0) ys[t][ch] = yp + Dv * xv;
      }
    }
    if (FINAL) {
      __syncthreads();
      for (int i = threadIdx.x; i < SC_SUB * SC_CH; i += SC_THREADS) {
        const int t = i / SC_CH, cc = i % SC_CH, tt = t0 + t, dx_ = d0 + cc;
        if (tt < t_end && dx_ < p.D) {
          float y = ys[t][cc];
          if (p.z) y *= silu(ldbf(p.z + b * p.zsb + tt * p.zst + dx_));
          p.out[b * p.osb + tt * p.ost + dx_] = float_to_h16(y);
        }
      }
    }
  }
  if (!FINAL && dv_ok) {
    const long long o = ((long long)b * p.NC + c) * p.D + d;
#pragma unroll
    for (int j = 0; j < 4; ++j) p.chunk_state[o * 16 + q * 4 + j] = h[j];
    if (q == 0) p.chunk_sumdt[o] = sdt;
  }
}

struct ScanStageBwd {
  float xs[SC_SUB][SC_CH], dl[SC_SUB][SC_CH], sg[SC_SUB][SC_CH], dys[SC_SUB][SC_CH], dzf[SC_SUB][SC_CH];
  float Bs[SC_SUB][16], Cs[SC_SUB][16];
  float o_dx[SC_SUB][SC_CH], o_ddt[SC_SUB][SC_CH], o_dz[SC_SUB][SC_CH];
  float ck[SC_NSUB][4][SC_THREADS];
  float bc[SC_THREADS / 32][SC_SUB][32];
};

__device__ __forceinline__ void stage_bwd(const ScanParams& p, ScanStageBwd& s, int b, int d0, int t0, int t_end,
                                          bool light) {
  for (int i = threadIdx.x; i < SC_SUB * SC_CH; i += SC_THREADS) {
    const int t = i / SC_CH, c = i % SC_CH, tt = t0 + t, d = d0 + c;
    float xv = 0.f, dv = 0.f, sg = 0.f, dys = 0.f, dzf = 0.f;
    if (tt < t_end && d < p.D) {
      const float raw = ldbf(p.dt + b * p.dsb + tt * p.dst + d) + p.dt_bias[d];
      dv = softplus_f(raw);
      sg = raw > 20.f ? 1.f : sigmoid_f(raw);
      const float g = ldbf(p.dout + b * p.gsb + tt * p.gst + d);
      if (p.z) {
        const float zv = ldbf(p.z + b * p.zsb + tt * p.zst + d);
        dys = g * silu(zv);
        dzf = g * silu_grad(zv);
      } else {
        dys = g;
      }
      if (!light) xv = ldbf(p.x + b * p.xsb + tt * p.xst + d);
    }
    s.xs[t][c] = xv; s.dl[t][c] = dv; s.sg[t][c] = sg; s.dys[t][c] = dys; s.dzf[t][c] = dzf;
  }
  for (int i = threadIdx.x; i < SC_SUB * 16; i += SC_THREADS) {
    const int t = i / 16, n = i % 16, tt = t0 + t;
    const bool ok = tt < t_end;
    s.Bs[t][n] = ok ? ldbf(p.Bm + b * p.bsb + tt * p.bst + n) : 0.f;
    s.Cs[t][n] = ok ? ldbf(p.Cm + b * p.csb + tt * p.cst + n) : 0.f;
  }
}

// Reverse recurrence from a zero carry: E[c] = what chunk c hands to chunk c-1.
__global__ void __launch_bounds__(SC_THREADS)
scan_bwd_local_kernel(const ScanParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  ScanStageBwd& s = *reinterpret_cast<ScanStageBwd*>(smem_raw);
  const int ch = threadIdx.x >> 2, q = threadIdx.x & 3;
  const int d0 = blockIdx.x * SC_CH, d = d0 + ch;
  const int c = blockIdx.y, b = blockIdx.z;
  const bool dv_ok = d < p.D;
  const int dd = dv_ok ? d : 0;
  float A[4], r[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 4; ++j) A[j] = p.A[dd * 16 + q * 4 + j];
  const int tc0 = c * SC_CHUNK, t_end = min(tc0 + SC_CHUNK, p.L);
  for (int sub = SC_NSUB - 1; sub >= 0; --sub) {
    const int t0 = tc0 + sub * SC_SUB;
    if (t0 >= t_end) continue;
    __syncthreads();
    stage_bwd(p, s, b, d0, t0, t_end, true);
    __syncthreads();
#pragma unroll
    for (int t = SC_SUB - 1; t >= 0; --t) {
      const float dl = s.dl[t][ch], dys = s.dys[t][ch];
#pragma unroll
      for (int j = 0; j < 4; ++j) r[j] = __expf(dl * A[j]) * (s.Cs[t][q * 4 + j] * dys + r[j]);
    }
  }
  if (dv_ok) {
    const long long o = ((long long)b * p.NC + c) * p.D + d;
#pragma unroll
    for (int j = 0; j < 4; ++j) p.chunk_E[o * 16 + q * 4 + j] = r[j];
  }
}

__global__ void __launch_bounds__(SC_THREADS)
scan_bwd_final_kernel(const ScanParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  ScanStageBwd& s = *reinterpret_cast<ScanStageBwd*>(smem_raw);
  const int ch = threadIdx.x >> 2, q = threadIdx.x & 3;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int d0 = blockIdx.x * SC_CH, d = d0 + ch;
  const int c = blockIdx.y, b = blockIdx.z;
  const bool dv_ok = d < p.D;
  const int dd = dv_ok ? d : 0;
  float A[4], h[4], r[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 4; ++j) A[j] = p.A[dd * 16 + q * 4 + j];
  const float Dv = p.Dv ? p.Dv[dd] : 0.f;
  {
    const long long o = ((long long)b * p.NC + c) * p.D + dd;
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = p.chunk_h0[o * 16 + q * 4 + j];
  }
  for (int cp = p.NC - 1; cp > c; --cp) {
    const long long o = ((long long)b * p.NC + cp) * p.D + dd;
    const float sd = p.chunk_sumdt[o];
#pragma unroll
    for (int j = 0; j < 4; ++j) r[j] = p.chunk_E[o * 16 + q * 4 + j] + __expf(A[j] * sd) * r[j];
  }
  const int tc0 = c * SC_CHUNK, t_end = min(tc0 + SC_CHUNK, p.L);
  // forward over the chunk, keeping the state at the start of every sub-chunk
  for (int sub = 0; sub < SC_NSUB; ++sub) {
    const int t0 = tc0 + sub * SC_SUB;
#pragma unroll
    for (int j = 0; j < 4; ++j) s.ck[sub][j][threadIdx.x] = h[j];
    if (t0 >= t_end || sub == SC_NSUB - 1) continue;
    __syncthreads();
    for (int i = threadIdx.x; i < SC_SUB * SC_CH; i += SC_THREADS) {
      const int t = i / SC_CH, cc = i % SC_CH, tt = t0 + t, dx_ = d0 + cc;
      float xv = 0.f, dv = 0.f;
      if (tt < t_end && dx_ < p.D) {
        xv = ldbf(p.x + b * p.xsb + tt * p.xst + dx_);
        dv = softplus_f(ldbf(p.dt + b * p.dsb + tt * p.dst + dx_) + p.dt_bias[dx_]);
      }
      s.xs[t][cc] = xv; s.dl[t][cc] = dv;
    }
    for (int i = threadIdx.x; i < SC_SUB * 16; i += SC_THREADS) {
      const int t = i / 16, n = i % 16, tt = t0 + t;
      s.Bs[t][n] = tt < t_end ? ldbf(p.Bm + b * p.bsb + tt * p.bst + n) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int t = 0; t < SC_SUB; ++t) {
      const float xv = s.xs[t][ch], dl = s.dl[t][ch];
#pragma unroll
      for (int j = 0; j < 4; ++j) h[j] = __expf(dl * A[j]) * h[j] + dl * s.Bs[t][q * 4 + j] * xv;
    }
  }
  float dA[4] = {0.f, 0.f, 0.f, 0.f}, dD = 0.f, dbias = 0.f;
  const bool b2 = lane & 4, b3 = lane & 8, b4 = lane & 16;
  const int idx = (b2 ? 4 : 0) + (b3 ? 2 : 0) + (b4 ? 1 : 0);
  const int col = idx < 4 ? q * 4 + idx : 16 + q * 4 + (idx - 4);
  for (int sub = SC_NSUB - 1; sub >= 0; --sub) {
    const int t0 = tc0 + sub * SC_SUB;
    if (t0 >= t_end) continue;
    __syncthreads();
    stage_bwd(p, s, b, d0, t0, t_end, false);
    __syncthreads();
    float hist[SC_SUB][4];
    float h0[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) h0[j] = s.ck[sub][j][threadIdx.x];
#pragma unroll
    for (int t = 0; t < SC_SUB; ++t) {
      const float xv = s.xs[t][ch], dl = s.dl[t][ch];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        hist[t][j] = __expf(dl * A[j]) * (t == 0 ? h0[j] : hist[t - 1][j]) + dl * s.Bs[t][q * 4 + j] * xv;
    }
#pragma unroll
    for (int t = SC_SUB - 1; t >= 0; --t) {
      const float xv = s.xs[t][ch], dl = s.dl[t][ch], dys = s.dys[t][ch];
      float ddl = 0.f, dxp = 0.f, yp = 0.f, v[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float Bv = s.Bs[t][q * 4 + j], Cv = s.Cs[t][q * 4 + j];
        const float a = __expf(dl * A[j]);
        const float g = Cv * dys + r[j];
        const float hp = t == 0 ? h0[j] : hist[t - 1][j];
        const float da = g * hp * a;
        ddl += da * A[j] + g * Bv * xv;
        dA[j] += da * dl;
        dxp += g * dl * Bv;
        yp += hist[t][j] * Cv;
        v[j] = g * dl * xv;            // dB
        v[4 + j] = dys * hist[t][j];   // dC
        r[j] = a * g;
      }
      ddl = quad_sum(ddl); dxp = quad_sum(dxp); yp = quad_sum(yp);
      if (q == 0) {
        const float ddt_raw = ddl * s.sg[t][ch];
        s.o_dx[t][ch] = dxp + Dv * dys;
        s.o_ddt[t][ch] = ddt_raw;
        s.o_dz[t][ch] = s.dzf[t][ch] * (yp + Dv * xv);
        dD += dys * xv;
        dbias += ddt_raw;
      }
      // sum dB / dC over the 8 channels of the warp, halving the value set at every exchange
      float w4[4], w2[2], w1;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float send = b2 ? v[j] : v[4 + j], keep = b2 ? v[4 + j] : v[j];
        w4[j] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float send = b3 ? w4[j] : w4[2 + j], keep = b3 ? w4[2 + j] : w4[j];
        w2[j] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
      }
      {
        const float send = b4 ? w2[0] : w2[1], keep = b4 ? w2[1] : w2[0];
        w1 = keep + __shfl_xor_sync(0xffffffffu, send, 16);
      }
      s.bc[warp][t][col] = w1;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < SC_SUB * SC_CH; i += SC_THREADS) {
      const int t = i / SC_CH, cc = i % SC_CH, tt = t0 + t, dx_ = d0 + cc;
      if (tt < t_end && dx_ < p.D) {
        const long long o = b * p.osb + tt * p.ost + dx_;
        p.dx[o] = float_to_h16(s.o_dx[t][cc]);
        p.ddt[o] = float_to_h16(s.o_ddt[t][cc]);
        if (p.dz) p.dz[o] = float_to_h16(s.o_dz[t][cc]);
      }
    }
    for (int i = threadIdx.x; i < SC_SUB * 32; i += SC_THREADS) {
      const int t = i / 32, cl = i % 32, tt = t0 + t;
      if (tt < t_end) {
        float acc = 0.f;
#pragma unroll
        for (int wv = 0; wv < SC_THREADS / 32; ++wv) acc += s.bc[wv][t][cl];
        p.partBC[(((long long)blockIdx.x * p.B + b) * p.L + tt) * 32 + cl] = acc;
      }
    }
  }
  if (dv_ok) {
#pragma unroll
    for (int j = 0; j < 4; ++j) atomicAdd(p.dA + d * 16 + q * 4 + j, dA[j]);
    if (q == 0) {
      if (p.dD) atomicAdd(p.dD + d, dD);
      atomicAdd(p.dbias + d, dbias);
    }
  }
}

NX_API int NX_SYM(nx_scan_chunks)(int L) { return (L + SC_CHUNK - 1) / SC_CHUNK; }
NX_API int NX_SYM(nx_scan_channel_blocks)(int D) { return (D + SC_CH - 1) / SC_CH; }

// A [D,16] fp32 (negative), Dv [D] fp32 or null, dt_bias [D] fp32; x/dt/z/out bf16 addressed by
// (batch stride, time stride); Bm/Cm bf16 [.., 16]. Scratch (fp32): chunk_state / chunk_h0
// [B, NC, D, 16], chunk_sumdt [B, NC, D].
NX_API int NX_SYM(nx_selective_scan_fwd)(const void* x, long long xsb, long long xst, const void* dt, long long dsb,
                                 long long dst, const void* z, long long zsb, long long zst, const void* Bm,
                                 long long bsb, long long bst, const void* Cm, long long csb, long long cst,
                                 const void* A, const void* Dv, const void* dt_bias, void* out, long long osb,
                                 long long ost, void* chunk_state, void* chunk_sumdt, void* chunk_h0, int B,
                                 int L, int D, cudaStream_t stream) {
  ScanParams p{};
  p.x = (const h16*)x; p.xsb = xsb; p.xst = xst;
  p.dt = (const h16*)dt; p.dsb = dsb; p.dst = dst;
  p.z = (const h16*)z; p.zsb = zsb; p.zst = zst;
  p.Bm = (const h16*)Bm; p.bsb = bsb; p.bst = bst;
  p.Cm = (const h16*)Cm; p.csb = csb; p.cst = cst;
  p.A = (const float*)A; p.Dv = (const float*)Dv; p.dt_bias = (const float*)dt_bias;
  p.out = (h16*)out; p.osb = osb; p.ost = ost;
  p.chunk_state = (float*)chunk_state; p.chunk_sumdt = (float*)chunk_sumdt; p.chunk_h0 = (float*)chunk_h0;
  p.B = B; p.L = L; p.D = D; p.NC = (L + SC_CHUNK - 1) / SC_CHUNK;
  dim3 grid((D + SC_CH - 1) / SC_CH, p.NC, B);
  if (p.NC > 1) {
    scan_fwd_kernel<false><<<grid, SC_THREADS, 0, stream>>>(p);
    NX_LAUNCH_CHECK();
  }
  scan_fwd_kernel<true><<<grid, SC_THREADS, 0, stream>>>(p);
  NX_LAUNCH_CHECK();
  return NX_OK;
}

// dx / ddt / dz: bf16 with strides (osb, ost). partBC fp32 [ceil(D/64), B, L, 32] (written fully);
// dA [D,16], dD [D], dbias [D] fp32, zeroed by the caller. chunk_* from the forward; chunk_E scratch.
NX_API int NX_SYM(nx_selective_scan_bwd)(const void* x, long long xsb, long long xst, const void* dt, long long dsb,
                                 long long dst, const void* z, long long zsb, long long zst, const void* Bm,
                                 long long bsb, long long bst, const void* Cm, long long csb, long long cst,
                                 const void* A, const void* Dv, const void* dt_bias, const void* dout,
                                 long long gsb, long long gst, void* dx, void* ddt, void* dz, long long osb,
                                 long long ost, void* partBC, void* dA, void* dD, void* dbias,
                                 void* chunk_sumdt, void* chunk_h0, void* chunk_E, int B, int L, int D,
                                 cudaStream_t stream) {
  ScanParams p{};
  p.x = (const h16*)x; p.xsb = xsb; p.xst = xst;
  p.dt = (const h16*)dt; p.dsb = dsb; p.dst = dst;
  p.z = (const h16*)z; p.zsb = zsb; p.zst = zst;
  p.Bm = (const h16*)Bm; p.bsb = bsb; p.bst = bst;
  p.Cm = (const h16*)Cm; p.csb = csb; p.cst = cst;
  p.dout = (const h16*)dout; p.gsb = gsb; p.gst = gst;
  p.A = (const float*)A; p.Dv = (const float*)Dv; p.dt_bias = (const float*)dt_bias;
  p.dx = (h16*)dx; p.ddt = (h16*)ddt; p.dz = (h16*)dz; p.osb = osb; p.ost = ost;
  p.partBC = (float*)partBC; p.dA = (float*)dA; p.dD = (float*)dD; p.dbias = (float*)dbias;
  p.chunk_sumdt = (float*)chunk_sumdt; p.chunk_h0 = (float*)chunk_h0; p.chunk_E = (float*)chunk_E;
  p.B = B; p.L = L; p.D = D; p.NC = (L + SC_CHUNK - 1) / SC_CHUNK;
  dim3 grid((D + SC_CH - 1) / SC_CH, p.NC, B);
  const int smem = (int)sizeof(ScanStageBwd);
  static bool attr_set = false;
  if (!attr_set) {
    NX_CUDA_CHECK(cudaFuncSetAttribute(scan_bwd_local_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    NX_CUDA_CHECK(cudaFuncSetAttribute(scan_bwd_final_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set = true;
  }
  if (p.NC > 1) {
    scan_bwd_local_kernel<<<grid, SC_THREADS, smem, stream>>>(p);
    NX_LAUNCH_CHECK();
  }
  scan_bwd_final_kernel<<<grid, SC_THREADS, smem, stream>>>(p);
  NX_LAUNCH_CHECK();
  return NX_OK;
}

}  // namespace nx
