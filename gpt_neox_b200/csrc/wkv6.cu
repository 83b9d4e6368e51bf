// RWKV-6 WKV recurrence, forward and backward, with no compile-time sequence length.
//
//   y_t[j]   = sum_i r_t[i] * (u[i] * k_t[i] * v_t[j] + S_{t-1}[i][j])
//   S_t[i][j] = d_t[i] * S_{t-1}[i][j] + k_t[i] * v_t[j],      d_t[i] = exp(-exp(w_t[i]))
//
// Counterpart in the reference: megatron/model/rwkv/v6/cuda/wkv6_cuda.cu:6-241 (kernel_forward,
// kernel_backward_111 / _222), which walks the whole sequence in one thread per channel and needs
// the sequence length as a compile-time constant for a per-thread array.
//
// Here the sequence is cut into chunks of 128 steps that run in parallel.  The recurrence is linear
// in the state, so a chunk's end state is  P (.) S_start + S_local  with P[i] = prod_t d_t[i]:
//   wkv_local : every chunk from a zero state -> S_local and sum_t(-exp(w_t)) per chunk
//   wkv_fold  : sequential over the (few) chunks -> the state at the start of every chunk
//   wkv_sweep : every chunk from its true start state -> outputs
// The same three kernels run time-reversed for the gradient state G (dL/dS).  Two thread mappings:
// "column" (a thread owns S[:, j], output indexed by j: y and gv) and "row" (a thread owns S[i, :],
// output indexed by i: gr and gk).  The decay gradient needs no kernel of its own: with
// Q_t[i] = sum_j G_t[i][j] S_t[i][j] one has Q_{t-1} - Q_t = r_t gr_t - k_t gk_t, so it follows from
// gr and gk by a reverse cumulative sum (done by the caller).
#include "common.h"
#include "ptx.cuh"

namespace nx {

constexpr int WK_CHUNK = 128;
constexpr int WK_SUB = 16;

struct WkvParams {
  // "a/b/c" roles: column sweep out[j] = sum_i a[i] (u[i] b[i] c[j] + S[i][j]),  S += b[i] c[j]
  //                row sweep    out[i] = sum_j a[j] (u[i] b[i] c[j] + S[i][j]),  S += b[i] c[j]
  const h16 *a, *b, *c, *w;
  long long sb, st;                 // batch / time strides (elements) shared by a, b, c, w
  const float* u;                   // [H, N]
  void* out;                        // [B, T, C] contiguous in (osb, ost); bf16 or fp32
  long long osb, ost;
  int out_f32;
  float* local;                     // [B, H, NC, N, N] chunk-local end states
  float* start;                     // [B, H, NC, N, N] chunk start states
  float* sumew;                     // [B, H, NC, N]
  int B, T, H, NC;
};

__device__ __forceinline__ float ldb(const h16* p) { return h16_to_float(*p); }

template <int N>
struct WkvStage {
  float a[WK_SUB][N], b[WK_SUB][N], c[WK_SUB][N], d[WK_SUB][N], ew[WK_SUB][N];
};

template <int N>
__device__ __forceinline__ void wkv_stage(const WkvParams& p, WkvStage<N>& s, int bi, int h, int t0, int t_lo,
                                          int t_hi, bool need_a) {
  for (int i = threadIdx.x; i < WK_SUB * N; i += N) {
    const int t = i / N, n = i % N, tt = t0 + t;
    float av = 0.f, bv = 0.f, cv = 0.f, ew = 0.f;
    if (tt >= t_lo && tt < t_hi) {
      const long long o = bi * p.sb + tt * p.st + h * N + n;
      if (need_a) av = ldb(p.a + o);
      bv = ldb(p.b + o);
      cv = ldb(p.c + o);
      ew = -__expf(ldb(p.w + o));
    }
    s.a[t][n] = av; s.b[t][n] = bv; s.c[t][n] = cv; s.ew[t][n] = ew; s.d[t][n] = __expf(ew);
  }
}

// Chunk-local end state from zero (column mapping) and the chunk's sum of ew.
template <int N, bool REV>
__global__ void __launch_bounds__(N) wkv_local_kernel(const WkvParams p) {
  __shared__ WkvStage<N> s;
  const int j = threadIdx.x, c = blockIdx.x, h = blockIdx.y, bi = blockIdx.z;
  const int t_lo = c * WK_CHUNK, t_hi = min(t_lo + WK_CHUNK, p.T);
  float S[N];
#pragma unroll
  for (int i = 0; i < N; ++i) S[i] = 0.f;
  float sew = 0.f;
  const int nsub = (t_hi - t_lo + WK_SUB - 1) / WK_SUB;
  for (int q = 0; q < nsub; ++q) {
    const int sub = REV ? nsub - 1 - q : q;
    const int t0 = t_lo + sub * WK_SUB;
    __syncthreads();
    wkv_stage<N>(p, s, bi, h, t0, t_lo, t_hi, false);
    __syncthreads();
#pragma unroll 1
    for (int tq = 0; tq < WK_SUB; ++tq) {
      const int t = REV ? WK_SUB - 1 - tq : tq;
      if (t0 + t >= t_hi) continue;
      const float cj = s.c[t][j];
      sew += s.ew[t][j];
#pragma unroll
      for (int i = 0; i < N; ++i) S[i] = S[i] * s.d[t][i] + s.b[t][i] * cj;
    }
  }
  const long long base = (((long long)bi * p.H + h) * p.NC + c);
#pragma unroll
  for (int i = 0; i < N; ++i) p.local[(base * N + i) * N + j] = S[i];
  p.sumew[base * N + j] = sew;
}

// start[c] for every chunk: forward  start[0] = 0, start[c+1] = P_c start[c] + local[c];
//                           reverse  start[NC-1] = 0, start[c-1] = P_c start[c] + local[c].
template <int N, bool REV>
__global__ void __launch_bounds__(N) wkv_fold_kernel(const WkvParams p) {
  const int j = threadIdx.x, h = blockIdx.y, bi = blockIdx.z;
  float S[N];
#pragma unroll
  for (int i = 0; i < N; ++i) S[i] = 0.f;
  for (int q = 0; q < p.NC; ++q) {
    const int c = REV ? p.NC - 1 - q : q;
    const long long base = (((long long)bi * p.H + h) * p.NC + c);
#pragma unroll
    for (int i = 0; i < N; ++i) {
      p.start[(base * N + i) * N + j] = S[i];
      S[i] = S[i] * __expf(p.sumew[base * N + i]) + p.local[(base * N + i) * N + j];
    }
  }
}

template <int N>
__device__ __forceinline__ void wkv_store(const WkvParams& p, long long o, float v) {
  if (p.out_f32) reinterpret_cast<float*>(p.out)[o] = v;
  else reinterpret_cast<h16*>(p.out)[o] = float_to_h16(v);
}

// ROW = false: thread j owns S[:, j]; ROW = true: thread i owns S[i, :].
template <int N, bool REV, bool ROW>
__global__ void __launch_bounds__(N) wkv_sweep_kernel(const WkvParams p) {
  __shared__ WkvStage<N> s;
  __shared__ float us[N];
  const int me = threadIdx.x, c = blockIdx.x, h = blockIdx.y, bi = blockIdx.z;
  const int t_lo = c * WK_CHUNK, t_hi = min(t_lo + WK_CHUNK, p.T);
  us[me] = p.u[h * N + me];
  float S[N];
  const long long base = (((long long)bi * p.H + h) * p.NC + c);
#pragma unroll
  for (int x = 0; x < N; ++x) S[x] = ROW ? p.start[(base * N + me) * N + x] : p.start[(base * N + x) * N + me];
  const int nsub = (t_hi - t_lo + WK_SUB - 1) / WK_SUB;
  for (int q = 0; q < nsub; ++q) {
    const int sub = REV ? nsub - 1 - q : q;
    const int t0 = t_lo + sub * WK_SUB;
    __syncthreads();
    wkv_stage<N>(p, s, bi, h, t0, t_lo, t_hi, true);
    __syncthreads();
#pragma unroll 1
    for (int tq = 0; tq < WK_SUB; ++tq) {
      const int t = REV ? WK_SUB - 1 - tq : tq;
      if (t0 + t >= t_hi) continue;
      float acc = 0.f;
      if (!ROW) {
        const float cj = s.c[t][me];
#pragma unroll
        for (int i = 0; i < N; ++i) {
          const float x = s.b[t][i] * cj;
          acc += s.a[t][i] * (us[i] * x + S[i]);
          S[i] = S[i] * s.d[t][i] + x;
        }
      } else {
        const float bi_ = s.b[t][me], di = s.d[t][me], ui = us[me];
#pragma unroll
        for (int jx = 0; jx < N; ++jx) {
          const float x = bi_ * s.c[t][jx];
          acc += s.a[t][jx] * (ui * x + S[jx]);
          S[jx] = S[jx] * di + x;
        }
      }
      wkv_store<N>(p, bi * p.osb + (long long)(t0 + t) * p.ost + h * N + me, acc);
    }
  }
}

template <int N>
static int wkv_run(const WkvParams& p, int mode, cudaStream_t stream) {
  dim3 grid(p.NC, p.H, p.B), gridf(1, p.H, p.B);
  switch (mode) {
    case 0: wkv_local_kernel<N, false><<<grid, N, 0, stream>>>(p); break;
    case 1: wkv_local_kernel<N, true><<<grid, N, 0, stream>>>(p); break;
    case 2: wkv_fold_kernel<N, false><<<gridf, N, 0, stream>>>(p); break;
    case 3: wkv_fold_kernel<N, true><<<gridf, N, 0, stream>>>(p); break;
    case 4: wkv_sweep_kernel<N, false, false><<<grid, N, 0, stream>>>(p); break;   // forward, column (y)
    case 5: wkv_sweep_kernel<N, true, false><<<grid, N, 0, stream>>>(p); break;    // reverse, column (gv)
    case 6: wkv_sweep_kernel<N, false, true><<<grid, N, 0, stream>>>(p); break;    // forward, row (gr)
    case 7: wkv_sweep_kernel<N, true, true><<<grid, N, 0, stream>>>(p); break;     // reverse, row (gk)
    default: return NX_ERR_ARG;
  }
  NX_LAUNCH_CHECK();
  return NX_OK;
}

NX_API int NX_SYM(nx_wkv6_chunks)(int T) { return (T + WK_CHUNK - 1) / WK_CHUNK; }

// mode: 0/1 local state fwd/rev, 2/3 fold fwd/rev, 4 y, 5 gv, 6 gr, 7 gk (see wkv_run).
// a, b, c, w: bf16 [B, T, H*N] addressed by (sb, st); u fp32 [H, N]; out bf16 or fp32 by (osb, ost).
// local / start: fp32 [B, H, NC, N, N]; sumew fp32 [B, H, NC, N].
NX_API int NX_SYM(nx_wkv6_pass)(int mode, const void* a, const void* b, const void* c, const void* w, long long sb,
                        long long st, const void* u, void* out, long long osb, long long ost, int out_f32,
                        void* local, void* start, void* sumew, int B, int T, int H, int N, cudaStream_t stream) {
  NX_REQUIRE(N == 64 || N == 32, "wkv6: head size %d not supported (32 or 64)", N);
  WkvParams p{};
  p.a = (const h16*)a; p.b = (const h16*)b; p.c = (const h16*)c;
  p.w = (const h16*)w; p.sb = sb; p.st = st; p.u = (const float*)u;
  p.out = out; p.osb = osb; p.ost = ost; p.out_f32 = out_f32;
  p.local = (float*)local; p.start = (float*)start; p.sumew = (float*)sumew;
  p.B = B; p.T = T; p.H = H; p.NC = (T + WK_CHUNK - 1) / WK_CHUNK;
  return N == 64 ? wkv_run<64>(p, mode, stream) : wkv_run<32>(p, mode, stream);
}

}  // namespace nx
