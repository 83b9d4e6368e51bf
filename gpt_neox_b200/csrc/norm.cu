// LayerNorm / RMSNorm forward and backward (bf16 in/out, fp32 statistics).
//
// Replaces apex's FusedLayerNorm / FusedRMSNorm used by the reference
// (megatron/model/fused_layer_norm.py:34-262) and the unfused modules in
// megatron/model/norms.py:62-99.  Two fusions the reference does not have:
//   * "dual" forward: the GPT-J parallel-residual block applies two different norms to the
//     same input (megatron/model/transformer.py:1083); both outputs are produced from one
//     read of x and one set of statistics.
//   * backward takes both upstream gradients of a dual norm and an incoming residual-stream
//     gradient (dx = dx_in + ...): the sum of the residual path and the two norm paths is one
//     pass over x, dy1, dy2, dx_in.
// Memory-bound: one block per row in forward, persistent blocks in backward (row-strided) so
// that dgamma / dbeta accumulate in registers and are reduced across blocks by a second tiny
// kernel through a caller-provided fp32 workspace [blocks, 2 or 4, H].
#include <algorithm>
#include <cstdint>
#include <cstdlib>

#include "common.h"
#include "ptx.cuh"
#include "reduce.cuh"

namespace nx {

constexpr int MAXV = 4;  // 16-byte vectors cached per thread

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const float2 a = unpack_h16x2(u.x), b = unpack_h16x2(u.y), c = unpack_h16x2(u.z),
               d = unpack_h16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_h16x2(f[0], f[1]);
  u.y = pack_h16x2(f[2], f[3]);
  u.z = pack_h16x2(f[4], f[5]);
  u.w = pack_h16x2(f[6], f[7]);
  return u;
}

template <bool RMS>
__global__ void norm_fwd_kernel(const h16* __restrict__ x,
                                const h16* __restrict__ g1,
                                const h16* __restrict__ b1, h16* __restrict__ y1,
                                const h16* __restrict__ g2,
                                const h16* __restrict__ b2, h16* __restrict__ y2,
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

// Backward of one norm (DUAL = false) or of two norms of the same input (DUAL = true: the upstream
// gradients dy1 / dy2 meet in one dx, from one read of x and one pair of row reductions, because
// dx is linear in w = dy1 * gamma1 + dy2 * gamma2).  Persistent blocks stride over the rows; a thread
// owns VPT 16-byte column groups and keeps their dgamma / dbeta partial sums in registers (gamma is
// re-read per row: it stays in L1).  VPT = 1 (64 registers, up to 1024 threads: two resident blocks per SM
// up to H = 4096, one up to 8192) is the fast form; wider rows take 4 or 8 groups per thread.
template <bool RMS, int VPT, bool DUAL>
__global__ void __launch_bounds__(VPT == 1 ? 1024 : 512, 1)
norm_bwd_kernel(const h16* __restrict__ dy1, const h16* __restrict__ dy2,
                const h16* __restrict__ x, const float* __restrict__ mean_in,
                const float* __restrict__ rstd_in, const h16* __restrict__ gamma1,
                const h16* __restrict__ gamma2, const h16* __restrict__ dx_in,
                h16* __restrict__ dx, float* __restrict__ ws, long long rows, int H) {
  __shared__ float sh[64];
  constexpr int NOUT = DUAL ? 4 : 2;
  const int nv = H >> 3;
  float dg1[VPT][8], db1[VPT][8], dg2[DUAL ? VPT : 1][8], db2[DUAL ? VPT : 1][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dg1[i][j] = db1[i][j] = 0.f;
      if (DUAL) dg2[i][j] = db2[i][j] = 0.f;
    }
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mean = RMS ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float xh[VPT][8], w[VPT][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      if (idx < nv) {
        const uint4 xu = reinterpret_cast<const uint4*>(x + row * H)[idx];
        const uint4 du = reinterpret_cast<const uint4*>(dy1 + row * H)[idx];
        uint4 eu = make_uint4(0u, 0u, 0u, 0u);
        if (DUAL) eu = reinterpret_cast<const uint4*>(dy2 + row * H)[idx];
        float xv[8], dv[8], g[8];
        unpack8(xu, xv);
        unpack8(du, dv);
        unpack8(reinterpret_cast<const uint4*>(gamma1)[idx], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xv[j] - mean) * rstd;
          w[i][j] = dv[j] * g[j];
          dg1[i][j] += dv[j] * xh[i][j];
          db1[i][j] += dv[j];
        }
        if (DUAL) {
          unpack8(eu, dv);
          unpack8(reinterpret_cast<const uint4*>(gamma2)[idx], g);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            w[i][j] += dv[j] * g[j];
            dg2[i][j] += dv[j] * xh[i][j];
            db2[i][j] += dv[j];
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s1 += w[i][j] * xh[i][j];
          s2 += w[i][j];
        }
      }
    }
    const float2 r = block_sum2(s1, s2, sh);
    const float c1 = r.x / H, c2 = RMS ? 0.f : r.y / H;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      if (idx < nv) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (w[i][j] - c2 - xh[i][j] * c1);
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
  float* wg = ws + static_cast<long long>(blockIdx.x) * NOUT * H;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nv) {
      float4* p = reinterpret_cast<float4*>(wg + idx * 8);
      p[0] = make_float4(dg1[i][0], dg1[i][1], dg1[i][2], dg1[i][3]);
      p[1] = make_float4(dg1[i][4], dg1[i][5], dg1[i][6], dg1[i][7]);
      p = reinterpret_cast<float4*>(wg + H + idx * 8);
      p[0] = make_float4(db1[i][0], db1[i][1], db1[i][2], db1[i][3]);
      p[1] = make_float4(db1[i][4], db1[i][5], db1[i][6], db1[i][7]);
      if (DUAL) {
        p = reinterpret_cast<float4*>(wg + 2 * H + idx * 8);
        p[0] = make_float4(dg2[i][0], dg2[i][1], dg2[i][2], dg2[i][3]);
        p[1] = make_float4(dg2[i][4], dg2[i][5], dg2[i][6], dg2[i][7]);
        p = reinterpret_cast<float4*>(wg + 3 * H + idx * 8);
        p[0] = make_float4(db2[i][0], db2[i][1], db2[i][2], db2[i][3]);
        p[1] = make_float4(db2[i][4], db2[i][5], db2[i][6], db2[i][7]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Ring variants: persistent blocks whose rows arrive through a ring of shared-memory stages filled by bulk
// asynchronous copies (cp.async.bulk, completion on an mbarrier).  The bytes in flight per SM are then set by
// the ring (up to ~200 KB), not by how many 16-byte loads the resident threads can hold in registers, and
// the loads of the next rows run during the row reductions and the stores of the current one.  One thread
// refills a stage as soon as every thread has taken its part of the row into registers (the barrier inside
// the first block reduction).  Rows up to 8192 elements; wider rows use the kernels above.
// ---------------------------------------------------------------------------------------------
constexpr int RING_MAX_STAGES = 8;

// After a wait on the ring ran out: give the copies that may still be in flight a bounded time to land before the
// block (and its shared memory) goes away.  Stage s was last filled for iteration i_s = first i >= it with i % nst == s.
__device__ __forceinline__ void ring_drain(uint32_t bar0, int nst, int it, long long row, long long rows) {
  if (threadIdx.x != 0) return;
  for (int k = 0; k < nst; ++k) {
    const int i = it + k;
    if (row + static_cast<long long>(k) * gridDim.x >= rows) break;
    for (int spin = 0; spin < 4096 && !mbar_try_wait(bar0 + 8 * (i % nst), (i / nst) & 1); ++spin) __nanosleep(64);
  }
}

template <bool RMS>
__global__ void norm_fwd_ring_kernel(const h16* __restrict__ x, const h16* __restrict__ g1,
                                     const h16* __restrict__ b1, h16* __restrict__ y1,
                                     const h16* __restrict__ g2, const h16* __restrict__ b2,
                                     h16* __restrict__ y2, float* __restrict__ mean_out,
                                     float* __restrict__ rstd_out, long long rows, int H, float eps, int nst,
                                     int* err) {
  extern __shared__ __align__(128) unsigned char ring[];
  __shared__ float sh[64];
  __shared__ __align__(8) unsigned long long bars[RING_MAX_STAGES];
  const int nv = H >> 3;
  const uint32_t row_bytes = static_cast<uint32_t>(H) * 2u;
  const uint32_t ring0 = smem_u32(ring), bar0 = smem_u32(bars);
  if (threadIdx.x == 0) {
    for (int s = 0; s < nst; ++s) mbar_init(bar0 + 8 * s, 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int s = 0; s < nst; ++s) {
      const long long r = blockIdx.x + static_cast<long long>(s) * gridDim.x;
      if (r < rows) {
        mbar_expect_tx(bar0 + 8 * s, row_bytes);
        bulk_load_1d(ring0 + s * row_bytes, x + r * H, row_bytes, bar0 + 8 * s);
      }
    }
  }
  int it = 0;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x, ++it) {
    const int st = it % nst;
    const bool ok = mbar_wait(bar0 + 8 * st, (it / nst) & 1, err, 60);
    if (!__syncthreads_and(ok ? 1 : 0)) {
      ring_drain(bar0, nst, it, row, rows);
      break;
    }
    const uint4* xr = reinterpret_cast<const uint4*>(ring + static_cast<size_t>(st) * row_bytes);
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
    const float tot = block_sum(s, sh);      // every thread has read its part of the stage once this returns
    if (threadIdx.x == 0) {
      const long long nr = row + static_cast<long long>(nst) * gridDim.x;
      if (nr < rows) {
        mbar_expect_tx(bar0 + 8 * st, row_bytes);
        bulk_load_1d(ring0 + st * row_bytes, x + nr * H, row_bytes, bar0 + 8 * st);
      }
    }
    if (RMS) {
      rstd = rsqrtf(tot / H + eps);
    } else {
      mean = tot / H;
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
      rstd = rsqrtf(block_sum(v, sh) / H + eps);
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
        for (int j = 0; j < 8; ++j) o[j] = (xv[i][j] - mean) * rstd * g[j] + (b1 != nullptr ? b[j] : 0.f);
        reinterpret_cast<uint4*>(y1 + row * H)[idx] = pack8(o);
        if (g2 != nullptr) {
          unpack8(reinterpret_cast<const uint4*>(g2)[idx], g);
          if (b2 != nullptr) unpack8(reinterpret_cast<const uint4*>(b2)[idx], b);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = (xv[i][j] - mean) * rstd * g[j] + (b2 != nullptr ? b[j] : 0.f);
          reinterpret_cast<uint4*>(y2 + row * H)[idx] = pack8(o);
        }
      }
    }
  }
}

// Backward (one 16-byte column group per thread, as norm_bwd_kernel<*, 1, *>): a stage holds the row of x, dy1,
// (dy2,) (dx_in) back to back.
template <bool RMS, bool DUAL>
__global__ void __launch_bounds__(1024, 1)
norm_bwd_ring_kernel(const h16* __restrict__ dy1, const h16* __restrict__ dy2, const h16* __restrict__ x,
                     const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                     const h16* __restrict__ gamma1, const h16* __restrict__ gamma2,
                     const h16* __restrict__ dx_in, h16* __restrict__ dx, float* __restrict__ ws, long long rows,
                     int H, int nst, int* err) {
  extern __shared__ __align__(128) unsigned char ring[];
  __shared__ float sh[64];
  __shared__ __align__(8) unsigned long long bars[RING_MAX_STAGES];
  constexpr int NOUT = DUAL ? 4 : 2;
  const int nv = H >> 3;
  const int idx = threadIdx.x;
  const bool live = idx < nv;
  const uint32_t row_bytes = static_cast<uint32_t>(H) * 2u;
  const int ntens = 2 + (DUAL ? 1 : 0) + (dx_in != nullptr ? 1 : 0);
  const uint32_t stage_bytes = row_bytes * ntens;
  const uint32_t ring0 = smem_u32(ring), bar0 = smem_u32(bars);
  auto fill = [&](int st, long long r) {
    const uint32_t dst = ring0 + st * stage_bytes, bar = bar0 + 8 * st;
    mbar_expect_tx(bar, stage_bytes);
    bulk_load_1d(dst, x + r * H, row_bytes, bar);
    bulk_load_1d(dst + row_bytes, dy1 + r * H, row_bytes, bar);
    if (DUAL) bulk_load_1d(dst + 2 * row_bytes, dy2 + r * H, row_bytes, bar);
    if (dx_in != nullptr) bulk_load_1d(dst + (DUAL ? 3 : 2) * row_bytes, dx_in + r * H, row_bytes, bar);
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < nst; ++s) mbar_init(bar0 + 8 * s, 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int s = 0; s < nst; ++s) {
      const long long r = blockIdx.x + static_cast<long long>(s) * gridDim.x;
      if (r < rows) fill(s, r);
    }
  }
  float dg1[8], db1[8], dg2[8], db2[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) dg1[j] = db1[j] = dg2[j] = db2[j] = 0.f;
  float mean_n = 0.f, rstd_n = 0.f;       // statistics of the next row, fetched one row ahead
  if (blockIdx.x < rows) {
    mean_n = RMS ? 0.f : mean_in[blockIdx.x];
    rstd_n = rstd_in[blockIdx.x];
  }
  int it = 0;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x, ++it) {
    const int st = it % nst;
    const float mean = mean_n, rstd = rstd_n;
    if (row + gridDim.x < rows) {
      mean_n = RMS ? 0.f : mean_in[row + gridDim.x];
      rstd_n = rstd_in[row + gridDim.x];
    }
    const bool ok = mbar_wait(bar0 + 8 * st, (it / nst) & 1, err, 61);
    if (!__syncthreads_and(ok ? 1 : 0)) {
      ring_drain(bar0, nst, it, row, rows);
      break;
    }
    const unsigned char* stage = ring + static_cast<size_t>(st) * stage_bytes;
    float xh[8], w[8];
    uint4 au = make_uint4(0u, 0u, 0u, 0u);
    float s1 = 0.f, s2 = 0.f;
    if (live) {
      float xv[8], dv[8], gv[8];            // gamma is re-read per row: it stays in L1 and costs no registers
      unpack8(reinterpret_cast<const uint4*>(stage)[idx], xv);
      unpack8(reinterpret_cast<const uint4*>(stage + row_bytes)[idx], dv);
      unpack8(reinterpret_cast<const uint4*>(gamma1)[idx], gv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        xh[j] = (xv[j] - mean) * rstd;
        w[j] = dv[j] * gv[j];
        dg1[j] += dv[j] * xh[j];
        db1[j] += dv[j];
      }
      if (DUAL) {
        unpack8(reinterpret_cast<const uint4*>(stage + 2 * row_bytes)[idx], dv);
        unpack8(reinterpret_cast<const uint4*>(gamma2)[idx], gv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          w[j] += dv[j] * gv[j];
          dg2[j] += dv[j] * xh[j];
          db2[j] += dv[j];
        }
      }
      if (dx_in != nullptr) au = reinterpret_cast<const uint4*>(stage + (DUAL ? 3 : 2) * row_bytes)[idx];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s1 += w[j] * xh[j];
        s2 += w[j];
      }
    }
    const float2 r = block_sum2(s1, s2, sh);   // every thread has read its part of the stage once this returns
    if (threadIdx.x == 0) {
      const long long nr = row + static_cast<long long>(nst) * gridDim.x;
      if (nr < rows) fill(st, nr);
    }
    const float c1 = r.x / H, c2 = RMS ? 0.f : r.y / H;
    if (live) {
      float o[8], a[8];
      unpack8(au, a);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rstd * (w[j] - c2 - xh[j] * c1) + a[j];
      reinterpret_cast<uint4*>(dx + row * H)[idx] = pack8(o);
    }
  }
  if (live) {
    float* wg = ws + static_cast<long long>(blockIdx.x) * NOUT * H;
    float4* p = reinterpret_cast<float4*>(wg + idx * 8);
    p[0] = make_float4(dg1[0], dg1[1], dg1[2], dg1[3]);
    p[1] = make_float4(dg1[4], dg1[5], dg1[6], dg1[7]);
    p = reinterpret_cast<float4*>(wg + H + idx * 8);
    p[0] = make_float4(db1[0], db1[1], db1[2], db1[3]);
    p[1] = make_float4(db1[4], db1[5], db1[6], db1[7]);
    if (DUAL) {
      p = reinterpret_cast<float4*>(wg + 2 * H + idx * 8);
      p[0] = make_float4(dg2[0], dg2[1], dg2[2], dg2[3]);
      p[1] = make_float4(dg2[4], dg2[5], dg2[6], dg2[7]);
      p = reinterpret_cast<float4*>(wg + 3 * H + idx * 8);
      p[0] = make_float4(db2[0], db2[1], db2[2], db2[3]);
      p[1] = make_float4(db2[4], db2[5], db2[6], db2[7]);
    }
  }
}

// Shared memory the ring kernels may use per SM (the rest is left to L1) and whether the ring path is on
// (NEOX_NORM_RING=0 selects the register-resident kernels for every shape).
constexpr int RING_SMEM_PER_SM = 200 * 1024;
static bool ring_enabled() {
  static const bool on = [] {
    const char* e = getenv("NEOX_NORM_RING");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct NormGradOut {
  float* out[4];  // dgamma1, dbeta1, dgamma2, dbeta2 (null = not wanted)
};

// out[which][c] (+)= sum_b ws[b, which, c]; blockIdx.y = which.  Block = 128 columns x 8 row groups:
// each thread sums every 8th partial row (eight independent load chains per column instead of one
// long one), then the groups are combined through shared memory.
__global__ void __launch_bounds__(1024)
norm_param_grad_reduce(const float* __restrict__ ws, int nblocks, int nout, int H, NormGradOut o,
                       int accumulate) {
  __shared__ float sa[8][128];
  float* dst = o.out[blockIdx.y];
  if (dst == nullptr) return;
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int g = threadIdx.y;
  float a = 0.f;
  if (c < H) {
    const float* src = ws + static_cast<long long>(blockIdx.y) * H + c;
    for (int i = g; i < nblocks; i += 8) a += src[static_cast<long long>(i) * nout * H];
  }
  sa[g][threadIdx.x] = a;
  __syncthreads();
  if (g == 0 && c < H) {
#pragma unroll
    for (int k = 1; k < 8; ++k) a += sa[k][threadIdx.x];
    if (accumulate) dst[c] += a;
    else dst[c] = a;
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
NX_API int NX_SYM(nx_norm_fwd)(int kind, const void* x, const void* g1, const void* b1, void* y1,
                       const void* g2, const void* b2, void* y2, void* mean, void* rstd,
                       long long rows, int H, float eps, void* stream_) {
  using namespace nx;
  if (rows <= 0) return NX_OK;
  NX_REQUIRE(H % 8 == 0 && H <= 8 * MAXV * 1024, "norm: H=%d must be a multiple of 8 and <= %d", H,
             8 * MAXV * 1024);
  NX_REQUIRE(rows < (1ll << 31), "norm: too many rows");
  auto s = static_cast<cudaStream_t>(stream_);
  const int t = threads_for(H);
  using bf = h16;
  // The ring form of the forward pass measured slower than one block per row (0.171 against 0.104 ms for 32768 x 4096:
  // with one input stream the many small resident blocks already keep enough loads in flight), so it is opt-in.
  static const bool fwd_ring = [] { const char* e = getenv("NEOX_NORM_FWD_RING"); return e != nullptr && e[0] == '1'; }();
  if (fwd_ring && ring_enabled() && H <= 8192 && rows >= 2 * sm_count() && aligned16(x)) {
    // blocks per SM: as many as the threads allow (<= 4); each gets an equal part of the ring budget
    const int bps = std::max(1, std::min(4, 2048 / t));
    const int nst = std::min(RING_MAX_STAGES, RING_SMEM_PER_SM / bps / (H * 2));
    if (nst >= 2) {
      const int smem = nst * H * 2;
      const int grid = static_cast<int>(std::min<long long>(rows, static_cast<long long>(sm_count()) * bps));
      auto kern = kind == 0 ? norm_fwd_ring_kernel<false> : norm_fwd_ring_kernel<true>;
      NX_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      kern<<<grid, t, smem, s>>>((const bf*)x, (const bf*)g1, (const bf*)b1, (bf*)y1, (const bf*)g2, (const bf*)b2,
                                 (bf*)y2, (float*)mean, (float*)rstd, rows, H, eps, nst, device_error_word());
      NX_LAUNCH_CHECK();
      return NX_OK;
    }
  }
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

// Number of persistent blocks the backward uses == rows of the fp32 workspace [blocks, 2 or 4, H].
NX_API int NX_SYM(nx_norm_bwd_blocks)(long long rows) {
  const long long cap = static_cast<long long>(nx::sm_count()) * 2;
  return static_cast<int>(rows < cap ? rows : cap);
}

namespace nx {
template <bool RMS, int VPT, bool DUAL>
static void launch_norm_bwd(int blocks, int threads, cudaStream_t s, const void* dy1, const void* dy2,
                            const void* x, const void* mean, const void* rstd, const void* g1,
                            const void* g2, const void* dx_in, void* dx, void* ws, long long rows,
                            int H) {
  using bf = h16;
  norm_bwd_kernel<RMS, VPT, DUAL><<<blocks, threads, 0, s>>>(
      (const bf*)dy1, (const bf*)dy2, (const bf*)x, (const float*)mean, (const float*)rstd,
      (const bf*)g1, (const bf*)g2, (const bf*)dx_in, (bf*)dx, (float*)ws, rows, H);
}
}  // namespace nx

// dx = dx_in (optional) + backward of the norm(s) of x.  dy2 / gamma2 non-null: the two norms of a
// dual forward, both gradients in one pass.  dgamma* / dbeta* fp32 (a null one is skipped;
// accumulate != 0 adds into them).  ws: fp32 workspace of nx_norm_bwd_blocks(rows) * (dy2 ? 4 : 2) * H.
NX_API int NX_SYM(nx_norm_bwd)(int kind, const void* dy1, const void* dy2, const void* x, const void* mean,
                       const void* rstd, const void* gamma1, const void* gamma2, const void* dx_in,
                       void* dx, void* dgamma1, void* dbeta1, void* dgamma2, void* dbeta2, void* ws,
                       long long rows, int H, int accumulate, void* stream_) {
  using namespace nx;
  if (rows <= 0) return NX_OK;
  NX_REQUIRE(H % 8 == 0 && H <= 8 * MAXV * 1024, "norm: H=%d unsupported", H);
  NX_REQUIRE(ws != nullptr, "norm_bwd: workspace is null");
  NX_REQUIRE((dy2 == nullptr) == (gamma2 == nullptr), "norm_bwd: dy2 and gamma2 go together");
  auto s = static_cast<cudaStream_t>(stream_);
  const int nv = H / 8;
  const int vpt = nv <= 1024 ? 1 : (nv <= 2048 ? 4 : 8);
  int threads = ((nv + vpt - 1) / vpt + 31) / 32 * 32;
  if (threads < 64) threads = 64;
  int blocks = NX_SYM(nx_norm_bwd_blocks)(rows);
  const bool dual = dy2 != nullptr, rms = kind != 0;
  bool done = false;
  if (ring_enabled() && vpt == 1 && rows >= 2 * sm_count() && aligned16(x) && aligned16(dy1) && aligned16(dy2) &&
      aligned16(dx_in)) {
    const int ntens = 2 + (dual ? 1 : 0) + (dx_in != nullptr ? 1 : 0);
    const int bps = threads <= 512 ? 2 : 1;            // 64 registers x 1024 threads per SM
    const int nst = std::min(RING_MAX_STAGES, RING_SMEM_PER_SM / bps / (ntens * H * 2));
    if (nst >= 2) {
      const int smem = nst * ntens * H * 2;
      blocks = static_cast<int>(std::min<long long>(blocks, static_cast<long long>(sm_count()) * bps));
      auto kern = rms ? (dual ? norm_bwd_ring_kernel<true, true> : norm_bwd_ring_kernel<true, false>)
                      : (dual ? norm_bwd_ring_kernel<false, true> : norm_bwd_ring_kernel<false, false>);
      NX_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      using bf = h16;
      kern<<<blocks, threads, smem, s>>>((const bf*)dy1, (const bf*)dy2, (const bf*)x, (const float*)mean,
                                         (const float*)rstd, (const bf*)gamma1, (const bf*)gamma2, (const bf*)dx_in,
                                         (bf*)dx, (float*)ws, rows, H, nst, device_error_word());
      done = true;
    }
  }
#define NX_NORM_BWD(R, V, D)                                                                        \
  launch_norm_bwd<R, V, D>(blocks, threads, s, dy1, dy2, x, mean, rstd, gamma1, gamma2, dx_in, dx, \
                           ws, rows, H)
#define NX_NORM_BWD_V(R, D)                  \
  do {                                       \
    if (vpt == 1) NX_NORM_BWD(R, 1, D);      \
    else if (vpt == 4) NX_NORM_BWD(R, 4, D); \
    else NX_NORM_BWD(R, 8, D);               \
  } while (0)
  if (done) {
  } else if (rms) {
    if (dual) NX_NORM_BWD_V(true, true);
    else NX_NORM_BWD_V(true, false);
  } else {
    if (dual) NX_NORM_BWD_V(false, true);
    else NX_NORM_BWD_V(false, false);
  }
#undef NX_NORM_BWD_V
#undef NX_NORM_BWD
  NX_LAUNCH_CHECK();
  const int nout = dual ? 4 : 2;
  NormGradOut o{{(float*)dgamma1, (float*)dbeta1, (float*)dgamma2, (float*)dbeta2}};
  norm_param_grad_reduce<<<dim3((H + 127) / 128, nout), dim3(128, 8), 0, s>>>(
      (const float*)ws, blocks, nout, H, o, accumulate);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
