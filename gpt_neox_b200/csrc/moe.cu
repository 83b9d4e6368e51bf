// Mixture-of-experts routing plan and token permutation, entirely on the device (no host read of the
// routing result anywhere in the layer).
//
// Given the top-k expert ids of T tokens (C = T*k routed copies) the plan kernels produce a *padded
// permuted layout*: the copies of expert e occupy rows [offsets[e], offsets[e] + counts[e]) of a matrix
// whose expert segments start at multiples of 128 rows, in the original (token, slot) order (a stable
// counting sort).  Segment alignment means a 128-row GEMM tile never straddles two experts, so the
// grouped GEMM (csrc/gemm_tcgen05.cu, GROUP_ROWS / GROUP_K) needs only a tile -> expert table, and the
// padding rows are zero so weight-gradient reductions over a segment are exact.
//
// Counterparts in the reference: megablocks ops.sort / histogram / inclusive_cumsum / gather / scatter
// called at megatron/model/moe.py:62-83,128,153.
#include "common.h"
#include "ptx.cuh"

namespace nx {

constexpr int MOE_BLOCK = 1024;
constexpr int MOE_MAX_E = 256;
constexpr int MOE_ALIGN = 128;

// hist[b][e] = number of copies of expert e among copies [b*1024, (b+1)*1024)
__global__ void __launch_bounds__(MOE_BLOCK)
moe_hist_kernel(const long long* __restrict__ expert, int C, int E, int* __restrict__ hist) {
  __shared__ int h[MOE_MAX_E];
  for (int i = threadIdx.x; i < E; i += MOE_BLOCK) h[i] = 0;
  __syncthreads();
  const int c = blockIdx.x * MOE_BLOCK + threadIdx.x;
  if (c < C && expert[c] >= 0) atomicAdd(&h[static_cast<int>(expert[c])], 1);   // id < 0: not routed here
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += MOE_BLOCK) hist[blockIdx.x * E + i] = h[i];
}

// One block.  base[b][e] = copies of expert e in earlier blocks; counts[e]; offsets[e] (segment starts,
// multiples of 128, offsets[E] = padded total); tile_expert[t] for every 128-row tile (-1 past the end).
__global__ void __launch_bounds__(MOE_MAX_E)
moe_plan_kernel(const int* __restrict__ hist, int nblk, int E, int* __restrict__ base, int* __restrict__ counts,
                int* __restrict__ offsets, int* __restrict__ tile_expert, int max_tiles) {
  __shared__ int cnt[MOE_MAX_E], off[MOE_MAX_E + 1];
  const int e = threadIdx.x;
  if (e < E) {
    int run = 0;
    for (int b = 0; b < nblk; ++b) {
      base[b * E + e] = run;
      run += hist[b * E + e];
    }
    cnt[e] = run;
    counts[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0;
    for (int i = 0; i < E; ++i) {
      off[i] = o;
      o += (cnt[i] + MOE_ALIGN - 1) / MOE_ALIGN * MOE_ALIGN;
    }
    off[E] = o;
  }
  __syncthreads();
  for (int i = threadIdx.x; i <= E; i += MOE_MAX_E) offsets[i] = off[i];
  if (e < E)
    for (int t = off[e] / MOE_ALIGN; t < off[e + 1] / MOE_ALIGN; ++t) tile_expert[t] = e;
  for (int t = off[E] / MOE_ALIGN + threadIdx.x; t < max_tiles; t += MOE_MAX_E) tile_expert[t] = -1;
}

// dest_row[c] = offsets[e] + base[block][e] + (copies of e earlier in this block); src_copy[dest] = c.
// A copy with a negative expert id (expert parallelism: an expert of another rank) gets dest_row -1.
__global__ void __launch_bounds__(MOE_BLOCK)
moe_rank_kernel(const long long* __restrict__ expert, int C, int E, const int* __restrict__ base,
                const int* __restrict__ offsets, int* __restrict__ dest_row, int* __restrict__ src_copy) {
  extern __shared__ int wcount[];   // [32 warps][E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 32 * E; i += MOE_BLOCK) wcount[i] = 0;
  __syncthreads();
  const int c = blockIdx.x * MOE_BLOCK + threadIdx.x;
  const int e = c < C ? static_cast<int>(expert[c]) : -1;
  const unsigned mask = __match_any_sync(0xffffffffu, e);
  const int rank_in_warp = __popc(mask & ((1u << lane) - 1u));
  if (e >= 0 && rank_in_warp == 0) wcount[warp * E + e] = __popc(mask);
  __syncthreads();
  if (e >= 0) {
    int before = 0;
    for (int w = 0; w < warp; ++w) before += wcount[w * E + e];
    const int d = offsets[e] + base[blockIdx.x * E + e] + before + rank_in_warp;
    dest_row[c] = d;
    src_copy[d] = c;
  } else if (c < C) {
    dest_row[c] = -1;   // copy of an expert that lives on another rank
  }
}

// Row gather by destination: out[row] = scale * src[src_copy[row] / k] (zeros for padding rows).
// scale: per-copy weights (indexed by copy id) or null.  One warp per row; H % 8 == 0.
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const h16* __restrict__ src, long long lds, const int* __restrict__ src_copy,
                       const h16* __restrict__ scale, int k, h16* __restrict__ out, int rows,
                       int H) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int c = src_copy[row];
  uint4* o = reinterpret_cast<uint4*>(out + static_cast<long long>(row) * H);
  if (c < 0) {
    for (int v = lane; v < H / 8; v += 32) o[v] = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  const uint4* s = reinterpret_cast<const uint4*>(src + static_cast<long long>(c / k) * lds);
  if (scale == nullptr) {
    for (int v = lane; v < H / 8; v += 32) o[v] = s[v];
  } else {
    const float w = h16_to_float(scale[c]);
    for (int v = lane; v < H / 8; v += 32) {
      const uint4 u = s[v];
      const float2 a = unpack_h16x2(u.x), b = unpack_h16x2(u.y), cc = unpack_h16x2(u.z), d = unpack_h16x2(u.w);
      uint4 r;
      r.x = pack_h16x2(a.x * w, a.y * w); r.y = pack_h16x2(b.x * w, b.y * w);
      r.z = pack_h16x2(cc.x * w, cc.y * w); r.w = pack_h16x2(d.x * w, d.y * w);
      o[v] = r;
    }
  }
}

// Weighted combine by token: out[t] = sum_j w[t*k+j] * y[dest_row[t*k+j]] (w null: unit weights).
// One warp per token, fp32 accumulation, deterministic.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const h16* __restrict__ y, const int* __restrict__ dest_row,
                   const h16* __restrict__ w, int k, h16* __restrict__ out, int T, int H) {
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= T) return;
  const int lane = threadIdx.x & 31;
  for (int v = lane; v < H / 8; v += 32) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      const int c = t * k + j;
      const float wj = w ? h16_to_float(w[c]) : 1.f;
      const uint4 u = reinterpret_cast<const uint4*>(y + static_cast<long long>(dest_row[c]) * H)[v];
      const float2 a = unpack_h16x2(u.x), b = unpack_h16x2(u.y), cc = unpack_h16x2(u.z), d = unpack_h16x2(u.w);
      acc[0] += wj * a.x; acc[1] += wj * a.y; acc[2] += wj * b.x; acc[3] += wj * b.y;
      acc[4] += wj * cc.x; acc[5] += wj * cc.y; acc[6] += wj * d.x; acc[7] += wj * d.y;
    }
    uint4 r;
    r.x = pack_h16x2(acc[0], acc[1]); r.y = pack_h16x2(acc[2], acc[3]);
    r.z = pack_h16x2(acc[4], acc[5]); r.w = pack_h16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + static_cast<long long>(t) * H)[v] = r;
  }
}

// Gradient of the routing weights: dw[c] = <g[c / k], y[dest_row[c]]>.  One warp per copy.
__global__ void __launch_bounds__(256)
moe_weight_grad_kernel(const h16* __restrict__ g, const h16* __restrict__ y,
                       const int* __restrict__ dest_row, int k, h16* __restrict__ dw, int C, int H) {
  const int c = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (c >= C) return;
  const int lane = threadIdx.x & 31;
  const uint4* gp = reinterpret_cast<const uint4*>(g + static_cast<long long>(c / k) * H);
  const uint4* yp = reinterpret_cast<const uint4*>(y + static_cast<long long>(dest_row[c]) * H);
  float acc = 0.f;
  for (int v = lane; v < H / 8; v += 32) {
    const uint4 a = gp[v], b = yp[v];
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 x = unpack_h16x2(aw[q]), z = unpack_h16x2(bw[q]);
      acc += x.x * z.x + x.y * z.y;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) dw[c] = float_to_h16(acc);
}

NX_API int NX_SYM(nx_moe_blocks)(int C) { return (C + MOE_BLOCK - 1) / MOE_BLOCK; }
NX_API int NX_SYM(nx_moe_max_rows)(int C, int E) { return (C + E * (MOE_ALIGN - 1) + MOE_ALIGN - 1) / MOE_ALIGN * MOE_ALIGN; }

// expert: int64 [C]; scratch hist / base: int32 [blocks * E]; outputs: counts [E], offsets [E+1],
// tile_expert [max_rows / 128], dest_row [C], src_copy [max_rows] (filled with -1 here).
NX_API int NX_SYM(nx_moe_plan)(const void* expert, int C, int E, void* hist, void* base, void* counts, void* offsets,
                       void* tile_expert, void* dest_row, void* src_copy, cudaStream_t stream) {
  NX_REQUIRE(E >= 1 && E <= MOE_MAX_E, "moe_plan: %d experts (max %d)", E, MOE_MAX_E);
  NX_REQUIRE(C > 0, "moe_plan: no routed copies");
  const int nblk = (C + MOE_BLOCK - 1) / MOE_BLOCK;
  const int max_rows = NX_SYM(nx_moe_max_rows)(C, E);
  NX_CUDA_CHECK(cudaMemsetAsync(src_copy, 0xff, sizeof(int) * static_cast<size_t>(max_rows), stream));
  moe_hist_kernel<<<nblk, MOE_BLOCK, 0, stream>>>((const long long*)expert, C, E, (int*)hist);
  NX_LAUNCH_CHECK();
  moe_plan_kernel<<<1, MOE_MAX_E, 0, stream>>>((const int*)hist, nblk, E, (int*)base, (int*)counts, (int*)offsets,
                                               (int*)tile_expert, max_rows / MOE_ALIGN);
  NX_LAUNCH_CHECK();
  moe_rank_kernel<<<nblk, MOE_BLOCK, sizeof(int) * 32 * E, stream>>>((const long long*)expert, C, E, (const int*)base,
                                                                     (const int*)offsets, (int*)dest_row, (int*)src_copy);
  NX_LAUNCH_CHECK();
  return NX_OK;
}

NX_API int NX_SYM(nx_moe_gather_rows)(const void* src, long long lds, const void* src_copy, const void* scale, int k, void* out,
                              int rows, int H, cudaStream_t stream) {
  NX_REQUIRE(H % 8 == 0 && lds % 8 == 0, "moe_gather_rows: hidden size must be a multiple of 8");
  moe_gather_rows_kernel<<<(rows + 7) / 8, 256, 0, stream>>>((const h16*)src, lds, (const int*)src_copy,
                                                             (const h16*)scale, k, (h16*)out, rows, H);
  NX_LAUNCH_CHECK();
  return NX_OK;
}

NX_API int NX_SYM(nx_moe_combine)(const void* y, const void* dest_row, const void* w, int k, void* out, int T, int H,
                          cudaStream_t stream) {
  NX_REQUIRE(H % 8 == 0, "moe_combine: hidden size must be a multiple of 8");
  moe_combine_kernel<<<(T + 7) / 8, 256, 0, stream>>>((const h16*)y, (const int*)dest_row,
                                                      (const h16*)w, k, (h16*)out, T, H);
  NX_LAUNCH_CHECK();
  return NX_OK;
}

NX_API int NX_SYM(nx_moe_weight_grad)(const void* g, const void* y, const void* dest_row, int k, void* dw, int C, int H,
                              cudaStream_t stream) {
  NX_REQUIRE(H % 8 == 0, "moe_weight_grad: hidden size must be a multiple of 8");
  moe_weight_grad_kernel<<<(C + 7) / 8, 256, 0, stream>>>((const h16*)g, (const h16*)y,
                                                          (const int*)dest_row, k, (h16*)dw, C, H);
  NX_LAUNCH_CHECK();
  return NX_OK;
}

}  // namespace nx
