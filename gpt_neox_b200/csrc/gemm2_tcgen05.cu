// bf16 GEMM on CTA pairs: two SMs of a cluster cooperate on one 256 x 256 output tile with
// tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of A and one half (128 rows of the N
// dimension) of B per K block, so a pair moves half as many B bytes through shared memory as two
// independent 128 x 256 tiles would, and one MMA instruction covers 256 x 256 x 16.
//
//   CTA rank 0 ("leader") : its elected MMA thread issues every tcgen05.mma for the pair and commits
//                           to the mbarriers of both CTAs (tcgen05.commit ... multicast::cluster).
//   both CTAs             : a TMA producer warp fills the CTA's own shared memory; the transaction
//                           bytes of both CTAs are counted on the leader's "full" barrier (the
//                           cta_group::2 form of the bulk tensor load may signal the peer's barrier);
//                           four epilogue warps drain the CTA's own 128 TMEM lanes (its 128 rows of
//                           the tile, all 256 columns) and report to the leader's "tmem empty" barrier.
//
// Same contract as nx_gemm_bf16 (csrc/gemm_tcgen05.cu): C[M,N] = epilogue(op(A) * op(B)), layouts
// NT / NN / TN / TT, epilogue flags bias, GeLU (+ pre-activation out), GeLU', residual, scale,
// accumulate, fp32 output.  No loads with cluster multicast are used anywhere.
#include <cooperative_groups.h>

#include "common.h"
#include "ptx.cuh"

namespace nx {
namespace g2 {

constexpr int BM = 128;          // rows per CTA (256 per pair)
constexpr int BNH = 128;         // B rows (N) staged per CTA; the pair's tile is 256 wide
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UK = 16;
constexpr int STAGES = 6;
constexpr int THREADS = 192;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BNH * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
constexpr int DYN_BYTES = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 1024;

enum Epi : int { BIAS = 1, GELU_ERF = 2, GELU_TANH = 4, AUX_OUT = 8, DGELU_ERF = 16, DGELU_TANH = 32, RESIDUAL = 64,
                 ACCUM = 128, OUT_F32 = 256, SCALE = 512 };

struct Params {
  int M, N, K;
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* aux_in;
  __nv_bfloat16* aux_out;
  const __nv_bfloat16* residual;
  long long ld_aux;
  int flags;
  float alpha;
  int tiles_m, tiles_n;    // 256-row x 256-column tiles
  int* err;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_result_addr, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result_addr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_bf16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive (once all tcgen05 ops issued so far are done) on the barrier at this offset in both CTAs.
__device__ __forceinline__ void umma2_commit_both(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(mask)
      : "memory");
}
// Bulk tensor load into this CTA's shared memory whose completion is counted on `bar`, which may be the
// peer CTA's barrier (shared::cluster address).
__device__ __forceinline__ void tma2_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tile_coords2(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int GROUP = 8;
  const int per_group = GROUP * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP;
  const int gsize = min(GROUP, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + (r % gsize);
  tn = r / gsize;
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
    gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + BAR_OFFSET + 8 * (2 * STAGES + 4));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  constexpr uint32_t TMEM_COLS = 512;          // two 256-column accumulators

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);               // leader: one expect_tx arrival + the bytes of both CTAs
      mbar_init(empty_bar(s), 1);              // one multicast commit per use
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), 8);         // leader: four epilogue warps of each CTA
    }
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  __syncthreads();
  cluster_sync_all();                          // the peer's barriers exist before anything signals them
  if (warp == 1) {
    tmem_alloc2(tmem_slot, TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  bool aborted = false;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = pair; tile < num_tiles && !aborted; tile += pairs) {
        int tm, tn;
        tile_coords2(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * (2 * BM) + rank * BM;
        const int n0 = tn * BN + rank * BNH;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, p.err, 11)) {
            aborted = true;
            break;
          }
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
          const uint32_t b_dst = a_dst + A_BYTES;
          // completion bytes of both CTAs go to the leader's barrier of this stage
          const uint32_t bar = map_to_cta(full_bar(stage), 0);
          if (leader) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
          const int k0 = kb * BK;
          if constexpr (!A_MN) {
            tma2_load_2d(a_dst, &tmA, bar, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma2_load_2d(a_dst + j * (BK * 128), &tmA, bar, m0 + j * 64, k0);
          }
          if constexpr (!B_MN) {
            tma2_load_2d(b_dst, &tmB, bar, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j) tma2_load_2d(b_dst + j * (BK * 128), &tmB, bar, n0 + j * 64, k0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      constexpr uint32_t A_LBO = A_MN ? BK * 128 : 0, B_LBO = B_MN ? BK * 128 : 0;
      constexpr uint32_t A_KADV = A_MN ? UK * 128 : UK * 2;
      constexpr uint32_t B_KADV = B_MN ? UK * 128 : UK * 2;
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (int tile = pair; tile < num_tiles && !aborted; tile += pairs) {
        if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1, p.err, 12)) {
          aborted = true;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, p.err, 13)) {
            aborted = true;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_base + stage * STAGE_BYTES;
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            const uint64_t adesc = umma_smem_desc_sw128(a_addr + k * A_KADV, A_LBO, 1024);
            const uint64_t bdesc = umma_smem_desc_sw128(b_addr + k * B_KADV, B_LBO, 1024);
            umma2_bf16_ss(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma2_commit_both(empty_bar(stage));       // frees this stage in both CTAs
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (aborted) break;
        umma2_commit_both(tmem_full_bar(acc));        // accumulator ready in both CTAs
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    const int flags = p.flags;
    for (int tile = pair; tile < num_tiles; tile += pairs) {
      int tm, tn;
      tile_coords2(tile, p.tiles_m, p.tiles_n, tm, tn);
      const int m0 = tm * (2 * BM) + rank * BM, n0 = tn * BN;
      if (!mbar_wait(tmem_full_bar(acc), acc_phase, p.err, 14)) {
        aborted = true;
        break;
      }
      tc_fence_after_sync();
      const long long row = m0 + row_in_tile;
      const bool row_ok = row < p.M;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(quad * 32) << 16), r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (flags & SCALE) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
        }
        if (flags & BIAS) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (col0 + j < p.N) {
              const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.bias + col0 + j));
              const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z),
                           b3 = unpack_bf16x2(b.w);
              v[j + 0] += b0.x; v[j + 1] += b0.y; v[j + 2] += b1.x; v[j + 3] += b1.y;
              v[j + 4] += b2.x; v[j + 5] += b2.y; v[j + 6] += b3.x; v[j + 7] += b3.y;
            }
          }
        }
        if (row_ok) {
          if (flags & AUX_OUT) {
            __nv_bfloat16* ap = p.aux_out + row * p.ld_aux + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < p.N) {
                uint4 o;
                o.x = pack_bf16x2(v[j], v[j + 1]); o.y = pack_bf16x2(v[j + 2], v[j + 3]);
                o.z = pack_bf16x2(v[j + 4], v[j + 5]); o.w = pack_bf16x2(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4*>(ap + j) = o;
              }
            }
          }
          if (flags & (DGELU_ERF | DGELU_TANH)) {
            const __nv_bfloat16* ap = p.aux_in + row * p.ld_aux + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < p.N) {
                const uint4 a = *reinterpret_cast<const uint4*>(ap + j);
                const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const float2 x = unpack_bf16x2(aw[q]);
                  if (flags & DGELU_ERF) {
                    v[j + 2 * q] *= gelu_erf_grad(x.x);
                    v[j + 2 * q + 1] *= gelu_erf_grad(x.y);
                  } else {
                    v[j + 2 * q] *= gelu_tanh_grad(x.x);
                    v[j + 2 * q + 1] *= gelu_tanh_grad(x.y);
                  }
                }
              }
            }
          }
          if (flags & GELU_ERF) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
          } else if (flags & GELU_TANH) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
          }
          if (flags & RESIDUAL) {
            const __nv_bfloat16* rp = p.residual + row * p.ld_aux + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < p.N) {
                const uint4 a = *reinterpret_cast<const uint4*>(rp + j);
                const float2 x0 = unpack_bf16x2(a.x), x1 = unpack_bf16x2(a.y), x2 = unpack_bf16x2(a.z),
                             x3 = unpack_bf16x2(a.w);
                v[j + 0] += x0.x; v[j + 1] += x0.y; v[j + 2] += x1.x; v[j + 3] += x1.y;
                v[j + 4] += x2.x; v[j + 5] += x2.y; v[j + 6] += x3.x; v[j + 7] += x3.y;
              }
            }
          }
          if (flags & OUT_F32) {
            float* cp = reinterpret_cast<float*>(p.C) + row * p.ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col0 + j < p.N) {
                float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                if (flags & ACCUM) {
                  const float4 old = *reinterpret_cast<const float4*>(cp + j);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(cp + j) = o;
              }
            }
          } else {
            __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < p.N) {
                if (flags & ACCUM) {
                  const uint4 a = *reinterpret_cast<const uint4*>(cp + j);
                  const float2 x0 = unpack_bf16x2(a.x), x1 = unpack_bf16x2(a.y), x2 = unpack_bf16x2(a.z),
                               x3 = unpack_bf16x2(a.w);
                  v[j + 0] += x0.x; v[j + 1] += x0.y; v[j + 2] += x1.x; v[j + 3] += x1.y;
                  v[j + 4] += x2.x; v[j + 5] += x2.y; v[j + 6] += x3.x; v[j + 7] += x3.y;
                }
                uint4 o;
                o.x = pack_bf16x2(v[j], v[j + 1]); o.y = pack_bf16x2(v[j + 2], v[j + 3]);
                o.z = pack_bf16x2(v[j + 4], v[j + 5]); o.w = pack_bf16x2(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4*>(cp + j) = o;
              }
            }
          }
        }
      }
      // this warp is done with the accumulator: tell the leader's MMA thread
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tmem_empty_bar(acc), 0));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (aborted) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();          // nobody leaves while the peer may still signal this CTA's barriers
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN>
static int launch2(const CUtensorMap& tmA, const CUtensorMap& tmB, const Params& p, cudaStream_t stream) {
  auto kern = gemm2_kernel<A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    NX_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DYN_BYTES));
    configured = true;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int max_pairs = sm_count() / 2;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  kern<<<2 * pairs, THREADS, DYN_BYTES, stream>>>(tmA, tmB, p);     // cluster dims are compiled in
  NX_LAUNCH_CHECK();
  return NX_OK;
}

}  // namespace g2

// Same arguments as nx_gemm_bf16.
NX_API int nx_gemm2_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                         long long ldc, int transA, int transB, const void* bias, const void* aux_in, void* aux_out,
                         const void* residual, long long ld_aux, int flags, float alpha, void* stream_) {
  using namespace g2;
  if (M <= 0 || N <= 0) return NX_OK;
  NX_REQUIRE(K > 0, "gemm2: K must be positive");
  NX_REQUIRE(N % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0, "gemm2: N / lda / ldb must be multiples of 8");
  NX_REQUIRE(ldc % ((flags & OUT_F32) ? 4 : 8) == 0, "gemm2: ldc alignment");
  NX_REQUIRE((reinterpret_cast<uintptr_t>(C) & 15) == 0, "gemm2: C must be 16-byte aligned");
  CUtensorMap tmA, tmB;
  bool ok;
  if (!transA) ok = make_tma_2d(&tmA, A, M, K, lda * 2, BM, BK, 2);
  else         ok = make_tma_2d(&tmA, A, K, M, lda * 2, BK, 64, 2);
  if (!ok) return NX_ERR_ARG;
  if (!transB) ok = make_tma_2d(&tmB, B, N, K, ldb * 2, BNH, BK, 2);
  else         ok = make_tma_2d(&tmB, B, K, N, ldb * 2, BK, 64, 2);
  if (!ok) return NX_ERR_ARG;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.aux_in = static_cast<const __nv_bfloat16*>(aux_in);
  p.aux_out = static_cast<__nv_bfloat16*>(aux_out);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ld_aux = ld_aux; p.flags = flags; p.alpha = alpha;
  p.tiles_m = (M + 2 * BM - 1) / (2 * BM);
  p.tiles_n = (N + BN - 1) / BN;
  p.err = device_error_word();
  auto s = static_cast<cudaStream_t>(stream_);
  if (!transA && !transB) return launch2<false, false>(tmA, tmB, p, s);
  if (!transA && transB) return launch2<false, true>(tmA, tmB, p, s);
  if (transA && !transB) return launch2<true, false>(tmA, tmB, p, s);
  return launch2<true, true>(tmA, tmB, p, s);
}

}  // namespace nx
