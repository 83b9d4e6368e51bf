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

#include <cstdlib>

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
constexpr int THREADS = 320;        // producer, MMA issuer, 4 epilogue warps, 4 all-gather push warps
constexpr int RS_ROW_BYTES = 144;    // 64 bf16 columns + 16 B pad
constexpr int RS_STAGE_BYTES = 4 * 32 * RS_ROW_BYTES;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BNH * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
constexpr int RS_OFFSET = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 8 * 8;   // tmem slot, abort word, 8 chunk barriers
constexpr int DYN_BYTES = RS_OFFSET + RS_STAGE_BYTES + 1024;
enum Comm : int { COMM_NONE = 0, COMM_RS = 1, COMM_AG = 2, COMM_AR = 3 };

enum Epi : int { BIAS = 1, GELU_ERF = 2, GELU_TANH = 4, AUX_OUT = 8, DGELU_ERF = 16, DGELU_TANH = 32, RESIDUAL = 64,
                 ACCUM = 128, OUT_F32 = 256, SCALE = 512,
                 AUX_DERIV = 1024,   // aux_out receives gelu'(pre-activation) instead of the pre-activation
                 MUL_AUX = 2048 };   // multiply by aux_in (the stored derivative): no erf / exp in the backward epilogue

struct Params {
  int M, N, K;
  void* C;
  long long ldc;
  const h16* bias;
  const h16* aux_in;
  h16* aux_out;
  const h16* residual;
  long long ld_aux;
  int flags;
  float alpha;
  int tiles_m, tiles_n;    // 256-row x 256-column tiles
  int* err;
  // ---- fused tensor-parallel collective (same protocol as csrc/gemm_tcgen05.cu, 256-row tiles)
  int comm, tp_rank, ws;
  int tiles_m_chunk;            // row tiles per rank chunk: (M / ws) / 256
  int rs_lag;                   // reduce-scatter tile order: 0 = peers' chunks first, own chunk last; > 0 = interleaved (below)
  int num_slots;                // length of the tile sequence the CTA pairs walk (== tiles unless interleaved)
  uint32_t epoch;
  h16* rs_stage[8];   // on rank q: staging [src rank][M / ws, N]
  uint32_t* rs_flags[8];        // on rank q: flags[tile in chunk][src rank][cta of pair][warp]
  const h16* residual2;
  long long ld_res2;
  const h16* ag_src;  // this rank's [M / ws, K] shard
  long long ag_ld;
  h16* ag_dst[8];     // on rank q: gather buffer [M, K]
  uint32_t* ag_flags[8];        // on rank q: flags[src][cta]
  // all-reduce mode (reduce-scatter as above, then the owner of a chunk writes the reduced tiles into every
  // rank's full [M, N] output and bumps that rank's delivery counter once per 32-row band)
  h16* ar_out[8];     // on rank q: output [M, N], leading dimension N
  uint32_t* ar_count[8];        // on rank q: delivery counter
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

// Tile order under a fused collective: whole rank chunks of rows at a time (reduce-scatter: peers' chunks
// first, own last; all-gather: own chunk first, then the peers' as their shards arrive).
// Interleaved reduce-scatter order (rs_lag > 0): the sequence is made of groups of ws slots; group q holds tile q
// of every peer's chunk and, in its last slot, tile q - rs_lag of the own chunk.  Every rank walks the same
// order, so the partial sums an own tile needs were produced by the peers about rs_lag groups (at least one
// whole wave of CTA pairs) earlier, and the partial tiles cross NVLink evenly over the whole kernel instead of
// all within its first (ws - 1) / ws.  Slots without a tile (the first rs_lag own slots, the last rs_lag peer
// groups) return false and are skipped by every role alike.
__device__ __forceinline__ bool tile_coords2_p(int tile, const Params& p, int& tm, int& tn, int& chunk) {
  if (p.comm == COMM_NONE) {
    tile_coords2(tile, p.tiles_m, p.tiles_n, tm, tn);
    chunk = 0;
    return true;
  }
  const int per_chunk = p.tiles_m_chunk * p.tiles_n;
  if (p.rs_lag > 0) {
    const int q = tile / p.ws, s = tile - q * p.ws;
    int idx;
    if (s < p.ws - 1) {
      if (q >= per_chunk) return false;
      chunk = (p.tp_rank + 1 + s) % p.ws;
      idx = q;
    } else {
      if (q < p.rs_lag) return false;
      chunk = p.tp_rank;
      idx = q - p.rs_lag;
    }
    int tl;
    tile_coords2(idx, p.tiles_m_chunk, p.tiles_n, tl, tn);
    tm = chunk * p.tiles_m_chunk + tl;
    return true;
  }
  const int order = tile / per_chunk;
  chunk = p.comm != COMM_AG ? (p.tp_rank + 1 + order) % p.ws : (p.tp_rank + order) % p.ws;
  int tl;
  tile_coords2(tile - order * per_chunk, p.tiles_m_chunk, p.tiles_n, tl, tn);
  tm = chunk * p.tiles_m_chunk + tl;
  return true;
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
    gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmA2, const Params p) {
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
  auto ag_bar = [&](int k) { return bar_base + 8u * (2 * STAGES + 6 + k); };
  volatile int* ag_abort = reinterpret_cast<volatile int*>(smem_gen + BAR_OFFSET + 8 * (2 * STAGES + 5));

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
    for (int k = 0; k < 8; ++k) mbar_init(ag_bar(k), 4);   // one arrival per push warp
    *ag_abort = 0;
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

  const int num_tiles = p.num_slots;
  const int num_kb = (p.K + BK - 1) / BK;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  bool aborted = false;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int ag_ready_chunk = -1;
      for (int tile = pair; tile < num_tiles && !aborted; tile += pairs) {
        int tm, tn, chunk;
        if (!tile_coords2_p(tile, p, tm, tn, chunk)) continue;
        int m0 = tm * (2 * BM) + rank * BM;
        const int n0 = tn * BN + rank * BNH;
        const CUtensorMap* mapA = &tmA;
        if (p.comm == COMM_AG) {
          if (chunk == p.tp_rank) {
            mapA = &tmA2;                                   // own shard: read it where it already is
            m0 -= chunk * p.tiles_m_chunk * (2 * BM);
          } else if (chunk != ag_ready_chunk) {
            const int order = (chunk - p.tp_rank + p.ws) % p.ws;
            if (!mbar_wait(ag_bar(order - 1), 0, p.err, 17) || *ag_abort) {
              aborted = true;
              break;
            }
            asm volatile("fence.proxy.async;" ::: "memory");
            ag_ready_chunk = chunk;
          }
        }
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
            tma2_load_2d(a_dst, mapA, bar, k0, m0);
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
        {
          int tm_, tn_, chunk_;
          if (!tile_coords2_p(tile, p, tm_, tn_, chunk_)) continue;
        }
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
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    const int flags = p.flags;
    const long long chunk_rows = static_cast<long long>(p.tiles_m_chunk) * (2 * BM);
    for (int tile = pair; tile < num_tiles; tile += pairs) {
      int tm, tn, chunk;
      if (!tile_coords2_p(tile, p, tm, tn, chunk)) continue;
      const int m0 = tm * (2 * BM) + rank * BM, n0 = tn * BN;
      if (!mbar_wait(tmem_full_bar(acc), acc_phase, p.err, 14)) {
        aborted = true;
        break;
      }
      tc_fence_after_sync();
      const long long row = m0 + row_in_tile;
      const bool row_ok = row < p.M;
      const int tile_in_chunk = (tm - chunk * p.tiles_m_chunk) * p.tiles_n + tn;
      const int warp_slot = static_cast<int>(rank) * 4 + quad;       // which 32-row band of the 256-row tile
      const bool rs_like = p.comm == COMM_RS || p.comm == COMM_AR;
      if (rs_like && chunk == p.tp_rank) {
        // own rows: every peer's warp of the same band must have delivered its partial tile
        bool ok = true;
        if (lane < p.ws && lane != p.tp_rank)
          ok = wait_flag_ge(p.rs_flags[p.tp_rank] + (static_cast<long long>(tile_in_chunk) * p.ws + lane) * 8 + warp_slot,
                            p.epoch, p.err, 18);
        if (!__all_sync(0xffffffffu, ok)) {
          aborted = true;
          break;
        }
      }
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
        if ((flags & BIAS) && !rs_like) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (col0 + j < p.N) {
              const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.bias + col0 + j));
              const float2 b0 = unpack_h16x2(b.x), b1 = unpack_h16x2(b.y), b2 = unpack_h16x2(b.z),
                           b3 = unpack_h16x2(b.w);
              v[j + 0] += b0.x; v[j + 1] += b0.y; v[j + 2] += b1.x; v[j + 3] += b1.y;
              v[j + 4] += b2.x; v[j + 5] += b2.y; v[j + 6] += b3.x; v[j + 7] += b3.y;
            }
          }
        }
        if (row_ok) {
          if (flags & AUX_OUT) {
            h16* ap = p.aux_out + row * p.ld_aux + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < p.N) {
                float d[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                  d[q] = v[j + q];
                  if (flags & AUX_DERIV) {   // derivative out, activation in place (the GeLU step below is skipped)
                    if (flags & GELU_TANH) gelu_tanh_both(v[j + q], v[j + q], d[q]);
                    else gelu_erf_both(v[j + q], v[j + q], d[q]);
                  }
                }
                uint4 o;
                o.x = pack_h16x2(d[0], d[1]); o.y = pack_h16x2(d[2], d[3]);
                o.z = pack_h16x2(d[4], d[5]); o.w = pack_h16x2(d[6], d[7]);
                *reinterpret_cast<uint4*>(ap + j) = o;
              }
            }
          }
          if (flags & (DGELU_ERF | DGELU_TANH | MUL_AUX)) {
            const h16* ap = p.aux_in + row * p.ld_aux + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < p.N) {
                const uint4 a = *reinterpret_cast<const uint4*>(ap + j);
                const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const float2 x = unpack_h16x2(aw[q]);
                  if (flags & MUL_AUX) {
                    v[j + 2 * q] *= x.x;
                    v[j + 2 * q + 1] *= x.y;
                  } else if (flags & DGELU_ERF) {
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
          if (flags & AUX_DERIV) {
            // activation already applied together with its derivative
          } else if (flags & GELU_ERF) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
          } else if (flags & GELU_TANH) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
          }
          if (flags & RESIDUAL) {
            const h16* rp = p.residual + row * p.ld_aux + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < p.N) {
                const uint4 a = *reinterpret_cast<const uint4*>(rp + j);
                const float2 x0 = unpack_h16x2(a.x), x1 = unpack_h16x2(a.y), x2 = unpack_h16x2(a.z),
                             x3 = unpack_h16x2(a.w);
                v[j + 0] += x0.x; v[j + 1] += x0.y; v[j + 2] += x1.x; v[j + 3] += x1.y;
                v[j + 4] += x2.x; v[j + 5] += x2.y; v[j + 6] += x3.x; v[j + 7] += x3.y;
              }
            }
          }
          if (rs_like) {
            const long long crow = row - chunk * chunk_rows;
            if (chunk != p.tp_rank) {
              // partial tile of a peer's rows -> that peer's staging slot for this rank, as full 128-byte lines
              uint8_t* slab = smem_gen + RS_OFFSET + (warp - 2) * (32 * RS_ROW_BYTES);
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 o;
                o.x = pack_h16x2(v[j], v[j + 1]); o.y = pack_h16x2(v[j + 2], v[j + 3]);
                o.z = pack_h16x2(v[j + 4], v[j + 5]); o.w = pack_h16x2(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4*>(slab + lane * RS_ROW_BYTES + (c & 1) * 64 + j * 2) = o;
              }
              const bool last_group = (c == BN / 32 - 1) || (col0 + 32 >= p.N);
              if ((c & 1) || last_group) {
                __syncwarp();
                const int colp = n0 + (c & ~1) * 32;
                const int oct = lane & 7;
                const long long base_row = p.tp_rank * chunk_rows + (m0 + quad * 32 - chunk * chunk_rows);
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                  const int rr = it * 4 + (lane >> 3);
                  const int col = colp + oct * 8;
                  if (col < p.N && (oct < 4 || (c & 1)))
                    *reinterpret_cast<uint4*>(p.rs_stage[chunk] + (base_row + rr) * p.N + col) =
                        *reinterpret_cast<const uint4*>(slab + rr * RS_ROW_BYTES + oct * 16);
                }
                __syncwarp();
              }
            } else {
              for (int sr = 0; sr < p.ws; ++sr) {
                if (sr == p.tp_rank) continue;
                const h16* sp = p.rs_stage[p.tp_rank] + (sr * chunk_rows + crow) * p.N + col0;
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  if (col0 + j < p.N) {
                    const uint4 a = *reinterpret_cast<const uint4*>(sp + j);
                    const float2 x0 = unpack_h16x2(a.x), x1 = unpack_h16x2(a.y), x2 = unpack_h16x2(a.z),
                                 x3 = unpack_h16x2(a.w);
                    v[j + 0] += x0.x; v[j + 1] += x0.y; v[j + 2] += x1.x; v[j + 3] += x1.y;
                    v[j + 4] += x2.x; v[j + 5] += x2.y; v[j + 6] += x3.x; v[j + 7] += x3.y;
                  }
                }
              }
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                if (col0 + j < p.N) {
                  if (flags & BIAS) {
                    const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.bias + col0 + j));
                    const float2 b0 = unpack_h16x2(b.x), b1 = unpack_h16x2(b.y), b2 = unpack_h16x2(b.z),
                                 b3 = unpack_h16x2(b.w);
                    v[j + 0] += b0.x; v[j + 1] += b0.y; v[j + 2] += b1.x; v[j + 3] += b1.y;
                    v[j + 4] += b2.x; v[j + 5] += b2.y; v[j + 6] += b3.x; v[j + 7] += b3.y;
                  }
                  if (p.residual2 != nullptr) {
                    const uint4 a = *reinterpret_cast<const uint4*>(p.residual2 + crow * p.ld_res2 + col0 + j);
                    const float2 x0 = unpack_h16x2(a.x), x1 = unpack_h16x2(a.y), x2 = unpack_h16x2(a.z),
                                 x3 = unpack_h16x2(a.w);
                    v[j + 0] += x0.x; v[j + 1] += x0.y; v[j + 2] += x1.x; v[j + 3] += x1.y;
                    v[j + 4] += x2.x; v[j + 5] += x2.y; v[j + 6] += x3.x; v[j + 7] += x3.y;
                  }
                  uint4 o;
                  o.x = pack_h16x2(v[j], v[j + 1]); o.y = pack_h16x2(v[j + 2], v[j + 3]);
                  o.z = pack_h16x2(v[j + 4], v[j + 5]); o.w = pack_h16x2(v[j + 6], v[j + 7]);
                  if (p.comm == COMM_RS) {
                    *reinterpret_cast<uint4*>(reinterpret_cast<h16*>(p.C) + crow * p.ldc + col0 + j) = o;
                  } else {
                    uint8_t* slab = smem_gen + RS_OFFSET + (warp - 2) * (32 * RS_ROW_BYTES);
                    *reinterpret_cast<uint4*>(slab + lane * RS_ROW_BYTES + (c & 1) * 64 + j * 2) = o;
                  }
                }
              }
              if (p.comm == COMM_AR) {
                // reduced rows of this band: out through shared memory as full 128-byte lines, to every rank
                const uint8_t* slab = smem_gen + RS_OFFSET + (warp - 2) * (32 * RS_ROW_BYTES);
                const bool last_group = (c == BN / 32 - 1) || (col0 + 32 >= p.N);
                if ((c & 1) || last_group) {
                  __syncwarp();
                  const int colp = n0 + (c & ~1) * 32;
                  const int oct = lane & 7;
                  const long long grow0 = m0 + quad * 32;
#pragma unroll
                  for (int it = 0; it < 8; ++it) {
                    const int rr = it * 4 + (lane >> 3);
                    const int col = colp + oct * 8;
                    if (col < p.N && (oct < 4 || (c & 1))) {
                      const uint4 val = *reinterpret_cast<const uint4*>(slab + rr * RS_ROW_BYTES + oct * 16);
                      for (int q = 0; q < p.ws; ++q)
                        *reinterpret_cast<uint4*>(p.ar_out[q] + (grow0 + rr) * p.N + col) = val;
                    }
                  }
                  __syncwarp();
                }
              }
            }
          } else if (flags & OUT_F32) {
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
            h16* cp = reinterpret_cast<h16*>(p.C) + row * p.ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < p.N) {
                if (flags & ACCUM) {
                  const uint4 a = *reinterpret_cast<const uint4*>(cp + j);
                  const float2 x0 = unpack_h16x2(a.x), x1 = unpack_h16x2(a.y), x2 = unpack_h16x2(a.z),
                               x3 = unpack_h16x2(a.w);
                  v[j + 0] += x0.x; v[j + 1] += x0.y; v[j + 2] += x1.x; v[j + 3] += x1.y;
                  v[j + 4] += x2.x; v[j + 5] += x2.y; v[j + 6] += x3.x; v[j + 7] += x3.y;
                }
                uint4 o;
                o.x = pack_h16x2(v[j], v[j + 1]); o.y = pack_h16x2(v[j + 2], v[j + 3]);
                o.z = pack_h16x2(v[j + 4], v[j + 5]); o.w = pack_h16x2(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4*>(cp + j) = o;
              }
            }
          }
        }
      }
      if (p.comm == COMM_AR && chunk == p.tp_rank) {
        // this band of the reduced tile is in every rank's output: count the delivery on each of them
        __threadfence_system();
        __syncwarp();
        if (lane < p.ws && lane != p.tp_rank)
          asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.ar_count[lane]) : "memory");
      }
      if (rs_like && chunk != p.tp_rank) {
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          comm_jitter(p.err, static_cast<uint32_t>(tile_in_chunk));
          st_release_sys(p.rs_flags[chunk] + (static_cast<long long>(tile_in_chunk) * p.ws + p.tp_rank) * 8 + warp_slot,
                         p.epoch);
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
  } else if (p.comm == COMM_AG) {
    // ------------------------------------------------------------------ all-gather push (warps 6..9, both CTAs)
    const long long chunk_rows = static_cast<long long>(p.tiles_m_chunk) * (2 * BM);
    const int kv = p.K >> 3;
    const long long total = chunk_rows * kv;
    const int pt = threadIdx.x - 192;
    const long long stride = static_cast<long long>(gridDim.x) * 128;
    long long v = static_cast<long long>(blockIdx.x) * 128 + pt;
    constexpr int U = 4;
    for (; v + (U - 1) * stride < total; v += U * stride) {
      uint4 x[U];
      long long off[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long vv = v + u * stride;
        const long long r = vv / kv;
        const int c = static_cast<int>(vv - r * kv) * 8;
        x[u] = *reinterpret_cast<const uint4*>(p.ag_src + r * p.ag_ld + c);
        off[u] = (p.tp_rank * chunk_rows + r) * p.K + c;
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
        for (int q = 0; q < p.ws; ++q) *reinterpret_cast<uint4*>(p.ag_dst[q] + off[u]) = x[u];
    }
    for (; v < total; v += stride) {
      const long long r = v / kv;
      const int c = static_cast<int>(v - r * kv) * 8;
      const uint4 x = *reinterpret_cast<const uint4*>(p.ag_src + r * p.ag_ld + c);
      for (int q = 0; q < p.ws; ++q) *reinterpret_cast<uint4*>(p.ag_dst[q] + (p.tp_rank * chunk_rows + r) * p.K + c) = x;
    }
    __threadfence_system();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (pt < p.ws && pt != p.tp_rank) {
      comm_jitter(p.err, static_cast<uint32_t>(pt));
      st_release_sys(p.ag_flags[pt] + p.tp_rank * 256 + blockIdx.x, p.epoch);
    }
    for (int order = 1; order < p.ws; ++order) {
      const int chunk = (p.tp_rank + order) % p.ws;
      bool ok = true;
      for (int c = pt; c < static_cast<int>(gridDim.x) && ok; c += 128)
        ok = wait_flag_ge(p.ag_flags[p.tp_rank] + chunk * 256 + c, p.epoch, p.err, 19);
      if (!ok) *ag_abort = 1;
      __threadfence_block();
      __syncwarp();
      if (lane == 0) mbar_arrive(ag_bar(order - 1));
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
static int launch2(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmA2, const Params& p,
                   cudaStream_t stream) {
  auto kern = gemm2_kernel<A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    NX_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DYN_BYTES));
    configured = true;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int max_pairs = sm_count() / 2;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  kern<<<2 * pairs, THREADS, DYN_BYTES, stream>>>(tmA, tmB, tmA2, p);     // cluster dims are compiled in
  NX_LAUNCH_CHECK();
  return NX_OK;
}

}  // namespace g2

struct Comm2Args {
  int mode = 0, rank = 0, ws = 1;
  unsigned int epoch = 0;
  const unsigned long long* data_ptrs = nullptr;
  const unsigned long long* flag_ptrs = nullptr;
  const void* residual2 = nullptr;
  long long ld_res2 = 0;
  const void* ag_src = nullptr;
  long long ag_ld = 0;
  const unsigned long long* ar_out_ptrs = nullptr;     // all-reduce mode: per-rank [M, N] outputs
  const unsigned long long* ar_count_ptrs = nullptr;   // and delivery counters
};

// NEOX_RS_ORDER=chunks selects the older order (all peers' chunks first); default: interleaved.
static bool rs_interleave() {
  static const bool on = [] {
    const char* e = getenv("NEOX_RS_ORDER");
    return !(e != nullptr && e[0] == 'c');
  }();
  return on;
}

static int gemm2_common(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                        long long ldc, int transA, int transB, const void* bias, const void* aux_in, void* aux_out,
                        const void* residual, long long ld_aux, int flags, float alpha, const Comm2Args& ca,
                        cudaStream_t s) {
  using namespace g2;
  if (M <= 0 || N <= 0) return NX_OK;
  NX_REQUIRE(K > 0, "gemm2: K must be positive");
  NX_REQUIRE(N % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0, "gemm2: N / lda / ldb must be multiples of 8");
  NX_REQUIRE(ldc % ((flags & OUT_F32) ? 4 : 8) == 0, "gemm2: ldc alignment");
  NX_REQUIRE((reinterpret_cast<uintptr_t>(C) & 15) == 0, "gemm2: C must be 16-byte aligned");
  if (flags & (DGELU_ERF | DGELU_TANH | MUL_AUX))
    NX_REQUIRE(aux_in != nullptr && ld_aux % 8 == 0, "gemm2: aux_in is required by the epilogue flags");
  if (flags & AUX_OUT) NX_REQUIRE(aux_out != nullptr && ld_aux % 8 == 0, "gemm2: aux_out is required by the flags");
  if (flags & RESIDUAL) NX_REQUIRE(residual != nullptr && ld_aux % 8 == 0, "gemm2: residual is required by the flags");
  if (flags & BIAS) NX_REQUIRE(bias != nullptr, "gemm2: bias is required by the flags");
  CUtensorMap tmA, tmB, tmA2;
  bool ok;
  if (!transA) ok = make_tma_2d(&tmA, A, M, K, lda * 2, BM, BK, 2);
  else         ok = make_tma_2d(&tmA, A, K, M, lda * 2, BK, 64, 2);
  if (!ok) return NX_ERR_ARG;
  if (!transB) ok = make_tma_2d(&tmB, B, N, K, ldb * 2, BNH, BK, 2);
  else         ok = make_tma_2d(&tmB, B, K, N, ldb * 2, BK, 64, 2);
  if (!ok) return NX_ERR_ARG;
  tmA2 = tmA;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc;
  p.bias = static_cast<const h16*>(bias);
  p.aux_in = static_cast<const h16*>(aux_in);
  p.aux_out = static_cast<h16*>(aux_out);
  p.residual = static_cast<const h16*>(residual);
  p.ld_aux = ld_aux; p.flags = flags; p.alpha = alpha;
  p.tiles_m = (M + 2 * BM - 1) / (2 * BM);
  p.tiles_n = (N + BN - 1) / BN;
  p.err = device_error_word();
  p.comm = ca.mode;
  p.num_slots = p.tiles_m * p.tiles_n;
  p.rs_lag = 0;
  if (ca.mode != COMM_NONE) {
    NX_REQUIRE(ca.ws >= 2 && ca.ws <= 8 && ca.rank >= 0 && ca.rank < ca.ws, "gemm2_comm: bad rank/world %d/%d", ca.rank, ca.ws);
    NX_REQUIRE(!transA && M % (ca.ws * 2 * BM) == 0, "gemm2_comm: row-major A and M (%d) %% (ws * 256) == 0 required", M);
    NX_REQUIRE(!(flags & (OUT_F32 | ACCUM)), "gemm2_comm: fp32 / accumulate outputs are not supported");
    NX_REQUIRE(ca.data_ptrs != nullptr && ca.flag_ptrs != nullptr, "gemm2_comm: null peer tables");
    p.tp_rank = ca.rank; p.ws = ca.ws; p.epoch = ca.epoch;
    p.tiles_m_chunk = (M / ca.ws) / (2 * BM);
    if ((ca.mode == COMM_RS || ca.mode == COMM_AR) && rs_interleave()) {
      // own tiles trail the peers' by a little more than one wave of CTA pairs
      const int tiles = p.tiles_m * p.tiles_n;
      const int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
      p.rs_lag = (pairs + ca.ws - 1) / ca.ws + 4;
      p.num_slots = ca.ws * (p.tiles_m_chunk * p.tiles_n + p.rs_lag);
    }
    for (int i = 0; i < ca.ws; ++i) {
      if (ca.mode == COMM_RS || ca.mode == COMM_AR) {
        p.rs_stage[i] = reinterpret_cast<h16*>(ca.data_ptrs[i]);
        p.rs_flags[i] = reinterpret_cast<uint32_t*>(ca.flag_ptrs[i]);
        if (ca.mode == COMM_AR) {
          NX_REQUIRE(ca.ar_out_ptrs != nullptr && ca.ar_count_ptrs != nullptr, "gemm2_comm: all-reduce tables are null");
          p.ar_out[i] = reinterpret_cast<h16*>(ca.ar_out_ptrs[i]);
          p.ar_count[i] = reinterpret_cast<uint32_t*>(ca.ar_count_ptrs[i]);
        }
      } else {
        p.ag_dst[i] = reinterpret_cast<h16*>(ca.data_ptrs[i]);
        p.ag_flags[i] = reinterpret_cast<uint32_t*>(ca.flag_ptrs[i]);
      }
    }
    p.residual2 = static_cast<const h16*>(ca.residual2);
    p.ld_res2 = ca.ld_res2;
    p.ag_src = static_cast<const h16*>(ca.ag_src);
    p.ag_ld = ca.ag_ld;
    if (ca.mode != COMM_AG && ca.residual2 != nullptr) NX_REQUIRE(ca.ld_res2 % 8 == 0, "gemm2_comm: residual2 ld");
    if (ca.mode == COMM_AG) {
      NX_REQUIRE(ca.ag_src != nullptr && ca.ag_ld % 8 == 0 && K % 8 == 0 && lda == K,
                 "gemm2_comm: all-gather mode needs a dense [M, K] gather buffer and an aligned shard");
      NX_REQUIRE(sm_count() <= 256, "gemm2_comm: flag table holds 256 CTAs per rank");
      if (!make_tma_2d(&tmA2, ca.ag_src, M / ca.ws, K, ca.ag_ld * 2, BM, BK, 2)) return NX_ERR_ARG;
    }
  }
  if (!transA && !transB) return launch2<false, false>(tmA, tmB, tmA2, p, s);
  if (!transA && transB) return launch2<false, true>(tmA, tmB, tmA2, p, s);
  if (transA && !transB) return launch2<true, false>(tmA, tmB, tmA2, p, s);
  return launch2<true, true>(tmA, tmB, tmA2, p, s);
}

// Same arguments as nx_gemm_bf16.
NX_API int NX_SYM(nx_gemm2_bf16)(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                         long long ldc, int transA, int transB, const void* bias, const void* aux_in, void* aux_out,
                         const void* residual, long long ld_aux, int flags, float alpha, void* stream_) {
  Comm2Args ca;
  return gemm2_common(A, B, C, M, N, K, lda, ldb, ldc, transA, transB, bias, aux_in, aux_out, residual, ld_aux, flags,
                      alpha, ca, static_cast<cudaStream_t>(stream_));
}

// Same arguments as nx_gemm_bf16_comm; reduce-scatter flags are laid out [tile][src rank][8 warp bands].
NX_API int NX_SYM(nx_gemm2_bf16_comm)(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                              long long ldc, int transB, const void* bias, const void* aux_in, void* aux_out,
                              const void* residual, long long ld_aux, int flags, int mode, int rank, int ws,
                              unsigned int epoch, const unsigned long long* data_ptrs,
                              const unsigned long long* flag_ptrs, const void* residual2, long long ld_res2,
                              const void* ag_src, long long ag_ld, void* stream_) {
  Comm2Args ca;
  ca.mode = mode; ca.rank = rank; ca.ws = ws; ca.epoch = epoch;
  ca.data_ptrs = data_ptrs; ca.flag_ptrs = flag_ptrs;
  ca.residual2 = residual2; ca.ld_res2 = ld_res2; ca.ag_src = ag_src; ca.ag_ld = ag_ld;
  return gemm2_common(A, B, C, M, N, K, lda, ldb, ldc, 0, transB, bias, aux_in, aux_out, residual, ld_aux, flags, 1.0f,
                      ca, static_cast<cudaStream_t>(stream_));
}

namespace g2 {
// Bounded wait until the delivery counter reaches `target` (all peers' reduced tiles have landed).
__global__ void wait_counter_kernel(const uint32_t* counter, uint32_t target, int* err) {
  if (threadIdx.x == 0) wait_flag_ge(counter, target, err, 20);
}
}  // namespace g2

// GEMM -> all-reduce over the rows' owners: reduce-scatter as in mode 1, then every owner writes its reduced
// chunk (+ bias) into each rank's [M, N] output (out_ptrs, leading dimension N) and counts deliveries;
// a one-thread kernel behind the GEMM waits (bounded) until this rank has received `count_target` bands.
NX_API int NX_SYM(nx_gemm2_bf16_allreduce)(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                                   int transB, const void* bias, const void* residual, long long ld_aux, int flags,
                                   int rank, int ws, unsigned int epoch, const unsigned long long* stage_ptrs,
                                   const unsigned long long* flag_ptrs, const unsigned long long* out_ptrs,
                                   const unsigned long long* count_ptrs, unsigned int count_target, void* stream_) {
  Comm2Args ca;
  ca.mode = 3; ca.rank = rank; ca.ws = ws; ca.epoch = epoch;
  ca.data_ptrs = stage_ptrs; ca.flag_ptrs = flag_ptrs;
  ca.ar_out_ptrs = out_ptrs; ca.ar_count_ptrs = count_ptrs;
  void* c_local = reinterpret_cast<void*>(out_ptrs[rank]);
  int st = gemm2_common(A, B, c_local, M, N, K, lda, ldb, N, 0, transB, bias, nullptr, nullptr, residual, ld_aux, flags,
                        1.0f, ca, static_cast<cudaStream_t>(stream_));
  if (st != NX_OK) return st;
  g2::wait_counter_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(
      reinterpret_cast<const uint32_t*>(count_ptrs[rank]), count_target, device_error_word());
  NX_LAUNCH_CHECK();
  return NX_OK;
}

// The delivery wait on its own: returns once *counter >= target or the wait budget ran out (then the
// device error word holds {ERR_PEER_TIMEOUT, site 20}).
NX_API int NX_SYM(nx_wait_counter)(const void* counter, unsigned int target, void* stream_) {
  g2::wait_counter_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(static_cast<const uint32_t*>(counter), target,
                                                                            device_error_word());
  NX_LAUNCH_CHECK();
  return NX_OK;
}

}  // namespace nx
