// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory),
// operands staged by TMA into a 128-byte-swizzled shared-memory ring.
//
// Replaces the cuBLAS calls behind every dense projection of the reference
// (megatron/mpu/layers.py:576,773 and megatron/model/transformer.py:1240-1242) and fuses the
// element-wise work the reference runs as separate torch.jit kernels
// (megatron/model/activations.py:78-112, megatron/model/fused_bias_dropout.py:44-55) into the
// epilogue.
//
// Kernel shape: persistent, one CTA per SM, 192 threads:
//   warp 0      TMA producer  (one elected lane)
//   warp 1      TMEM allocator + tcgen05.mma issuer (one elected lane)
//   warps 2..5  epilogue: tcgen05.ld from TMEM -> registers -> fused math -> global stores
// Tile 128 x BN x 64 with a STAGES-deep operand ring and two TMEM accumulators, so the
// epilogue of tile i overlaps the main loop of tile i+1.
//
// Operand layouts (all row-major in memory):
//   transA = 0: A is [M, K]  (K contiguous)      transA = 1: A is [K, M]  (M contiguous)
//   transB = 0: B is [N, K]  (K contiguous, the nn.Linear weight layout)
//   transB = 1: B is [K, N]  (N contiguous)
// so that  forward = (0,0),  input-gradient = (0,1),  weight-gradient = (1,1).
#include <string.h>

#include "common.h"
#include "ptx.cuh"

namespace nx {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 320;   // producer, MMA issuer, 4 epilogue warps, 4 all-gather push warps
constexpr int RS_ROW_BYTES = 144;    // 64 bf16 columns + 16 B pad: conflict-free 16-byte rows in shared memory
constexpr int RS_STAGE_BYTES = 4 * 32 * RS_ROW_BYTES;   // one 32-row x 64-column slab per epilogue warp

enum EpiFlags : int {
  EPI_BIAS = 1,         // + bias[n]
  EPI_GELU_ERF = 2,     // exact GeLU
  EPI_GELU_TANH = 4,    // tanh-approximated GeLU
  EPI_AUX_OUT = 8,      // store the pre-activation (after bias) as bf16 into aux_out
  EPI_DGELU_ERF = 16,   // multiply by gelu_erf'(aux_in)
  EPI_DGELU_TANH = 32,  // multiply by gelu_tanh'(aux_in)
  EPI_RESIDUAL = 64,    // + residual (bf16, same shape / leading dimension as aux ld)
  EPI_ACCUM = 128,      // C += result (read-modify-write)
  EPI_OUT_F32 = 256,    // C is fp32 instead of bf16
  EPI_SCALE = 512,      // result *= alpha (applied first)
  EPI_AUX_DERIV = 1024, // with AUX_OUT + a GeLU flag: aux_out receives gelu'(pre-activation) instead of it, so
                        // that the backward GEMM's epilogue is one multiply (EPI_MUL_AUX) with no erf / exp
  EPI_MUL_AUX = 2048,   // multiply by aux_in
};

struct GemmParams {
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
  int tiles_m, tiles_n;
  int* err;
  // ---- grouped (mixture-of-experts) modes; group_mode == GROUP_NONE leaves them unused
  //  GROUP_ROWS: the rows of A / C are expert segments aligned to BM; grp_tile_expert[tm] names the expert of
  //              row tile tm (-1: tile unused); B holds the experts' matrices stacked, grp_b_rows apart.
  //  GROUP_K   : one output matrix per expert (grp_c_stride apart), reduction over the expert's row segment
  //              [grp_row_offsets[e], grp_row_offsets[e+1]) of MN-major A and B (weight gradients).
  int group_mode, total_tiles;
  const int* grp_tile_expert;
  const int* grp_row_offsets;
  int grp_b_rows;
  long long grp_c_stride;
  // ---- fused collective (tensor-parallel group of `ws` ranks, this rank = `rank`); comm == COMM_NONE
  //      leaves everything below unused
  int comm, rank, ws;
  int tiles_m_chunk;            // row tiles per rank chunk: (M / ws) / BM
  uint32_t epoch;               // value written to / expected in the flags of this call
  // COMM_RS (GEMM -> reduce-scatter over rows): C points to this rank's [M/ws, N] output.
  h16* rs_stage[8];   // on rank q: staging area [ws][M/ws, N]; slot = source rank
  uint32_t* rs_flags[8];        // on rank q: flags[tile_in_chunk][src][4 epilogue warps]
  const h16* residual2;  // [M/ws, N] added on the owner after the reduction (may be null)
  long long ld_res2;
  // COMM_AG (all-gather over rows -> GEMM): A's shard is pushed to every rank's gather buffer first
  const h16* ag_src;  // this rank's shard [M/ws, K], leading dimension ag_ld
  long long ag_ld;
  h16* ag_dst[8];     // on rank q: gather buffer [M, K] (dense, leading dimension K)
  uint32_t* ag_flags[8];        // on rank q: flags[src][cta]
};

enum CommMode : int { COMM_NONE = 0, COMM_RS = 1, COMM_AG = 2 };
enum GroupMode : int { GROUP_NONE = 0, GROUP_ROWS = 1, GROUP_K = 2 };

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], tmem base word
  static constexpr int RS_OFFSET = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 8 * 8;   // + 8 chunk-ready barriers
  static constexpr int TOTAL = RS_OFFSET + RS_STAGE_BYTES;
  static constexpr int DYN_BYTES = TOTAL + 1024;  // slack for manual 1024-byte alignment
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  // Group 8 row-tiles together so that concurrently running CTAs share B panels in L2.
  constexpr int GROUP = 8;
  const int per_group = GROUP * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP;
  const int gsize = min(GROUP, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + (r % gsize);
  tn = r / gsize;
}

// Tile order under a fused collective: whole rank-chunks of rows at a time.  Reduce-scatter computes the
// peers' chunks first (so they can finish early) and its own last; all-gather computes its own
// chunk first (its operand is already local) and the peers' as their shards arrive.
__device__ __forceinline__ void tile_coords_p(int tile, const GemmParams& p, int& tm, int& tn, int& chunk) {
  if (p.comm == COMM_NONE) {
    tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
    chunk = 0;
    return;
  }
  const int per_chunk = p.tiles_m_chunk * p.tiles_n;
  const int order = tile / per_chunk;
  chunk = p.comm == COMM_RS ? (p.rank + 1 + order) % p.ws : (p.rank + order) % p.ws;
  int tl;
  tile_coords(tile - order * per_chunk, p.tiles_m_chunk, p.tiles_n, tl, tn);
  tm = chunk * p.tiles_m_chunk + tl;
}


// Grouped modes: expert of the tile and the range of K blocks it reduces over.  Returns false for a tile
// that has no work (unused row tile / expert without rows); every warp role skips it the same way.
__device__ __forceinline__ bool group_tile(int tile, const GemmParams& p, int num_kb, int& tm, int& tn, int& chunk,
                                           int& e, int& kb0, int& kb1) {
  e = 0;
  kb0 = 0;
  kb1 = num_kb;
  if (p.group_mode == GROUP_K) {
    const int per = p.tiles_m * p.tiles_n;
    e = tile / per;
    chunk = 0;
    tile_coords(tile - e * per, p.tiles_m, p.tiles_n, tm, tn);
    kb0 = p.grp_row_offsets[e] / BK;
    kb1 = p.grp_row_offsets[e + 1] / BK;
    return kb1 > kb0;
  }
  tile_coords_p(tile, p, tm, tn, chunk);
  if (p.group_mode == GROUP_ROWS) {
    e = p.grp_tile_expert[tm];
    return e >= 0;
  }
  return true;
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmA2, const GemmParams p) {
  using L = SmemLayout<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t bar_base = smem_base + L::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);
  // all-gather mode: barrier k completes when the k-th peer chunk (in consumption order) has arrived
  auto ag_bar = [&](int k) { return bar_base + 8u * (2 * STAGES + 6 + k); };
  volatile int* ag_abort = reinterpret_cast<volatile int*>(smem_gen + L::BAR_OFFSET + 8 * (2 * STAGES + 5));
  volatile uint32_t* tmem_slot_gen =
      reinterpret_cast<volatile uint32_t*>(smem_gen + L::BAR_OFFSET + 8 * (2 * STAGES + 4));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), 4);  // one arrival per epilogue warp
    }
    for (int k = 0; k < 8; ++k) mbar_init(ag_bar(k), 4);  // one arrival per push warp
    *ag_abort = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;

  const int num_tiles = p.total_tiles;
  const int num_kb = (p.K + BK - 1) / BK;
  bool aborted = false;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int ag_ready_chunk = -1;
      for (int tile = blockIdx.x; tile < num_tiles && !aborted; tile += gridDim.x) {
        int tm, tn, chunk, ge, kb0, kb1;
        if (!group_tile(tile, p, num_kb, tm, tn, chunk, ge, kb0, kb1)) continue;
        int m0 = tm * BM;
        const int n0 = tn * BN;
        const int b_off = p.group_mode == GROUP_ROWS ? ge * p.grp_b_rows : 0;   // expert's block of stacked B
        const CUtensorMap* mapA = &tmA;
        if (p.comm == COMM_AG) {
          if (chunk == p.rank) {
            // own shard: read it where it already is
            mapA = &tmA2;
            m0 -= chunk * p.tiles_m_chunk * BM;
          } else if (chunk != ag_ready_chunk) {
            // peer shard: the push warps poll the peer's per-CTA flags in parallel and complete the
            // chunk's barrier; then make those generic-proxy writes visible to TMA
            const int order = (chunk - p.rank + p.ws) % p.ws;     // 1 .. ws-1
            if (!mbar_wait(ag_bar(order - 1), 0, p.err, 7) || *ag_abort) {
              aborted = true;
              break;
            }
            asm volatile("fence.proxy.async;" ::: "memory");
            ag_ready_chunk = chunk;
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, p.err, 1)) {
            aborted = true;
            break;
          }
          const uint32_t a_dst = smem_base + stage * L::STAGE_BYTES;
          const uint32_t b_dst = a_dst + L::A_BYTES;
          mbar_expect_tx(full_bar(stage), L::STAGE_BYTES);
          const int k0 = kb * BK;
          if constexpr (!A_MN) {
            tma_load_2d(a_dst, mapA, full_bar(stage), k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(a_dst + j * (BK * 128), &tmA, full_bar(stage), m0 + j * 64, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(b_dst, &tmB, full_bar(stage), k0, n0 + b_off);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(b_dst + j * (BK * 128), &tmB, full_bar(stage), n0 + j * 64, k0 + b_off);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      // K-major: 8-row groups are 1024 B apart (SBO), 16 K-elements advance 32 B.
      // MN-major: 64-element column blocks are BK*128 B apart (LBO), 8-row K groups 1024 B
      // apart (SBO), 16 K-rows advance 2048 B.
      constexpr uint32_t A_LBO = A_MN ? BK * 128 : 0, B_LBO = B_MN ? BK * 128 : 0;
      constexpr uint32_t A_KADV = A_MN ? UMMA_K * 128 : UMMA_K * 2;
      constexpr uint32_t B_KADV = B_MN ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !aborted; tile += gridDim.x) {
        int tm_, tn_, chunk_, ge_, kb0, kb1;
        if (!group_tile(tile, p, num_kb, tm_, tn_, chunk_, ge_, kb0, kb1)) continue;
        if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1, p.err, 2)) {
          aborted = true;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, p.err, 3)) {
            aborted = true;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_base + stage * L::STAGE_BYTES;
          const uint32_t b_addr = a_addr + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = umma_smem_desc_sw128(a_addr + k * A_KADV, A_LBO, 1024);
            const uint64_t bdesc = umma_smem_desc_sw128(b_addr + k * B_KADV, B_LBO, 1024);
            umma_bf16_ss(d_tmem, adesc, bdesc, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));  // frees the smem slot once these MMAs retire
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (aborted) break;
        umma_commit(tmem_full_bar(acc));  // accumulator complete -> epilogue
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    const int flags = p.flags;
    const long long chunk_rows = static_cast<long long>(p.tiles_m_chunk) * BM;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int tm, tn, chunk, ge, kb0_, kb1_;
      if (!group_tile(tile, p, num_kb, tm, tn, chunk, ge, kb0_, kb1_)) continue;
      const int m0 = tm * BM, n0 = tn * BN;
      const long long c_off = p.group_mode == GROUP_K ? ge * p.grp_c_stride : 0;
      if (!mbar_wait(tmem_full_bar(acc), acc_phase, p.err, 4)) {
        aborted = true;
        break;
      }
      tc_fence_after_sync();
      const long long row = m0 + row_in_tile;
      const bool row_ok = row < p.M;
      const int tile_in_chunk = (tm - chunk * p.tiles_m_chunk) * p.tiles_n + tn;
      if (p.comm == COMM_RS && chunk == p.rank) {
        // own rows: every peer's four epilogue warps must have delivered this tile
        bool ok = true;
        if (lane < p.ws * 4 && (lane >> 2) != p.rank)
          ok = wait_flag_ge(p.rs_flags[p.rank] + (static_cast<long long>(tile_in_chunk) * p.ws) * 4 + lane, p.epoch,
                            p.err, 8);
        if (!__all_sync(0xffffffffu, ok)) {
          aborted = true;
          break;
        }
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;  // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(quad * 32) << 16), r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (flags & EPI_SCALE) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
        }
        if ((flags & EPI_BIAS) && p.comm != COMM_RS) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (col0 + j < p.N) {
              const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.bias + col0 + j));
              const float2 b0 = unpack_h16x2(b.x), b1 = unpack_h16x2(b.y),
                           b2 = unpack_h16x2(b.z), b3 = unpack_h16x2(b.w);
              v[j + 0] += b0.x; v[j + 1] += b0.y; v[j + 2] += b1.x; v[j + 3] += b1.y;
              v[j + 4] += b2.x; v[j + 5] += b2.y; v[j + 6] += b3.x; v[j + 7] += b3.y;
            }
          }
        }
        if (row_ok) {
          if (flags & EPI_AUX_OUT) {
            h16* ap = p.aux_out + row * p.ld_aux + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < p.N) {
                float d[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                  d[q] = v[j + q];
                  if (flags & EPI_AUX_DERIV) {   // derivative out, activation in place (the GeLU step below is skipped)
                    if (flags & EPI_GELU_TANH) gelu_tanh_both(v[j + q], v[j + q], d[q]);
                    else gelu_erf_both(v[j + q], v[j + q], d[q]);
                  }
                }
                uint4 o;
                o.x = pack_h16x2(d[0], d[1]);
                o.y = pack_h16x2(d[2], d[3]);
                o.z = pack_h16x2(d[4], d[5]);
                o.w = pack_h16x2(d[6], d[7]);
                *reinterpret_cast<uint4*>(ap + j) = o;
              }
            }
          }
          if (flags & (EPI_DGELU_ERF | EPI_DGELU_TANH | EPI_MUL_AUX)) {
            const h16* ap = p.aux_in + row * p.ld_aux + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < p.N) {
                const uint4 a = *reinterpret_cast<const uint4*>(ap + j);
                const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const float2 x = unpack_h16x2(aw[q]);
                  if (flags & EPI_MUL_AUX) {
                    v[j + 2 * q] *= x.x;
                    v[j + 2 * q + 1] *= x.y;
                  } else if (flags & EPI_DGELU_ERF) {
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
          if (flags & EPI_AUX_DERIV) {
            // activation already applied together with its derivative
          } else if (flags & EPI_GELU_ERF) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
          } else if (flags & EPI_GELU_TANH) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
          }
          if (flags & EPI_RESIDUAL) {
            const h16* rp = p.residual + row * p.ld_aux + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < p.N) {
                const uint4 a = *reinterpret_cast<const uint4*>(rp + j);
                const float2 x0 = unpack_h16x2(a.x), x1 = unpack_h16x2(a.y),
                             x2 = unpack_h16x2(a.z), x3 = unpack_h16x2(a.w);
                v[j + 0] += x0.x; v[j + 1] += x0.y; v[j + 2] += x1.x; v[j + 3] += x1.y;
                v[j + 4] += x2.x; v[j + 5] += x2.y; v[j + 6] += x3.x; v[j + 7] += x3.y;
              }
            }
          }
          if (p.comm == COMM_RS) {
            const long long crow = row - chunk * chunk_rows;
            if (chunk != p.rank) {
              // partial tile of a peer's rows: goes into that peer's staging slot for this rank.  A lane owns
              // a row, so direct stores would scatter 16-byte pieces over 32 rows per instruction; two column
              // groups are transposed through shared memory and leave as full 128-byte lines instead.
              uint8_t* slab = smem_gen + L::RS_OFFSET + (warp - 2) * (32 * RS_ROW_BYTES);
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 o;
                o.x = pack_h16x2(v[j], v[j + 1]);
                o.y = pack_h16x2(v[j + 2], v[j + 3]);
                o.z = pack_h16x2(v[j + 4], v[j + 5]);
                o.w = pack_h16x2(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4*>(slab + lane * RS_ROW_BYTES + (c & 1) * 64 + j * 2) = o;
              }
              const bool last_group = (c == BN / 32 - 1) || (col0 + 32 >= p.N);
              if ((c & 1) || last_group) {
                __syncwarp();
                const int colp = n0 + (c & ~1) * 32;            // first column of the pair
                const int oct = lane & 7;
                const long long base_row = (p.rank * chunk_rows + (m0 + quad * 32 - chunk * chunk_rows));
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
                if (sr == p.rank) continue;
                const h16* sp = p.rs_stage[p.rank] + (sr * chunk_rows + crow) * p.N + col0;
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  if (col0 + j < p.N) {
                    const uint4 a = *reinterpret_cast<const uint4*>(sp + j);
                    const float2 x0 = unpack_h16x2(a.x), x1 = unpack_h16x2(a.y),
                                 x2 = unpack_h16x2(a.z), x3 = unpack_h16x2(a.w);
                    v[j + 0] += x0.x; v[j + 1] += x0.y; v[j + 2] += x1.x; v[j + 3] += x1.y;
                    v[j + 4] += x2.x; v[j + 5] += x2.y; v[j + 6] += x3.x; v[j + 7] += x3.y;
                  }
                }
              }
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                if (col0 + j < p.N) {
                  if (flags & EPI_BIAS) {
                    const uint4 b = __ldg(reinterpret_cast<const uint4*>(p.bias + col0 + j));
                    const float2 b0 = unpack_h16x2(b.x), b1 = unpack_h16x2(b.y),
                                 b2 = unpack_h16x2(b.z), b3 = unpack_h16x2(b.w);
                    v[j + 0] += b0.x; v[j + 1] += b0.y; v[j + 2] += b1.x; v[j + 3] += b1.y;
                    v[j + 4] += b2.x; v[j + 5] += b2.y; v[j + 6] += b3.x; v[j + 7] += b3.y;
                  }
                  if (p.residual2 != nullptr) {
                    const uint4 a = *reinterpret_cast<const uint4*>(p.residual2 + crow * p.ld_res2 + col0 + j);
                    const float2 x0 = unpack_h16x2(a.x), x1 = unpack_h16x2(a.y),
                                 x2 = unpack_h16x2(a.z), x3 = unpack_h16x2(a.w);
                    v[j + 0] += x0.x; v[j + 1] += x0.y; v[j + 2] += x1.x; v[j + 3] += x1.y;
                    v[j + 4] += x2.x; v[j + 5] += x2.y; v[j + 6] += x3.x; v[j + 7] += x3.y;
                  }
                  uint4 o;
                  o.x = pack_h16x2(v[j], v[j + 1]);
                  o.y = pack_h16x2(v[j + 2], v[j + 3]);
                  o.z = pack_h16x2(v[j + 4], v[j + 5]);
                  o.w = pack_h16x2(v[j + 6], v[j + 7]);
                  *reinterpret_cast<uint4*>(reinterpret_cast<h16*>(p.C) + crow * p.ldc + col0 + j) = o;
                }
              }
            }
          } else if (flags & EPI_OUT_F32) {
            float* cp = reinterpret_cast<float*>(p.C) + c_off + row * p.ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col0 + j < p.N) {
                float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                if (flags & EPI_ACCUM) {
                  const float4 old = *reinterpret_cast<const float4*>(cp + j);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(cp + j) = o;
              }
            }
          } else {
            h16* cp = reinterpret_cast<h16*>(p.C) + c_off + row * p.ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < p.N) {
                if (flags & EPI_ACCUM) {
                  const uint4 a = *reinterpret_cast<const uint4*>(cp + j);
                  const float2 x0 = unpack_h16x2(a.x), x1 = unpack_h16x2(a.y),
                               x2 = unpack_h16x2(a.z), x3 = unpack_h16x2(a.w);
                  v[j + 0] += x0.x; v[j + 1] += x0.y; v[j + 2] += x1.x; v[j + 3] += x1.y;
                  v[j + 4] += x2.x; v[j + 5] += x2.y; v[j + 6] += x3.x; v[j + 7] += x3.y;
                }
                uint4 o;
                o.x = pack_h16x2(v[j], v[j + 1]);
                o.y = pack_h16x2(v[j + 2], v[j + 3]);
                o.z = pack_h16x2(v[j + 4], v[j + 5]);
                o.w = pack_h16x2(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4*>(cp + j) = o;
              }
            }
          }
        }
      }
      if (p.comm == COMM_RS && chunk != p.rank) {
        // this warp's 32 rows of the tile are in the peer's memory: publish them
        __threadfence_system();
        __syncwarp();
        if (lane == 0)
          st_release_sys(p.rs_flags[chunk] + (static_cast<long long>(tile_in_chunk) * p.ws + p.rank) * 4 + quad,
                         p.epoch);
      }
      // This warp is done reading the accumulator: hand it back to the MMA issuer.
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar(acc));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  } else if (p.comm == COMM_AG) {
    // ------------------------------------------------------------------ all-gather push (warps 6..9)
    // Copy this rank's shard of A into every rank's gather buffer (coalesced 16-byte peer stores over
    // NVLink, several loads in flight per thread) while the main loop already works on the local chunk;
    // then publish "CTA b of rank r is done".  Kept off the epilogue warps so that accumulators drain
    // while the push is running.
    const long long chunk_rows = static_cast<long long>(p.tiles_m_chunk) * BM;
    const int kv = p.K >> 3;
    const long long total = chunk_rows * kv;
    const int pt = threadIdx.x - 192;  // 0..127 among the push threads
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
        off[u] = (p.rank * chunk_rows + r) * p.K + c;
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
        for (int q = 0; q < p.ws; ++q) *reinterpret_cast<uint4*>(p.ag_dst[q] + off[u]) = x[u];
    }
    for (; v < total; v += stride) {
      const long long r = v / kv;
      const int c = static_cast<int>(v - r * kv) * 8;
      const uint4 x = *reinterpret_cast<const uint4*>(p.ag_src + r * p.ag_ld + c);
      for (int q = 0; q < p.ws; ++q)
        *reinterpret_cast<uint4*>(p.ag_dst[q] + (p.rank * chunk_rows + r) * p.K + c) = x;
    }
    __threadfence_system();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (pt < p.ws && pt != p.rank) st_release_sys(p.ag_flags[pt] + p.rank * 256 + blockIdx.x, p.epoch);
    // wait for the peers' shards in the order the main loop consumes them: 128 threads poll the
    // gridDim.x flags of a chunk in parallel (one dependent acquire-load each instead of a serial chain)
    for (int order = 1; order < p.ws; ++order) {
      const int chunk = (p.rank + order) % p.ws;
      bool ok = true;
      for (int c = pt; c < static_cast<int>(gridDim.x) && ok; c += 128)
        ok = wait_flag_ge(p.ag_flags[p.rank] + chunk * 256 + c, p.epoch, p.err, 7);
      if (!ok) *ag_abort = 1;
      __threadfence_block();
      __syncwarp();
      if (lane == 0) mbar_arrive(ag_bar(order - 1));
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (aborted) {
    // A bounded wait ran out: give copies already in flight time to land before the CTA's
    // shared memory is released.
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmA2,
                       const GemmParams& p, cudaStream_t stream) {
  using L = SmemLayout<BN, STAGES>;
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    NX_CUDA_CHECK(
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_BYTES));
    configured = true;
  }
  const int tiles = p.total_tiles;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, GEMM_THREADS, L::DYN_BYTES, stream>>>(tmA, tmB, tmA2, p);
  NX_LAUNCH_CHECK();
  return NX_OK;
}

template <int BN, int STAGES>
static int dispatch_layout(int transA, int transB, const CUtensorMap& tmA, const CUtensorMap& tmB,
                           const CUtensorMap& tmA2, const GemmParams& p, cudaStream_t stream) {
  if (!transA && !transB) return launch_gemm<BN, STAGES, false, false>(tmA, tmB, tmA2, p, stream);
  if (!transA && transB) return launch_gemm<BN, STAGES, false, true>(tmA, tmB, tmA2, p, stream);
  if (transA && !transB) return launch_gemm<BN, STAGES, true, false>(tmA, tmB, tmA2, p, stream);
  return launch_gemm<BN, STAGES, true, true>(tmA, tmB, tmA2, p, stream);
}

}  // namespace nx

struct CommArgs {
  int mode = 0, rank = 0, ws = 1;
  unsigned int epoch = 0;
  const unsigned long long* data_ptrs = nullptr;  // per rank: RS staging area / AG gather buffer
  const unsigned long long* flag_ptrs = nullptr;  // per rank: flag array of that mode
  const void* residual2 = nullptr;
  long long ld_res2 = 0;
  const void* ag_src = nullptr;
  long long ag_ld = 0;
  // grouped (mixture-of-experts) modes
  int group_mode = 0, experts = 1;
  const int* tile_expert = nullptr;
  const int* row_offsets = nullptr;
  long long c_stride = 0;
};

static int gemm_common(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                       long long ldc, int transA, int transB, const void* bias, const void* aux_in, void* aux_out,
                       const void* residual, long long ld_aux, int flags, float alpha, const CommArgs& ca,
                       cudaStream_t stream) {
  using namespace nx;
  if (M <= 0 || N <= 0) return NX_OK;
  NX_REQUIRE(K > 0, "gemm: K must be positive");
  NX_REQUIRE(N % 8 == 0, "gemm: N (%d) must be a multiple of 8", N);
  NX_REQUIRE(lda % 8 == 0 && ldb % 8 == 0, "gemm: lda/ldb must be multiples of 8 elements");
  NX_REQUIRE(ldc % ((flags & EPI_OUT_F32) ? 4 : 8) == 0, "gemm: ldc alignment");
  NX_REQUIRE((reinterpret_cast<uintptr_t>(C) & 15) == 0, "gemm: C must be 16-byte aligned");
  if (flags & EPI_BIAS) NX_REQUIRE(bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 15) == 0, "gemm: bias null/unaligned");
  if (flags & (EPI_DGELU_ERF | EPI_DGELU_TANH | EPI_MUL_AUX))
    NX_REQUIRE(aux_in != nullptr && ld_aux % 8 == 0, "gemm: aux_in");
  if (flags & EPI_AUX_OUT) NX_REQUIRE(aux_out != nullptr && ld_aux % 8 == 0, "gemm: aux_out");
  if (flags & EPI_RESIDUAL) NX_REQUIRE(residual != nullptr && ld_aux % 8 == 0, "gemm: residual");

  const int BN = (N <= 128) ? 128 : 256;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.comm = ca.mode;
  if (ca.mode != COMM_NONE) {
    NX_REQUIRE(ca.ws >= 2 && ca.ws <= 8 && ca.rank >= 0 && ca.rank < ca.ws, "gemm_comm: bad rank/world %d/%d", ca.rank, ca.ws);
    NX_REQUIRE(!transA, "gemm_comm: A must be row-major [M, K]");
    NX_REQUIRE(M % (ca.ws * BM) == 0, "gemm_comm: M (%d) must be a multiple of ws * %d", M, BM);
    NX_REQUIRE(!(flags & (EPI_OUT_F32 | EPI_ACCUM)), "gemm_comm: fp32 / accumulate outputs are not supported");
    NX_REQUIRE(ca.data_ptrs != nullptr && ca.flag_ptrs != nullptr, "gemm_comm: null peer tables");
    p.rank = ca.rank; p.ws = ca.ws; p.epoch = ca.epoch;
    p.tiles_m_chunk = (M / ca.ws) / BM;
    for (int i = 0; i < ca.ws; ++i) {
      if (ca.mode == COMM_RS) {
        p.rs_stage[i] = reinterpret_cast<h16*>(ca.data_ptrs[i]);
        p.rs_flags[i] = reinterpret_cast<uint32_t*>(ca.flag_ptrs[i]);
      } else {
        p.ag_dst[i] = reinterpret_cast<h16*>(ca.data_ptrs[i]);
        p.ag_flags[i] = reinterpret_cast<uint32_t*>(ca.flag_ptrs[i]);
      }
    }
    p.residual2 = static_cast<const h16*>(ca.residual2);
    p.ld_res2 = ca.ld_res2;
    p.ag_src = static_cast<const h16*>(ca.ag_src);
    p.ag_ld = ca.ag_ld;
    if (ca.mode == COMM_RS && ca.residual2 != nullptr) NX_REQUIRE(ca.ld_res2 % 8 == 0, "gemm_comm: residual2 ld");
    if (ca.mode == COMM_AG) {
      NX_REQUIRE(ca.ag_src != nullptr && ca.ag_ld % 8 == 0 && K % 8 == 0 && lda == K,
                 "gemm_comm: all-gather mode needs a dense [M, K] gather buffer and an aligned shard");
      NX_REQUIRE(sm_count() <= 256, "gemm_comm: flag table holds 256 CTAs per rank");
    }
  }
  CUtensorMap tmA, tmB, tmA2;
  bool ok;
  if (!transA) ok = make_tma_2d(&tmA, A, M, K, lda * 2, BM, BK, 2);
  else         ok = make_tma_2d(&tmA, A, K, M, lda * 2, BK, 64, 2);
  if (!ok) return NX_ERR_ARG;
  const long long eb = ca.group_mode == GROUP_ROWS ? ca.experts : 1;    // stacked expert matrices
  if (!transB) ok = make_tma_2d(&tmB, B, eb * N, K, ldb * 2, BN, BK, 2);
  else         ok = make_tma_2d(&tmB, B, eb * K, N, ldb * 2, BK, 64, 2);
  if (!ok) return NX_ERR_ARG;
  tmA2 = tmA;
  if (ca.mode == COMM_AG) {
    if (!make_tma_2d(&tmA2, ca.ag_src, M / ca.ws, K, ca.ag_ld * 2, BM, BK, 2)) return NX_ERR_ARG;
  }
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.bias = static_cast<const h16*>(bias);
  p.aux_in = static_cast<const h16*>(aux_in);
  p.aux_out = static_cast<h16*>(aux_out);
  p.residual = static_cast<const h16*>(residual);
  p.ld_aux = ld_aux;
  p.flags = flags;
  p.alpha = alpha;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.total_tiles = p.tiles_m * p.tiles_n;
  p.group_mode = ca.group_mode;
  if (ca.group_mode == GROUP_ROWS) {
    NX_REQUIRE(!transA && ca.mode == COMM_NONE && ca.tile_expert != nullptr && M % BM == 0,
               "gemm_grouped: row mode needs row-major A, a tile->expert table and M %% %d == 0", BM);
    p.grp_tile_expert = ca.tile_expert;
    p.grp_b_rows = transB ? K : N;
  } else if (ca.group_mode == GROUP_K) {
    NX_REQUIRE(transA && transB && ca.mode == COMM_NONE && ca.row_offsets != nullptr,
               "gemm_grouped: reduction mode needs MN-major A and B and the experts' row offsets");
    p.grp_row_offsets = ca.row_offsets;
    p.grp_c_stride = ca.c_stride;
    p.total_tiles = p.tiles_m * p.tiles_n * ca.experts;
  }
  p.err = device_error_word();
  if (BN == 128) return dispatch_layout<128, 6>(transA, transB, tmA, tmB, tmA2, p, stream);
  return dispatch_layout<256, 4>(transA, transB, tmA, tmB, tmA2, p, stream);
}

// C[M,N] = epilogue(op(A) * op(B)).  Leading dimensions in elements.  bias/aux/residual may be
// null when their flag is clear.  ld_aux is the leading dimension shared by aux_in, aux_out
// and residual.  Returns an NxStatus.
NX_API int NX_SYM(nx_gemm_bf16)(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                        long long ldb, long long ldc, int transA, int transB, const void* bias,
                        const void* aux_in, void* aux_out, const void* residual, long long ld_aux,
                        int flags, float alpha, void* stream_) {
  CommArgs ca;
  return gemm_common(A, B, C, M, N, K, lda, ldb, ldc, transA, transB, bias, aux_in, aux_out, residual, ld_aux,
                     flags, alpha, ca, static_cast<cudaStream_t>(stream_));
}

// Grouped GEMMs over expert row segments that are aligned to 128 rows (the layout the MoE permute kernel
// writes).  mode 1: C[rows, N] = A[rows, K] * op(B_e) with B the experts' matrices stacked ([E*N, K] for
// transB = 0, [E*K, N] for transB = 1) and tile_expert[row tile] -> expert (or -1).  mode 2: per-expert
// weight gradient C_e[M, N] (+)= A[rows_e, M]^T * B[rows_e, N], rows_e = [row_offsets[e], row_offsets[e+1]);
// C_e = C + e * c_stride; experts without rows are left untouched.  All tables live on the device: no host
// synchronisation on the routing result.
NX_API int NX_SYM(nx_gemm_bf16_grouped)(int mode, const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                long long ldb, long long ldc, int transB, int experts, const void* tile_expert,
                                const void* row_offsets, long long c_stride, const void* aux_in, void* aux_out,
                                long long ld_aux, int flags, void* stream_) {
  CommArgs ca;
  ca.group_mode = mode; ca.experts = experts;
  ca.tile_expert = static_cast<const int*>(tile_expert);
  ca.row_offsets = static_cast<const int*>(row_offsets);
  ca.c_stride = c_stride;
  return gemm_common(A, B, C, M, N, K, lda, ldb, ldc, mode == 2 ? 1 : 0, mode == 2 ? 1 : transB, nullptr, aux_in,
                     aux_out, nullptr, ld_aux, flags, 1.0f, ca, static_cast<cudaStream_t>(stream_));
}

// Number of CTAs the GEMM of this shape launches (the all-gather mode's flag count per source rank).
NX_API int NX_SYM(nx_gemm_grid)(int M, int N) {
  const int BN = (N <= 128) ? 128 : 256;
  const long long tiles = static_cast<long long>((M + nx::BM - 1) / nx::BM) * ((N + BN - 1) / BN);
  return static_cast<int>(tiles < nx::sm_count() ? tiles : nx::sm_count());
}

// GEMM fused with its tensor-parallel collective over peer memory (mode 1: GEMM -> reduce-scatter of
// the rows, C = this rank's [M/ws, N] slice, bias / residual2 applied after the reduction;
// mode 2: all-gather of the rows of A -> GEMM, A = this rank's dense [M, K] gather buffer, ag_src =
// this rank's [M/ws, K] shard).  data_ptrs / flag_ptrs: per-rank addresses (as mapped on this
// rank) of the staging / gather area and of its flag array; epoch: this call's flag value.
NX_API int NX_SYM(nx_gemm_bf16_comm)(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                             long long ldb, long long ldc, int transB, const void* bias, const void* aux_in,
                             void* aux_out, const void* residual, long long ld_aux, int flags, int mode,
                             int rank, int ws, unsigned int epoch, const unsigned long long* data_ptrs,
                             const unsigned long long* flag_ptrs, const void* residual2, long long ld_res2,
                             const void* ag_src, long long ag_ld, void* stream_) {
  CommArgs ca;
  ca.mode = mode; ca.rank = rank; ca.ws = ws; ca.epoch = epoch;
  ca.data_ptrs = data_ptrs; ca.flag_ptrs = flag_ptrs;
  ca.residual2 = residual2; ca.ld_res2 = ld_res2; ca.ag_src = ag_src; ca.ag_ld = ag_ld;
  return gemm_common(A, B, C, M, N, K, lda, ldb, ldc, 0, transB, bias, aux_in, aux_out, residual, ld_aux, flags,
                     1.0f, ca, static_cast<cudaStream_t>(stream_));
}
