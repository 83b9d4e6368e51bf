// Flash attention backward on tcgen05 (causal / sliding window / ALiBi / GQA).
//
// Three launches, no atomics, no fp32 scratch for dQ, deterministic:
//   1. attn_delta_kernel    delta[b,h,q] = sum_d O * dO
//   2. attn_bwd_dq_kernel   one CTA per 128 query rows: loops over key blocks, recomputes
//                           S = Q K^T and dP = dO V^T on the tensor cores, forms
//                           dS = P o (dP - delta) * scale per row (thread == query row), writes it
//                           as bf16 into TMEM and accumulates dQ += dS K  (A operand from TMEM).
//   3. attn_bwd_dkv_kernel  one CTA per 128 keys (per kv head; loops over the query heads of the
//                           GQA group and over query blocks): computes the transposed tiles
//                           S^T = K Q^T and dP^T = V dO^T so that thread == key row, writes P^T and
//                           dS^T (bf16) over the same TMEM columns and accumulates
//                           dV += P^T dO,  dK += dS^T Q.
// Recomputing S and dP in both kernels costs 7 tile GEMMs instead of 5 but keeps every
// accumulator in TMEM from first to last block.  Counterpart of the flash-attn 2 backward the
// reference calls through autograd (megatron/model/transformer.py:573-690).
#include <cstdlib>

#include "common.h"
#include "ptx.cuh"
#include "reduce.cuh"

namespace nx {

constexpr int AB = 128;  // rows per tile in every role
// Threads per CTA: producer warp, MMA warp and 4 * HALVES element-wise warps.  HALVES = 2 (default) puts two warps
// on every TMEM lane quadrant, each taking half of the 128 columns of a block (one warp per scheduler leaves the
// exponential / convert pipes idle during the serial S -> P -> dS chain); HALVES = 1 is the four-warp form
// (NEOX_ATTN_BWD_WARPS=4 selects it).
constexpr int ab_threads(int halves) { return 64 + 128 * halves; }
constexpr float LOG2E = 1.4426950408889634f;

struct AttnBwdParams {
  const float* lse;    // [B,H,Sq_pad] base-2 log-sum-exp, +inf in the padding
  const float* delta;  // [B,H,Sq_pad], 0 in the padding
  const float* alibi;
  h16 *dq, *dk, *dv;
  long long dq_sb, dq_sh, dq_ss, dk_sb, dk_sh, dk_ss, dv_sb, dv_sh, dv_ss;
  int B, H, Hk, Sq, Sk, D, Sq_pad;
  float scale, scale_log2;
  int causal, window;
  int* err;
  // dropout as in the forward (same seed and threshold): dP is masked and scaled before delta is subtracted,
  // and the P^T that feeds dV is the dropped one
  uint32_t drop_thr, seed_lo, seed_hi;
  float drop_rp;
  // block-sparse layout tables of the forward (null = dense): blk_rows[q * blk_nkt + kt] bit j = row q attends to
  // key sub-block j of key tile kt; blk_any[qt * blk_nkt + kt] != 0 = tile (qt, kt) has any live block
  const uint8_t* blk_rows;
  const uint8_t* blk_any;
  int blk_shift, blk_nkt;
};

// delta = rowsum(O * dO); one warp per (b, h, q) row.
__global__ void attn_delta_kernel(const h16* __restrict__ o,
                                  const h16* __restrict__ dO, float* __restrict__ delta,
                                  int B, int H, int Sq, int Sq_pad, int D, long long o_sb, long long o_sh,
                                  long long o_ss, long long d_sb, long long d_sh, long long d_ss) {
  const long long row = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long total = static_cast<long long>(B) * H * Sq;
  if (row >= total) return;
  const int lane = threadIdx.x & 31;
  const int q = static_cast<int>(row % Sq);
  const int h = static_cast<int>((row / Sq) % H);
  const int b = static_cast<int>(row / (static_cast<long long>(Sq) * H));
  const h16* op = o + b * o_sb + h * o_sh + q * o_ss;
  const h16* dp = dO + b * d_sb + h * d_sh + q * d_ss;
  float s = 0.f;
  for (int d = lane * 2; d < D; d += 64) {
    const float2 a = unpack_h16x2(*reinterpret_cast<const uint32_t*>(op + d));
    const float2 g = unpack_h16x2(*reinterpret_cast<const uint32_t*>(dp + d));
    s += a.x * g.x + a.y * g.y;
  }
  s = warp_sum(s);
  if (lane == 0) delta[(static_cast<long long>(b) * H + h) * Sq_pad + q] = s;
}

// Same for head dims 64 / 128 with 16-byte aligned rows: a group of D/8 lanes reads one row with one 16-byte
// load per lane and tensor, so a warp covers 32 / (D/8) rows per pass (the scalar-pair form above moves
// 4 bytes per lane and load).
template <int LPR>   // lanes per row = D / 8, a power of two
__global__ void attn_delta_vec8_kernel(const h16* __restrict__ o, const h16* __restrict__ dO,
                                       float* __restrict__ delta, int B, int H, int Sq, int Sq_pad, long long o_sb,
                                       long long o_sh, long long o_ss, long long d_sb, long long d_sh,
                                       long long d_ss) {
  constexpr int RPW = 32 / LPR;  // rows per warp
  const int lane = threadIdx.x & 31;
  const long long warp = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long row = warp * RPW + lane / LPR;
  const long long total = static_cast<long long>(B) * H * Sq;
  float s = 0.f;
  int q = 0, h = 0, b = 0;
  const bool live = row < total;
  if (live) {
    q = static_cast<int>(row % Sq);
    h = static_cast<int>((row / Sq) % H);
    b = static_cast<int>(row / (static_cast<long long>(Sq) * H));
    const int c = (lane % LPR) * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(o + b * o_sb + h * o_sh + q * o_ss + c);
    const uint4 g = *reinterpret_cast<const uint4*>(dO + b * d_sb + h * d_sh + q * d_ss + c);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 x = unpack_h16x2(aw[k]), y = unpack_h16x2(gw[k]);
      s += x.x * y.x + x.y * y.y;
    }
  }
#pragma unroll
  for (int off = LPR / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (live && (lane % LPR) == 0) delta[(static_cast<long long>(b) * H + h) * Sq_pad + q] = s;
}

// AND of a predicate over the 64 threads (two warps) that meet at named barrier `id`.
__device__ __forceinline__ bool pair_all(bool ok, int id) {
  uint32_t out;
  asm volatile(
      "{\n"
      ".reg .pred pi, po;\n"
      "setp.ne.u32 pi, %1, 0;\n"
      "bar.red.and.pred po, %2, 64, pi;\n"
      "selp.u32 %0, 1, 0, po;\n"
      "}\n"
      : "=r"(out)
      : "r"(ok ? 1u : 0u), "r"(id)
      : "memory");
  return out != 0;
}

template <int DP>
struct BwdSmem {
  static constexpr int TILE = AB * DP * 2;
  static constexpr int BAR_OFF = 6 * TILE;  // two resident tiles + 2 x 2 streamed tiles
  static constexpr int NBAR = 24;
  static constexpr int VEC_OFF = BAR_OFF + NBAR * 8;  // lse / delta staging: 2 stages x 2 x 128 floats
  static constexpr int TOTAL = VEC_OFF + 4 * AB * 4 + 16;
  static constexpr int DYN = TOTAL + 1024;
};

// Loads one [128 x DP] tile (rows contiguous in d) as DP/64 swizzled boxes.
template <int DP>
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap* m, uint32_t bar, int row0,
                                          int head, int batch) {
#pragma unroll
  for (int c = 0; c < DP / 64; ++c) tma_load_4d(dst + c * (AB * 128), m, bar, c * 64, row0, head, batch);
}
// D[128 x N] = A[128 x DP] * B[N x DP]^T, both K-major (head dim contiguous); b points at the first of the N rows.
template <int DP, int N = AB>
__device__ __forceinline__ void mma_nt(uint32_t d_tmem, uint32_t a, uint32_t b) {
  constexpr uint32_t idesc = umma_idesc_bf16(AB, N, 0, 0);
#pragma unroll
  for (int k = 0; k < DP / 16; ++k) {
    const uint32_t o = (k >> 2) * (AB * 128) + (k & 3) * 32;
    umma_bf16_ss(d_tmem, umma_smem_desc_sw128(a + o, 0, 1024), umma_smem_desc_sw128(b + o, 0, 1024),
                 idesc, k != 0 ? 1u : 0u);
  }
}
// D[128 x DP] (+)= A_tmem[128 x 128 (bf16, 64 columns)] * B[128 x DP] with B's head dim contiguous
// (MN-major B operand).
// KR: rows of B (the contraction length), 128 or 64; b points at the first of them.
template <int DP, int KR = AB>
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b, bool accumulate) {
  constexpr uint32_t idesc = umma_idesc_bf16(AB, DP, 0, 1);
#pragma unroll
  for (int k = 0; k < KR / 16; ++k) {
    umma_bf16_ts(d_tmem, a_tmem + k * 8, umma_smem_desc_sw128(b + k * 2048, AB * 128, 1024), idesc,
                 (accumulate || k != 0) ? 1u : 0u);
  }
}

// ------------------------------------------------------------------------------------------------
// dQ kernel.  smem tiles: 0 = Q, 1 = dO, 2..3 = K ring, 4..5 = V ring.
// TMEM: S [0,128) dP [128,256) dQ [256,256+DP) dS0 [384,448) dS1 [448,512)
// PIPE (default, eight element-wise warps): the 128 keys of a block are handled as two halves of 64 with their own
// S / dP columns (S_h at [64 h, ...), dP_h at [128 + 64 h, ...)), dS_h at [384 + 32 h, ...) and their own barriers.
// The MMA warp issues S / dP of half u + 1 before it waits for dS of half u, so the tensor core computes the next
// half (and dQ += dS K of the previous one) while the element-wise warps work on the current one; without PIPE
// the tensor core and the element-wise warps take turns.
// ------------------------------------------------------------------------------------------------
template <int DP, bool DROP, int HALVES, bool PIPE>
__global__ void __launch_bounds__(ab_threads(HALVES), 1)
    attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                       const AttnBwdParams p) {
  using L = BwdSmem<DP>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t bar0 = sbase + L::BAR_OFF;
  static_assert(!PIPE || HALVES == 2, "the pipelined form gives each of a half's 64 columns' halves to one warp");
  enum { QDO_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7, SDP_FULL = 9, DS_FULL = 11, DQ_DONE = 13,
         SDP_EMPTY = 15, NUSED = 16 };
  auto bar = [&](int which, int idx) { return bar0 + 8u * (which + idx); };
  const uint32_t tmem_slot = bar0 + 8u * 23;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(sgen + L::BAR_OFF + 8 * 23);
  auto tile = [&](int i) { return sbase + i * L::TILE; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.H / p.Hk);
  const int q0 = qt * AB;
  const int off = p.Sk - p.Sq;
  int kv_end = p.Sk;
  if (p.causal) kv_end = min(p.Sk, q0 + AB + off);
  int kv_begin = 0;
  if (p.window >= 0) kv_begin = max(0, q0 + off - p.window);
  const int jb = kv_begin / AB;
  const int nblk = max((kv_end + AB - 1) / AB - jb, 0);
  // block-sparse layouts: key tiles without a live block for this query tile are skipped by every role; ring
  // stages and barrier phases count the live tiles
  auto tile_live = [&](int kt) { return p.blk_any == nullptr || p.blk_any[static_cast<long long>(qt) * p.blk_nkt + kt] != 0; };

  if (threadIdx.x == 0) {
    for (int i = 0; i < NUSED; ++i) {
      const bool by_softmax = (i == SDP_EMPTY) || (i >= DS_FULL && i < DS_FULL + 2);
      mbar_init(bar0 + 8u * i, by_softmax ? 4 * HALVES : 1);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot_gen;
  const uint32_t T_S = tmem, T_DP = tmem + 128, T_DQ = tmem + 256, T_DS = tmem + 384;
  bool aborted = false;

  if (warp == 0) {
    if (elect_one() && nblk > 0) {
      mbar_expect_tx(bar(QDO_FULL, 0), 2 * L::TILE);
      load_tile<DP>(tile(0), &tmQ, bar(QDO_FULL, 0), q0, head, batch);
      load_tile<DP>(tile(1), &tmDO, bar(QDO_FULL, 0), q0, head, batch);
      for (int t = 0, n = 0; t < nblk; ++t) {
        if (!tile_live(jb + t)) continue;
        const int i = n++;
        const int st = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        const int k0 = (jb + t) * AB;
        if (!mbar_wait(bar(K_EMPTY, st), ph ^ 1, p.err, 31)) { aborted = true; break; }
        mbar_expect_tx(bar(K_FULL, st), L::TILE);
        load_tile<DP>(tile(2 + st), &tmK, bar(K_FULL, st), k0, kv_head, batch);
        if (!mbar_wait(bar(V_EMPTY, st), ph ^ 1, p.err, 32)) { aborted = true; break; }
        mbar_expect_tx(bar(V_FULL, st), L::TILE);
        load_tile<DP>(tile(4 + st), &tmV, bar(V_FULL, st), k0, kv_head, batch);
      }
    }
  } else if (warp == 1) {
    if (elect_one() && nblk > 0) {
      auto issue_dq = [&](int i) -> bool {
        const int st = i & 1;
        if (!mbar_wait(bar(DS_FULL, st), (i >> 1) & 1, p.err, 33)) return false;
        tc_fence_after_sync();
        mma_ts<DP>(T_DQ, T_DS + st * 64, tile(2 + st), i != 0);
        umma_commit(bar(DQ_DONE, st));
        umma_commit(bar(K_EMPTY, st));
        return true;
      };
      if (!mbar_wait(bar(QDO_FULL, 0), 0, p.err, 34)) aborted = true;
      int n = 0;
      if (PIPE) {
        // sub-step u = 2 i + h of live block i: S_h = Q K_h^T, dP_h = dO V_h^T (64 keys), later dQ += dS_h K_h
        int nl = 0;
        for (int t = 0; t < nblk; ++t) nl += tile_live(jb + t) ? 1 : 0;
        auto issue_m1 = [&](int u) -> bool {
          const int i = u >> 1, h = u & 1, st = i & 1;
          if (h == 0) {
            if (!mbar_wait(bar(K_FULL, st), (i >> 1) & 1, p.err, 35)) return false;
            if (!mbar_wait(bar(V_FULL, st), (i >> 1) & 1, p.err, 36)) return false;
          }
          tc_fence_after_sync();
          mma_nt<DP, 64>(T_S + h * 64, tile(0), tile(2 + st) + h * (64 * 128));
          mma_nt<DP, 64>(T_DP + h * 64, tile(1), tile(4 + st) + h * (64 * 128));
          umma_commit(bar(SDP_FULL, h));
          if (h == 1) umma_commit(bar(V_EMPTY, st));
          return true;
        };
        const int nsub = 2 * nl;
        if (!aborted && nsub > 0 && !issue_m1(0)) aborted = true;
        for (int u = 0; u < nsub && !aborted; ++u) {
          const int i = u >> 1, h = u & 1, st = i & 1;
          if (u + 1 < nsub && !issue_m1(u + 1)) { aborted = true; break; }
          if (!mbar_wait(bar(DS_FULL, h), i & 1, p.err, 33)) { aborted = true; break; }
          tc_fence_after_sync();
          mma_ts<DP, 64>(T_DQ, T_DS + h * 32, tile(2 + st) + h * (64 * 128), u != 0);    // dQ += dS_h K_h
          if (h == 1) umma_commit(bar(K_EMPTY, st));
        }
        if (!aborted && nsub > 0) umma_commit(bar(DQ_DONE, 0));
        n = 0;      // (the loop below is the unpipelined form)
      }
      for (int t = 0; !PIPE && t < nblk && !aborted; ++t) {
        if (!tile_live(jb + t)) continue;
        const int i = n++;
        const int st = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        if (!mbar_wait(bar(K_FULL, st), ph, p.err, 35)) { aborted = true; break; }
        if (!mbar_wait(bar(V_FULL, st), ph, p.err, 36)) { aborted = true; break; }
        if (!mbar_wait(bar(SDP_EMPTY, 0), (i & 1) ^ 1, p.err, 37)) { aborted = true; break; }
        tc_fence_after_sync();
        mma_nt<DP>(T_S, tile(0), tile(2 + st));
        mma_nt<DP>(T_DP, tile(1), tile(4 + st));
        umma_commit(bar(SDP_FULL, 0));
        umma_commit(bar(V_EMPTY, st));
        if (i > 0 && !issue_dq(i - 1)) { aborted = true; break; }
      }
      if (!PIPE && !aborted && n > 0 && !issue_dq(n - 1)) aborted = true;
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;    // HALVES = 2: which 64 of the 128 key columns of a block (and half of dQ's columns)
    constexpr int CPW = (AB / 32) / HALVES;   // 32-column chunks per warp and block
    const int r = quad * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const int qi = q0 + r;
    const int qpos = qi + off;
    const bool row_ok = qi < p.Sq;
    const long long stat_idx = (static_cast<long long>(batch) * p.H + head) * p.Sq_pad + qi;
    const float lse2 = p.lse[stat_idx];     // +inf for rows past Sq -> P = 0
    const float delta = p.delta[stat_idx];
    const float slope2 = p.alibi != nullptr ? p.alibi[head] * LOG2E : 0.f;
    int nlive = 0;
    for (int t = 0; t < nblk; ++t) {
      if (!tile_live(jb + t)) continue;
      const int i = nlive++;
      const int st = i & 1;
      const int k0 = (jb + t) * AB;
      uint32_t bits = 0xffffffffu;
      if (p.blk_rows != nullptr)
        bits = row_ok ? p.blk_rows[static_cast<long long>(qi) * p.blk_nkt + (jb + t)] : 0u;
      const uint32_t full_bits = (1u << (AB >> p.blk_shift)) - 1u;
      const bool blk_partial = p.blk_rows != nullptr && !__all_sync(0xffffffffu, (bits & full_bits) == full_bits);
      if (!PIPE) {
        if (!mbar_wait(bar(SDP_FULL, 0), i & 1, p.err, 38)) { aborted = true; break; }
        if (i >= 2 && !mbar_wait(bar(DQ_DONE, st), ((i - 2) >> 1) & 1, p.err, 39)) { aborted = true; break; }
        tc_fence_after_sync();
      }
      const bool need_mask = (k0 + AB > p.Sk) || (p.causal && k0 + AB - 1 > q0 + quad * 32 + off) ||
                             (p.window >= 0 && k0 < q0 + quad * 32 + 31 + off - p.window) || blk_partial;
      const int rel0 = k0 - qpos;
      int hi = p.Sk - k0 - 1;
      if (p.causal) hi = min(hi, -rel0);
      const int lo = p.window >= 0 ? -rel0 - p.window : -(1 << 30);
      const float bias0 = slope2 * static_cast<float>(rel0) - lse2;  // folded into the exponent
      // PIPE: pass h = 0, 1 over the block's halves, this warp's chunk in each is c = 2 h + half (block columns
      // 32 c ..), read from the half's own S / dP columns after its own barrier; otherwise CPW chunks of the one buffer.
#pragma unroll 1
      for (int cc = 0; cc < (PIPE ? 2 : CPW); ++cc) {
        const int c = PIPE ? cc * 2 + half : half * CPW + cc;
        if (PIPE) {
          if (!mbar_wait(bar(SDP_FULL, cc), i & 1, p.err, 38)) { aborted = true; break; }
          tc_fence_after_sync();
        }
        uint32_t sv[32], dv[32];
        tmem_ld_32x32b_x32(T_S + c * 32 + lane_off, sv);
        tmem_ld_32x32b_x32(T_DP + c * 32 + lane_off, dv);
        tmem_ld_wait();
        if (DROP) {
          // dP of a dropped probability is zero, of a kept one it carries the 1 / (1 - p) factor
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const int kk = k0 + c * 32 + j;
            const uint32_t patch = dropout_patch(p.seed_lo, p.seed_hi, static_cast<uint32_t>(batch * p.H + head),
                                                 static_cast<uint32_t>(qi) >> 1, static_cast<uint32_t>(kk) >> 1);
            dv[j] = dropout_keep(patch, qi, kk, p.drop_thr) ? __float_as_uint(__uint_as_float(dv[j]) * p.drop_rp) : 0u;
            dv[j + 1] = dropout_keep(patch, qi, kk + 1, p.drop_thr)
                            ? __float_as_uint(__uint_as_float(dv[j + 1]) * p.drop_rp) : 0u;
          }
        }
        uint32_t pk[16];
        if (!need_mask && p.alibi == nullptr) {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            // the softmax scale of dS is applied once, to dQ, in the epilogue
            const float p0 = exp2f(fmaf(__uint_as_float(sv[j]), p.scale_log2, -lse2));
            const float p1 = exp2f(fmaf(__uint_as_float(sv[j + 1]), p.scale_log2, -lse2));
            pk[j >> 1] = pack_h16x2(p0 * (__uint_as_float(dv[j]) - delta),
                                     p1 * (__uint_as_float(dv[j + 1]) - delta));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float ds[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int idx = c * 32 + j + e;
              float x = fmaf(__uint_as_float(sv[j + e]), p.scale_log2,
                             fmaf(slope2, static_cast<float>(idx), bias0));
              float pr = exp2f(x);
              if (idx < lo || idx > hi || !((bits >> (idx >> p.blk_shift)) & 1u)) pr = 0.f;
              ds[e] = pr * (__uint_as_float(dv[j + e]) - delta);
            }
            pk[j >> 1] = pack_h16x2(ds[0], ds[1]);
          }
        }
        if (PIPE) {
          // dS_h sits at [384 + 32 h, ...): the chunk's 16 columns at 16 c (c = 2 h + half)
          tmem_st_32x32b_x16(T_DS + c * 16 + lane_off, pk);
          tmem_st_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(DS_FULL, cc));
        } else {
          tmem_st_32x32b_x16(T_DS + st * 64 + c * 16 + lane_off, pk);
        }
      }
      if (aborted) break;
      if (!PIPE) {
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bar(SDP_EMPTY, 0));
          mbar_arrive(bar(DS_FULL, st));
        }
      }
    }
    if (!aborted && nlive > 0) {
      if (PIPE ? !mbar_wait(bar(DQ_DONE, 0), 0, p.err, 40)
               : !mbar_wait(bar(DQ_DONE, (nlive - 1) & 1), ((nlive - 1) >> 1) & 1, p.err, 40)) aborted = true;
      tc_fence_after_sync();
    }
    if (!aborted) {
      h16* orow = p.dq + batch * p.dq_sb + head * p.dq_sh + static_cast<long long>(qi) * p.dq_ss;
#pragma unroll 1
      for (int c = half * (DP / 32 / HALVES); c < (half + 1) * (DP / 32 / HALVES); ++c) {   // this warp's dQ columns
        uint32_t ov[32];
        if (nlive > 0) {  // warp-uniform: every lane takes part in the collective TMEM load
          tmem_ld_32x32b_x32(T_DQ + c * 32 + lane_off, ov);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) ov[j] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (c * 32 + j < p.D) {
              const float sc = p.scale;
              uint4 o4;
              o4.x = pack_h16x2(__uint_as_float(ov[j]) * sc, __uint_as_float(ov[j + 1]) * sc);
              o4.y = pack_h16x2(__uint_as_float(ov[j + 2]) * sc, __uint_as_float(ov[j + 3]) * sc);
              o4.z = pack_h16x2(__uint_as_float(ov[j + 4]) * sc, __uint_as_float(ov[j + 5]) * sc);
              o4.w = pack_h16x2(__uint_as_float(ov[j + 6]) * sc, __uint_as_float(ov[j + 7]) * sc);
              *reinterpret_cast<uint4*>(orow + c * 32 + j) = o4;
            }
          }
        }
      }
    }
  }
  __syncwarp();
  if (aborted) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// dK / dV kernel.  smem tiles: 0 = K, 1 = V, 2..3 = Q ring, 4..5 = dO ring.
// TMEM: S^T [0,128) (P^T bf16 overwrites cols [0,64)), dP^T [128,256) (dS^T bf16 over [128,192)),
//       dK [256,256+DP), dV [384,384+DP)
// PIPE (default, eight element-wise warps): a step's 128 query columns are handled as two halves of 64 with their
// own S^T / dP^T buffers (S^T_h at [64 h, 64 h + 64), dP^T_h at [128 + 64 h, ...)) and their own barriers.  The MMA
// warp issues S^T / dP^T of half u + 1 before it waits for P^T / dS^T of half u, so the tensor core works on the
// next half (and on dV / dK of the previous one) while the element-wise warps are busy with the current one;
// without PIPE the four phases of a step run one after the other.
// ------------------------------------------------------------------------------------------------
template <int DP, bool DROP, int HALVES, bool PIPE>
__global__ void __launch_bounds__(ab_threads(HALVES), 1)
    attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                        const AttnBwdParams p) {
  using L = BwdSmem<DP>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t bar0 = sbase + L::BAR_OFF;
  static_assert(!PIPE || HALVES == 2, "the pipelined form splits a half's 64 columns over two warps per quadrant");
  enum { KV_FULL = 0, Q_FULL = 1, Q_EMPTY = 3, ST_FULL = 5, PT_FULL = 7, ACC_DONE = 9, NUSED = 10 };
  auto bar = [&](int which, int idx) { return bar0 + 8u * (which + idx); };
  const uint32_t tmem_slot = bar0 + 8u * 23;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(sgen + L::BAR_OFF + 8 * 23);
  auto tile = [&](int i) { return sbase + i * L::TILE; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x;
  const int kv_head = blockIdx.y, batch = blockIdx.z;
  const int group = p.H / p.Hk;
  const int k0 = kt * AB;
  const int off = p.Sk - p.Sq;
  // query rows that can see this key block: qpos >= k0 (causal), qpos <= k_last + window
  int q_begin = 0, q_end = p.Sq;
  if (p.causal) q_begin = max(0, k0 - off);
  if (p.window >= 0) q_end = min(p.Sq, k0 + AB - 1 + p.window - off + 1);
  const int ib = q_begin / AB;
  const int nq = max((q_end + AB - 1) / AB - ib, 0);
  const int nsteps = nq * group;
  // block-sparse layouts: query tiles without a live block for this key tile are skipped by every role
  auto step_live = [&](int t) {
    return p.blk_any == nullptr || p.blk_any[static_cast<long long>(ib + t % nq) * p.blk_nkt + kt] != 0;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < NUSED; ++i) mbar_init(bar0 + 8u * i, (i == PT_FULL || i == PT_FULL + 1) ? 4 * HALVES : 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot_gen;
  const uint32_t T_ST = tmem, T_DPT = tmem + 128, T_DK = tmem + 256, T_DV = tmem + 384;
  bool aborted = false;

  if (warp == 0) {
    if (elect_one() && nsteps > 0) {
      mbar_expect_tx(bar(KV_FULL, 0), 2 * L::TILE);
      load_tile<DP>(tile(0), &tmK, bar(KV_FULL, 0), k0, kv_head, batch);
      load_tile<DP>(tile(1), &tmV, bar(KV_FULL, 0), k0, kv_head, batch);
      for (int t = 0, n = 0; t < nsteps; ++t) {
        if (!step_live(t)) continue;
        const int st = n & 1;
        const uint32_t ph = (n >> 1) & 1;
        ++n;
        const int head = kv_head * group + t / nq;
        const int q0 = (ib + t % nq) * AB;
        if (!mbar_wait(bar(Q_EMPTY, st), ph ^ 1, p.err, 51)) { aborted = true; break; }
        mbar_expect_tx(bar(Q_FULL, st), 2 * L::TILE + 2 * AB * 4);
        load_tile<DP>(tile(2 + st), &tmQ, bar(Q_FULL, st), q0, head, batch);
        load_tile<DP>(tile(4 + st), &tmDO, bar(Q_FULL, st), q0, head, batch);
        const long long stat0 = (static_cast<long long>(batch) * p.H + head) * p.Sq_pad + q0;
        bulk_load_1d(sbase + L::VEC_OFF + st * (2 * AB * 4), p.lse + stat0, AB * 4, bar(Q_FULL, st));
        bulk_load_1d(sbase + L::VEC_OFF + st * (2 * AB * 4) + AB * 4, p.delta + stat0, AB * 4,
                     bar(Q_FULL, st));
      }
    }
  } else if (warp == 1) {
    if (elect_one() && nsteps > 0) {
      if (!mbar_wait(bar(KV_FULL, 0), 0, p.err, 52)) aborted = true;
      int n = 0;
      if (PIPE) {
        // sub-step u = 2 t + h of live step t: S^T_h = K Q_h^T, dP^T_h = V dO_h^T (64 query rows), later
        // dV += P^T_h dO_h, dK += dS^T_h Q_h
        int nl = 0;
        for (int tt = 0; tt < nsteps; ++tt) nl += step_live(tt) ? 1 : 0;
        auto issue_m1 = [&](int u) -> bool {
          const int t = u >> 1, h = u & 1, st = t & 1;
          if (h == 0 && !mbar_wait(bar(Q_FULL, st), (t >> 1) & 1, p.err, 53)) return false;
          tc_fence_after_sync();
          mma_nt<DP, 64>(T_ST + h * 64, tile(0), tile(2 + st) + h * (64 * 128));
          mma_nt<DP, 64>(T_DPT + h * 64, tile(1), tile(4 + st) + h * (64 * 128));
          umma_commit(bar(ST_FULL, h));
          return true;
        };
        const int nsub = 2 * nl;
        if (!aborted && nsub > 0 && !issue_m1(0)) aborted = true;
        for (int u = 0; u < nsub && !aborted; ++u) {
          const int t = u >> 1, h = u & 1, st = t & 1;
          if (u + 1 < nsub && !issue_m1(u + 1)) { aborted = true; break; }
          if (!mbar_wait(bar(PT_FULL, h), t & 1, p.err, 54)) { aborted = true; break; }
          tc_fence_after_sync();
          mma_ts<DP, 64>(T_DV, T_ST + h * 64, tile(4 + st) + h * (64 * 128), u != 0);    // dV += P^T_h dO_h
          mma_ts<DP, 64>(T_DK, T_DPT + h * 64, tile(2 + st) + h * (64 * 128), u != 0);   // dK += dS^T_h Q_h
          if (h == 1) umma_commit(bar(Q_EMPTY, st));
        }
        n = nl;
      }
      for (int tt = 0; !PIPE && tt < nsteps && !aborted; ++tt) {
        if (!step_live(tt)) continue;
        const int t = n++;          // live steps: ring stages, barrier phases and the accumulate flags count these
        const int st = t & 1;
        if (!mbar_wait(bar(Q_FULL, st), (t >> 1) & 1, p.err, 53)) { aborted = true; break; }
        tc_fence_after_sync();
        mma_nt<DP>(T_ST, tile(0), tile(2 + st));   // S^T  = K Q^T
        mma_nt<DP>(T_DPT, tile(1), tile(4 + st));  // dP^T = V dO^T
        umma_commit(bar(ST_FULL, 0));
        if (!mbar_wait(bar(PT_FULL, 0), t & 1, p.err, 54)) { aborted = true; break; }
        tc_fence_after_sync();
        mma_ts<DP>(T_DV, T_ST, tile(4 + st), t != 0);   // dV += P^T dO
        mma_ts<DP>(T_DK, T_DPT, tile(2 + st), t != 0);  // dK += dS^T Q
        umma_commit(bar(Q_EMPTY, st));
      }
      if (!aborted && n > 0) umma_commit(bar(ACC_DONE, 0));
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;   // which 64 of the 128 query columns of a step (and which half of dK / dV)
    const int r = quad * 32 + lane;  // key row in tile
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const int kcol = k0 + r;
    const bool key_ok = kcol < p.Sk;
    int nlive = 0;
    for (int tt = 0; tt < nsteps; ++tt) {
      if (!step_live(tt)) continue;
      const int t = nlive++;
      const int head = kv_head * group + tt / nq;
      const int q0 = (ib + tt % nq) * AB;
      const float slope2 = p.alibi != nullptr ? p.alibi[head] * LOG2E : 0.f;
      const int st = t & 1;
      // lse / delta of this query block were bulk-copied next to the Q / dO tiles
      bool ok = mbar_wait(bar(Q_FULL, st), (t >> 1) & 1, p.err, 57);
      const float4* v_lse = reinterpret_cast<const float4*>(sgen + L::VEC_OFF + st * (2 * AB * 4));
      const float4* v_del = v_lse + AB / 4;
      if (!PIPE) {
        if (ok) ok = mbar_wait(bar(ST_FULL, 0), t & 1, p.err, 55);
        // the two warps of a quadrant meet at a named barrier further down: they must take the same decision here
        // (a wait that ran out on one of them ends the loop for both)
        if (HALVES == 2 ? !pair_all(ok, 5 + quad) : !ok) { aborted = true; break; }
        tc_fence_after_sync();
      }
      // query columns qq (0..127) of this block are alive for lo <= qq <= hi
      const int rel0 = kcol - q0 - off;  // key position minus position of query column 0
      int lo = p.causal ? rel0 : -(1 << 30);
      int hi = p.window >= 0 ? rel0 + p.window : (1 << 30);
      if (!key_ok) hi = -(1 << 30);
      const bool need_mask = __any_sync(0xffffffffu, lo > 0 || hi < AB - 1) || p.blk_rows != nullptr;
      const float bias0 = slope2 * static_cast<float>(rel0);
      const uint32_t kbit = 1u << (r >> p.blk_shift);      // this key row's sub-block within the key tile
      const bool plain = !need_mask && p.alibi == nullptr;   // warp-uniform: no per-element compares in the hot path
      // P^T and dS^T (16 bit) go over the columns S^T and dP^T were read from, and the partner warp of this
      // quadrant reads the other half of those columns: both chunks of this warp are kept in registers until the
      // two warps have finished reading (named barrier of the quadrant's 64 threads), then everything is stored.
      // (With four warps a thread takes all four chunks, two at a time; its own earlier stores never reach columns
      //  it has yet to read.)
      // PIPE: two passes (the halves of the step), one 32-column chunk per warp and pass, each pass with its own
      // S^T / dP^T buffer and barriers; otherwise 2 / HALVES passes over two chunks each in the one buffer.
      constexpr int NGRP = PIPE ? 2 : 2 / HALVES;
      constexpr int NCC = PIPE ? 1 : 2;
#pragma unroll 1
      for (int grp = 0; grp < NGRP; ++grp) {
      const int cbase = PIPE ? grp * 2 + half : (half * (2 / HALVES) + grp) * 2;
      // where this pass's chunks sit in TMEM: columns of the S^T buffer read / of the 16-bit result written
      const uint32_t rd0 = PIPE ? grp * 64 + half * 32 : cbase * 32;
      const uint32_t wr0 = PIPE ? grp * 64 + half * 16 : cbase * 16;
      if (PIPE) {
        if (ok) ok = mbar_wait(bar(ST_FULL, grp), t & 1, p.err, 55);
        if (!pair_all(ok, 5 + quad)) { aborted = true; break; }
        tc_fence_after_sync();
      }
      uint32_t pp_all[NCC][16], pd_all[NCC][16];
#pragma unroll
      for (int cc = 0; cc < NCC; ++cc) {
        const int c = cbase + cc;
        uint32_t (&pp)[16] = pp_all[cc];
        uint32_t (&pd)[16] = pd_all[cc];
        uint32_t sv[32], dv[32];
        tmem_ld_32x32b_x32(T_ST + rd0 + cc * 32 + lane_off, sv);
        tmem_ld_32x32b_x32(T_DPT + rd0 + cc * 32 + lane_off, dv);
        tmem_ld_wait();
        float keepf[32];      // DROP: 0 or 1 / (1 - p) per query column of this chunk (unused otherwise)
        if (DROP) {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const int qq = q0 + c * 32 + j;
            const uint32_t patch = dropout_patch(p.seed_lo, p.seed_hi, static_cast<uint32_t>(batch * p.H + head),
                                                 static_cast<uint32_t>(qq) >> 1, static_cast<uint32_t>(kcol) >> 1);
            keepf[j] = dropout_keep(patch, qq, kcol, p.drop_thr) ? p.drop_rp : 0.f;
            keepf[j + 1] = dropout_keep(patch, qq + 1, kcol, p.drop_thr) ? p.drop_rp : 0.f;
          }
        }
        if (plain) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 l4 = v_lse[(c * 32 + j) >> 2];
            const float4 d4 = v_del[(c * 32 + j) >> 2];
            const float lq[4] = {l4.x, l4.y, l4.z, l4.w}, dq_[4] = {d4.x, d4.y, d4.z, d4.w};
            float pr[4], ds[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              pr[e] = exp2f(fmaf(__uint_as_float(sv[j + e]), p.scale_log2, -lq[e]));
              const float dpe = DROP ? __uint_as_float(dv[j + e]) * keepf[j + e] : __uint_as_float(dv[j + e]);
              ds[e] = pr[e] * (dpe - dq_[e]);     // softmax scale: once, on dK, in the epilogue
              if (DROP) pr[e] *= keepf[j + e];    // dV takes the dropped probabilities
            }
            pp[j >> 1] = pack_h16x2(pr[0], pr[1]);
            pp[(j >> 1) + 1] = pack_h16x2(pr[2], pr[3]);
            pd[j >> 1] = pack_h16x2(ds[0], ds[1]);
            pd[(j >> 1) + 1] = pack_h16x2(ds[2], ds[3]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 l4 = v_lse[(c * 32 + j) >> 2];
            const float4 d4 = v_del[(c * 32 + j) >> 2];
            const float lq[4] = {l4.x, l4.y, l4.z, l4.w}, dq_[4] = {d4.x, d4.y, d4.z, d4.w};
            float pr[4], ds[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int idx = c * 32 + j + e;
              float x = fmaf(__uint_as_float(sv[j + e]), p.scale_log2, -lq[e]);
              if (p.alibi != nullptr) x += fmaf(-slope2, static_cast<float>(idx), bias0);
              pr[e] = exp2f(x);
              if (idx < lo || idx > hi) pr[e] = 0.f;
              if (p.blk_rows != nullptr) {   // the layout byte of query row q0 + idx (the same for the whole warp)
                const int qq = min(q0 + idx, p.Sq - 1);
                if (!(p.blk_rows[static_cast<long long>(qq) * p.blk_nkt + kt] & kbit)) pr[e] = 0.f;
              }
              const float dpe = DROP ? __uint_as_float(dv[j + e]) * keepf[j + e] : __uint_as_float(dv[j + e]);
              ds[e] = pr[e] * (dpe - dq_[e]);
              if (DROP) pr[e] *= keepf[j + e];
            }
            pp[j >> 1] = pack_h16x2(pr[0], pr[1]);
            pp[(j >> 1) + 1] = pack_h16x2(pr[2], pr[3]);
            pd[j >> 1] = pack_h16x2(ds[0], ds[1]);
            pd[(j >> 1) + 1] = pack_h16x2(ds[2], ds[3]);
          }
        }
      }
      if (HALVES == 2) asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");
#pragma unroll
      for (int cc = 0; cc < NCC; ++cc) {
        tmem_st_32x32b_x16(T_ST + wr0 + cc * 16 + lane_off, pp_all[cc]);
        tmem_st_32x32b_x16(T_DPT + wr0 + cc * 16 + lane_off, pd_all[cc]);
      }
      if (PIPE) {
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(PT_FULL, grp));
      }
      }
      if (aborted) break;
      if (!PIPE) {
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(PT_FULL, 0));
      }
    }
    if (!aborted && nlive > 0) {
      if (!mbar_wait(bar(ACC_DONE, 0), 0, p.err, 56)) aborted = true;
      tc_fence_after_sync();
    }
    if (!aborted) {
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t T = which == 0 ? T_DK : T_DV;
        h16* base = which == 0 ? p.dk : p.dv;
        const long long sb = which == 0 ? p.dk_sb : p.dv_sb, sh = which == 0 ? p.dk_sh : p.dv_sh,
                        ss = which == 0 ? p.dk_ss : p.dv_ss;
        h16* orow = base + batch * sb + kv_head * sh + static_cast<long long>(kcol) * ss;
#pragma unroll 1
        for (int c = half * (DP / 32 / HALVES); c < (half + 1) * (DP / 32 / HALVES); ++c) {   // this warp's columns
          uint32_t ov[32];
          if (nlive > 0) {
            tmem_ld_32x32b_x32(T + c * 32 + lane_off, ov);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) ov[j] = 0u;
          }
          if (key_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (c * 32 + j < p.D) {
                const float sc = which == 0 ? p.scale : 1.f;     // dK carries the softmax scale of dS
                uint4 o4;
                o4.x = pack_h16x2(__uint_as_float(ov[j]) * sc, __uint_as_float(ov[j + 1]) * sc);
                o4.y = pack_h16x2(__uint_as_float(ov[j + 2]) * sc, __uint_as_float(ov[j + 3]) * sc);
                o4.z = pack_h16x2(__uint_as_float(ov[j + 4]) * sc, __uint_as_float(ov[j + 5]) * sc);
                o4.w = pack_h16x2(__uint_as_float(ov[j + 6]) * sc, __uint_as_float(ov[j + 7]) * sc);
                *reinterpret_cast<uint4*>(orow + c * 32 + j) = o4;
              }
            }
          }
        }
      }
    }
  }
  __syncwarp();
  if (aborted) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

static bool bwd_map(CUtensorMap* m, const void* base, int B, int Hh, int S, int D, long long sb,
                    long long sh, long long ss) {
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)S, (uint64_t)Hh, (uint64_t)B};
  const uint64_t strides[3] = {(uint64_t)ss * 2, (uint64_t)sh * 2, (uint64_t)sb * 2};
  const uint32_t box[4] = {64, AB, 1, 1};
  return make_tma_4d(m, base, dims, strides, box, 2, true);
}

template <int DP, bool DROP, int HALVES>
static int launch_bwd_h(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                      const CUtensorMap& tdo, const AttnBwdParams& p, cudaStream_t s) {
  static bool cfg = false;
  if (!cfg) {
    NX_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_dq_kernel<DP, DROP, HALVES, false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<DP>::DYN));
    NX_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_dq_kernel<DP, DROP, HALVES, HALVES == 2>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<DP>::DYN));
    NX_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_dkv_kernel<DP, DROP, HALVES, false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<DP>::DYN));
    NX_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_dkv_kernel<DP, DROP, HALVES, HALVES == 2>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<DP>::DYN));
    cfg = true;
  }
  dim3 gq((p.Sq + AB - 1) / AB, p.H, p.B);
  static const bool serial_q = [] {        // NEOX_ATTN_DQ_PIPE=0: the unpipelined form
    const char* e = getenv("NEOX_ATTN_DQ_PIPE");
    return e != nullptr && atoi(e) == 0;
  }();
  if (HALVES == 2 && !serial_q)
    attn_bwd_dq_kernel<DP, DROP, HALVES, HALVES == 2><<<gq, ab_threads(HALVES), BwdSmem<DP>::DYN, s>>>(tq, tk, tv, tdo, p);
  else
    attn_bwd_dq_kernel<DP, DROP, HALVES, false><<<gq, ab_threads(HALVES), BwdSmem<DP>::DYN, s>>>(tq, tk, tv, tdo, p);
  NX_LAUNCH_CHECK();
  dim3 gk((p.Sk + AB - 1) / AB, p.Hk, p.B);
  static const bool serial = [] {        // NEOX_ATTN_DKV_PIPE=0: the unpipelined form
    const char* e = getenv("NEOX_ATTN_DKV_PIPE");
    return e != nullptr && atoi(e) == 0;
  }();
  if (HALVES == 2 && !serial)
    attn_bwd_dkv_kernel<DP, DROP, HALVES, HALVES == 2><<<gk, ab_threads(HALVES), BwdSmem<DP>::DYN, s>>>(tq, tk, tv, tdo, p);
  else
    attn_bwd_dkv_kernel<DP, DROP, HALVES, false><<<gk, ab_threads(HALVES), BwdSmem<DP>::DYN, s>>>(tq, tk, tv, tdo, p);
  NX_LAUNCH_CHECK();
  return NX_OK;
}

template <int DP, bool DROP>
static int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                      const CUtensorMap& tdo, const AttnBwdParams& p, cudaStream_t s) {
  static const bool four = [] {
    const char* e = getenv("NEOX_ATTN_BWD_WARPS");
    return e != nullptr && atoi(e) == 4;
  }();
  return four ? launch_bwd_h<DP, DROP, 1>(tq, tk, tv, tdo, p, s) : launch_bwd_h<DP, DROP, 2>(tq, tk, tv, tdo, p, s);
}

}  // namespace nx

// Views as in nx_flash_attn_fwd (element strides batch, head, seq).  delta: fp32 scratch [B,H,Sq]
// provided by the caller.  dq/dk/dv: 16-bit strided outputs, fully overwritten.  dropout_p / seed: the
// values the forward was given; blk_rows / blk_any / blk_size: the forward's block-sparse layout tables.
NX_API int NX_SYM(nx_flash_attn_bwd)(const void* q, const void* k, const void* v, const void* o, const void* dO,
                             const void* lse, void* delta, void* dq, void* dk, void* dv,
                             const void* alibi, int B, int H, int Hk, int Sq, int Sk, int D,
                             long long q_sb, long long q_sh, long long q_ss, long long k_sb,
                             long long k_sh, long long k_ss, long long v_sb, long long v_sh,
                             long long v_ss, long long o_sb, long long o_sh, long long o_ss,
                             long long do_sb, long long do_sh, long long do_ss, long long dq_sb,
                             long long dq_sh, long long dq_ss, long long dk_sb, long long dk_sh,
                             long long dk_ss, long long dv_sb, long long dv_sh, long long dv_ss,
                             float scale, int causal, int window, float dropout_p,
                             unsigned long long seed, const void* blk_rows, const void* blk_any, int blk_size,
                             void* stream_) {
  using namespace nx;
  if (B == 0 || H == 0 || Sq == 0 || Sk == 0) return NX_OK;
  NX_REQUIRE((blk_rows == nullptr) == (blk_any == nullptr), "flash_attn_bwd: both block-layout tables or none");
  NX_REQUIRE(blk_rows == nullptr || blk_size == 16 || blk_size == 32 || blk_size == 64 || blk_size == 128,
             "flash_attn_bwd: block-sparse layouts need a block size of 16, 32, 64 or 128 (got %d)", blk_size);
  NX_REQUIRE(dropout_p >= 0.f && dropout_p < 1.f, "flash_attn_bwd: dropout probability %f outside [0, 1)", dropout_p);
  NX_REQUIRE(D % 8 == 0 && D <= 128 && D > 0, "flash_attn_bwd: head dim %d unsupported", D);
  NX_REQUIRE(Hk > 0 && H % Hk == 0, "flash_attn_bwd: H=%d not a multiple of Hk=%d", H, Hk);
  auto aligned = [](const void* ptr, long long a, long long b, long long c) {
    return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && a % 8 == 0 && b % 8 == 0 && c % 8 == 0;
  };
  NX_REQUIRE(aligned(dq, dq_sb, dq_sh, dq_ss) && aligned(dk, dk_sb, dk_sh, dk_ss) &&
                 aligned(dv, dv_sb, dv_sh, dv_ss),
             "flash_attn_bwd: gradient views must be 16-byte aligned");
  auto s = (cudaStream_t)stream_;
  {
    const long long rows = static_cast<long long>(B) * H * Sq;
    const int wpb = 8;
    const int sq_pad = (Sq + AB - 1) / AB * AB;
    const bool aligned = ((o_sb | o_sh | o_ss | do_sb | do_sh | do_ss) % 8) == 0 &&
                         ((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(dO)) & 15) == 0;
    if (aligned && (D == 128 || D == 64)) {
      const int rpw = D == 128 ? 2 : 4;
      const long long warps = (rows + rpw - 1) / rpw;
      const unsigned grid = (unsigned)((warps + wpb - 1) / wpb);
      if (D == 128)
        attn_delta_vec8_kernel<16><<<grid, wpb * 32, 0, s>>>((const h16*)o, (const h16*)dO,
                                                            (float*)delta, B, H, Sq, sq_pad, o_sb, o_sh, o_ss, do_sb,
                                                            do_sh, do_ss);
      else
        attn_delta_vec8_kernel<8><<<grid, wpb * 32, 0, s>>>((const h16*)o, (const h16*)dO,
                                                           (float*)delta, B, H, Sq, sq_pad, o_sb, o_sh, o_ss, do_sb,
                                                           do_sh, do_ss);
    } else {
      attn_delta_kernel<<<(unsigned)((rows + wpb - 1) / wpb), wpb * 32, 0, s>>>(
          (const h16*)o, (const h16*)dO, (float*)delta, B, H, Sq, sq_pad, D, o_sb, o_sh, o_ss,
          do_sb, do_sh, do_ss);
    }
    NX_LAUNCH_CHECK();
  }
  CUtensorMap tq, tk, tv, tdo;
  if (!bwd_map(&tq, q, B, H, Sq, D, q_sb, q_sh, q_ss)) return NX_ERR_ARG;
  if (!bwd_map(&tk, k, B, Hk, Sk, D, k_sb, k_sh, k_ss)) return NX_ERR_ARG;
  if (!bwd_map(&tv, v, B, Hk, Sk, D, v_sb, v_sh, v_ss)) return NX_ERR_ARG;
  if (!bwd_map(&tdo, dO, B, H, Sq, D, do_sb, do_sh, do_ss)) return NX_ERR_ARG;
  AttnBwdParams p;
  p.lse = (const float*)lse; p.delta = (const float*)delta; p.alibi = (const float*)alibi;
  p.dq = (h16*)dq; p.dk = (h16*)dk; p.dv = (h16*)dv;
  p.dq_sb = dq_sb; p.dq_sh = dq_sh; p.dq_ss = dq_ss;
  p.dk_sb = dk_sb; p.dk_sh = dk_sh; p.dk_ss = dk_ss;
  p.dv_sb = dv_sb; p.dv_sh = dv_sh; p.dv_ss = dv_ss;
  p.B = B; p.H = H; p.Hk = Hk; p.Sq = Sq; p.Sk = Sk; p.D = D;
  p.Sq_pad = (Sq + AB - 1) / AB * AB;
  p.scale = scale; p.scale_log2 = scale * LOG2E;
  p.causal = causal; p.window = window;
  p.err = device_error_word();
  p.drop_thr = static_cast<uint32_t>(dropout_p * 256.f + 0.5f);
  if (p.drop_thr > 255u) p.drop_thr = 255u;
  p.drop_rp = 256.f / static_cast<float>(256u - p.drop_thr);
  p.seed_lo = static_cast<uint32_t>(seed);
  p.seed_hi = static_cast<uint32_t>(seed >> 32);
  p.blk_rows = static_cast<const uint8_t*>(blk_rows);
  p.blk_any = static_cast<const uint8_t*>(blk_any);
  p.blk_nkt = (Sk + AB - 1) / AB;
  p.blk_shift = blk_size == 16 ? 4 : blk_size == 32 ? 5 : blk_size == 64 ? 6 : 7;
  if (p.drop_thr > 0u) return D <= 64 ? launch_bwd<64, true>(tq, tk, tv, tdo, p, s) : launch_bwd<128, true>(tq, tk, tv, tdo, p, s);
  if (D <= 64) return launch_bwd<64, false>(tq, tk, tv, tdo, p, s);
  return launch_bwd<128, false>(tq, tk, tv, tdo, p, s);
}
