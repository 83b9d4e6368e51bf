// Flash attention forward on tcgen05: causal / sliding-window / ALiBi / GQA, bf16 in, bf16 out,
// fp32 log-sum-exp saved for the backward.
//
// Replaces the flash-attn 2 calls of the reference (megatron/model/transformer.py:573-690;
// flash_attn_func with causal=True, window_size, alibi_slopes) and, for the "global" path, the
// baddbmm -> fused softmax -> bmm chain (megatron/model/transformer.py:473-571).
//
// One CTA per (128 query rows, head, batch); 320 threads:
//   warp 0      TMA producer: Q once, then K_j / V_j blocks of 128 keys through a 2-deep ring
//   warp 1      tcgen05.mma issuer:  S_j = Q K_j^T  (two S buffers in TMEM, so S_{j+1} is computed
//               while the softmax warps work on S_j),  O += P_j V_j  with P_j read from TMEM
//   warps 2..9  softmax: two warps per TMEM lane quadrant, each owning 64 of the block's 128 key
//               columns of its 32 query rows (eight warps keep the exp2 pipe busy where four, one per
//               scheduler, left it half idle).  A thread reads its half row of S from TMEM, applies
//               scale / masks / ALiBi, exchanges the half-row maximum with its partner through shared
//               memory (a tagged word polled with a bound, never a blocking barrier), keeps online max
//               and sum in base 2, writes P (bf16) back to TMEM, rescales its half of the O columns only
//               when the running max moved by more than 2^8 (lazy rescale), and finally normalises and
//               stores its half of O.
// TMEM columns: S0 [0,128) S1 [128,256) O [256,256+DP) P0 [384,448) P1 [448,512).
// Head dims up to 128 are zero-padded to DP in {64,128} by TMA out-of-bounds fill.
//
// Second shape of the same kernel (template parameters BN = 64, HALVES = 1; the default): 64-key blocks, four
// softmax warps (a thread owns a whole row of the block: no max exchange), P_j written over the columns of S_j,
// so a CTA needs 256 TMEM columns, 96 KB of shared memory and 192 threads, and TWO CTAs share an SM: while one
// waits in its S -> softmax -> P -> PV chain the other one's MMAs run, which is what a single CTA per SM could
// not do (tensor pipe 23 - 28 % active in the first shape).  TMEM columns: S0 [0,64) S1 [64,128) O [128,128+DP),
// P_j = the first 32 columns of S_j.  NEOX_ATTN_FWD_SHAPE=1 selects the first shape.
#include <cstdlib>

#include "common.h"
#include "ptx.cuh"

namespace nx {

constexpr int ATT_BM = 128;  // query rows per CTA
constexpr int att_threads(int halves) { return 64 + 128 * halves; }

struct AttnFwdParams {
  h16* o;
  float* lse;
  const float* alibi;  // per query head, or null
  int B, H, Hk, Sq, Sk, D, Sq_pad;
  long long o_sb, o_sh, o_ss;
  float scale_log2;  // softmax scale * log2(e)
  int causal;
  int window;  // < 0: unlimited look-back
  int* err;
  // dropout on the normalised probabilities (DROP kernels only): keep iff hash byte >= drop_thr, kept
  // values scaled by drop_rp = 256 / (256 - drop_thr)
  uint32_t drop_thr, seed_lo, seed_hi;
  float drop_rp;
  // block-sparse layout (null = dense): key blocks of (1 << blk_shift) tokens, 16 <= block <= 128, one layout
  // for all heads.  blk_rows[q * blk_nkt + kt]: bit j = query row q attends to sub-block j of key tile kt (128 keys);
  // blk_any[qt * blk_nkt + kt] != 0: query tile qt (128 rows) has any live sub-block in key tile kt (else the tile
  // is skipped by every role).
  const uint8_t* blk_rows;
  const uint8_t* blk_any;
  int blk_shift, blk_nkt;
};

template <int DP, int BN>
struct AttnSmem {
  static constexpr int TILE = ATT_BM * DP * 2;  // the Q tile
  static constexpr int KV_TILE = BN * DP * 2;   // one K / V tile
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = TILE;
  static constexpr int V_OFF = TILE + 2 * KV_TILE;
  static constexpr int BAR_OFF = TILE + 4 * KV_TILE;
  // q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_empty[2], p_full[2],
  // pv_done[2]  = 17 barriers, then the TMEM base word in slot 17
  static constexpr int NBAR = 18;
  // max / sum exchange between the two column halves: [parity][half][row] 8-byte tagged words
  static constexpr int XCH_OFF = BAR_OFF + NBAR * 8 + 16;
  static constexpr int TOTAL = XCH_OFF + 2 * 2 * ATT_BM * 8;
  static constexpr int DYN = TOTAL + 1024;
};

// Row maximum of raw scores (no mask, no ALiBi), four independent chains for ILP.
template <int NC>
__device__ __forceinline__ float row_max_plain(const uint32_t (&sv)[NC][32]) {
  float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      m0 = fmax3(m0, __uint_as_float(sv[c][j]), __uint_as_float(sv[c][j + 1]));
      m1 = fmax3(m1, __uint_as_float(sv[c][j + 2]), __uint_as_float(sv[c][j + 3]));
      m2 = fmax3(m2, __uint_as_float(sv[c][j + 4]), __uint_as_float(sv[c][j + 5]));
      m3 = fmax3(m3, __uint_as_float(sv[c][j + 6]), __uint_as_float(sv[c][j + 7]));
    }
  }
  return fmaxf(fmax3(m0, m1, m2), m3);
}
// Rewrites raw scores in place as base-2 logits: x = s * scale_log2 (+ slope2 * (col - qpos)),
// -inf outside the live column range [lo, hi] of this block; returns the row maximum.
// rel0 = (first column of the block) - (query position); col0 = first block column of this half row.
// bits / shift: block-sparse layout of this row in this key tile (bit (idx >> shift) set = column idx is attended);
// 0xffffffff with any shift for a dense layout.
template <bool ALIBI, int NC>
__device__ __forceinline__ float prep_scores(uint32_t (&sv)[NC][32], float scale_log2, float slope2,
                                             int rel0, int lo, int hi, int col0, uint32_t bits, int shift) {
  float m0 = -INFINITY, m1 = -INFINITY;
  const float bias0 = ALIBI ? slope2 * static_cast<float>(rel0) : 0.f;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int idx = col0 + c * 32 + j;
      float x = __uint_as_float(sv[c][j]) * scale_log2;
      if (ALIBI) x += fmaf(slope2, static_cast<float>(idx), bias0);
      if (idx < lo || idx > hi || !((bits >> (idx >> shift)) & 1u)) x = -INFINITY;
      sv[c][j] = __float_as_uint(x);
      if (j & 1) m1 = fmaxf(m1, x); else m0 = fmaxf(m0, x);
    }
  }
  return fmaxf(m0, m1);
}

// exp2 on the FMA / ALU pipes: round-to-nearest split x = n + f, f in [-0.5, 0.5], cubic for 2^f
// (relative error 1.9e-4, below the bf16 rounding of P), n added into the exponent field.  Sharing the
// exponentials between this and the MUFU ex2 unit, and packing P to bf16 with integer adds + a byte
// permute instead of the float->bf16 convert (which issues on the same 16-lane pipe as ex2), unloads
// that pipe; kept as a selectable variant.
__device__ __forceinline__ float exp2_poly(float x) {
  x = fmaxf(x, -126.f);
  const float t = __fadd_rn(x, 12582912.f);  // 1.5 * 2^23: the rounded integer lands in the low mantissa bits
  const float f = __fsub_rn(x, __fsub_rn(t, 12582912.f));
  float q = fmaf(f, 0.05587554f, 0.24229462f);
  q = fmaf(q, f, 0.69312727f);
  q = fmaf(q, f, 0.99994826f);
  return __uint_as_float(__float_as_uint(q) + (__float_as_uint(t) << 23));
}
// (lo, hi) -> packed 16-bit pair (bf16: round-half-up on the magnitude; inputs finite and non-negative.
__device__ __forceinline__ uint32_t pack_h16x2_alu(float lo, float hi) {
#ifdef NX_HALF
  return pack_h16x2(lo, hi);      // the byte-permute trick only holds for bf16 (the top half of an fp32)
#else
  return __byte_perm(__float_as_uint(lo) + 0x8000u, __float_as_uint(hi) + 0x8000u, 0x7632);
#endif
}

// EXPV: 0 = every exp2 on the MUFU unit, convert instruction for the packing (default: fastest as measured,
// 0.306 ms against 0.313 / 0.331 ms for batch 4, 32 heads, 2048 x 128: the softmax warps are bound by the
// S -> P dependency chain per block, not by the MUFU pipe, so extra ALU instructions cost more than they
// save); 1 = MUFU + integer packing; 2 = every second exp2 as the polynomial + integer packing
// (NEOX_ATTN_EXP selects).
// DROP: dropout on the probabilities (the row sum stays that of the undropped softmax).
template <int DP, int EXPV, bool DROP, int BN, int HALVES>
__global__ void __launch_bounds__(att_threads(HALVES), BN == 64 ? 2 : 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const AttnFwdParams p) {
  static_assert((BN == 128 && HALVES == 2) || BN == 64, "a softmax thread owns 64 columns, or 32 in the third shape");
  constexpr int CPT = BN / HALVES;      // key columns of a block per softmax thread
  constexpr int NC = CPT / 32;          // ... in 32-column TMEM loads
  constexpr int ATT_BN = BN;
  constexpr int ATT_THREADS = att_threads(HALVES);
  constexpr uint32_t TMEM_COLS = BN == 128 ? 512 : 256;
  using L = AttnSmem<DP, BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t bar0 = sbase + L::BAR_OFF;
  enum { Q_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7, S_FULL = 9, S_EMPTY = 11,
         P_FULL = 13, PV_DONE = 15 };
  auto bar = [&](int which, int idx) { return bar0 + 8u * (which + idx); };
  const uint32_t tmem_slot = bar0 + 8u * 17;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(sgen + L::BAR_OFF + 8 * 17);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;  // heavy (late) query tiles first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.H / p.Hk);
  const int q0 = qt * ATT_BM;
  const int off = p.Sk - p.Sq;  // query i sits at absolute position i + off

  // key range this query tile can see
  int kv_end = p.Sk;
  if (p.causal) kv_end = min(p.Sk, q0 + ATT_BM + off);
  int kv_begin = 0;
  if (p.window >= 0) kv_begin = max(0, q0 + off - p.window);
  const int jb = kv_begin / ATT_BN;
  const int je = (kv_end + ATT_BN - 1) / ATT_BN;  // exclusive
  const int nblk = max(je - jb, 0);
  // block-sparse layouts: key tiles without a live block for this query tile are skipped by every role
  // (the layout tables are kept per 128-key tile; a 64-key block looks up the tile it lies in)
  constexpr int KT_SHIFT = BN == 64 ? 1 : 0;
  auto tile_live = [&](int kt) {
    return p.blk_any == nullptr || p.blk_any[static_cast<long long>(qt) * p.blk_nkt + (kt >> KT_SHIFT)] != 0;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < 17; ++i) {
      const bool softmax_arrives = (i >= S_EMPTY && i < S_EMPTY + 2) || (i >= P_FULL && i < P_FULL + 2);
      mbar_init(bar0 + 8u * i, softmax_arrives ? 4 * HALVES : 1);
    }
    fence_barrier_init();
  }
  for (int i = threadIdx.x; i < 2 * 2 * ATT_BM; i += ATT_THREADS)
    reinterpret_cast<unsigned long long*>(sgen + L::XCH_OFF)[i] = 0ull;
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot_gen;
  // S_j at T_S + j * BN; P_j (16 bit: BN / 2 columns) in its own columns (first shape) or over the first columns of
  // S_j (second shape: the thread that writes a row of P_j has read that row of S_j into registers before)
  // (third shape, BN = 64 with two warps per lane quadrant: the second half row's P lands on columns the FIRST half
  // row's thread reads; that thread has them in registers before it publishes its maximum, which the partner waits for)
  const uint32_t T_S = tmem, T_O = tmem + 2 * BN, T_P = BN == 128 ? tmem + 384 : tmem;
  constexpr uint32_t P_STRIDE = BN == 128 ? BN / 2 : BN;
  bool aborted = false;

  if (warp == 0) {
    if (elect_one() && nblk > 0) {
      // ---------------------------------------------------------------- producer
      mbar_expect_tx(bar(Q_FULL, 0), L::TILE);
#pragma unroll
      for (int c = 0; c < DP / 64; ++c)
        tma_load_4d(sbase + L::Q_OFF + c * (ATT_BM * 128), &tmQ, bar(Q_FULL, 0), c * 64, q0, head, batch);
      for (int i = 0, n = 0; i < nblk; ++i) {
        if (!tile_live(jb + i)) continue;
        const int st = n & 1;
        const uint32_t ph = (n >> 1) & 1;
        ++n;
        const int k0 = (jb + i) * ATT_BN;
        if (!mbar_wait(bar(K_EMPTY, st), ph ^ 1, p.err, 11)) { aborted = true; break; }
        mbar_expect_tx(bar(K_FULL, st), L::KV_TILE);
#pragma unroll
        for (int c = 0; c < DP / 64; ++c)
          tma_load_4d(sbase + L::K_OFF + st * L::KV_TILE + c * (ATT_BN * 128), &tmK, bar(K_FULL, st),
                      c * 64, k0, kv_head, batch);
        if (!mbar_wait(bar(V_EMPTY, st), ph ^ 1, p.err, 12)) { aborted = true; break; }
        mbar_expect_tx(bar(V_FULL, st), L::KV_TILE);
#pragma unroll
        for (int c = 0; c < DP / 64; ++c)
          tma_load_4d(sbase + L::V_OFF + st * L::KV_TILE + c * (ATT_BN * 128), &tmV, bar(V_FULL, st),
                      c * 64, k0, kv_head, batch);
      }
    }
  } else if (warp == 1) {
    if (elect_one() && nblk > 0) {
      // ---------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_s = umma_idesc_bf16(ATT_BM, ATT_BN, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(ATT_BM, DP, 0, 1);
      auto issue_pv = [&](int i) -> bool {
        const int st = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        if (!mbar_wait(bar(P_FULL, st), ph, p.err, 13)) return false;
        if (!mbar_wait(bar(V_FULL, st), ph, p.err, 14)) return false;
        tc_fence_after_sync();
        const uint32_t vb = sbase + L::V_OFF + st * L::KV_TILE;
#pragma unroll
        for (int k = 0; k < ATT_BN / 16; ++k) {
          // V tile is [BN keys][DP] with the head dim contiguous: MN-major B operand.
          const uint64_t bdesc = umma_smem_desc_sw128(vb + k * 2048, ATT_BN * 128, 1024);
          umma_bf16_ts(T_O, T_P + st * P_STRIDE + k * 8, bdesc, idesc_o, (i | k) != 0 ? 1u : 0u);
        }
        umma_commit(bar(PV_DONE, st));
        umma_commit(bar(V_EMPTY, st));
        return true;
      };
      if (!mbar_wait(bar(Q_FULL, 0), 0, p.err, 15)) aborted = true;
      int n = 0;      // live key tiles so far: ring stages and barrier phases count these, not the tile index
      for (int t = 0; t < nblk && !aborted; ++t) {
        if (!tile_live(jb + t)) continue;
        const int i = n++;
        const int st = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        if (!mbar_wait(bar(K_FULL, st), ph, p.err, 16)) { aborted = true; break; }
        if (!mbar_wait(bar(S_EMPTY, st), ph ^ 1, p.err, 17)) { aborted = true; break; }
        tc_fence_after_sync();
        const uint32_t qb = sbase + L::Q_OFF, kb = sbase + L::K_OFF + st * L::KV_TILE;
#pragma unroll
        for (int k = 0; k < DP / 16; ++k) {
          const uint32_t oq = (k >> 2) * (ATT_BM * 128) + (k & 3) * 32;
          const uint32_t ok = (k >> 2) * (ATT_BN * 128) + (k & 3) * 32;
          umma_bf16_ss(T_S + st * BN, umma_smem_desc_sw128(qb + oq, 0, 1024),
                       umma_smem_desc_sw128(kb + ok, 0, 1024), idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit(bar(S_FULL, st));
        umma_commit(bar(K_EMPTY, st));
        if (i > 0 && !issue_pv(i - 1)) { aborted = true; break; }
      }
      if (!aborted && n > 0 && !issue_pv(n - 1)) aborted = true;
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue
    const int quad = warp & 3;
    const int half = HALVES == 2 ? (warp - 2) >> 2 : 0;  // first shape: which 64 of the block's 128 key columns (and half of O)
    const int col0 = half * CPT;
    const int r = quad * 32 + lane;  // row in tile == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    volatile unsigned long long* xch = reinterpret_cast<volatile unsigned long long*>(sgen + L::XCH_OFF);
    // publish `v` under tag `seq` and fetch the partner's value with the same tag (bounded poll)
    auto exchange = [&](float v, uint32_t seq, float& other) -> bool {
      const int par = seq & 1;
      xch[(par * 2 + half) * ATT_BM + r] = (static_cast<unsigned long long>(seq) << 32) | __float_as_uint(v);
      volatile unsigned long long* src = xch + (par * 2 + (half ^ 1)) * ATT_BM + r;
      for (int spin = 0; spin < (1 << 22); ++spin) {
        const unsigned long long w = *src;
        if (static_cast<uint32_t>(w >> 32) == seq) {
          other = __uint_as_float(static_cast<uint32_t>(w));
          return true;
        }
        if (spin > 4096) __nanosleep(64);
      }
      if (p.err != nullptr) atomicExch(p.err, 22);
      return false;
    };
    const int qi = q0 + r;
    const int qpos = qi + off;
    float m_used = -INFINITY, l = 0.f;
    const float slope2 = p.alibi != nullptr ? p.alibi[head] * 1.4426950408889634f : 0.f;
    int nlive = 0;
    for (int t = 0; t < nblk; ++t) {
      if (!tile_live(jb + t)) continue;
      const int i = nlive++;
      const int st = i & 1;
      const uint32_t ph = (i >> 1) & 1;
      const int k0 = (jb + t) * ATT_BN;
      // block-sparse: which 16..128-key sub-blocks of this key tile the row attends to
      uint32_t bits = 0xffffffffu;
      if (p.blk_rows != nullptr) {
        bits = qi < p.Sq ? p.blk_rows[static_cast<long long>(qi) * p.blk_nkt + ((jb + t) >> KT_SHIFT)] : 0u;
        if (BN == 64) bits >>= ((jb + t) & 1) * (64 >> p.blk_shift);      // the 64-key half of the 128-key tile
      }
      const uint32_t full_bits = (1u << max(1, ATT_BN >> p.blk_shift)) - 1u;
      const bool blk_partial = p.blk_rows != nullptr && !__all_sync(0xffffffffu, (bits & full_bits) == full_bits);
      if (!mbar_wait(bar(S_FULL, st), ph, p.err, 18)) { aborted = true; break; }
      tc_fence_after_sync();
      // One read of the whole score row into registers.
      uint32_t sv[NC][32];
#pragma unroll
      for (int c = 0; c < NC; ++c) tmem_ld_32x32b_x32(T_S + st * BN + col0 + c * 32 + lane_off, sv[c]);
      tmem_ld_wait();
      // Does this block need per-element masking?  (warp-uniform decision)
      const bool need_mask = (k0 + ATT_BN > p.Sk) || (p.causal && k0 + ATT_BN - 1 > q0 + quad * 32 + off) ||
                             (p.window >= 0 && k0 < q0 + quad * 32 + 31 + off - p.window) || blk_partial;
      const bool plain = !need_mask && p.alibi == nullptr;
      float mx;
      if (plain) {
        mx = row_max_plain<NC>(sv) * p.scale_log2;
      } else {
        // columns idx (0..127) of this block are alive for lo <= idx <= hi
        const int rel0 = k0 - qpos;
        int hi = p.Sk - k0 - 1;
        if (p.causal) hi = min(hi, -rel0);
        const int lo = p.window >= 0 ? -rel0 - p.window : -(1 << 30);
        mx = p.alibi != nullptr ? prep_scores<true, NC>(sv, p.scale_log2, slope2, rel0, lo, hi, col0, bits, p.blk_shift)
                                : prep_scores<false, NC>(sv, p.scale_log2, slope2, rel0, lo, hi, col0, bits, p.blk_shift);
      }
      if (HALVES == 2) {
        // the row maximum over both column halves: both partners then take identical decisions
        float other;
        bool ok = exchange(mx, static_cast<uint32_t>(i + 1), other);
        if (!__all_sync(0xffffffffu, ok)) { aborted = true; break; }
        mx = fmaxf(mx, other);
      }
      float alpha = 1.f;
      bool rescale = false;
      if (mx > m_used + 8.f || m_used == -INFINITY) {
        const float m_new = fmaxf(m_used, mx);
        if (m_used != -INFINITY) {
          alpha = exp2f(m_used - m_new);
          rescale = true;
        }
        m_used = m_new;
        l *= alpha;
      }
      if (i > 0 && __any_sync(0xffffffffu, rescale)) {
        // O must be complete up to block i-1 before it is rescaled.
        if (!mbar_wait(bar(PV_DONE, (i - 1) & 1), ((i - 1) >> 1) & 1, p.err, 19)) { aborted = true; break; }
        tc_fence_after_sync();
#pragma unroll 1
        for (int c = half * (DP / 32 / HALVES); c < (half + 1) * (DP / 32 / HALVES); ++c) {   // this warp's O columns
          uint32_t ov[32];
          tmem_ld_32x32b_x32(T_O + c * 32 + lane_off, ov);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float2 o2 = fmul2(u2f2(ov[j], ov[j + 1]), make_float2(alpha, alpha));
            ov[j] = __float_as_uint(o2.x);
            ov[j + 1] = __float_as_uint(o2.y);
          }
          tmem_st_32x32b_x32(T_O + c * 32 + lane_off, ov);
        }
        tmem_st_wait();
      }
      // P buffer `st` was last read by PV_{i-2}.
      if (i >= 2) {
        if (!mbar_wait(bar(PV_DONE, st), ((i - 2) >> 1) & 1, p.err, 20)) { aborted = true; break; }
      }
      // probabilities (base 2), packed to bf16 and written to TMEM as the A operand of P V
      const float msub = m_used == -INFINITY ? 0.f : m_used;
      // (packed fp32 pairs: one FFMA2 scales and shifts two scores, one FADD2 adds two probabilities to the row sums)
      float2 rs[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
      const float2 sc2 = make_float2(plain ? p.scale_log2 : 1.f, plain ? p.scale_log2 : 1.f);
      const float2 nm2 = make_float2(-msub, -msub);
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float2 x = ffma2(u2f2(sv[c][j], sv[c][j + 1]), sc2, nm2);
          float p0 = exp2f(x.x);
          float p1 = EXPV == 2 ? exp2_poly(x.y) : exp2f(x.y);
          rs[(j >> 1) & 3] = fadd2(rs[(j >> 1) & 3], make_float2(p0, p1));
          if (DROP) {
            const int kk = k0 + col0 + c * 32 + j;        // even: (kk, kk + 1) share one patch
            const uint32_t patch = dropout_patch(p.seed_lo, p.seed_hi, static_cast<uint32_t>(batch * p.H + head),
                                                 static_cast<uint32_t>(qi) >> 1, static_cast<uint32_t>(kk) >> 1);
            if (!dropout_keep(patch, qi, kk, p.drop_thr)) p0 = 0.f;
            if (!dropout_keep(patch, qi, kk + 1, p.drop_thr)) p1 = 0.f;
          }
          pk[j >> 1] = EXPV == 0 ? pack_h16x2(p0, p1) : pack_h16x2_alu(p0, p1);
        }
        tmem_st_32x32b_x16(T_P + st * P_STRIDE + half * (CPT / 2) + c * 16 + lane_off, pk);
      }
      const float2 rs01 = fadd2(fadd2(rs[0], rs[1]), fadd2(rs[2], rs[3]));
      const float rowsum = rs01.x + rs01.y;
      l += rowsum;
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar(S_EMPTY, st));
        mbar_arrive(bar(P_FULL, st));
      }
    }
    // ---- epilogue: O / l -> global, lse
    const int nblk_live = nlive;      // (below, "nblk" means the key tiles that were really processed)
    if (!aborted && nblk_live > 0) {
      if (!mbar_wait(bar(PV_DONE, (nblk_live - 1) & 1), ((nblk_live - 1) >> 1) & 1, p.err, 21)) aborted = true;
      tc_fence_after_sync();
    }
    if (HALVES == 2 && !aborted) {
      // total row sum = this half's + the partner's (same running max on both sides)
      float other = 0.f;
      const bool ok = exchange(l, static_cast<uint32_t>(nblk_live + 1), other);
      if (!__all_sync(0xffffffffu, ok)) aborted = true;
      l += other;
    }
    if (!aborted) {
      const float inv_l = (l > 0.f ? 1.f / l : 0.f) * (DROP ? p.drop_rp : 1.f);
      const bool row_ok = qi < p.Sq;
      h16* orow = p.o + batch * p.o_sb + head * p.o_sh + static_cast<long long>(qi) * p.o_ss;
#pragma unroll 1
      for (int c = half * (DP / 32 / HALVES); c < (half + 1) * (DP / 32 / HALVES); ++c) {
        uint32_t ov[32];
        if (nblk_live > 0) {
          tmem_ld_32x32b_x32(T_O + c * 32 + lane_off, ov);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) ov[j] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (c * 32 + j < p.D) {
              uint4 o4;
              o4.x = pack_h16x2(__uint_as_float(ov[j]) * inv_l, __uint_as_float(ov[j + 1]) * inv_l);
              o4.y = pack_h16x2(__uint_as_float(ov[j + 2]) * inv_l, __uint_as_float(ov[j + 3]) * inv_l);
              o4.z = pack_h16x2(__uint_as_float(ov[j + 4]) * inv_l, __uint_as_float(ov[j + 5]) * inv_l);
              o4.w = pack_h16x2(__uint_as_float(ov[j + 6]) * inv_l, __uint_as_float(ov[j + 7]) * inv_l);
              *reinterpret_cast<uint4*>(orow + c * 32 + j) = o4;
            }
          }
        }
      }
      if (row_ok && half == 0) {
        // base-2 log-sum-exp of the scaled scores; rows are padded to a multiple of 128
        const float lse2 = l > 0.f ? m_used + log2f(l) : -INFINITY;
        p.lse[(static_cast<long long>(batch) * p.H + head) * p.Sq_pad + qi] = lse2;
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
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// Builds the 4-D (d, s, head, batch) tensor map of a [B, heads, S, D] view given element strides.
static bool attn_map(CUtensorMap* m, const void* base, int B, int Hh, int S, int D, long long sb,
                     long long sh, long long ss, int box_rows) {
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)S, (uint64_t)Hh, (uint64_t)B};
  const uint64_t strides[3] = {(uint64_t)ss * 2, (uint64_t)sh * 2, (uint64_t)sb * 2};
  const uint32_t box[4] = {64, (uint32_t)box_rows, 1, 1};
  return make_tma_4d(m, base, dims, strides, box, 2, true);
}

}  // namespace nx

// q [B,H,Sq,D], k/v [B,Hk,Sk,D], o [B,H,Sq,D] as strided views (element strides for batch, head,
// sequence; head dim contiguous); lse: fp32 [B,H,Sq_pad] (Sq rounded up to 128), receives the
// base-2 log-sum-exp of the scaled scores for rows < Sq (the caller pre-fills it with +inf).  alibi: fp32 [H] or null.
// window < 0: no sliding window.  D % 8 == 0, D <= 128.  dropout_p > 0: dropout on the probabilities with
// the mask of dropout_patch() under `seed` (the backward must be given the same p and seed).
// blk_rows / blk_any (both or neither): block-sparse layout tables, uint8 [Sq, ceil(Sk / 128)] and
// [ceil(Sq / 128), ceil(Sk / 128)] (see AttnFwdParams), blk_size the layout's block size in tokens.
NX_API int NX_SYM(nx_flash_attn_fwd)(const void* q, const void* k, const void* v, void* o, void* lse,
                             const void* alibi, int B, int H, int Hk, int Sq, int Sk, int D,
                             long long q_sb, long long q_sh, long long q_ss, long long k_sb,
                             long long k_sh, long long k_ss, long long v_sb, long long v_sh,
                             long long v_ss, long long o_sb, long long o_sh, long long o_ss,
                             float scale, int causal, int window, float dropout_p,
                             unsigned long long seed, const void* blk_rows, const void* blk_any, int blk_size,
                             void* stream_) {
  using namespace nx;
  if (B == 0 || H == 0 || Sq == 0) return NX_OK;
  NX_REQUIRE(D % 8 == 0 && D <= 128 && D > 0, "flash_attn: head dim %d unsupported (need %%8, <=128)", D);
  NX_REQUIRE((blk_rows == nullptr) == (blk_any == nullptr), "flash_attn: both block-layout tables or none");
  NX_REQUIRE(blk_rows == nullptr || blk_size == 16 || blk_size == 32 || blk_size == 64 || blk_size == 128,
             "flash_attn: block-sparse layouts need a block size of 16, 32, 64 or 128 (got %d)", blk_size);
  NX_REQUIRE(dropout_p >= 0.f && dropout_p < 1.f, "flash_attn: dropout probability %f outside [0, 1)", dropout_p);
  NX_REQUIRE(dropout_p == 0.f || (Sq <= 131072 && Sk <= 131072), "flash_attn: dropout needs sequences <= 131072");
  NX_REQUIRE(Hk > 0 && H % Hk == 0, "flash_attn: H=%d not a multiple of Hk=%d", H, Hk);
  NX_REQUIRE(Sk >= 1, "flash_attn: empty key sequence");
  NX_REQUIRE((o_ss % 8) == 0 && (o_sh % 8) == 0 && (o_sb % 8) == 0 &&
                 (reinterpret_cast<uintptr_t>(o) & 15) == 0,
             "flash_attn: output view must be 16-byte aligned");
  CUtensorMap tq, tk, tv;
  // 2 (default): 64-key blocks, four softmax warps, two CTAs per SM; 1: 128-key blocks, eight softmax warps, one CTA per
  // SM; 3: 64-key blocks, eight softmax warps on 32-column half rows, two CTAs per SM
  static const int shape = [] {
    const char* e = getenv("NEOX_ATTN_FWD_SHAPE");
    const int v = e != nullptr ? atoi(e) : 2;
    return v == 1 || v == 3 ? v : 2;
  }();
  const int bn = shape == 1 ? 128 : 64;
  if (!attn_map(&tq, q, B, H, Sq, D, q_sb, q_sh, q_ss, ATT_BM)) return NX_ERR_ARG;
  if (!attn_map(&tk, k, B, Hk, Sk, D, k_sb, k_sh, k_ss, bn)) return NX_ERR_ARG;
  if (!attn_map(&tv, v, B, Hk, Sk, D, v_sb, v_sh, v_ss, bn)) return NX_ERR_ARG;
  AttnFwdParams p;
  p.o = (h16*)o; p.lse = (float*)lse; p.alibi = (const float*)alibi;
  p.B = B; p.H = H; p.Hk = Hk; p.Sq = Sq; p.Sk = Sk; p.D = D;
  p.Sq_pad = (Sq + ATT_BM - 1) / ATT_BM * ATT_BM;
  p.o_sb = o_sb; p.o_sh = o_sh; p.o_ss = o_ss;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal; p.window = window;
  p.err = device_error_word();
  p.drop_thr = static_cast<uint32_t>(dropout_p * 256.f + 0.5f);     // p in steps of 1 / 256
  if (p.drop_thr > 255u) p.drop_thr = 255u;
  p.drop_rp = 256.f / static_cast<float>(256u - p.drop_thr);
  p.seed_lo = static_cast<uint32_t>(seed);
  p.seed_hi = static_cast<uint32_t>(seed >> 32);
  p.blk_rows = static_cast<const uint8_t*>(blk_rows);
  p.blk_any = static_cast<const uint8_t*>(blk_any);
  p.blk_nkt = (Sk + 127) / 128;
  p.blk_shift = blk_size == 16 ? 4 : blk_size == 32 ? 5 : blk_size == 64 ? 6 : 7;
  const bool drop = p.drop_thr > 0u;
  dim3 grid((Sq + ATT_BM - 1) / ATT_BM, H, B);
  auto s = (cudaStream_t)stream_;
  static const int expv = [] {
    const char* e = getenv("NEOX_ATTN_EXP");
    const int v = e ? atoi(e) : 0;
    return v < 0 || v > 2 ? 0 : v;
  }();
#define NX_ATTN_LAUNCH(DPV, EV, DR, BNV, HV)                                                                 \
  do {                                                                                                       \
    static bool cfg = false;                                                                                 \
    auto kern = attn_fwd_kernel<DPV, EV, DR, BNV, HV>;                                                       \
    if (!cfg) {                                                                                              \
      NX_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,                  \
                                         AttnSmem<DPV, BNV>::DYN));                                          \
      cfg = true;                                                                                            \
    }                                                                                                        \
    kern<<<grid, att_threads(HV), AttnSmem<DPV, BNV>::DYN, s>>>(tq, tk, tv, p);                              \
  } while (0)
  if (shape == 3) {
    if (drop) {
      if (D <= 64) NX_ATTN_LAUNCH(64, 0, true, 64, 2);
      else NX_ATTN_LAUNCH(128, 0, true, 64, 2);
    } else if (D <= 64) {
      NX_ATTN_LAUNCH(64, 0, false, 64, 2);
    } else {
      NX_ATTN_LAUNCH(128, 0, false, 64, 2);
    }
  } else if (shape == 2) {
    if (drop) {
      if (D <= 64) NX_ATTN_LAUNCH(64, 0, true, 64, 1);
      else NX_ATTN_LAUNCH(128, 0, true, 64, 1);
    } else if (D <= 64) {
      NX_ATTN_LAUNCH(64, 0, false, 64, 1);
    } else {
      NX_ATTN_LAUNCH(128, 0, false, 64, 1);
    }
  } else if (drop) {
    if (D <= 64) NX_ATTN_LAUNCH(64, 0, true, 128, 2);
    else NX_ATTN_LAUNCH(128, 0, true, 128, 2);
  } else if (D <= 64) {
    if (expv == 0) NX_ATTN_LAUNCH(64, 0, false, 128, 2);
    else if (expv == 1) NX_ATTN_LAUNCH(64, 1, false, 128, 2);
    else NX_ATTN_LAUNCH(64, 2, false, 128, 2);
  } else {
    if (expv == 0) NX_ATTN_LAUNCH(128, 0, false, 128, 2);
    else if (expv == 1) NX_ATTN_LAUNCH(128, 1, false, 128, 2);
    else NX_ATTN_LAUNCH(128, 2, false, 128, 2);
  }
#undef NX_ATTN_LAUNCH
  NX_LAUNCH_CHECK();
  return NX_OK;
}
