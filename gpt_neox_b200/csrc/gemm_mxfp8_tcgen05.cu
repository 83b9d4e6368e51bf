// Block-scaled FP8 GEMM (MXFP8) on the 5th-generation tensor cores:
//   C[M,N] = alpha * sum_k (A[m,k] * 2^(sa[m, k/32] - 127)) * (B[n,k] * 2^(sb[n, k/32] - 127))  (+ bias)
// A [M,K] and B [N,K] in e4m3 / e5m2 (one byte per element, K-major), one power-of-two (ue8m0) scale per 32
// consecutive K elements of every row of A and of B, applied by the tensor core itself
// (tcgen05.mma.kind::mxf8f6f4.block_scale), fp32 accumulation in tensor memory, 16-bit or fp32 output.
//
// Counterpart in the reference: Transformer Engine's fp8 Linear with a block-scaling (MXFP8) recipe
// (megatron/model/transformer_engine.py:247-517 builds its layers on TE, whose Blackwell recipe is this format).
//
// Scale factors.  The instruction reads them from tensor memory: for the 128 rows of an operand tile and the four
// K = 32 steps of a 128-element K block, 4 columns of 32-bit cells whose cell (lane l, column c) holds the four scale
// bytes (one per K step, selected by the scale-factor id in the instruction descriptor) of tile row 32 c + (l mod 32),
// the same in all four 32-lane quarters.  Host side they are stored as words: sf[kb][row] = the four ue8m0 bytes of
// K groups 4 kb .. 4 kb + 3 of that row (little endian), rows padded to a multiple of 128 with 0x7f (scale 1).
// Four warps bring the words of a K block to tensor memory (tcgen05.st, each warp its own lane quarter) one ring
// stage ahead of the MMA warp.
//
// Pipeline: one persistent CTA per SM, 128 x BN tiles; warp 0 issues TMA loads into a shared-memory ring
// (128-byte swizzle: a row of a tile is 128 fp8 values), warp 1 issues the MMAs, warps 2-5 drain the TMEM
// accumulators, warps 6-9 stage the scale factors.  TMEM: accumulator stages [0, NACC * BN), then 16 columns per ring
// stage for the scale cells.  The accumulators cannot be 2 x 256 columns as in the per-tensor kernel (the scale cells
// need room), so the tile is 128 x 256 with one accumulator stage (the default: fastest as measured) or narrower with two.
//
// Plus the quantiser: 16-bit -> fp8 with one scale per 32 elements of a row, emitted in the layout above.
#include <cuda_fp8.h>

#include "common.h"
#include "ptx.cuh"

namespace nx {

namespace mx {
constexpr int BM = 128, BK = 128, UK = 32, THREADS = 320;
constexpr uint32_t TMEM_COLS = 512;
constexpr int SF_STRIDE = 16;             // TMEM columns per scale stage: A in 0..3, B in 4..4 + BN / 32
// Tile shapes.  BN columns per tile, NACC accumulator stages, ring stages such that the TMEM columns
// (NACC * BN + 16 per stage) fit 512 and the operand ring fits shared memory.
template <int BN_, int NACC_, int STAGES_>
struct Cfg {
  static constexpr int BN = BN_, NACC = NACC_, STAGES = STAGES_;
  static constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int NBAR = 3 * STAGES + 4;
  static constexpr int DYN_BYTES = BAR_OFFSET + NBAR * 8 + 16 + 1024;
  static constexpr uint32_t SF_COL0 = NACC * BN;      // first scale-factor column
  static_assert(NACC * BN + STAGES * SF_STRIDE <= 512, "tensor memory");
  static_assert(DYN_BYTES <= 227 * 1024, "shared memory");
  static_assert(BN % 32 == 0 && BN <= 256 && 4 + BN / 32 <= SF_STRIDE, "tile width");
};
}  // namespace mx

struct MxGemmParams {
  int M, N, K;
  void* C;
  long long ldc;
  const float* alpha;               // device scalar or null (= 1)
  const h16* bias;
  const uint32_t* sfa;              // [num_kb][ld_sfa] scale words of A
  const uint32_t* sfb;              // [num_kb][ld_sfb] scale words of B
  long long ld_sfa, ld_sfb;
  int out_f32, accumulate;
  int tiles_m, tiles_n;
  uint32_t idesc;
  int* err;
};

__device__ __forceinline__ void umma_mxf8_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb), "r"(accumulate)
      : "memory");
}

// Block-scaled instruction descriptor: scale-factor id of B at bits [4,6), a / b format at bits 7 / 10 (0 = e4m3,
// 1 = e5m2), both K-major, N >> 3 at bit 17, scale type at bit 23 (1 = ue8m0), M >> 4 at bit 24, scale-factor id of
// A at bits [29,31).  The ids (which of the four bytes of a scale cell a K step uses) are or-ed in per instruction.
static uint32_t idesc_mxf8(int a_e5m2, int b_e5m2, int bn) {
  return (static_cast<uint32_t>(a_e5m2) << 7) | (static_cast<uint32_t>(b_e5m2) << 10) |
         (static_cast<uint32_t>(bn >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(mx::BM >> 4) << 24);
}

template <class C>
__global__ void __launch_bounds__(mx::THREADS, 1)
    gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const MxGemmParams p) {
  using namespace mx;
  constexpr int BN = C::BN, NACC = C::NACC, STAGES = C::STAGES, A_BYTES = C::A_BYTES, STAGE_BYTES = C::STAGE_BYTES,
                BAR_OFFSET = C::BAR_OFFSET, NBAR = C::NBAR;
  constexpr uint32_t SF_COL0 = C::SF_COL0;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto sf_full_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (3 * STAGES + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (3 * STAGES + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * NBAR;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + BAR_OFFSET + 8 * NBAR);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(sf_full_bar(s), 4);
    }
    for (int a = 0; a < NACC; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), 4);
    }
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
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;
  bool aborted = false;

  if (warp == 0) {
    if (elect_one()) {
      // ------------------------------------------------------------------ TMA producer
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !aborted; tile += gridDim.x) {
        const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, p.err, 71)) {
            aborted = true;
            break;
          }
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          tma_load_2d(a_dst, &tmA, full_bar(stage), kb * BK, tm * BM);
          tma_load_2d(a_dst + A_BYTES, &tmB, full_bar(stage), kb * BK, tn * BN);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      // ------------------------------------------------------------------ MMA issuer
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !aborted; tile += gridDim.x) {
        if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1, p.err, 72)) {
          aborted = true;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, p.err, 73) || !mbar_wait(sf_full_bar(stage), phase, p.err, 74)) {
            aborted = true;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_base + stage * STAGE_BYTES;
          const uint32_t b_addr = a_addr + A_BYTES;
          const uint32_t t_sfa = tmem_base + SF_COL0 + stage * SF_STRIDE, t_sfb = t_sfa + 4;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            // K-major, 128-byte swizzle: 8-row groups 1024 B apart; 32 fp8 K-elements advance 32 B; K step k uses
            // byte k of the scale cells
            const uint64_t adesc = umma_smem_desc_sw128(a_addr + k * UK, 0, 1024);
            const uint64_t bdesc = umma_smem_desc_sw128(b_addr + k * UK, 0, 1024);
            const uint32_t idesc = p.idesc | (static_cast<uint32_t>(k) << 29) | (static_cast<uint32_t>(k) << 4);
            umma_mxf8_ss(d_tmem, adesc, bdesc, idesc, t_sfa, t_sfb, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));       // frees the operand stage AND its scale-factor columns
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (aborted) break;
        umma_commit(tmem_full_bar(acc));
        if (++acc == NACC) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else if (warp >= 6) {
    // -------------------------------------------------------------------- scale-factor staging (warps 6..9)
    const int quad = warp & 3;                 // the TMEM lane quarter this warp may write
    int stage = 0;
    uint32_t phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles && !aborted; tile += gridDim.x) {
      const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
      const long long m0 = static_cast<long long>(tm) * BM, n0 = static_cast<long long>(tn) * BN;
      for (int kb = 0; kb < num_kb; ++kb) {
        // cell (lane l, column c) = the scale word of tile row 32 c + l: A in columns 0..3, B in 4..4 + BN / 32; rows past
        // the padded end of the scale array (a tile width that is not a multiple of 128) re-read its last word: the
        // operand rows there are zero-filled by TMA and their outputs are never stored
        uint32_t w[16];
        const uint32_t* ra = p.sfa + kb * p.ld_sfa;
        const uint32_t* rb = p.sfb + kb * p.ld_sfb;
#pragma unroll
        for (int c = 0; c < 4; ++c) w[c] = __ldg(ra + min(m0 + 32 * c + lane, p.ld_sfa - 1));
#pragma unroll
        for (int c = 0; c < 12; ++c)
          w[4 + c] = c < BN / 32 ? __ldg(rb + min(n0 + 32 * c + lane, p.ld_sfb - 1)) : 0x7f7f7f7fu;
        bool ok = mbar_wait(empty_bar(stage), phase ^ 1, p.err, 75);
        if (!__all_sync(0xffffffffu, ok)) {
          aborted = true;
          break;
        }
        tc_fence_after_sync();
        tmem_st_32x32b_x16(tmem_base + SF_COL0 + stage * SF_STRIDE + (static_cast<uint32_t>(quad * 32) << 16), w);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(sf_full_bar(stage));
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // -------------------------------------------------------------------- epilogue (warps 2..5)
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    const float alpha = p.alpha != nullptr ? *p.alpha : 1.f;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
      const int m0 = tm * BM, n0 = tn * BN;
      if (!mbar_wait(tmem_full_bar(acc), acc_phase, p.err, 76)) {
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
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * alpha;
        if (p.bias != nullptr) {
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
          if (p.out_f32) {
            float* cp = reinterpret_cast<float*>(p.C) + row * p.ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col0 + j < p.N) {
                float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                if (p.accumulate) {
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
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar(acc));
      if (++acc == NACC) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }
  __syncwarp();
  if (aborted) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);      // copies / MMAs still in flight finish before TMEM goes
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

namespace mx {
template <class C>
static int launch(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb, MxGemmParams p,
                  int a_e5m2, int b_e5m2, cudaStream_t stream) {
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + C::BN - 1) / C::BN;
  p.idesc = idesc_mxf8(a_e5m2, b_e5m2, C::BN);
  CUtensorMap tmA, tmB;
  if (!make_tma_2d(&tmA, A, M, K, lda, BM, BK, 1)) return NX_ERR_ARG;
  if (!make_tma_2d(&tmB, B, N, K, ldb, C::BN, BK, 1)) return NX_ERR_ARG;
  static bool configured = false;
  if (!configured) {
    NX_CUDA_CHECK(cudaFuncSetAttribute(gemm_mxfp8_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::DYN_BYTES));
    configured = true;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  gemm_mxfp8_kernel<C><<<grid, THREADS, C::DYN_BYTES, stream>>>(tmA, tmB, p);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
}  // namespace mx

// A [M, K] and B [N, K]: fp8 bytes, leading dimensions in elements (multiples of 16); sfa / sfb: scale words
// [ceil(K / 128)][ld_sf*] with ld_sfa >= round_up(M, 128), ld_sfb >= round_up(N, 128) (padding rows hold 0x7f7f7f7f);
// a_e5m2 / b_e5m2 select the operand formats.  C: 16-bit [M, N] or fp32 (out_f32; accumulate adds into it).
// tile: 0 = chosen here; 128 / 192 / 224 / 256 = that tile width (256: one accumulator stage).
NX_API int NX_SYM(nx_gemm_mxfp8)(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                 long long ldb, long long ldc, const void* sfa, const void* sfb, long long ld_sfa,
                                 long long ld_sfb, int a_e5m2, int b_e5m2, const void* alpha, const void* bias,
                                 int out_f32, int accumulate, int tile, cudaStream_t stream) {
  using namespace mx;
  NX_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_mxfp8: empty problem");
  NX_REQUIRE(lda % 16 == 0 && ldb % 16 == 0 && K % 32 == 0, "gemm_mxfp8: K must be a multiple of 32, leading dimensions of 16");
  NX_REQUIRE(N % 8 == 0 && ldc % (out_f32 ? 4 : 8) == 0, "gemm_mxfp8: N / ldc alignment");
  NX_REQUIRE((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) % 16 == 0,
             "gemm_mxfp8: operands must be 16-byte aligned");
  NX_REQUIRE(sfa != nullptr && sfb != nullptr, "gemm_mxfp8: scale factors are required");
  NX_REQUIRE(ld_sfa >= (M + 127) / 128 * 128 && ld_sfb >= (N + 127) / 128 * 128,
             "gemm_mxfp8: scale rows must be padded to multiples of 128 (ld_sfa %lld, ld_sfb %lld)", ld_sfa, ld_sfb);
  MxGemmParams p{};
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc;
  p.alpha = static_cast<const float*>(alpha);
  p.bias = static_cast<const h16*>(bias);
  p.sfa = static_cast<const uint32_t*>(sfa); p.sfb = static_cast<const uint32_t*>(sfb);
  p.ld_sfa = ld_sfa; p.ld_sfb = ld_sfb;
  p.out_f32 = out_f32; p.accumulate = accumulate;
  p.err = device_error_word();
  // measured (8192 x 12288 x 4096 / 8192 x 4096 x 16384): 128: 1287 / 1050, 192: 1724 / 1390, 224: 1909 / 1530,
  // 256 with one accumulator stage: 2056 / 1899 TFLOP/s -- the wide tile outweighs the unhidden epilogue
  if (tile == 0) tile = N <= 128 ? 128 : 256;
  switch (tile) {
    case 128: return launch<Cfg<128, 2, 6>>(A, B, M, N, K, lda, ldb, p, a_e5m2, b_e5m2, stream);
    case 192: return launch<Cfg<192, 2, 5>>(A, B, M, N, K, lda, ldb, p, a_e5m2, b_e5m2, stream);
    case 224: return launch<Cfg<224, 2, 4>>(A, B, M, N, K, lda, ldb, p, a_e5m2, b_e5m2, stream);
    case 256: return launch<Cfg<256, 1, 4>>(A, B, M, N, K, lda, ldb, p, a_e5m2, b_e5m2, stream);
    default: NX_REQUIRE(false, "gemm_mxfp8: tile width %d (128, 192, 224 or 256)", tile);
  }
  return NX_ERR_ARG;
}

// ---------------------------------------------------------------------------------------------
// Quantiser: one thread per (row, group of 32 columns).  scale = 2^e with e = ceil(log2(amax / fp8_max)) (the
// smallest power of two that brings the group into range), stored as the ue8m0 byte e + 127 in byte (g mod 4) of
// word sf[g / 4][row]; values are multiplied by 2^-e and converted with saturation.
// ---------------------------------------------------------------------------------------------
template <bool E5M2>
__global__ void __launch_bounds__(256)
mxfp8_quantize_kernel(const h16* __restrict__ x, long long ldx, uint8_t* __restrict__ out, long long ldo,
                      uint8_t* __restrict__ sf, long long ld_sf, int rows, int groups) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= static_cast<long long>(rows) * groups) return;
  const int row = static_cast<int>(t / groups), g = static_cast<int>(t % groups);
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(row) * ldx + g * 32);
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 u = src[i];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_h16x2(w[j]);
      v[i * 8 + 2 * j] = f.x;
      v[i * 8 + 2 * j + 1] = f.y;
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  constexpr float FP8_MAX = E5M2 ? 57344.f : 448.f;
  int e = 0;
  if (amax > 0.f && amax < INFINITY) {
    const uint32_t bits = __float_as_uint(amax / FP8_MAX);
    e = static_cast<int>((bits >> 23) & 0xffu) - 127 + ((bits & 0x7fffffu) != 0u ? 1 : 0);
    e = max(-127, min(127, e));
  }
  const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);        // 2^-e (e = 127 gives a denormal: 0)
  uint32_t q[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint32_t wq = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      wq |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(v[i * 4 + j] * inv, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3))
            << (8 * j);
    q[i] = wq;
  }
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(row) * ldo + g * 32);
  dst[0] = make_uint4(q[0], q[1], q[2], q[3]);
  dst[1] = make_uint4(q[4], q[5], q[6], q[7]);
  sf[(static_cast<long long>(g >> 2) * ld_sf + row) * 4 + (g & 3)] = static_cast<uint8_t>(e + 127);
}

// Both forms from one read: the row-wise form above (scale blocks along the columns: the operand of a GEMM that
// contracts over the columns) and the column-wise form (out_t [cols, rows] with scale blocks along the ROWS of x: the
// operand of a GEMM that contracts over the rows, which both backward GEMMs of a linear layer need).  A block takes
// a 32-row x 256-column tile: thread (row t / 8, group t mod 8) quantises its 32 row elements and leaves the 16-bit
// values in shared memory, then thread t quantises column t of the tile (32 values down the rows).
template <bool E5M2>
__device__ __forceinline__ uint8_t mx_scale_and_quantize(const float (&v)[32], float amax, uint32_t (&q)[8]) {
  constexpr float FP8_MAX = E5M2 ? 57344.f : 448.f;
  int e = 0;
  if (amax > 0.f && amax < INFINITY) {
    const uint32_t bits = __float_as_uint(amax / FP8_MAX);
    e = static_cast<int>((bits >> 23) & 0xffu) - 127 + ((bits & 0x7fffffu) != 0u ? 1 : 0);
    e = max(-127, min(127, e));
  }
  const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint32_t wq = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      wq |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(v[i * 4 + j] * inv, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3))
            << (8 * j);
    q[i] = wq;
  }
  return static_cast<uint8_t>(e + 127);
}

template <bool E5M2>
__global__ void __launch_bounds__(256)
mxfp8_quantize_dual_kernel(const h16* __restrict__ x, long long ldx, uint8_t* __restrict__ out, long long ldo,
                           uint8_t* __restrict__ sf, long long ld_sf, uint8_t* __restrict__ out_t, long long ldt,
                           uint8_t* __restrict__ sf_t, long long ld_sft, int rows, int cols) {
  __shared__ __align__(16) h16 tile[32][256 + 8];
  const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 256;
  const int t = threadIdx.x;
  {
    const int r = t >> 3, g = t & 7;
    const int row = r0 + r, col = c0 + g * 32;
    if (row < rows && col < cols) {
      const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(row) * ldx + col);
      float v[32];
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 u = src[i];
        *reinterpret_cast<uint4*>(&tile[r][g * 32 + i * 8]) = u;
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_h16x2(w[j]);
          v[i * 8 + 2 * j] = f.x;
          v[i * 8 + 2 * j + 1] = f.y;
          amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
      }
      uint32_t q[8];
      const uint8_t sb = mx_scale_and_quantize<E5M2>(v, amax, q);
      uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(row) * ldo + col);
      dst[0] = make_uint4(q[0], q[1], q[2], q[3]);
      dst[1] = make_uint4(q[4], q[5], q[6], q[7]);
      const int gg = col >> 5;
      sf[(static_cast<long long>(gg >> 2) * ld_sf + row) * 4 + (gg & 3)] = sb;
    }
  }
  __syncthreads();
  const int col = c0 + t;
  if (col < cols && r0 + 32 <= rows) {
    float v[32];
    float amax = 0.f;
#pragma unroll
    for (int r = 0; r < 32; ++r) {
      v[r] = h16_to_float(tile[r][t]);
      amax = fmaxf(amax, fabsf(v[r]));
    }
    uint32_t q[8];
    const uint8_t sb = mx_scale_and_quantize<E5M2>(v, amax, q);
    uint4* dst = reinterpret_cast<uint4*>(out_t + static_cast<long long>(col) * ldt + r0);
    dst[0] = make_uint4(q[0], q[1], q[2], q[3]);
    dst[1] = make_uint4(q[4], q[5], q[6], q[7]);
    const int gg = r0 >> 5;
    sf_t[(static_cast<long long>(gg >> 2) * ld_sft + col) * 4 + (gg & 3)] = sb;
  }
}

// x 16-bit [rows, cols] (rows and cols multiples of 32): out [rows, cols] + sf as nx_mxfp8_quantize, and out_t
// [cols, rows] + sf_t = the same for x transposed (scale blocks along the rows of x).  Both scale arrays pre-filled
// with 0x7f7f7f7f by the caller.
NX_API int NX_SYM(nx_mxfp8_quantize_dual)(const void* x, long long ldx, void* out, long long ldo, void* sf,
                                          long long ld_sf, void* out_t, long long ldt, void* sf_t, long long ld_sft,
                                          int rows, int cols, int e5m2, cudaStream_t stream) {
  NX_REQUIRE(rows % 32 == 0 && cols % 32 == 0 && ldx % 8 == 0 && ldo % 16 == 0 && ldt % 16 == 0,
             "mxfp8_quantize_dual: rows and columns must be multiples of 32");
  NX_REQUIRE(ld_sf >= rows && ld_sft >= cols, "mxfp8_quantize_dual: scale rows");
  NX_REQUIRE((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(out_t)) % 16 == 0,
             "mxfp8_quantize_dual: alignment");
  if (rows <= 0 || cols <= 0) return NX_OK;
  dim3 grid((cols + 255) / 256, rows / 32);
  if (e5m2)
    mxfp8_quantize_dual_kernel<true><<<grid, 256, 0, stream>>>((const h16*)x, ldx, (uint8_t*)out, ldo, (uint8_t*)sf, ld_sf,
                                                               (uint8_t*)out_t, ldt, (uint8_t*)sf_t, ld_sft, rows, cols);
  else
    mxfp8_quantize_dual_kernel<false><<<grid, 256, 0, stream>>>((const h16*)x, ldx, (uint8_t*)out, ldo, (uint8_t*)sf, ld_sf,
                                                                (uint8_t*)out_t, ldt, (uint8_t*)sf_t, ld_sft, rows, cols);
  NX_LAUNCH_CHECK();
  return NX_OK;
}

// x 16-bit [rows, cols] (cols % 32 == 0); out fp8 [rows, cols]; sf: scale words [ceil(cols / 128)][ld_sf], which the
// caller has filled with 0x7f7f7f7f (the kernel writes only the bytes of real rows and groups).
NX_API int NX_SYM(nx_mxfp8_quantize)(const void* x, long long ldx, void* out, long long ldo, void* sf, long long ld_sf,
                                     int rows, int cols, int e5m2, cudaStream_t stream) {
  NX_REQUIRE(cols % 32 == 0 && ldx % 8 == 0 && ldo % 16 == 0, "mxfp8_quantize: columns must be a multiple of 32");
  NX_REQUIRE(ld_sf >= rows, "mxfp8_quantize: scale rows");
  NX_REQUIRE((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) % 16 == 0, "mxfp8_quantize: alignment");
  if (rows <= 0 || cols <= 0) return NX_OK;
  const int groups = cols / 32;
  const long long n = static_cast<long long>(rows) * groups;
  const unsigned grid = static_cast<unsigned>((n + 255) / 256);
  if (e5m2)
    mxfp8_quantize_kernel<true><<<grid, 256, 0, stream>>>((const h16*)x, ldx, (uint8_t*)out, ldo, (uint8_t*)sf, ld_sf,
                                                          rows, groups);
  else
    mxfp8_quantize_kernel<false><<<grid, 256, 0, stream>>>((const h16*)x, ldx, (uint8_t*)out, ldo, (uint8_t*)sf, ld_sf,
                                                           rows, groups);
  NX_LAUNCH_CHECK();
  return NX_OK;
}

}  // namespace nx
