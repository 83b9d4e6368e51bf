// FP8 GEMM on the 5th-generation tensor cores: C[M,N] = alpha * A[M,K] * B[N,K]^T (+ bias), A and B in
// e4m3 or e5m2 (one byte per element, both K-major), fp32 accumulation in tensor memory, bf16 or
// (accumulating) fp32 output.  alpha is read from device memory: it is the product of the two tensors'
// de-quantisation scales, which the delayed-scaling recipe keeps on the device.
//
// Plus the quantisation kernels around it: bf16 -> fp8 with a per-tensor scale, the running absolute
// maximum (for the next step's scale) and, optionally, the transposed copy that the backward GEMMs need
// (both operands of tcgen05.mma kind::f8f6f4 are consumed K-major here).
//
// Counterpart in the reference: Transformer Engine's fp8 Linear under `fp8_autocast` with the
// DelayedScaling recipe (megatron/model/transformer_engine.py:102-156,633-670).
//
// Same pipeline as csrc/gemm_tcgen05.cu: one persistent CTA per SM; warp 0 issues TMA loads into a
// 4-stage shared-memory ring (128-byte swizzle: a row of a tile is 128 fp8 values), warp 1 issues
// tcgen05.mma (K = 32 per instruction), warps 2-5 drain the two TMEM accumulators.
#include <cuda_fp8.h>

#include "common.h"
#include "ptx.cuh"

namespace nx {

namespace f8 {
constexpr int BM = 128, BN = 256, BK = 128, UK = 32, STAGES = 4, THREADS = 192;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
constexpr int DYN_BYTES = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 1024;
}  // namespace f8

struct Fp8GemmParams {
  int M, N, K;
  void* C;
  long long ldc;
  const float* alpha;               // device scalar
  const h16* bias;
  int out_f32, accumulate;
  int tiles_m, tiles_n;
  uint32_t idesc;
  int* err;
};

__device__ __forceinline__ void umma_f8_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// c_format F32 (1) at bit 4; a / b format at bits 7 / 10 (0 = e4m3, 1 = e5m2); both K-major;
// N >> 3 at bit 17, M >> 4 at bit 24.
static uint32_t idesc_f8(int a_e5m2, int b_e5m2) {
  return (1u << 4) | (static_cast<uint32_t>(a_e5m2) << 7) | (static_cast<uint32_t>(b_e5m2) << 10) |
         (static_cast<uint32_t>(f8::BN >> 3) << 17) | (static_cast<uint32_t>(f8::BM >> 4) << 24);
}

__global__ void __launch_bounds__(f8::THREADS, 1)
    gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const Fp8GemmParams p) {
  using namespace f8;
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
  constexpr uint32_t TMEM_COLS = 512;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
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
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !aborted; tile += gridDim.x) {
        const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, p.err, 1)) {
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
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !aborted; tile += gridDim.x) {
        if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1, p.err, 2)) {
          aborted = true;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, p.err, 3)) {
            aborted = true;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_base + stage * STAGE_BYTES;
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            // K-major, 128-byte swizzle: 8-row groups 1024 B apart; 32 fp8 K-elements advance 32 B
            const uint64_t adesc = umma_smem_desc_sw128(a_addr + k * UK, 0, 1024);
            const uint64_t bdesc = umma_smem_desc_sw128(b_addr + k * UK, 0, 1024);
            umma_f8_ss(d_tmem, adesc, bdesc, p.idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (aborted) break;
        umma_commit(tmem_full_bar(acc));
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    const float alpha = *p.alpha;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
      const int m0 = tm * BM, n0 = tn * BN;
      if (!mbar_wait(tmem_full_bar(acc), acc_phase, p.err, 4)) {
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
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
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
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// A [M, K] and B [N, K]: fp8 bytes, leading dimensions in elements (multiples of 16); a_e5m2 / b_e5m2
// select the operand formats.  C: bf16 [M, N] or fp32 (out_f32; accumulate adds into it).
NX_API int NX_SYM(nx_gemm_fp8)(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                       long long ldc, int a_e5m2, int b_e5m2, const void* alpha, const void* bias, int out_f32,
                       int accumulate, cudaStream_t stream) {
  using namespace f8;
  NX_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_fp8: empty problem");
  NX_REQUIRE(lda % 16 == 0 && ldb % 16 == 0 && K % 16 == 0, "gemm_fp8: K and leading dimensions must be multiples of 16");
  NX_REQUIRE(N % 8 == 0 && ldc % (out_f32 ? 4 : 8) == 0, "gemm_fp8: N / ldc alignment");
  NX_REQUIRE((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) % 16 == 0,
             "gemm_fp8: operands must be 16-byte aligned");
  NX_REQUIRE(alpha != nullptr, "gemm_fp8: alpha (device scalar) is required");
  CUtensorMap tmA, tmB;
  if (!make_tma_2d(&tmA, A, M, K, lda, BM, BK, 1)) return NX_ERR_ARG;
  if (!make_tma_2d(&tmB, B, N, K, ldb, BN, BK, 1)) return NX_ERR_ARG;
  Fp8GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc;
  p.alpha = static_cast<const float*>(alpha);
  p.bias = static_cast<const h16*>(bias);
  p.out_f32 = out_f32; p.accumulate = accumulate;
  p.tiles_m = (M + BM - 1) / BM; p.tiles_n = (N + BN - 1) / BN;
  p.idesc = idesc_f8(a_e5m2, b_e5m2);
  p.err = device_error_word();
  static bool configured = false;
  if (!configured) {
    NX_CUDA_CHECK(cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DYN_BYTES));
    configured = true;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  gemm_fp8_kernel<<<grid, THREADS, DYN_BYTES, stream>>>(tmA, tmB, p);
  NX_LAUNCH_CHECK();
  return NX_OK;
}

// ---------------------------------------------------------------------------------------------
// quantisation: out = sat_fp8(x * scale); amax = max(amax, max|x|); optional transposed copy
// ---------------------------------------------------------------------------------------------
template <bool E5M2>
__device__ __forceinline__ uint8_t to_fp8(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3));
}

// 64 x 64 tiles; block 256 threads (each thread 16 elements: 2 rows x 8 columns per pass).
template <bool E5M2>
__global__ void __launch_bounds__(256)
fp8_quantize_kernel(const h16* __restrict__ x, long long ldx, const float* __restrict__ scale,
                    uint8_t* __restrict__ out, long long ldo, uint8_t* __restrict__ out_t, long long ldt,
                    float* __restrict__ amax, int rows, int cols) {
  __shared__ uint8_t tile[64][64 + 16];
  __shared__ float wmax[8];
  const float sc = *scale;
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int tr = threadIdx.x >> 3, tc = (threadIdx.x & 7) * 8;     // 32 row slots x 8 column groups
  float m = 0.f;
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    const int r = r0 + tr + pass * 32, c = c0 + tc;
    uint2 packed = make_uint2(0u, 0u);
    if (r < rows && c < cols) {
      const uint4 u = *reinterpret_cast<const uint4*>(x + static_cast<long long>(r) * ldx + c);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
      uint8_t q[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_h16x2(w[j]);
        m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
        q[2 * j] = to_fp8<E5M2>(f.x * sc);
        q[2 * j + 1] = to_fp8<E5M2>(f.y * sc);
      }
      packed.x = q[0] | (q[1] << 8) | (q[2] << 16) | (static_cast<uint32_t>(q[3]) << 24);
      packed.y = q[4] | (q[5] << 8) | (q[6] << 16) | (static_cast<uint32_t>(q[7]) << 24);
      *reinterpret_cast<uint2*>(out + static_cast<long long>(r) * ldo + c) = packed;
    }
    if (out_t != nullptr) *reinterpret_cast<uint2*>(&tile[tr + pass * 32][tc]) = packed;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float mm = wmax[0];
    for (int i = 1; i < 8; ++i) mm = fmaxf(mm, wmax[i]);
    atomicMax(reinterpret_cast<int*>(amax), __float_as_int(mm));   // non-negative floats order like ints
  }
  if (out_t != nullptr) {
    // transposed write: thread handles column (c0 + tr [+32]) and 8 consecutive rows
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      const int cc = tr + pass * 32, rr = tc;
      const int gc = c0 + cc, gr = r0 + rr;
      if (gc < cols && gr < rows) {
        uint8_t q[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = tile[rr + j][cc];
        uint2 packed;
        packed.x = q[0] | (q[1] << 8) | (q[2] << 16) | (static_cast<uint32_t>(q[3]) << 24);
        packed.y = q[4] | (q[5] << 8) | (q[6] << 16) | (static_cast<uint32_t>(q[7]) << 24);
        *reinterpret_cast<uint2*>(out_t + static_cast<long long>(gc) * ldt + gr) = packed;
      }
    }
  }
}

// x bf16 [rows, cols] (cols % 8 == 0, rows % 8 == 0 when the transpose is requested); scale / amax device
// floats; out [rows, cols] fp8; out_t [cols, rows] fp8 or null.
NX_API int NX_SYM(nx_fp8_quantize)(const void* x, long long ldx, const void* scale, void* out, long long ldo, void* out_t,
                           long long ldt, void* amax, int rows, int cols, int e5m2, cudaStream_t stream) {
  NX_REQUIRE(cols % 8 == 0 && ldx % 8 == 0 && ldo % 8 == 0, "fp8_quantize: columns / leading dimensions must be multiples of 8");
  NX_REQUIRE(out_t == nullptr || (rows % 8 == 0 && ldt % 8 == 0), "fp8_quantize: transpose needs rows % 8 == 0");
  dim3 grid((cols + 63) / 64, (rows + 63) / 64);
  if (e5m2)
    fp8_quantize_kernel<true><<<grid, 256, 0, stream>>>((const h16*)x, ldx, (const float*)scale, (uint8_t*)out,
                                                        ldo, (uint8_t*)out_t, ldt, (float*)amax, rows, cols);
  else
    fp8_quantize_kernel<false><<<grid, 256, 0, stream>>>((const h16*)x, ldx, (const float*)scale, (uint8_t*)out,
                                                         ldo, (uint8_t*)out_t, ldt, (float*)amax, rows, cols);
  NX_LAUNCH_CHECK();
  return NX_OK;
}

}  // namespace nx
