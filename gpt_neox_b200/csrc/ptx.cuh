// Thin inline-PTX wrappers for the Blackwell (sm_100a) execution model:
// mbarrier, TMA (cp.async.bulk.tensor, never with a cluster-broadcast qualifier),
// tcgen05 (TMEM alloc / mma / commit / ld) and NVLink multimem / system-scope
// signalling.  Every wait in here is bounded: it gives up after a clock budget
// and reports through an error word instead of spinning forever.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// The 16-bit floating-point storage type of this build of the kernels (see common.h: the same
// sources are compiled for bf16 and, with -DNX_HALF, for fp16).
#ifdef NX_HALF
using h16 = __half;
#else
using h16 = __nv_bfloat16;
#endif

namespace nx {

// ---------------------------------------------------------------------------
// error reporting (host-mapped word; 0 = ok)
// ---------------------------------------------------------------------------
enum ErrCode : int {
  ERR_NONE = 0,
  ERR_WAIT_TIMEOUT = 1,   // a bounded mbarrier / flag wait ran out
  ERR_BOUNDS = 2,         // a debug bounds check refused an access
  ERR_PEER_TIMEOUT = 3,   // a bounded wait on a peer's signal ran out
};

// Default wait budget in SM clock cycles (about 2 s at 2 GHz, longer at lower clocks).  The host can
// replace it at run time (nx_set_wait_budget_cycles): the error word is the first of four ints, and
// ints 2..3 hold the budget as one 64-bit value (0 = use the default).
#ifndef NX_WAIT_BUDGET_CYCLES
#define NX_WAIT_BUDGET_CYCLES (4000000000LL)
#endif

__device__ __forceinline__ long long wait_budget(const int* err_word) {
  long long b = 0;
  if (err_word != nullptr) b = *reinterpret_cast<const volatile long long*>(err_word + 2);
  return b > 0 ? b : NX_WAIT_BUDGET_CYCLES;
}

__device__ __forceinline__ void report_error(int* err_word, int code, int where) {
  if (err_word != nullptr) {
    atomicCAS(err_word, 0, (code & 0xff) | (where << 8));
  }
}

// ---------------------------------------------------------------------------
// debug aids for the communication kernels
//   * NEOX_DEBUG_BOUNDS build (python -m gpt_neox_b200.build --debug-bounds): every access into a symmetric
//     workspace is range-checked against the workspace size the host registered; a violation records
//     {ERR_BOUNDS, site} and the access is skipped (nothing traps).  In the normal build the check is no code.
//   * jitter: when the host sets a non-zero jitter (nx_set_comm_jitter_ns; int 1 of the error block), every
//     cross-rank signal is preceded by a pseudo-random sleep below that many nanoseconds, which reorders the
//     arrivals of flags and data between runs and shakes out protocol errors that need unlucky timing.
// ---------------------------------------------------------------------------
#ifdef NEOX_DEBUG_BOUNDS
__device__ __forceinline__ bool in_range(long long off, long long nbytes, long long limit, int* err_word, int where) {
  if (limit <= 0 || (off >= 0 && off + nbytes <= limit)) return true;
  report_error(err_word, ERR_BOUNDS, where);
  return false;
}
#define NX_IN_RANGE(off, nbytes, limit, err, where) in_range((off), (nbytes), (limit), (err), (where))
#else
#define NX_IN_RANGE(off, nbytes, limit, err, where) true
#endif

__device__ __forceinline__ void comm_jitter(const int* err_word, uint32_t salt) {
  if (err_word == nullptr) return;
  const int max_ns = *reinterpret_cast<const volatile int*>(err_word + 1);
  if (max_ns <= 0) return;
  uint32_t x = salt * 0x9e3779b9u + blockIdx.x * 0x85ebca6bu + static_cast<uint32_t>(clock64());
  x ^= x >> 15;
  x *= 0x2c1b3c6du;
  x ^= x >> 12;
  __nanosleep(x % static_cast<uint32_t>(max_ns));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
  uint32_t l;
  asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
  return l;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n"
      ".reg .pred P1;\n"
      "elect.sync _|P1, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, P1;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same test, but the thread may be suspended by the hardware for up to `hint_ns` nanoseconds while the phase
// is incomplete (it is woken when the phase completes).  A waiting warp then stops competing for issue slots with
// the warps that share its scheduler: with the plain form a waiting control warp re-polled every few dozen cycles
// and its loop took as many issue slots as a working warp.
__device__ __forceinline__ bool mbar_try_wait_suspend(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
#ifndef NX_MBAR_SUSPEND_NS
#define NX_MBAR_SUSPEND_NS 4000u
#endif
// Bounded wait. Returns false (and records ERR_WAIT_TIMEOUT) if the budget ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err_word, int where) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait_suspend(bar, parity, NX_MBAR_SUSPEND_NS)) {
    if ((++spins & 0x3f) == 0) {
      if (clock64() - t0 > wait_budget(err_word)) {
        report_error(err_word, ERR_WAIT_TIMEOUT, where);
        return false;
      }
      if (err_word != nullptr && *reinterpret_cast<volatile int*>(err_word) != 0) return false;
    }
  }
  return true;
}

// ---------------------------------------------------------------------------
// TMA (tiled bulk tensor copies, this GPU's memory -> this CTA's shared memory)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x,
                                            int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4, %5}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x,
                                            int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4, %5, %6}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
// Untiled bulk copy global -> this CTA's shared memory (both addresses 16-byte aligned, size a
// multiple of 16 bytes), completing on an mbarrier.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes,
                                             uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          dst),
      "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05: tensor memory + 5th-generation tensor core MMA
// ---------------------------------------------------------------------------
// Whole-warp calls.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result_addr, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_result_addr),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// One thread: D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void umma_bf16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One thread: D[tmem] (+)= A[tmem] * B[smem desc]   (A operand read from tensor memory)
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One thread: make `bar` complete once every tcgen05 op issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// Warp-collective: thread i reads 32 consecutive fp32 columns of TMEM lane (lane_base + i).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// Warp-collective: thread i writes 16 consecutive 32-bit columns of TMEM lane (lane_base + i).
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31])
      : "memory");
}

// Shared-memory matrix descriptor for tcgen05.mma operands laid out by TMA with the
// 128-byte swizzle.  Field layout (64 bit): start address >> 4 in [0,14), leading byte
// offset >> 4 in [16,30), stride byte offset >> 4 in [32,46), version (=1 on sm_100)
// in [46,48), swizzle mode in [61,64) (2 = 128 B).
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor for kind::f16 with 16-bit inputs (bf16, or fp16 in the NX_HALF build) and
// fp32 accumulation.  c_format (F32=1) at bit 4, a/b format (F16=0, BF16=1) at bits 7/10, a/b major
// (1 = MN-major) at bits 15/16, N>>3 at bit 17, M>>4 at bit 24.
#ifdef NX_HALF
constexpr uint32_t UMMA_AB_FORMAT = 0u;
#else
constexpr uint32_t UMMA_AB_FORMAT = 1u;
#endif
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N, int a_mn_major,
                                                       int b_mn_major) {
  return (1u << 4) | (UMMA_AB_FORMAT << 7) | (UMMA_AB_FORMAT << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}

// ---------------------------------------------------------------------------
// system-scope signalling and NVLink switch (multimem) operations
// ---------------------------------------------------------------------------
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_add_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait until *p >= target (monotone epoch counters; never reset).
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* p, uint32_t target, int* err_word,
                                             int where) {
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (static_cast<int32_t>(ld_acquire_sys(p) - target) < 0) {
    if ((++spins & 0xff) == 0) {
      if (clock64() - t0 > wait_budget(err_word)) {
        report_error(err_word, ERR_PEER_TIMEOUT, where);
        return false;
      }
    }
    __nanosleep(64);
  }
  return true;
}
// 16-byte switch-side reduction load of 8 bf16 values with fp32 accumulation.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_ptr) {
  uint4 v;
#ifdef NX_HALF
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
#else
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
#endif
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_ptr)
               : "memory");
  return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const void* mc_ptr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_ptr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_b128(void* mc_ptr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_ptr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}

// ---------------------------------------------------------------------------
// small math helpers shared by the element-wise epilogues
// ---------------------------------------------------------------------------
__device__ __forceinline__ float gelu_erf(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
}
__device__ __forceinline__ float gelu_erf_grad(float x) {
  const float cdf = 0.5f * (1.0f + erff(x * 0.70710678118654752440f));
  const float pdf = 0.39894228040143267794f * __expf(-0.5f * x * x);
  return cdf + x * pdf;
}
__device__ __forceinline__ float gelu_tanh(float x) {
  return 0.5f * x * (1.0f + tanhf(0.79788456f * x * (1.0f + 0.044715f * x * x)));
}
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float t = tanhf(0.79788456f * x * (1.0f + 0.044715f * x * x));
  return 0.5f * x * ((1.0f - t * t) * (0.79788456f + 0.1070322243f * x * x)) + 0.5f * (1.0f + t);
}
// GeLU and its derivative together, for the GEMM epilogue that stores the derivative for the backward pass.
// erf form: the normal CDF by Abramowitz-Stegun 7.1.26 (absolute error < 1e-7), which shares its exponential
// exp(-x^2/2) with the density term of the derivative: one ex2 + one reciprocal + a few FMAs for both values,
// with no cancellation in the negative tail (Phi(x) = q for x < 0, 1 - q otherwise).
__device__ __forceinline__ void gelu_erf_both(float x, float& g, float& dg) {
  const float ay = fabsf(x) * 0.70710678118654752440f;
  const float t = __fdividef(1.0f, fmaf(0.3275911f, ay, 1.0f));
  const float e = exp2f(x * x * -0.72134752044448170368f);  // exp(-x^2 / 2)
  float poly = fmaf(t, 1.061405429f, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  const float q = 0.5f * poly * t * e;
  const float cdf = x < 0.0f ? q : 1.0f - q;
  g = x * cdf;
  dg = fmaf(x * 0.39894228040143267794f, e, cdf);
}
__device__ __forceinline__ void gelu_tanh_both(float x, float& g, float& dg) {
  const float t = tanhf(0.79788456f * x * (1.0f + 0.044715f * x * x));
  const float h = 0.5f * (1.0f + t);
  g = x * h;
  dg = fmaf(0.5f * x * (1.0f - t * t), fmaf(0.1070322243f, x * x, 0.79788456f), h);
}
// ---------------------------------------------------------------------------
// attention dropout: the keep / drop decision of probability (q, k) of one (batch, head) is a pure
// function of (seed, batch * heads + head, q, k), so the forward and both backward kernels regenerate
// the same mask whatever their thread-to-element mapping.  One 32-bit hash serves the 2 x 2 patch
// (q & ~1, k & ~1): byte (q & 1) * 2 + (k & 1) is compared with the threshold.  p is quantised to 1/256.
// ---------------------------------------------------------------------------
// ---- packed fp32 pairs (sm_100 FFMA2 / FADD2 / FMUL2: one issue slot for two lanes of work) and the three-input
//      maximum; the element-wise halves of the attention kernels are issue-bound, so these halve their FMA-pipe
//      instruction count.
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 u2f2(uint32_t a, uint32_t b) { return make_float2(__uint_as_float(a), __uint_as_float(b)); }

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352du;
  x ^= x >> 15;
  x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}
// q2 = q >> 1, k2 = k >> 1 (each below 65536).
__device__ __forceinline__ uint32_t dropout_patch(uint32_t seed_lo, uint32_t seed_hi, uint32_t bh, uint32_t q2,
                                                  uint32_t k2) {
  uint32_t x = mix32(((q2 << 16) | k2) ^ seed_lo);
  return mix32(x + bh * 0x9e3779b9u + seed_hi);
}
__device__ __forceinline__ bool dropout_keep(uint32_t patch, int q, int k, uint32_t threshold) {
  return ((patch >> ((((q & 1) << 1) | (k & 1)) * 8)) & 0xffu) >= threshold;
}

__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }
__device__ __forceinline__ float silu_grad(float x) {
  const float s = 1.0f / (1.0f + __expf(-x));
  return s * (1.0f + x * (1.0f - s));
}

#ifdef NX_HALF
__device__ __forceinline__ uint32_t pack_h16x2(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_h16x2(uint32_t u) {
  __half2 v = *reinterpret_cast<__half2*>(&u);
  return __half22float2(v);
}
__device__ __forceinline__ float h16_to_float(h16 x) { return __half2float(x); }
__device__ __forceinline__ h16 float_to_h16(float x) { return __float2half_rn(x); }
#else
__device__ __forceinline__ uint32_t pack_h16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_h16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}
__device__ __forceinline__ float h16_to_float(h16 x) { return __bfloat162float(x); }
__device__ __forceinline__ h16 float_to_h16(float x) { return __float2bfloat16(x); }
#endif

}  // namespace nx
