// Library-wide host state: last error text, per-device error word, TMA descriptor encoder.
#include "common.h"
#include "ptx.cuh"

#include <cudaTypedefs.h>
#include <stdarg.h>
#include <string.h>

#include <mutex>

namespace nx {

static thread_local char g_last_error[1024] = "";

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

// [0] error word, [1] communication jitter in ns (0 = off), [2..3] run-time wait budget in cycles as one 64-bit value (0 = default)
__device__ __align__(16) int g_error_word[4] = {0, 0, 0, 0};

static int* g_err_ptr[64] = {nullptr};
static int g_sm_count[64] = {0};
static std::mutex g_mu;

int* device_error_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (g_err_ptr[dev] == nullptr) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_err_ptr[dev] == nullptr) {
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_error_word) != cudaSuccess) return nullptr;
      g_err_ptr[dev] = static_cast<int*>(p);
    }
  }
  return g_err_ptr[dev];
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

static CUtensorMapDataType dtype_of(int elem_bytes) {
  switch (elem_bytes) {
    case 1: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
    case 2: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    default: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  }
}

// The tensor-map encoder is a driver entry point and needs a current context in the calling thread.  A
// thread whose first CUDA activity is one of our launchers (an autograd worker thread that starts with a
// fused GEMM, for instance) may not have bound the primary context yet: any runtime call binds it.
static void ensure_thread_context() {
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

bool make_tma_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                 uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols, int elem_bytes,
                 bool swizzle128) {
  ensure_thread_context();
  auto fn = get_encode_fn();
  if (fn == nullptr) {
    set_last_error("cuTensorMapEncodeTiled entry point not available");
    return false;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_stride_bytes & 15) != 0) {
    set_last_error("TMA operand needs a 16-byte aligned base and row stride (base=%p stride=%llu)",
                   base, (unsigned long long)row_stride_bytes);
    return false;
  }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estride[2] = {1, 1};
  CUresult r = fn(map, dtype_of(elem_bytes), 2, const_cast<void*>(base), gdim, gstride, box, estride,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled failed (%d): rows=%llu cols=%llu stride=%llu box=%ux%u",
                   (int)r, (unsigned long long)rows, (unsigned long long)cols,
                   (unsigned long long)row_stride_bytes, box_rows, box_cols);
    return false;
  }
  return true;
}

bool make_tma_3d(CUtensorMap* map, const void* base, uint64_t d2, uint64_t d1, uint64_t d0,
                 uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box2, uint32_t box1,
                 uint32_t box0, int elem_bytes, bool swizzle128) {
  ensure_thread_context();
  auto fn = get_encode_fn();
  if (fn == nullptr) {
    set_last_error("cuTensorMapEncodeTiled entry point not available");
    return false;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (stride1_bytes & 15) != 0 ||
      (stride2_bytes & 15) != 0) {
    set_last_error("TMA operand needs 16-byte aligned base and strides");
    return false;
  }
  cuuint64_t gdim[3] = {d0, d1, d2};
  cuuint64_t gstride[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estride[3] = {1, 1, 1};
  CUresult r = fn(map, dtype_of(elem_bytes), 3, const_cast<void*>(base), gdim, gstride, box, estride,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled(3d) failed (%d)", (int)r);
    return false;
  }
  return true;
}

bool make_tma_4d(CUtensorMap* map, const void* base, const uint64_t dims[4],
                 const uint64_t strides_bytes[3], const uint32_t box[4], int elem_bytes,
                 bool swizzle128) {
  ensure_thread_context();
  auto fn = get_encode_fn();
  if (fn == nullptr) {
    set_last_error("cuTensorMapEncodeTiled entry point not available");
    return false;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (strides_bytes[0] & 15) != 0 ||
      (strides_bytes[1] & 15) != 0 || (strides_bytes[2] & 15) != 0) {
    set_last_error("TMA operand needs 16-byte aligned base and strides (base=%p strides=%llu,%llu,%llu)",
                   base, (unsigned long long)strides_bytes[0], (unsigned long long)strides_bytes[1],
                   (unsigned long long)strides_bytes[2]);
    return false;
  }
  cuuint64_t gdim[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t gstride[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
  cuuint32_t b[4] = {box[0], box[1], box[2], box[3]};
  cuuint32_t estride[4] = {1, 1, 1, 1};
  CUresult r = fn(map, dtype_of(elem_bytes), 4, const_cast<void*>(base), gdim, gstride, b, estride,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled(4d) failed (%d): dims=%llu,%llu,%llu,%llu", (int)r,
                   (unsigned long long)dims[0], (unsigned long long)dims[1],
                   (unsigned long long)dims[2], (unsigned long long)dims[3]);
    return false;
  }
  return true;
}

}  // namespace nx

NX_API const char* nx_last_error() { return nx::g_last_error; }

// Reads and clears the device error word of the current device (synchronises the device).
// Returns the raw word: low byte = nx::ErrCode, upper bits = site id; 0 = ok; -1 = CUDA failure.
NX_API int nx_read_device_error(int clear) {
  int* p = nx::device_error_word();
  if (p == nullptr) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (clear && v != 0) {
    int z = 0;
    cudaMemcpy(p, &z, sizeof(int), cudaMemcpyHostToDevice);
  }
  return v;
}

// Test hook: pre-set the device error word from the host (never stalls a GPU).
NX_API int nx_poison_device_error(int value) {
  int* p = nx::device_error_word();
  if (p == nullptr) return NX_ERR_CUDA;
  NX_CUDA_CHECK(cudaMemcpy(p, &value, sizeof(int), cudaMemcpyHostToDevice));
  return NX_OK;
}

// Replaces the cycle budget of every bounded wait on the current device (mbarrier and flag waits of
// all kernels launched afterwards); 0 restores the compile-time default.  Synchronises the device.
NX_API int nx_set_wait_budget_cycles(long long cycles) {
  int* p = nx::device_error_word();
  if (p == nullptr) return NX_ERR_CUDA;
  NX_REQUIRE(cycles >= 0, "wait budget must be >= 0");
  NX_CUDA_CHECK(cudaDeviceSynchronize());
  NX_CUDA_CHECK(cudaMemcpy(p + 2, &cycles, sizeof(long long), cudaMemcpyHostToDevice));
  return NX_OK;
}

// Upper bound (nanoseconds) of the pseudo-random sleep in front of every cross-rank signal of the communication
// kernels (debug aid against timing-dependent protocol errors); 0 = off.  Synchronises the device.
NX_API int nx_set_comm_jitter_ns(int max_ns) {
  int* p = nx::device_error_word();
  if (p == nullptr) return NX_ERR_CUDA;
  NX_REQUIRE(max_ns >= 0 && max_ns <= 1000000, "jitter must be within [0, 1 ms]");
  NX_CUDA_CHECK(cudaDeviceSynchronize());
  NX_CUDA_CHECK(cudaMemcpy(p + 1, &max_ns, sizeof(int), cudaMemcpyHostToDevice));
  return NX_OK;
}

namespace nx {
// Waits on an mbarrier that nothing ever arrives on: the bounded wait must give up, record
// {ERR_WAIT_TIMEOUT, site 21} and let the kernel return.  out[0] = 1 if the wait reported success.
__global__ void mbar_timeout_probe_kernel(int* err, int* out) {
  __shared__ __align__(8) unsigned long long bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    fence_barrier_init();
    out[0] = mbar_wait(smem_u32(&bar), 0, err, 21) ? 1 : 0;
  }
}
}  // namespace nx

// Self-test of the bounded mbarrier wait (see the kernel above).  Set a small budget first.
NX_API int nx_mbar_timeout_probe(void* out_i32, void* stream_) {
  nx::mbar_timeout_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(nx::device_error_word(),
                                                                                 static_cast<int*>(out_i32));
  NX_LAUNCH_CHECK();
  return NX_OK;
}

NX_API int nx_sm_count() { return nx::sm_count(); }
NX_API int nx_abi_version() { return 1; }
