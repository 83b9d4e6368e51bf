// Host-side helpers shared by every translation unit of libneox_b200: status codes,
// the device error word, SM count cache and TMA descriptor encoding through the
// driver entry point (no link-time dependency on libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define NX_API extern "C" __attribute__((visibility("default")))

enum NxStatus : int {
  NX_OK = 0,
  NX_ERR_CUDA = 1,       // a CUDA runtime call failed (see nx_last_error)
  NX_ERR_ARG = 2,        // shape / alignment / size precondition violated
  NX_ERR_UNSUPPORTED = 3,
  NX_ERR_DEVICE = 4,     // the device error word is set (bounded wait ran out, ...)
};

namespace nx {

void set_last_error(const char* fmt, ...);
int* device_error_word();  // per-device int in global memory, 0 = ok
int sm_count();

// Encodes a 2-D row-major bf16/fp32/u8 tensor [rows, cols] (cols contiguous, row stride in
// bytes) with box [box_rows, box_cols] and the 128-byte swizzle.
// elem_bytes in {1, 2, 4}. Returns false on failure.
bool make_tma_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                 uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols, int elem_bytes,
                 bool swizzle128 = true);
// 3-D variant: [d2, d1, d0] with d0 contiguous; strides for d1 and d2 in bytes.
bool make_tma_3d(CUtensorMap* map, const void* base, uint64_t d2, uint64_t d1, uint64_t d0,
                 uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box2, uint32_t box1,
                 uint32_t box0, int elem_bytes, bool swizzle128 = true);

// 4-D variant: dims / box given innermost first; strides (bytes) for dims 1..3.
bool make_tma_4d(CUtensorMap* map, const void* base, const uint64_t dims[4],
                 const uint64_t strides_bytes[3], const uint32_t box[4], int elem_bytes,
                 bool swizzle128 = true);

}  // namespace nx

// The kernels that work on 16-bit floating-point tensors are compiled twice from the same sources:
// once for bf16 (namespace nx, exported symbols nx_*) and once with -DNX_HALF for fp16 (namespace
// nxh, exported symbols nx_*_f16).  In the second build every `nx` below this point names `nxh`; the
// host helpers declared above stay shared through the using-directive.
#ifdef NX_HALF
namespace nxh {
using namespace nx;
}
#define nx nxh
#define NX_SYM(name) name##_f16
#else
#define NX_SYM(name) name
#endif

#define NX_CUDA_CHECK(expr)                                                              \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess) {                                                             \
      nx::set_last_error("%s:%d: %s -> %s", __FILE__, __LINE__, #expr, cudaGetErrorString(_e)); \
      return NX_ERR_CUDA;                                                                \
    }                                                                                    \
  } while (0)

#define NX_REQUIRE(cond, ...)            \
  do {                                   \
    if (!(cond)) {                       \
      nx::set_last_error(__VA_ARGS__);   \
      return NX_ERR_ARG;                 \
    }                                    \
  } while (0)

#define NX_LAUNCH_CHECK() NX_CUDA_CHECK(cudaGetLastError())
