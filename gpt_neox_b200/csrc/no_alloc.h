// Allocation-free entry point of libneox_b200 (no counterpart in the reference: GPT-NeoX only ever
// runs under PyTorch's caching allocator).
//
// nx_colsum_bf16_noalloc computes what nx_colsum_bf16 computes - out[c] = sum over rows of x[r, c],
// bf16 in, fp32 out, the bias-gradient reduction of every linear layer - but takes no workspace
// pointer and never calls cudaMalloc, cudaFree or any allocating routine (PyTorch's included).  It
// is for hosts that cannot allocate when they call in: a C or C++ runtime that embeds this library
// without PyTorch and has already given all of its device memory to its own arena, or a step
// function that runs under a fixed memory plan where a late cudaMalloc would either fail or
// stall the device.  The caller still owns the input and the output.
//
// The partial sums live in one file-scope __device__ array inside the library
// (NX_COLSUM_NOALLOC_MAX_FLOATS floats = 4 MiB, held by every GPU that loads the library until the
// process exits).  Consequences the caller must know:
//   * Sizes: nx_colsum_slabs(rows) * N must not exceed NX_COLSUM_NOALLOC_MAX_FLOATS
//     (N <= 16384 for any row count); larger requests are rejected with NX_ERR_ARG and a message in
//     nx_last_error().
//   * Set-up: the first call on each device resolves the array's device address
//     (cudaGetSymbolAddress) with that device current; with CUDA's lazy module loading it may also
//     be the call that loads this library's device code, which is when the driver sets the 4 MiB
//     aside.  Make that first call at start-up, before any stream capture begins on that device.
//     First calls from several host threads are serialised by a lock.  The cached address does
//     not survive cudaDeviceReset: do not call in again after resetting a device.
//   * Sharing: every call on a device uses the same array, which keeps the previous call's
//     contents.  Each call overwrites every element it later reads, so nothing has to be cleared,
//     but two calls that overlap on the GPU (different streams without ordering) race on it.
#pragma once

#define NX_COLSUM_NOALLOC_MAX_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

// x: bf16 [rows, N] with leading dimension ld (elements); out_f32: fp32 [N]; accumulate != 0 adds
// into out_f32 instead of overwriting it.  N and ld multiples of 8.  Returns an NxStatus.
int nx_colsum_bf16_noalloc(const void* x, void* out_f32, long long rows, int N, long long ld,
                           int accumulate, void* stream);

#ifdef __cplusplus
}
#endif
