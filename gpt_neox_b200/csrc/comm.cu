// Collectives over NVLink peer memory: all-reduce, all-gather and reduce-scatter kernels that read and
// write other GPUs' symmetric buffers directly (plain P2P ld/st, or NVLS multimem when a multicast
// address is given).  They replace the NCCL calls the reference issues from Python at
// megatron/mpu/mappings.py:44,210,248 in this framework's "fused" communication mode.
//
// Symmetric workspace layout (same on every rank; allocated and exchanged by comm/symm.py):
//   [0, FLAG_BYTES)        uint32 flags: flags[block][src_rank], monotone epoch counters, never reset
//   [FLAG_BYTES, ...)      payload
// Cross-rank barrier = every block b of every rank writes its epoch into flags[b][me] of every peer,
// then waits until its own flags[b][*] have reached that epoch.  All waits are bounded: on expiry
// the kernel records an error word and returns (outputs are then invalid; the host raises).
#include "common.h"
#include "ptx.cuh"

namespace nx {

constexpr int COMM_MAX_RANKS = 8;
constexpr int COMM_BLOCKS = 64;
constexpr int COMM_THREADS = 512;
constexpr int COMM_FLAG_BYTES = 64 * 1024;

struct PeerTable {
  void* ptr[COMM_MAX_RANKS];  // base of every rank's symmetric workspace, as mapped on this rank
  long long limit;            // size of one workspace in bytes if the host registered it (debug range checks), else 0
};

// Block-level barrier across ranks.  phase distinguishes the barriers of one launch.
__device__ __forceinline__ bool rank_barrier(const PeerTable& t, int me, int ws, uint32_t epoch,
                                             int* err, int where) {
  __syncthreads();
  bool ok = true;
  if (threadIdx.x < ws) {
    const int peer = threadIdx.x;
    uint32_t* remote = reinterpret_cast<uint32_t*>(t.ptr[peer]) + blockIdx.x * COMM_MAX_RANKS + me;
    __threadfence_system();
    comm_jitter(err, epoch + peer);
    st_release_sys(remote, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(t.ptr[me]) + blockIdx.x * COMM_MAX_RANKS + peer;
    ok = wait_flag_ge(mine, epoch, err, where);
  }
  ok = __syncthreads_and(ok ? 1 : 0) != 0;
  return ok;
}

__device__ __forceinline__ float4 add4(float4 a, float4 b) {
  return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}
__device__ __forceinline__ void acc_bf16x8(float (&acc)[8], uint4 u) {
  const float2 a = unpack_h16x2(u.x), b = unpack_h16x2(u.y), c = unpack_h16x2(u.z), d = unpack_h16x2(u.w);
  acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
  acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
}
__device__ __forceinline__ uint4 pack_acc(const float (&acc)[8]) {
  uint4 o;
  o.x = pack_h16x2(acc[0], acc[1]); o.y = pack_h16x2(acc[2], acc[3]);
  o.z = pack_h16x2(acc[4], acc[5]); o.w = pack_h16x2(acc[6], acc[7]);
  return o;
}

// Sum of the 16-byte vector at payload offset `off` over all ranks (fp32 accumulation).
template <bool BF16>
__device__ __forceinline__ uint4 reduce_vec(const PeerTable& t, int ws, const void* mc, long long pay, long long off) {
  if (mc != nullptr) {
    const char* p = reinterpret_cast<const char*>(mc) + pay + off;
    if (BF16) return multimem_ld_reduce_bf16x8(p);
    const float4 f = multimem_ld_reduce_f32x4(p);
    return make_uint4(__float_as_uint(f.x), __float_as_uint(f.y), __float_as_uint(f.z), __float_as_uint(f.w));
  }
  if (BF16) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < ws; ++r)
      acc_bf16x8(acc, *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(t.ptr[r]) + pay + off));
    return pack_acc(acc);
  }
  float4 s = make_float4(0, 0, 0, 0);
  for (int r = 0; r < ws; ++r)
    s = add4(s, *reinterpret_cast<const float4*>(reinterpret_cast<const char*>(t.ptr[r]) + pay + off));
  return make_uint4(__float_as_uint(s.x), __float_as_uint(s.y), __float_as_uint(s.z), __float_as_uint(s.w));
}

// Two-shot all-reduce of `bytes` of payload that every rank has placed at payload offset 0 of its
// own workspace: rank r reduces slice r and writes the result into every rank's workspace.
template <bool BF16>
__global__ void __launch_bounds__(COMM_THREADS) allreduce_kernel(PeerTable t, const void* mc, int me, int ws,
                                                                 long long pay, long long bytes, uint32_t epoch, int* err) {
  if (!rank_barrier(t, me, ws, epoch, err, 101)) return;
  const long long nvec = bytes / 16;
  const long long per = (nvec + ws - 1) / ws;
  const long long v0 = me * per, v1 = min(nvec, v0 + per);
  for (long long v = v0 + blockIdx.x * (long long)blockDim.x + threadIdx.x; v < v1;
       v += (long long)gridDim.x * blockDim.x) {
    if (!NX_IN_RANGE(pay + v * 16, 16, t.limit, err, 111)) continue;
    const uint4 s = reduce_vec<BF16>(t, ws, mc, pay, v * 16);
    if (mc != nullptr) {
      multimem_st_b128(reinterpret_cast<char*>(const_cast<void*>(mc)) + pay + v * 16, s);
    } else {
      for (int r = 0; r < ws; ++r)
        *reinterpret_cast<uint4*>(reinterpret_cast<char*>(t.ptr[r]) + pay + v * 16) = s;
    }
  }
  rank_barrier(t, me, ws, epoch + 1, err, 102);
}

// Reduce-scatter along dim 0: every rank has its full [ws * shard] payload at offset 0; rank r writes
// the sum of chunk r to `out` (its own memory).
template <bool BF16>
__global__ void __launch_bounds__(COMM_THREADS) reduce_scatter_kernel(PeerTable t, const void* mc, int me, int ws,
                                                                      long long pay, long long shard_bytes, void* out,
                                                                      uint32_t epoch, int* err) {
  if (!rank_barrier(t, me, ws, epoch, err, 103)) return;
  const long long nvec = shard_bytes / 16;
  const long long base = me * shard_bytes;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec;
       v += (long long)gridDim.x * blockDim.x) {
    if (!NX_IN_RANGE(pay + base + v * 16, 16, t.limit, err, 112)) continue;
    reinterpret_cast<uint4*>(out)[v] = reduce_vec<BF16>(t, ws, mc, pay, base + v * 16);
  }
  rank_barrier(t, me, ws, epoch + 1, err, 104);  // peers may overwrite their payload only after all reads
}

// All-gather along dim 0: rank r pushes its shard (`in`, own memory) to payload offset r * shard of
// every rank's workspace.
__global__ void __launch_bounds__(COMM_THREADS) allgather_kernel(PeerTable t, const void* mc, int me, int ws,
                                                                 long long pay, long long shard_bytes, const void* in,
                                                                 uint32_t epoch, int* err) {
  // the previous user of the workspace must be done on every rank before it is overwritten
  if (!rank_barrier(t, me, ws, epoch, err, 105)) return;
  const long long nvec = shard_bytes / 16;
  const long long base = pay + me * shard_bytes;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec;
       v += (long long)gridDim.x * blockDim.x) {
    if (!NX_IN_RANGE(base + v * 16, 16, t.limit, err, 113)) continue;
    const uint4 x = reinterpret_cast<const uint4*>(in)[v];
    if (mc != nullptr) {
      multimem_st_b128(reinterpret_cast<char*>(const_cast<void*>(mc)) + base + v * 16, x);
    } else {
      for (int r = 0; r < ws; ++r) *reinterpret_cast<uint4*>(reinterpret_cast<char*>(t.ptr[r]) + base + v * 16) = x;
    }
  }
  rank_barrier(t, me, ws, epoch + 1, err, 106);
}

// ---------------------------------------------------------------------------------------------
// ZeRO collectives on buffers that LIVE in the symmetric workspace (no staging copies):
//   zero_reduce_scatter: every rank's gradient buffer is at payload offset `pay`; rank r sums chunk r over
//     all ranks straight out of the peers' memory (coalesced 16-byte peer loads, four in flight per
//     thread) and writes the result over its own chunk r, in place.
//   zero_all_gather: rank r pushes chunk r of its parameter buffer into the same place of every peer.
// Both are bracketed by rank barriers: the first makes sure every rank's buffer is final (backward /
// optimizer step done), the second that nobody overwrites a buffer that a peer is still reading.
// ---------------------------------------------------------------------------------------------
template <bool BF16>
__global__ void __launch_bounds__(COMM_THREADS) zero_reduce_scatter_kernel(PeerTable t, int me, int ws, long long pay,
                                                                           long long shard_bytes, uint32_t epoch,
                                                                           int* err) {
  if (!rank_barrier(t, me, ws, epoch, err, 107)) return;
  long long nvec = shard_bytes / 16;
  const long long base = pay + me * shard_bytes;
  if (!NX_IN_RANGE(base, shard_bytes, t.limit, err, 114)) nvec = 0;       // nothing is touched; the barriers still run
  const long long stride = (long long)gridDim.x * blockDim.x;
  char* mine = reinterpret_cast<char*>(t.ptr[me]) + base;
  constexpr int U = 4;
  long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (; v + (U - 1) * stride < nvec; v += U * stride) {
    float acc[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
    for (int r = 0; r < ws; ++r) {
      const char* src = reinterpret_cast<const char*>(t.ptr[r]) + base;
      uint4 x[U];
#pragma unroll
      for (int u = 0; u < U; ++u) x[u] = *reinterpret_cast<const uint4*>(src + (v + u * stride) * 16);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (BF16) {
          acc_bf16x8(acc[u], x[u]);
        } else {
          acc[u][0] += __uint_as_float(x[u].x); acc[u][1] += __uint_as_float(x[u].y);
          acc[u][2] += __uint_as_float(x[u].z); acc[u][3] += __uint_as_float(x[u].w);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      uint4 o;
      if (BF16) o = pack_acc(acc[u]);
      else o = make_uint4(__float_as_uint(acc[u][0]), __float_as_uint(acc[u][1]), __float_as_uint(acc[u][2]),
                          __float_as_uint(acc[u][3]));
      *reinterpret_cast<uint4*>(mine + (v + u * stride) * 16) = o;
    }
  }
  for (; v < nvec; v += stride)
    *reinterpret_cast<uint4*>(mine + v * 16) = reduce_vec<BF16>(t, ws, nullptr, base, v * 16);
  rank_barrier(t, me, ws, epoch + 1, err, 108);
}

// Overlapped ZeRO gradient reduction of ONE bucket: the byte range [lo, hi) of the gradient buffer (a layer's
// gradients, complete while the backward pass of the layers below is still running).  The range's 16-byte
// vectors are dealt to the ranks in equal contiguous slices; a rank sums its slice over all ranks' buffers and
// writes the result into the buffer of the rank that owns that part of the flat space (owner = offset / shard
// bytes), so every bucket loads all ranks and all links evenly whichever shard it falls into.  Nobody else reads
// or writes a vector between the two barriers, so the result can go over the operand in place.
template <bool BF16>
__global__ void __launch_bounds__(COMM_THREADS) zero_reduce_range_kernel(PeerTable t, int me, int ws, long long pay,
                                                                         long long shard_bytes, long long lo,
                                                                         long long hi, uint32_t epoch, int* err) {
  if (!rank_barrier(t, me, ws, epoch, err, 116)) return;
  const long long nvec = (hi - lo) / 16;
  const long long per = (nvec + ws - 1) / ws;
  const long long v0 = me * per;
  long long v1 = min(nvec, v0 + per);
  if (!NX_IN_RANGE(pay + lo, hi - lo, t.limit, err, 117)) v1 = v0;        // nothing is touched; the barriers still run
  const long long stride = (long long)gridDim.x * blockDim.x;
  constexpr int U = 4;
  long long v = v0 + blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (; v + (U - 1) * stride < v1; v += U * stride) {
    float acc[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
    for (int r = 0; r < ws; ++r) {
      const char* src = reinterpret_cast<const char*>(t.ptr[r]) + pay + lo;
      uint4 x[U];
#pragma unroll
      for (int u = 0; u < U; ++u) x[u] = *reinterpret_cast<const uint4*>(src + (v + u * stride) * 16);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (BF16) {
          acc_bf16x8(acc[u], x[u]);
        } else {
          acc[u][0] += __uint_as_float(x[u].x); acc[u][1] += __uint_as_float(x[u].y);
          acc[u][2] += __uint_as_float(x[u].z); acc[u][3] += __uint_as_float(x[u].w);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      uint4 o;
      if (BF16) o = pack_acc(acc[u]);
      else o = make_uint4(__float_as_uint(acc[u][0]), __float_as_uint(acc[u][1]), __float_as_uint(acc[u][2]),
                          __float_as_uint(acc[u][3]));
      const long long off = lo + (v + u * stride) * 16;
      const int owner = static_cast<int>(min(off / shard_bytes, (long long)(ws - 1)));
      *reinterpret_cast<uint4*>(reinterpret_cast<char*>(t.ptr[owner]) + pay + off) = o;
    }
  }
  for (; v < v1; v += stride) {
    const long long off = lo + v * 16;
    const int owner = static_cast<int>(min(off / shard_bytes, (long long)(ws - 1)));
    *reinterpret_cast<uint4*>(reinterpret_cast<char*>(t.ptr[owner]) + pay + off) = reduce_vec<BF16>(t, ws, nullptr, pay, off);
  }
  rank_barrier(t, me, ws, epoch + 1, err, 118);
}

__global__ void __launch_bounds__(COMM_THREADS) zero_all_gather_kernel(PeerTable t, int me, int ws, long long pay,
                                                                       long long shard_bytes, uint32_t epoch,
                                                                       int* err) {
  if (!rank_barrier(t, me, ws, epoch, err, 109)) return;
  long long nvec = shard_bytes / 16;
  const long long base = pay + me * shard_bytes;
  if (!NX_IN_RANGE(base, shard_bytes, t.limit, err, 115)) nvec = 0;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const char* mine = reinterpret_cast<const char*>(t.ptr[me]) + base;
  constexpr int U = 4;
  long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (; v + (U - 1) * stride < nvec; v += U * stride) {
    uint4 x[U];
#pragma unroll
    for (int u = 0; u < U; ++u) x[u] = *reinterpret_cast<const uint4*>(mine + (v + u * stride) * 16);
    for (int r = 0; r < ws; ++r) {
      if (r == me) continue;
      char* dst = reinterpret_cast<char*>(t.ptr[r]) + base;
#pragma unroll
      for (int u = 0; u < U; ++u) *reinterpret_cast<uint4*>(dst + (v + u * stride) * 16) = x[u];
    }
  }
  for (; v < nvec; v += stride) {
    const uint4 x = *reinterpret_cast<const uint4*>(mine + v * 16);
    for (int r = 0; r < ws; ++r)
      if (r != me) *reinterpret_cast<uint4*>(reinterpret_cast<char*>(t.ptr[r]) + base + v * 16) = x;
  }
  rank_barrier(t, me, ws, epoch + 1, err, 110);
}

// Vocabulary-parallel embedding with the tensor-parallel reduction folded away (the reference looks the ids up
// against the local part of the table, zeroes the rows of foreign ids and all-reduces the result,
// megatron/mpu/layers.py:186-212; under sequence parallelism it then keeps one slice).  A token's row exists on
// exactly one rank, the owner of that part of the vocabulary: that rank stores the row straight into the output
// buffer (payload offset `pay` of the workspace) of every rank that needs it, which under sequence parallelism
// is the single rank that owns the token's part of the sequence.  Nothing is summed, and a row crosses NVLink once
// per destination.  ids: [B, S] row-major; output per rank: [B, S, H], or [B, S / ws, H] with sp != 0.
// One warp per token.  An id outside every rank's range leaves its output row unwritten.
__global__ void __launch_bounds__(COMM_THREADS) embed_push_kernel(PeerTable t, int me, int ws, long long pay,
                                                                  const long long* __restrict__ ids,
                                                                  const h16* __restrict__ table, int B, int S, int H,
                                                                  long long vocab_lo, long long vocab_n, int sp,
                                                                  uint32_t epoch, int* err) {
  if (!rank_barrier(t, me, ws, epoch, err, 119)) return;       // the previous readers of the buffers are done
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long T = static_cast<long long>(B) * S;
  const int s_loc = sp ? S / ws : S;
  const int nvec = H >> 3;
  const long long row_bytes = static_cast<long long>(H) * 2;
  for (long long tok = warp; tok < T; tok += nwarps) {
    const long long id = ids[tok] - vocab_lo;
    if (id < 0 || id >= vocab_n) continue;                     // another rank owns this part of the vocabulary
    const uint4* src = reinterpret_cast<const uint4*>(table + id * H);
    const int b = static_cast<int>(tok / S), sq = static_cast<int>(tok % S);
    const long long slot = sp ? static_cast<long long>(b) * s_loc + (sq % s_loc) : tok;
    const long long off = pay + slot * row_bytes;
    if (!NX_IN_RANGE(off, row_bytes, t.limit, err, 120)) continue;
    const int r0 = sp ? sq / s_loc : 0, r1 = sp ? r0 + 1 : ws;
    for (int v = lane; v < nvec; v += 32) {
      const uint4 x = src[v];
      for (int r = r0; r < r1; ++r) reinterpret_cast<uint4*>(reinterpret_cast<char*>(t.ptr[r]) + off)[v] = x;
    }
  }
  rank_barrier(t, me, ws, epoch + 1, err, 121);                // every row of every rank's output has landed
}

// Workspace sizes registered by the host (base address as seen by this rank -> bytes), for the debug range checks.
static unsigned long long g_ws_base[32];
static long long g_ws_bytes[32];
static int g_ws_n = 0;

static bool fill_table(PeerTable& t, const unsigned long long* ptrs, int ws, int me = -1) {
  if (ws < 1 || ws > COMM_MAX_RANKS) return false;
  for (int i = 0; i < COMM_MAX_RANKS; ++i) t.ptr[i] = i < ws ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  t.limit = 0;
  if (me >= 0 && me < ws)
    for (int i = 0; i < g_ws_n; ++i)
      if (g_ws_base[i] == ptrs[me]) t.limit = g_ws_bytes[i];
  return true;
}

}  // namespace nx

NX_API int NX_SYM(nx_comm_flag_bytes)() { return nx::COMM_FLAG_BYTES; }
// Tells the library how large the symmetric workspace that starts at `base` (this rank's own buffer) is.  Only the
// NEOX_DEBUG_BOUNDS build acts on it (range checks inside the kernels); the table holds the last 32 workspaces.
NX_API int NX_SYM(nx_comm_register_workspace)(unsigned long long base, long long bytes) {
  using namespace nx;
  for (int i = 0; i < g_ws_n; ++i)
    if (g_ws_base[i] == base) {
      g_ws_bytes[i] = bytes;
      return NX_OK;
    }
  const int slot = g_ws_n < 32 ? g_ws_n++ : 31;
  g_ws_base[slot] = base;
  g_ws_bytes[slot] = bytes;
  return NX_OK;
}
NX_API int NX_SYM(nx_comm_debug_bounds)() {
#ifdef NEOX_DEBUG_BOUNDS
  return 1;
#else
  return 0;
#endif
}
NX_API int NX_SYM(nx_comm_epochs_per_call)() { return 2; }

// dtype: 0 = bf16, 1 = fp32.  peer_ptrs: host array of ws workspace base addresses (as mapped here).
// mc_ptr: NVLS multicast address of the workspace or 0.  epoch: first of the two epochs this call
// consumes (the caller advances its counter by nx_comm_epochs_per_call()).
NX_API int NX_SYM(nx_comm_allreduce)(const unsigned long long* peer_ptrs, unsigned long long mc_ptr, int me, int ws,
                             long long payload_off, long long bytes, int dtype, unsigned int epoch, void* stream_) {
  using namespace nx;
  PeerTable t;
  NX_REQUIRE(fill_table(t, peer_ptrs, ws, me), "comm: world size %d out of range", ws);
  NX_REQUIRE(bytes % 16 == 0, "comm: payload must be a multiple of 16 bytes");
  auto s = (cudaStream_t)stream_;
  if (dtype == 0)
    allreduce_kernel<true><<<COMM_BLOCKS, COMM_THREADS, 0, s>>>(t, (const void*)mc_ptr, me, ws, payload_off, bytes, epoch,
                                                                device_error_word());
  else
    allreduce_kernel<false><<<COMM_BLOCKS, COMM_THREADS, 0, s>>>(t, (const void*)mc_ptr, me, ws, payload_off, bytes, epoch,
                                                                 device_error_word());
  NX_LAUNCH_CHECK();
  return NX_OK;
}
NX_API int NX_SYM(nx_comm_reduce_scatter)(const unsigned long long* peer_ptrs, unsigned long long mc_ptr, int me, int ws,
                                  long long payload_off, long long shard_bytes, void* out, int dtype, unsigned int epoch, void* stream_) {
  using namespace nx;
  PeerTable t;
  NX_REQUIRE(fill_table(t, peer_ptrs, ws, me), "comm: world size %d out of range", ws);
  NX_REQUIRE(shard_bytes % 16 == 0, "comm: shard must be a multiple of 16 bytes");
  auto s = (cudaStream_t)stream_;
  if (dtype == 0)
    reduce_scatter_kernel<true><<<COMM_BLOCKS, COMM_THREADS, 0, s>>>(t, (const void*)mc_ptr, me, ws, payload_off, shard_bytes,
                                                                     out, epoch, device_error_word());
  else
    reduce_scatter_kernel<false><<<COMM_BLOCKS, COMM_THREADS, 0, s>>>(t, (const void*)mc_ptr, me, ws, payload_off, shard_bytes,
                                                                      out, epoch, device_error_word());
  NX_LAUNCH_CHECK();
  return NX_OK;
}
NX_API int NX_SYM(nx_comm_allgather)(const unsigned long long* peer_ptrs, unsigned long long mc_ptr, int me, int ws,
                             long long payload_off, long long shard_bytes, const void* in, unsigned int epoch, void* stream_) {
  using namespace nx;
  PeerTable t;
  NX_REQUIRE(fill_table(t, peer_ptrs, ws, me), "comm: world size %d out of range", ws);
  NX_REQUIRE(shard_bytes % 16 == 0, "comm: shard must be a multiple of 16 bytes");
  allgather_kernel<<<COMM_BLOCKS, COMM_THREADS, 0, (cudaStream_t)stream_>>>(
      t, (const void*)mc_ptr, me, ws, payload_off, shard_bytes, in, epoch, device_error_word());
  NX_LAUNCH_CHECK();
  return NX_OK;
}

// Vocabulary-parallel embedding lookup whose rows are stored straight into the consumers' buffers (see
// embed_push_kernel).  table: this rank's [vocab_n, H] part (first id vocab_lo).  Output: payload_off of every
// rank's workspace.  Every rank passes the same ids, shapes, grid and epoch.
NX_API int NX_SYM(nx_comm_embed_push)(const unsigned long long* peer_ptrs, int me, int ws, long long payload_off,
                              const void* ids, const void* table, int B, int S, int H, long long vocab_lo,
                              long long vocab_n, int sp, int grid, unsigned int epoch, void* stream_) {
  using namespace nx;
  PeerTable t;
  NX_REQUIRE(fill_table(t, peer_ptrs, ws, me), "comm: world size %d out of range", ws);
  NX_REQUIRE(H % 8 == 0 && payload_off % 16 == 0, "embed_push: H=%d must be a multiple of 8", H);
  NX_REQUIRE(!sp || S % ws == 0, "embed_push: sequence length %d does not divide into %d ranks", S, ws);
  NX_REQUIRE(grid >= 1 && grid * COMM_MAX_RANKS * 4 <= COMM_FLAG_BYTES, "comm: grid %d does not fit the flag area", grid);
  embed_push_kernel<<<grid, COMM_THREADS, 0, (cudaStream_t)stream_>>>(
      t, me, ws, payload_off, (const long long*)ids, (const h16*)table, B, S, H, vocab_lo, vocab_n, sp, epoch,
      device_error_word());
  NX_LAUNCH_CHECK();
  return NX_OK;
}

// In-place ZeRO collectives over buffers inside the symmetric workspace (see the kernels above).
// grid: every rank must pass the same value (blocks pair up across ranks for the barriers).
NX_API int NX_SYM(nx_comm_zero_reduce_scatter)(const unsigned long long* peer_ptrs, int me, int ws, long long payload_off,
                                       long long shard_bytes, int dtype, int grid, unsigned int epoch, void* stream_) {
  using namespace nx;
  PeerTable t;
  NX_REQUIRE(fill_table(t, peer_ptrs, ws, me), "comm: world size %d out of range", ws);
  NX_REQUIRE(shard_bytes % 16 == 0 && payload_off % 16 == 0, "comm: shard / offset must be multiples of 16 bytes");
  NX_REQUIRE(grid >= 1 && grid * COMM_MAX_RANKS * 4 <= COMM_FLAG_BYTES, "comm: grid %d does not fit the flag area", grid);
  auto s = (cudaStream_t)stream_;
  if (dtype == 0)
    zero_reduce_scatter_kernel<true><<<grid, COMM_THREADS, 0, s>>>(t, me, ws, payload_off, shard_bytes, epoch,
                                                                   device_error_word());
  else
    zero_reduce_scatter_kernel<false><<<grid, COMM_THREADS, 0, s>>>(t, me, ws, payload_off, shard_bytes, epoch,
                                                                    device_error_word());
  NX_LAUNCH_CHECK();
  return NX_OK;
}
// One bucket of the overlapped ZeRO gradient reduction: bytes [lo, hi) of the gradient buffer at payload_off
// (see zero_reduce_range_kernel).  Every rank passes the same range, grid and epoch.  Small blocks (128 threads)
// fit into the registers the persistent GEMM CTAs of the backward pass leave free on an SM.
NX_API int NX_SYM(nx_comm_zero_reduce_range)(const unsigned long long* peer_ptrs, int me, int ws, long long payload_off,
                                     long long shard_bytes, long long lo, long long hi, int dtype, int grid,
                                     int threads, unsigned int epoch, void* stream_) {
  using namespace nx;
  PeerTable t;
  NX_REQUIRE(fill_table(t, peer_ptrs, ws, me), "comm: world size %d out of range", ws);
  NX_REQUIRE(shard_bytes > 0 && shard_bytes % 16 == 0 && payload_off % 16 == 0,
             "comm: shard / offset must be multiples of 16 bytes");
  NX_REQUIRE(lo >= 0 && hi >= lo && hi <= shard_bytes * ws && lo % 16 == 0 && hi % 16 == 0,
             "comm: range [%lld, %lld) must be 16-byte aligned and inside the buffer", lo, hi);
  NX_REQUIRE(grid >= 1 && grid * COMM_MAX_RANKS * 4 <= COMM_FLAG_BYTES, "comm: grid %d does not fit the flag area", grid);
  NX_REQUIRE(threads >= 32 && threads <= COMM_THREADS && threads % 32 == 0, "comm: %d threads per block", threads);
  auto s = (cudaStream_t)stream_;
  if (dtype == 0)
    zero_reduce_range_kernel<true><<<grid, threads, 0, s>>>(t, me, ws, payload_off, shard_bytes, lo, hi, epoch,
                                                            device_error_word());
  else
    zero_reduce_range_kernel<false><<<grid, threads, 0, s>>>(t, me, ws, payload_off, shard_bytes, lo, hi, epoch,
                                                             device_error_word());
  NX_LAUNCH_CHECK();
  return NX_OK;
}
NX_API int NX_SYM(nx_comm_zero_all_gather)(const unsigned long long* peer_ptrs, int me, int ws, long long payload_off,
                                   long long shard_bytes, int grid, unsigned int epoch, void* stream_) {
  using namespace nx;
  PeerTable t;
  NX_REQUIRE(fill_table(t, peer_ptrs, ws, me), "comm: world size %d out of range", ws);
  NX_REQUIRE(shard_bytes % 16 == 0 && payload_off % 16 == 0, "comm: shard / offset must be multiples of 16 bytes");
  NX_REQUIRE(grid >= 1 && grid * COMM_MAX_RANKS * 4 <= COMM_FLAG_BYTES, "comm: grid %d does not fit the flag area", grid);
  zero_all_gather_kernel<<<grid, COMM_THREADS, 0, (cudaStream_t)stream_>>>(t, me, ws, payload_off, shard_bytes, epoch,
                                                                           device_error_word());
  NX_LAUNCH_CHECK();
  return NX_OK;
}
