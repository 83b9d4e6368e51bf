// Expert-parallel MoE dispatch and combine over NVLink peer memory (no NCCL all-to-all, no host read
// of the routing result).
//
// Every rank of the expert-parallel group owns E_local = experts / ws experts and a symmetric
// workspace that its peers can load from.  One layer call is
//     publish (tokens + top-k expert ids into the own workspace)           -> rank barrier
//     plan over ALL ranks' routed copies, keeping those of the local experts (csrc/moe.cu)
//     gather: row r of the padded expert-sorted matrix is PULLED from the source rank's tokens
//             (the all-to-all dispatch and the permutation are one kernel)
//     grouped GEMMs on local rows, result rows + the copy -> row table into the own workspace
//                                                                           -> rank barrier
//     combine: token t sums its k expert outputs, each PULLED from the owner rank's result rows
//             (the return all-to-all and the weighted un-permutation are one kernel)
// The backward pass is the same two exchanges with the roles of tokens and rows swapped; the
// gradient of the routing weights is a per-row dot product computed on the owner and pulled back.
// Reference: megatron/model/moe.py:85-160 (dispatch by slicing replicated tokens + variable-size
// all-gather, mpu/mappings.py:147-183).
//
// All cross-rank loads are plain ld.global through peer mappings; waits are bounded and record an
// error word on expiry.
#include "common.h"
#include "ptx.cuh"

namespace nx {

constexpr int EP_MAX_RANKS = 8;

struct EpPeers {
  const char* base[EP_MAX_RANKS];  // every rank's workspace as mapped on this rank
};

// Single-block barrier over the ranks' workspaces: flags[0 .. ws) at the start of each workspace.
__global__ void ep_barrier_kernel(EpPeers p, int me, int ws, uint32_t epoch, int* err) {
  if (threadIdx.x < ws) {
    const int peer = threadIdx.x;
    uint32_t* remote = reinterpret_cast<uint32_t*>(const_cast<char*>(p.base[peer])) + me;
    __threadfence_system();
    st_release_sys(remote, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.base[me]) + peer;
    wait_flag_ge(mine, epoch, err, 40);
  }
}

// expert_local[r * Ck + c] = (id - e_lo) if rank r's copy c goes to one of this rank's experts, else -1.
__global__ void ep_stage_ids_kernel(EpPeers p, long long idx_off, int ws, int Ck, int e_lo, int E_local,
                                    long long* __restrict__ expert_local) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= ws * Ck) return;
  const int r = i / Ck, c = i - r * Ck;
  const int id = reinterpret_cast<const int*>(p.base[r] + idx_off)[c];
  const int e = id - e_lo;
  expert_local[i] = (e >= 0 && e < E_local) ? e : -1;
}

// out[row] = scale * tokens_of_rank(c / Ck)[(c % Ck) / k] with c = src_copy[row] (zeros for padding rows);
// scale (optional) = that rank's per-copy weight.  dot_with (optional, local [rows, H]): dot_out[row] =
// <unscaled source row, dot_with[row]>.  One warp per row.
__global__ void __launch_bounds__(256)
ep_gather_kernel(EpPeers p, long long tok_off, long long scale_off, const int* __restrict__ src_copy, int Ck, int k,
                 h16* __restrict__ out, int rows, int H, const h16* __restrict__ dot_with,
                 float* __restrict__ dot_out) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int c = src_copy[row];
  uint4* o = reinterpret_cast<uint4*>(out + static_cast<long long>(row) * H);
  if (c < 0) {
    for (int v = lane; v < H / 8; v += 32) o[v] = make_uint4(0u, 0u, 0u, 0u);
    if (dot_out != nullptr && lane == 0) dot_out[row] = 0.f;
    return;
  }
  const int r = c / Ck, lc = c - r * Ck;
  const uint4* s = reinterpret_cast<const uint4*>(p.base[r] + tok_off) + static_cast<long long>(lc / k) * (H / 8);
  float w = 1.f;
  if (scale_off >= 0) w = h16_to_float(reinterpret_cast<const h16*>(p.base[r] + scale_off)[lc]);
  const uint4* d = dot_with ? reinterpret_cast<const uint4*>(dot_with + static_cast<long long>(row) * H) : nullptr;
  float acc = 0.f;
  for (int v = lane; v < H / 8; v += 32) {
    const uint4 u = s[v];
    const uint32_t uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t ow[4];
    uint32_t dw[4] = {0u, 0u, 0u, 0u};
    if (d != nullptr) {
      const uint4 t = d[v];
      dw[0] = t.x; dw[1] = t.y; dw[2] = t.z; dw[3] = t.w;
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 a = unpack_h16x2(uw[q]);
      if (d != nullptr) {
        const float2 b = unpack_h16x2(dw[q]);
        acc += a.x * b.x + a.y * b.y;
      }
      ow[q] = scale_off >= 0 ? pack_h16x2(a.x * w, a.y * w) : uw[q];
    }
    o[v] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
  if (dot_out != nullptr) {
#pragma unroll
    for (int s2 = 16; s2 > 0; s2 >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s2);
    if (lane == 0) dot_out[row] = acc;
  }
}

// out[t] = sum_j w[t*k+j] * rows_of_owner[dest_of_owner[me*Ck + t*k + j]], owner = expert_id[t*k+j] / E_local
// (w null: unit weights).  aux_off >= 0: aux_out[t*k+j] = the owner's per-row scalar for that copy.
// One warp per token, fp32 accumulation, deterministic.
__global__ void __launch_bounds__(256)
ep_combine_kernel(EpPeers p, long long rows_off, long long dest_off, long long aux_off,
                  const int* __restrict__ expert_id, int E_local, int me, int ws, int Ck, int k,
                  const h16* __restrict__ w, h16* __restrict__ out, int T, int H,
                  h16* __restrict__ aux_out, int* err) {
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= T) return;
  const int lane = threadIdx.x & 31;
  constexpr int MAXK = 8;
  const uint4* src[MAXK];
  float wj[MAXK];
  for (int j = 0; j < k && j < MAXK; ++j) {
    const int c = t * k + j;
    const int owner = expert_id[c] / E_local;
    const int row = (owner >= 0 && owner < ws)
                        ? reinterpret_cast<const int*>(p.base[owner] + dest_off)[me * Ck + c] : -1;
    if (row < 0) {   // expert id out of range, or the owner did not place this copy (plans disagree)
      if (lane == 0) atomicExch(err, 41);
      src[j] = nullptr;
      wj[j] = 0.f;
      continue;
    }
    src[j] = reinterpret_cast<const uint4*>(p.base[owner] + rows_off) + static_cast<long long>(row) * (H / 8);
    wj[j] = w ? h16_to_float(w[c]) : 1.f;
    if (aux_off >= 0 && lane == 0)
      aux_out[c] = float_to_h16(reinterpret_cast<const float*>(p.base[owner] + aux_off)[row]);
  }
  for (int v = lane; v < H / 8; v += 32) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k && j < MAXK; ++j) {
      if (src[j] == nullptr) continue;
      const uint4 u = src[j][v];
      const float2 a = unpack_h16x2(u.x), b = unpack_h16x2(u.y), cc = unpack_h16x2(u.z), d = unpack_h16x2(u.w);
      acc[0] += wj[j] * a.x; acc[1] += wj[j] * a.y; acc[2] += wj[j] * b.x; acc[3] += wj[j] * b.y;
      acc[4] += wj[j] * cc.x; acc[5] += wj[j] * cc.y; acc[6] += wj[j] * d.x; acc[7] += wj[j] * d.y;
    }
    uint4 r;
    r.x = pack_h16x2(acc[0], acc[1]); r.y = pack_h16x2(acc[2], acc[3]);
    r.z = pack_h16x2(acc[4], acc[5]); r.w = pack_h16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + static_cast<long long>(t) * H)[v] = r;
  }
}

static EpPeers make_peers(const unsigned long long* ptrs, int ws) {
  EpPeers p;
  for (int i = 0; i < EP_MAX_RANKS; ++i) p.base[i] = i < ws ? reinterpret_cast<const char*>(ptrs[i]) : nullptr;
  return p;
}

}  // namespace nx

NX_API int NX_SYM(nx_moe_ep_flag_bytes)() { return 4096; }

NX_API int NX_SYM(nx_moe_ep_barrier)(const unsigned long long* peer_ptrs, int me, int ws, unsigned epoch, void* stream_) {
  using namespace nx;
  NX_REQUIRE(ws >= 1 && ws <= EP_MAX_RANKS && me >= 0 && me < ws, "moe_ep_barrier: rank %d of %d", me, ws);
  ep_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(make_peers(peer_ptrs, ws), me, ws, epoch,
                                                                       device_error_word());
  NX_LAUNCH_CHECK();
  return NX_OK;
}

// expert_local: int64 [ws * Ck] (input of nx_moe_plan with E_local experts).
NX_API int NX_SYM(nx_moe_ep_stage_ids)(const unsigned long long* peer_ptrs, int ws, long long idx_off, int Ck, int e_lo,
                               int E_local, void* expert_local, void* stream_) {
  using namespace nx;
  NX_REQUIRE(ws >= 1 && ws <= EP_MAX_RANKS && Ck > 0 && idx_off % 4 == 0, "moe_ep_stage_ids: bad arguments");
  const int n = ws * Ck;
  ep_stage_ids_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      make_peers(peer_ptrs, ws), idx_off, ws, Ck, e_lo, E_local, static_cast<long long*>(expert_local));
  NX_LAUNCH_CHECK();
  return NX_OK;
}

// scale_off < 0: no scaling.  dot_with / dot_out may be null.
NX_API int NX_SYM(nx_moe_ep_gather)(const unsigned long long* peer_ptrs, int ws, long long tok_off, long long scale_off,
                            const void* src_copy, int Ck, int k, void* out, int rows, int H, const void* dot_with,
                            void* dot_out, void* stream_) {
  using namespace nx;
  NX_REQUIRE(H % 8 == 0 && tok_off % 16 == 0 && (scale_off < 0 || scale_off % 2 == 0),
             "moe_ep_gather: hidden size must be a multiple of 8 and offsets aligned");
  NX_REQUIRE((dot_with == nullptr) == (dot_out == nullptr), "moe_ep_gather: dot_with and dot_out go together");
  ep_gather_kernel<<<(rows + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      make_peers(peer_ptrs, ws), tok_off, scale_off, static_cast<const int*>(src_copy), Ck, k,
      static_cast<h16*>(out), rows, H, static_cast<const h16*>(dot_with),
      static_cast<float*>(dot_out));
  NX_LAUNCH_CHECK();
  return NX_OK;
}

// aux_off < 0: no per-copy scalar.  w may be null (unit weights).
NX_API int NX_SYM(nx_moe_ep_combine)(const unsigned long long* peer_ptrs, int ws, int me, long long rows_off,
                             long long dest_off, long long aux_off, const void* expert_id, int E_local, int Ck, int k,
                             const void* w, void* out, int T, int H, void* aux_out, void* stream_) {
  using namespace nx;
  NX_REQUIRE(H % 8 == 0 && rows_off % 16 == 0 && dest_off % 4 == 0 && (aux_off < 0 || aux_off % 4 == 0),
             "moe_ep_combine: hidden size must be a multiple of 8 and offsets aligned");
  NX_REQUIRE(k >= 1 && k <= 8 && T * k == Ck, "moe_ep_combine: k=%d T=%d Ck=%d", k, T, Ck);
  ep_combine_kernel<<<(T + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      make_peers(peer_ptrs, ws), rows_off, dest_off, aux_off, static_cast<const int*>(expert_id), E_local, me, ws, Ck, k,
      static_cast<const h16*>(w), static_cast<h16*>(out), T, H,
      static_cast<h16*>(aux_out), device_error_word());
  NX_LAUNCH_CHECK();
  return NX_OK;
}
