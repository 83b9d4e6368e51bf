// Rotary position embedding (full or partial, strided, forward and backward) and the
// vocab-parallel embedding gather / scatter-add.
//
// Rotary: counterpart of megatron/fused_kernels/fused_rotary_positional_embedding.h:27-225 and
// megatron/model/positional_embeddings.py:103-127.  Convention: rotate_half over halves,
//   out[j]        = x[j]        * cos[j] - x[j + r/2] * sin[j]
//   out[j + r/2]  = x[j + r/2]  * cos[j] + x[j]       * sin[j]      (j < r/2, r = rotary dims)
// and dims >= r pass through (copied only when out != in).  The kernel works directly on a
// strided view, e.g. the q or k slice of the fused [s, b, heads, 3*hn] QKV projection output,
// so no de-interleave copy is needed.  Backward = same kernel with sin negated.
//
// Embedding: counterpart of VocabParallelEmbedding (megatron/mpu/layers.py:186-212): ids outside
// this rank's [vocab_start, vocab_start + V_local) produce zero rows (the cross-rank sum fills
// them in).
#include "common.h"
#include "ptx.cuh"

namespace nx {

struct RopeArgs {
  const h16* in;
  h16* out;
  const float* cos;  // [max_pos, r/2]
  const float* sin;
  int S, B, NH, D, R;
  long long is, ib, ih;  // input strides (elements) for s, b, head
  long long os, ob, oh;  // output strides
  int pos0;
  float sin_sign;
};

__global__ void rope_kernel(const RopeArgs a) {
  const int half = a.R >> 1;
  const bool copy_tail = (a.in != a.out);
  const int per_head = copy_tail ? (half + (a.D - a.R)) : half;  // work items per head
  const long long total = static_cast<long long>(a.S) * a.B * a.NH * per_head;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int j = static_cast<int>(i % per_head);
    long long t = i / per_head;
    const int h = static_cast<int>(t % a.NH);
    t /= a.NH;
    const int b = static_cast<int>(t % a.B);
    const int s = static_cast<int>(t / a.B);
    const h16* ip = a.in + s * a.is + b * a.ib + h * a.ih;
    h16* op = a.out + s * a.os + b * a.ob + h * a.oh;
    if (j < half) {
      const float c = a.cos[static_cast<long long>(a.pos0 + s) * half + j];
      const float sn = a.sin[static_cast<long long>(a.pos0 + s) * half + j] * a.sin_sign;
      const float x1 = h16_to_float(ip[j]), x2 = h16_to_float(ip[j + half]);
      op[j] = float_to_h16(x1 * c - x2 * sn);
      op[j + half] = float_to_h16(x2 * c + x1 * sn);
    } else {
      const int d = a.R + (j - half);
      op[d] = ip[d];
    }
  }
}

// In-place form for 16-byte aligned views with r/2 a multiple of 8: a thread rotates eight (j, j + r/2)
// pairs with two 16-byte loads and stores (the scalar kernel above moves 2 bytes per access, which costs a
// full sector each on the 64-byte rotary slice of a head).
__global__ void rope_vec8_kernel(const RopeArgs a) {
  const int half = a.R >> 1;
  const int groups = half >> 3;  // 8-wide groups per head
  const long long total = static_cast<long long>(a.S) * a.B * a.NH * groups;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int j = static_cast<int>(i % groups) * 8;
    long long t = i / groups;
    const int h = static_cast<int>(t % a.NH);
    t /= a.NH;
    const int b = static_cast<int>(t % a.B);
    const int s = static_cast<int>(t / a.B);
    h16* ptr = a.out + s * a.os + b * a.ob + h * a.oh;
    const uint4 u1 = *reinterpret_cast<const uint4*>(ptr + j);
    const uint4 u2 = *reinterpret_cast<const uint4*>(ptr + j + half);
    const float4* cp = reinterpret_cast<const float4*>(a.cos + static_cast<long long>(a.pos0 + s) * half + j);
    const float4* sp = reinterpret_cast<const float4*>(a.sin + static_cast<long long>(a.pos0 + s) * half + j);
    const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const uint32_t w1[4] = {u1.x, u1.y, u1.z, u1.w}, w2[4] = {u2.x, u2.y, u2.z, u2.w};
    uint32_t o1[4], o2[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 x1 = unpack_h16x2(w1[q]), x2 = unpack_h16x2(w2[q]);
      const float sa = sn[2 * q] * a.sin_sign, sb = sn[2 * q + 1] * a.sin_sign;
      o1[q] = pack_h16x2(x1.x * c[2 * q] - x2.x * sa, x1.y * c[2 * q + 1] - x2.y * sb);
      o2[q] = pack_h16x2(x2.x * c[2 * q] + x1.x * sa, x2.y * c[2 * q + 1] + x1.y * sb);
    }
    *reinterpret_cast<uint4*>(ptr + j) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
    *reinterpret_cast<uint4*>(ptr + j + half) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
  }
}

__global__ void embedding_fwd_kernel(const long long* __restrict__ ids,
                                     const h16* __restrict__ table,
                                     h16* __restrict__ out, long long n, int H,
                                     long long vocab_start, long long v_local) {
  const int h8 = H >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n * h8;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / h8;
    const int c = static_cast<int>(i - r * h8);
    const long long id = ids[r] - vocab_start;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (id >= 0 && id < v_local) v = reinterpret_cast<const uint4*>(table + id * H)[c];
    reinterpret_cast<uint4*>(out + r * H)[c] = v;
  }
}
// grad_table (fp32) [v_local, H] += dout rows
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids,
                                     const h16* __restrict__ dout,
                                     float* __restrict__ grad_table, long long n, int H,
                                     long long vocab_start, long long v_local) {
  const int h2 = H >> 1;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n * h2;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / h2;
    const int c = static_cast<int>(i - r * h2) * 2;
    const long long id = ids[r] - vocab_start;
    if (id >= 0 && id < v_local) {
      const float2 g = unpack_h16x2(*reinterpret_cast<const uint32_t*>(dout + r * H + c));
      atomicAdd(grad_table + id * H + c, g.x);
      atomicAdd(grad_table + id * H + c + 1, g.y);
    }
  }
}

}  // namespace nx

NX_API int NX_SYM(nx_rope)(const void* in, void* out, const void* cos, const void* sin, int S, int B, int NH,
                   int D, int R, long long is, long long ib, long long ih, long long os,
                   long long ob, long long oh, int pos0, int inverse, void* stream_) {
  using namespace nx;
  NX_REQUIRE(R % 2 == 0 && R <= D, "rope: rotary dims %d invalid for head dim %d", R, D);
  if (S == 0 || B == 0 || NH == 0 || (R == 0 && in == out)) return NX_OK;
  RopeArgs a;
  a.in = (const h16*)in; a.out = (h16*)out;
  a.cos = (const float*)cos; a.sin = (const float*)sin;
  a.S = S; a.B = B; a.NH = NH; a.D = D; a.R = R;
  a.is = is; a.ib = ib; a.ih = ih; a.os = os; a.ob = ob; a.oh = oh;
  a.pos0 = pos0; a.sin_sign = inverse ? -1.f : 1.f;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  const bool vec = in == out && (R / 2) % 8 == 0 && os % 8 == 0 && ob % 8 == 0 && oh % 8 == 0 &&
                   (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (reinterpret_cast<uintptr_t>(cos) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(sin) & 15) == 0;
  if (vec) {
    const long long total = static_cast<long long>(S) * B * NH * (R / 16);
    const long long g = (total + 255) / 256;
    rope_vec8_kernel<<<(int)(g < cap ? g : cap), 256, 0, (cudaStream_t)stream_>>>(a);
    NX_LAUNCH_CHECK();
    return NX_OK;
  }
  const int per_head = (in != out) ? (R / 2 + (D - R)) : R / 2;
  const long long total = static_cast<long long>(S) * B * NH * per_head;
  long long g = (total + 255) / 256;
  rope_kernel<<<(int)(g < cap ? g : cap), 256, 0, (cudaStream_t)stream_>>>(a);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
NX_API int NX_SYM(nx_embedding_fwd)(const void* ids, const void* table, void* out, long long n, int H,
                            long long vocab_start, long long v_local, void* stream_) {
  using namespace nx;
  NX_REQUIRE(H % 8 == 0, "embedding: H %% 8 != 0");
  if (n == 0) return NX_OK;
  long long g = (n * (H / 8) + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  embedding_fwd_kernel<<<(int)(g < cap ? g : cap), 256, 0, (cudaStream_t)stream_>>>(
      (const long long*)ids, (const h16*)table, (h16*)out, n, H, vocab_start,
      v_local);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
NX_API int NX_SYM(nx_embedding_bwd)(const void* ids, const void* dout, void* grad_table, long long n, int H,
                            long long vocab_start, long long v_local, void* stream_) {
  using namespace nx;
  NX_REQUIRE(H % 2 == 0, "embedding: H %% 2 != 0");
  if (n == 0) return NX_OK;
  long long g = (n * (H / 2) + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  embedding_bwd_kernel<<<(int)(g < cap ? g : cap), 256, 0, (cudaStream_t)stream_>>>(
      (const long long*)ids, (const h16*)dout, (float*)grad_table, n, H, vocab_start,
      v_local);
  NX_LAUNCH_CHECK();
  return NX_OK;
}
