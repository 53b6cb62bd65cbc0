// Per-head weightless RMS normalisation of the Q and K groups of packed QKV rows,
// forward (in place, rstd saved) and backward (in place on dQKV).
//
// Rows are [tokens, (Hq + Hkv + Hkv) * D] laid out (q heads | k heads | v heads). Each
// thread owns 8 consecutive elements (one 16-byte vector); the D/8 threads of a head
// reduce with shuffles, so a warp handles 4 heads (D = 64) or 2 heads (D = 128) and
// every global access is a full 16-byte vector.
//
//   forward : y = x * rsqrt(mean(x^2) + eps) (* q_scale for q heads)
//   backward: dx = scale * rstd * (dy - n * mean(dy * n)),  n = y / scale
//
// Reference counterparts: qk_rms_norm_packed_bf16_forward / _backward
// (neuralfn/csrc/tile_cuda/kernels.cu:19111-19155) and QKNormStage
// (neuralfn/torch_backend.py:2502).
#include "common.h"
#include "sm100_ptx.cuh"

namespace nfn {

__device__ __forceinline__ void qk_unpack8(const uint4& u, float (&f)[8]) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 qk_pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}
template <int GROUP>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = GROUP / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int D>
__global__ void __launch_bounds__(256)
qk_norm_fwd_kernel(__nv_bfloat16* __restrict__ qkv, float* __restrict__ rstd, long long n_heads_total,
                   int Hq, int Hkv, int ld, float eps, float q_scale) {
  constexpr int GROUP = D / 8;
  const long long t = (long long)blockIdx.x * 256 + threadIdx.x;
  const long long head_id = t / GROUP;          // (token, head) flattened
  const int part = (int)(t % GROUP);
  const bool live = head_id < n_heads_total;    // whole groups are live or dead together
  const int heads = Hq + Hkv;
  const long long tok = live ? head_id / heads : 0;
  const int h = live ? (int)(head_id % heads) : 0;
  __nv_bfloat16* ptr = qkv + tok * ld + h * D + part * 8;
  float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (live) qk_unpack8(*reinterpret_cast<const uint4*>(ptr), v);
  float sq = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) sq += v[j] * v[j];
  sq = group_sum<GROUP>(sq);
  if (!live) return;
  const float rs = rsqrtf(sq / D + eps);
  const float sc = rs * (h < Hq ? q_scale : 1.f);
  if (part == 0) rstd[head_id] = rs;
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] *= sc;
  *reinterpret_cast<uint4*>(ptr) = qk_pack8(v);
}

template <int D>
__global__ void __launch_bounds__(256)
qk_norm_bwd_kernel(__nv_bfloat16* __restrict__ dqkv, const __nv_bfloat16* __restrict__ qkv_normed,
                   const float* __restrict__ rstd, long long n_heads_total, int Hq, int Hkv, int ld,
                   float q_scale) {
  constexpr int GROUP = D / 8;
  const long long t = (long long)blockIdx.x * 256 + threadIdx.x;
  const long long head_id = t / GROUP;
  const int part = (int)(t % GROUP);
  const bool live = head_id < n_heads_total;
  const int heads = Hq + Hkv;
  const long long tok = live ? head_id / heads : 0;
  const int h = live ? (int)(head_id % heads) : 0;
  const size_t off = (size_t)tok * ld + h * D + part * 8;
  const float sc = (h < Hq ? q_scale : 1.f);
  float dy[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, n[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (live) {
    qk_unpack8(*reinterpret_cast<const uint4*>(dqkv + off), dy);
    qk_unpack8(*reinterpret_cast<const uint4*>(qkv_normed + off), n);
  }
  const float inv_sc = 1.f / sc;
  float dot = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) { n[j] *= inv_sc; dot += dy[j] * n[j]; }
  dot = group_sum<GROUP>(dot) / D;
  if (!live) return;
  const float rs = rstd[head_id] * sc;
  float o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = rs * (dy[j] - n[j] * dot);
  *reinterpret_cast<uint4*>(dqkv + off) = qk_pack8(o);
}

}  // namespace nfn

using namespace nfn;

extern "C" int nfn_qk_norm_forward(void* qkv, float* rstd, int tokens, int n_q_heads,
                                   int n_kv_heads, int head_dim, int ld, float eps, float q_scale,
                                   nfn_stream_t stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long heads_total = (long long)tokens * (n_q_heads + n_kv_heads);
  if (heads_total <= 0) return 0;
  if (ld % 8 || (reinterpret_cast<uintptr_t>(qkv) & 15)) return fail(-1, "qk_norm: misaligned rows");
  if (head_dim == 64) {
    const unsigned grid = (unsigned)((heads_total * 8 + 255) / 256);
    qk_norm_fwd_kernel<64><<<grid, 256, 0, st>>>((__nv_bfloat16*)qkv, rstd, heads_total, n_q_heads,
                                                 n_kv_heads, ld, eps, q_scale);
  } else if (head_dim == 128) {
    const unsigned grid = (unsigned)((heads_total * 16 + 255) / 256);
    qk_norm_fwd_kernel<128><<<grid, 256, 0, st>>>((__nv_bfloat16*)qkv, rstd, heads_total, n_q_heads,
                                                  n_kv_heads, ld, eps, q_scale);
  } else {
    return fail(-1, "qk_norm: head_dim must be 64 or 128");
  }
  return launch_check("qk_norm_fwd");
}

extern "C" int nfn_qk_norm_backward(void* dqkv, const void* qkv_normed, const float* rstd,
                                    int tokens, int n_q_heads, int n_kv_heads, int head_dim, int ld,
                                    float q_scale, nfn_stream_t stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long heads_total = (long long)tokens * (n_q_heads + n_kv_heads);
  if (heads_total <= 0) return 0;
  if (ld % 8) return fail(-1, "qk_norm: misaligned rows");
  if (head_dim == 64) {
    const unsigned grid = (unsigned)((heads_total * 8 + 255) / 256);
    qk_norm_bwd_kernel<64><<<grid, 256, 0, st>>>((__nv_bfloat16*)dqkv, (const __nv_bfloat16*)qkv_normed,
                                                 rstd, heads_total, n_q_heads, n_kv_heads, ld, q_scale);
  } else if (head_dim == 128) {
    const unsigned grid = (unsigned)((heads_total * 16 + 255) / 256);
    qk_norm_bwd_kernel<128><<<grid, 256, 0, st>>>((__nv_bfloat16*)dqkv, (const __nv_bfloat16*)qkv_normed,
                                                  rstd, heads_total, n_q_heads, n_kv_heads, ld, q_scale);
  } else {
    return fail(-1, "qk_norm: head_dim must be 64 or 128");
  }
  return launch_check("qk_norm_bwd");
}
