// Differential attention around the flash-attention kernels.
//
// A differential head splits its query and key into halves (q1 | q2), (k1 | k2), runs two softmax
// attentions over the same values and combines them:
//
//     a1 = softmax(q1 k1^T / sqrt(D/2)) v,  a2 = softmax(q2 k2^T / sqrt(D/2)) v
//     out = rms_norm(a1 - lambda * a2) * (1 - lambda_init)          (lambda: one learned scalar per layer)
//
// Both attentions go through ONE launch of the ordinary kernels: every head becomes two pseudo-heads
// whose queries are the head's query with the other half zeroed, (q1 | 0) and (0 | q2), sharing the
// head's unchanged key and value as a grouped-query pair. (q1 | 0) . (k1 | k2) = q1 . k1, so the scores
// are exact and no half-head-dimension kernel is needed; the flash kernels see 2 H query heads, H key /
// value heads and the scale 1 / sqrt(D/2). The kernels here are the memory-bound glue:
//
//   nfn_diff_q_expand      q [tokens, H D] -> q' [tokens, 2 H D]
//   nfn_diff_combine       a [tokens, 2 H D] -> out [tokens, H D], rstd [tokens, H]
//   nfn_diff_combine_bwd   d(out) -> d(a) [tokens, 2 H D] and d(lambda)
//   nfn_diff_q_collapse    d(q') -> d(q) (the zeroed halves' gradients are dropped)
//
// One thread owns 8 consecutive elements (a 16-byte vector); the D / 8 threads of a head reduce with
// shuffles. Reference counterparts: the packed differential attention kernels of
// neuralfn/csrc/tile_cuda/kernels.cu:19210-19554 and DifferentialAttentionStage
// (neuralfn/torch_backend.py), which materialise both score matrices.
#include "common.h"
#include "nfn_kernels.h"
#include "sm100_ptx.cuh"

namespace nfn {

__device__ __forceinline__ void da_unpack8(const uint4& u, float (&f)[8]) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 da_pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}
template <int GROUP>
__device__ __forceinline__ float da_group_sum(float v) {
#pragma unroll
  for (int o = GROUP / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// q' vector index e8 of a row of 2 H D / 8 vectors: pseudo-head p = 2 h + j keeps half j of head h.
__global__ void __launch_bounds__(256)
diff_q_expand_kernel(const __nv_bfloat16* __restrict__ q, int ldq, __nv_bfloat16* __restrict__ q2, long long tokens, int H, int D) {
  const int vec_per_row = 2 * H * D / 8, vec_per_head = D / 8;
  const long long total = tokens * vec_per_row;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const long long t = i / vec_per_row;
    const int e = (int)(i - t * vec_per_row), p = e / vec_per_head, d8 = e - p * vec_per_head;
    const int h = p >> 1, j = p & 1;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if ((d8 >= vec_per_head / 2) == (j == 1)) v = *reinterpret_cast<const uint4*>(q + t * ldq + h * D + d8 * 8);
    reinterpret_cast<uint4*>(q2)[i] = v;
  }
}

__global__ void __launch_bounds__(256)
diff_q_collapse_kernel(const __nv_bfloat16* __restrict__ dq2, __nv_bfloat16* __restrict__ dq, int lddq, long long tokens, int H, int D) {
  const int vec_per_row = H * D / 8, vec_per_head = D / 8;
  const long long total = tokens * vec_per_row;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const long long t = i / vec_per_row;
    const int e = (int)(i - t * vec_per_row), h = e / vec_per_head, d8 = e - h * vec_per_head;
    const int j = d8 >= vec_per_head / 2 ? 1 : 0;
    *reinterpret_cast<uint4*>(dq + t * lddq + h * D + d8 * 8) =
        reinterpret_cast<const uint4*>(dq2)[(t * 2 * H + 2 * h + j) * vec_per_head + d8];
  }
}

// group of D / 8 threads per (token, head)
template <int D>
__global__ void __launch_bounds__(256)
diff_combine_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ lambda, float out_scale, float eps,
                    __nv_bfloat16* __restrict__ out, float* __restrict__ rstd, long long heads_total) {
  constexpr int G = D / 8;
  const float lam = __bfloat162float(lambda[0]);
  const long long gid_raw = ((long long)blockIdx.x * 256 + threadIdx.x) / G;
  const int lane = threadIdx.x % G;
  // every lane of a warp takes part in the shuffles: groups past the end recompute the last head and store nothing
  const bool live = gid_raw < heads_total;
  const long long gid = live ? gid_raw : heads_total - 1;
  float a1[8], a2[8], x[8];
  da_unpack8(reinterpret_cast<const uint4*>(a)[(gid * 2) * G + lane], a1);
  da_unpack8(reinterpret_cast<const uint4*>(a)[(gid * 2 + 1) * G + lane], a2);
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    x[j] = a1[j] - lam * a2[j];
    ss += x[j] * x[j];
  }
  ss = da_group_sum<G>(ss);
  const float r = rsqrtf(ss / D + eps);
#pragma unroll
  for (int j = 0; j < 8; ++j) x[j] *= r * out_scale;
  if (live) {
    reinterpret_cast<uint4*>(out)[gid * G + lane] = da_pack8(x);
    if (lane == 0) rstd[gid] = r;
  }
}

// d(a1) = dx, d(a2) = -lambda dx with dx = c r (dy - n mean(dy n)), n = x r; d(lambda) = -sum(dx a2).
template <int D>
__global__ void __launch_bounds__(256)
diff_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ a,
                        const __nv_bfloat16* __restrict__ lambda, float out_scale, const float* __restrict__ rstd,
                        __nv_bfloat16* __restrict__ da, float* __restrict__ partial, long long heads_total) {
  constexpr int G = D / 8;
  __shared__ float red[8];
  const float lam = __bfloat162float(lambda[0]);
  const int lane = threadIdx.x % G;
  float dl = 0.f;
  // the loop bound is the same for all lanes of a warp (its first group), so the shuffles stay converged
  constexpr int GPW = 32 / G;   // groups per warp
  for (long long base = (((long long)blockIdx.x * 256 + threadIdx.x) / 32) * GPW; base < heads_total; base += (long long)gridDim.x * (256 / G)) {
    const long long gid_raw = base + (threadIdx.x & 31) / G;
    const bool live = gid_raw < heads_total;
    const long long gid = live ? gid_raw : heads_total - 1;
    float a1[8], a2[8], dy[8], n[8];
    da_unpack8(reinterpret_cast<const uint4*>(a)[(gid * 2) * G + lane], a1);
    da_unpack8(reinterpret_cast<const uint4*>(a)[(gid * 2 + 1) * G + lane], a2);
    da_unpack8(reinterpret_cast<const uint4*>(dout)[gid * G + lane], dy);
    const float r = rstd[gid];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      n[j] = (a1[j] - lam * a2[j]) * r;
      dot += dy[j] * n[j];
    }
    dot = da_group_sum<G>(dot) / D;
    float d1[8], d2[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float dx = out_scale * r * (dy[j] - n[j] * dot);
      d1[j] = dx;
      d2[j] = -lam * dx;
      if (live) dl -= dx * a2[j];
    }
    if (live) {
      reinterpret_cast<uint4*>(da)[(gid * 2) * G + lane] = da_pack8(d1);
      reinterpret_cast<uint4*>(da)[(gid * 2 + 1) * G + lane] = da_pack8(d2);
    }
  }
  dl = da_group_sum<32>(dl);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = dl;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w];
    partial[blockIdx.x] = t;
  }
}

// dlambda[0] = sum(partial) (elements 1..7 of the 8-element slot are zeroed)
__global__ void __launch_bounds__(256)
diff_lambda_final_kernel(const float* __restrict__ partial, int n, __nv_bfloat16* __restrict__ dlambda) {
  __shared__ float red[8];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += 256) s += partial[i];
  s = da_group_sum<32>(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 8) {
    float t = 0.f;
    if (threadIdx.x == 0) {
#pragma unroll
      for (int w = 0; w < 8; ++w) t += red[w];
    }
    dlambda[threadIdx.x] = __float2bfloat16(t);
  }
}

static int diff_grid(long long work_items, int per_block) {
  long long b = (work_items + per_block - 1) / per_block;
  const long long cap = (long long)sm_count() * 8;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

static int diff_check(const void* p, int ld, int H, int D, const char* what) {
  if (D != 64 && D != 128) return fail(-1, "differential attention: head_dim must be 64 or 128");
  if (H < 1 || (reinterpret_cast<uintptr_t>(p) & 15) || (ld % 8)) return fail(-1, what);
  return 0;
}

}  // namespace nfn

using namespace nfn;

extern "C" int nfn_diff_partials(void) { return sm_count() * 8; }

extern "C" int nfn_diff_q_expand(const void* q, int ldq, void* q2, long long tokens, int H, int D, nfn_stream_t stream) {
  if (int rc = diff_check(q, ldq, H, D, "diff_q_expand: q must be 16-byte aligned with a row stride that is a multiple of 8")) return rc;
  if (reinterpret_cast<uintptr_t>(q2) & 15) return fail(-1, "diff_q_expand: q2 must be 16-byte aligned");
  diff_q_expand_kernel<<<diff_grid(tokens * 2 * H * D / 8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(q), ldq, static_cast<__nv_bfloat16*>(q2), tokens, H, D);
  return launch_check("diff_q_expand");
}

extern "C" int nfn_diff_q_collapse(const void* dq2, void* dq, int lddq, long long tokens, int H, int D, nfn_stream_t stream) {
  if (int rc = diff_check(dq, lddq, H, D, "diff_q_collapse: dq must be 16-byte aligned with a row stride that is a multiple of 8")) return rc;
  if (reinterpret_cast<uintptr_t>(dq2) & 15) return fail(-1, "diff_q_collapse: dq2 must be 16-byte aligned");
  diff_q_collapse_kernel<<<diff_grid(tokens * H * D / 8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dq2), static_cast<__nv_bfloat16*>(dq), lddq, tokens, H, D);
  return launch_check("diff_q_collapse");
}

// a: [tokens, 2 H D] (pseudo-heads 2h, 2h + 1 of head h); lambda: bf16 (first element used); out: [tokens, H D];
// rstd: fp32 [tokens * H]. out_scale = 1 - lambda_init.
extern "C" int nfn_diff_combine(const void* a, const void* lambda, float out_scale, float eps, void* out, float* rstd,
                                long long tokens, int H, int D, nfn_stream_t stream) {
  if (int rc = diff_check(a, 8, H, D, "diff_combine: a must be 16-byte aligned")) return rc;
  if (reinterpret_cast<uintptr_t>(out) & 15) return fail(-1, "diff_combine: out must be 16-byte aligned");
  const long long heads = tokens * H;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long blocks = (heads * (D / 8) + 255) / 256;
  if (blocks > 0x7fffffffll) return fail(-1, "diff_combine: too many heads for one launch");
  if (D == 64)
    diff_combine_kernel<64><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(lambda),
                                                              out_scale, eps, static_cast<__nv_bfloat16*>(out), rstd, heads);
  else
    diff_combine_kernel<128><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(lambda),
                                                               out_scale, eps, static_cast<__nv_bfloat16*>(out), rstd, heads);
  return launch_check("diff_combine");
}

// da: [tokens, 2 H D]; partial: fp32 [nfn_diff_partials()]; dlambda: bf16, 8 elements (the parameter's slot).
extern "C" int nfn_diff_combine_backward(const void* dout, const void* a, const void* lambda, float out_scale, const float* rstd,
                                         void* da, float* partial, void* dlambda, long long tokens, int H, int D,
                                         nfn_stream_t stream) {
  if (int rc = diff_check(a, 8, H, D, "diff_combine_backward: a must be 16-byte aligned")) return rc;
  if ((reinterpret_cast<uintptr_t>(dout) & 15) || (reinterpret_cast<uintptr_t>(da) & 15))
    return fail(-1, "diff_combine_backward: dout and da must be 16-byte aligned");
  const long long heads = tokens * H;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = diff_grid(heads * (D / 8), 256);
  if (D == 64)
    diff_combine_bwd_kernel<64><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(a),
                                                      static_cast<const __nv_bfloat16*>(lambda), out_scale, rstd,
                                                      static_cast<__nv_bfloat16*>(da), partial, heads);
  else
    diff_combine_bwd_kernel<128><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(a),
                                                       static_cast<const __nv_bfloat16*>(lambda), out_scale, rstd,
                                                       static_cast<__nv_bfloat16*>(da), partial, heads);
  diff_lambda_final_kernel<<<1, 256, 0, st>>>(partial, grid, static_cast<__nv_bfloat16*>(dlambda));
  return launch_check("diff_combine_backward", 2);
}
