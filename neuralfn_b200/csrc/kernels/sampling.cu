// On-device token selection for the decode loop: row argmax (ties -> lowest index) and
// temperature / top-k / top-p sampling, so no logits ever cross PCIe.
//
// Sampling never sorts. Both truncations are "find the key threshold at which a weight
// sum, taken from the largest key downwards, reaches a target": weight 1 and target k for
// top-k, weight exp((x - max)/T) and target p * Z for top-p (Z taken over the top-k
// survivors, i.e. top-k is applied first, then top-p on the renormalised rest). The
// threshold is found by descending through 256-way equal-width value bins (three levels
// for bf16 logits, four for fp32); values that share the final bin are all kept.
// The draw itself is a Gumbel-max: argmax over survivors of x/T + G_i with
// G_i = -log(-log(u_i)), u_i from Philox4x32-10 keyed by (seed, row, offset), which is an
// exact sample from the truncated softmax and needs no prefix sum over the vocabulary.
//
// Host-side greedy choice in the reference: nfn_gpt2_native_train.cpp `select_token`;
// device argmax: kernels.cu:1564-1603.
#include <algorithm>
#include <cfloat>

#include "common.h"
#include "nfn_kernels.h"
#include "sm100_ptx.cuh"

namespace nfn {

__device__ __forceinline__ float ld_logit(const float* p, long long i) { return p[i]; }
__device__ __forceinline__ float ld_logit(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }

struct ValIdx {
  float v;
  int i;
};
__device__ __forceinline__ ValIdx better(ValIdx a, ValIdx b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ ValIdx warp_best(ValIdx x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ValIdx y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  return x;
}
// all threads of the block get the result; sm must hold 32 entries
__device__ ValIdx block_best(ValIdx x, ValIdx* sm) {
  x = warp_best(x);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) sm[w] = x;
  __syncthreads();
  ValIdx y = (l < nw) ? sm[l] : ValIdx{-FLT_MAX, 0x7fffffff};
  return warp_best(y);
}
__device__ float block_sum(float x, float* sm) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) sm[w] = x;
  __syncthreads();
  float y = (l < nw) ? sm[l] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
  return y;
}

// ---- argmax: grid (splits, rows) -> partial, then one warp per row ------------------------
template <typename T>
__global__ void __launch_bounds__(256)
argmax_partial_kernel(const T* __restrict__ logits, long long ld, int V, ValIdx* __restrict__ partial) {
  __shared__ ValIdx sm[32];
  const int row = blockIdx.y, splits = gridDim.x;
  const int per = (V + splits - 1) / splits, lo = blockIdx.x * per, hi = min(V, lo + per);
  const T* p = logits + (long long)row * ld;
  ValIdx best{-FLT_MAX, 0x7fffffff};
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = ld_logit(p, i);
    if (v == v) best = better(best, ValIdx{v, i});
  }
  best = block_best(best, sm);
  if (threadIdx.x == 0) partial[(long long)row * splits + blockIdx.x] = best;
}

__global__ void argmax_final_kernel(const ValIdx* __restrict__ partial, int splits, int rows, int* __restrict__ out_idx,
                                    float* __restrict__ out_val, int index_offset) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  ValIdx best{-FLT_MAX, 0x7fffffff};
  for (int s = lane; s < splits; s += 32) best = better(best, partial[(long long)row * splits + s]);
  best = warp_best(best);
  if (lane == 0) {
    out_idx[row] = best.i + index_offset;
    if (out_val) out_val[row] = best.v;
  }
}

// merge of per-rank winners (tensor-parallel vocabulary): vals/idx are [world, rows]
__global__ void argmax_merge_kernel(const float* __restrict__ vals, const int* __restrict__ idx, int world, int rows,
                                    int* __restrict__ out_idx, float* __restrict__ out_val) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  ValIdx best{-FLT_MAX, 0x7fffffff};
  for (int r = 0; r < world; ++r) best = better(best, ValIdx{vals[(long long)r * rows + row], idx[(long long)r * rows + row]});
  out_idx[row] = best.i;
  if (out_val) out_val[row] = best.v;
}

// ---- Philox4x32-10 --------------------------------------------------------------------------
__device__ __forceinline__ uint4 philox4x32(uint4 ctr, uint2 key) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, ctr.x), lo0 = 0xD2511F53u * ctr.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, ctr.z), lo1 = 0xCD9E8D57u * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += 0x9E3779B9u;
    key.y += 0xBB67AE85u;
  }
  return ctr;
}
__device__ __forceinline__ float gumbel(uint32_t bits) {
  const float u = ((float)(bits >> 8) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1)
  return -__logf(-__logf(u));
}

// ---- sampling: one 1024-thread block per row -----------------------------------------------------
// A threshold is a path through up to four levels of 256 equal-width value bins: level 0
// spans [lo0, lo0 + 256 * w0) (everything below lo0 falls into bin 0), each deeper level
// splits the chosen bin again. An element survives when its bin path is lexicographically
// >= the chosen path. Linear bins spread a row's logits over many counters, which keeps
// the shared-memory atomics from piling onto one address the way exponent-byte digits would.
struct BinPath {
  float lo0, w0;
  int levels;
  int sel[4];
};

__device__ __forceinline__ int bin_of(float x, float lo, float inv_w) {
  const float t = (x - lo) * inv_w;
  return t <= 0.f ? 0 : (t >= 255.f ? 255 : (int)t);
}

// compares x's bin path with the first `levels` chosen bins: >0 above, <0 below, 0 on the path;
// on return (lo, w) describe the bin x would be split into next
__device__ __forceinline__ int path_cmp(float x, const BinPath& p, int levels, float* lo_out, float* w_out) {
  float lo = p.lo0, w = p.w0;
  for (int l = 0; l < levels; ++l) {
    const int b = bin_of(x, lo, 1.f / w);
    if (b != p.sel[l]) return b > p.sel[l] ? 1 : -1;
    lo += (float)p.sel[l] * w;
    w *= (1.f / 256.f);
  }
  *lo_out = lo;
  *w_out = w;
  return 0;
}
__device__ __forceinline__ bool survives(float x, const BinPath& p) {
  if (p.levels == 0) return true;
  float lo, w;
  return path_cmp(x, p, p.levels, &lo, &w) >= 0;
}

// Descends until the weight sum taken from the top reaches `target`. `outer` restricts the
// population (top-k survivors when searching the top-p threshold).
template <typename T, bool kWeighted>
__device__ void find_threshold(const T* __restrict__ p, int V, float target, float row_max, float row_lo, float inv_temp,
                               const BinPath& outer, int n_levels, BinPath* path, float* hist, float* sh_above) {
  if (threadIdx.x == 0) {
    path->lo0 = row_lo;
    path->w0 = fmaxf((row_max - row_lo) * (1.f / 256.f) * 1.000001f, 1e-30f);
    path->levels = 0;
    *sh_above = 0.f;
  }
  __syncthreads();
  for (int level = 0; level < n_levels; ++level) {
    for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0.f;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float x = ld_logit(p, i);
      if (!(x == x) || !survives(x, outer)) continue;
      float lo, w;
      if (path_cmp(x, *path, level, &lo, &w) != 0) continue;
      atomicAdd(&hist[bin_of(x, lo, 1.f / w)], kWeighted ? __expf((x - row_max) * inv_temp) : 1.f);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float run = *sh_above;
      int bin = 0;
      for (int b = 255; b >= 0; --b) {
        bin = b;
        if (run + hist[b] >= target || b == 0) break;  // b == 0 unmet: keep the whole range
        run += hist[b];
      }
      path->sel[level] = bin;
      path->levels = level + 1;
      *sh_above = run;
    }
    __syncthreads();
  }
}

template <typename T>
__global__ void __launch_bounds__(1024)
sample_rows_kernel(const T* __restrict__ logits, long long ld, int V, int rows, int* __restrict__ out_idx,
                   float* __restrict__ out_logprob, float temperature, int top_k, float top_p,
                   const float* __restrict__ row_params, unsigned long long seed, unsigned long long offset,
                   const unsigned long long* __restrict__ offset_dev, int index_offset) {
  __shared__ float hist[256];
  __shared__ ValIdx sm_vi[32];
  __shared__ float sm_f[32];
  __shared__ BinPath path_k, path_p;
  __shared__ float sh_above;
  const int row = blockIdx.x;
  if (row >= rows) return;
  const T* p = logits + (long long)row * ld;
  if (row_params) {
    temperature = row_params[3 * row];
    top_k = (int)row_params[3 * row + 1];
    top_p = row_params[3 * row + 2];
  }
  const int n_levels = sizeof(T) == 2 ? 3 : 4;
  if (threadIdx.x == 0) path_k.levels = path_p.levels = 0;

  // pass 1: greedy winner (= row maximum) and the smallest finite value
  ValIdx best{-FLT_MAX, 0x7fffffff};
  float mn = FLT_MAX;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = ld_logit(p, i);
    if (v == v) {
      best = better(best, ValIdx{v, i});
      if (v > -FLT_MAX) mn = fminf(mn, v);
    }
  }
  best = block_best(best, sm_vi);
  if (!(temperature > 0.f) || top_k == 1) {
    if (threadIdx.x == 0) {
      out_idx[row] = best.i + index_offset;
      if (out_logprob) out_logprob[row] = 0.f;
    }
    return;
  }
  mn = -block_best(ValIdx{-mn, 0}, sm_vi).v;
  const float inv_temp = 1.f / temperature, row_max = best.v;
  // values more than 1e4 below the maximum (masked logits) share the lowest bin
  const float row_lo = fmaxf(mn, row_max - 1.0e4f);

  if (top_k > 0 && top_k < V)
    find_threshold<T, false>(p, V, (float)top_k, row_max, row_lo, inv_temp, path_p /* empty */, n_levels, &path_k, hist, &sh_above);
  __syncthreads();
  float z = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float x = ld_logit(p, i);
    if (x == x && survives(x, path_k)) z += __expf((x - row_max) * inv_temp);
  }
  z = block_sum(z, sm_f);
  if (top_p > 0.f && top_p < 1.f) {
    __shared__ BinPath path_tmp;
    find_threshold<T, true>(p, V, top_p * z, row_max, row_lo, inv_temp, path_k, n_levels, &path_tmp, hist, &sh_above);
    if (threadIdx.x == 0) path_p = path_tmp;
    __syncthreads();
    float z2 = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float x = ld_logit(p, i);
      if (x == x && survives(x, path_k) && survives(x, path_p)) z2 += __expf((x - row_max) * inv_temp);
    }
    z = block_sum(z2, sm_f);
  }
  __syncthreads();

  // Gumbel-max over the survivors; 4 uniforms per Philox call, counter = element quad
  const unsigned long long off = offset + (offset_dev ? *offset_dev : 0ull);
  const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
  ValIdx pick{-FLT_MAX, 0x7fffffff};
  for (int q = threadIdx.x; q * 4 < V; q += blockDim.x) {
    const uint4 r = philox4x32(make_uint4((uint32_t)q, (uint32_t)row, (uint32_t)off, (uint32_t)(off >> 32)), key);
    const uint32_t bits[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = q * 4 + e;
      if (i >= V) break;
      const float x = ld_logit(p, i);
      if (!(x == x) || !survives(x, path_k) || !survives(x, path_p)) continue;
      pick = better(pick, ValIdx{(x - row_max) * inv_temp + gumbel(bits[e]), i});
    }
  }
  pick = block_best(pick, sm_vi);
  if (threadIdx.x == 0) {
    const int chosen = pick.i == 0x7fffffff ? best.i : pick.i;
    out_idx[row] = chosen + index_offset;
    if (out_logprob) out_logprob[row] = (ld_logit(p, chosen) - row_max) * inv_temp - __logf(z);
  }
}

}  // namespace nfn

using namespace nfn;

extern "C" int nfn_argmax_rows(const void* logits, int is_fp32, long long ld, int rows, int V, int* out_idx, float* out_val,
                               void* workspace, long long workspace_bytes, int index_offset, nfn_stream_t stream) {
  if (rows <= 0) return 0;
  if (!logits || !out_idx || V <= 0 || ld < V) return fail(-1, "argmax_rows: bad arguments");
  int splits = 1;
  if ((long long)rows * 32 < 2LL * sm_count()) splits = (int)std::min<long long>(64, std::max<long long>(1, (2LL * sm_count()) / rows));
  splits = max(1, min(splits, (V + 2047) / 2048));
  if (!workspace || workspace_bytes < (long long)rows * splits * (long long)sizeof(ValIdx)) {
    if (!workspace || workspace_bytes < (long long)rows * (long long)sizeof(ValIdx)) return fail(-1, "argmax_rows: workspace needs rows * 8 bytes at least (rows * 512 for full parallelism)");
    splits = (int)std::min<long long>(splits, workspace_bytes / ((long long)rows * (long long)sizeof(ValIdx)));
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(splits, rows);
  if (is_fp32) argmax_partial_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(logits), ld, V, static_cast<ValIdx*>(workspace));
  else argmax_partial_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), ld, V, static_cast<ValIdx*>(workspace));
  argmax_final_kernel<<<(rows + 7) / 8, 256, 0, st>>>(static_cast<const ValIdx*>(workspace), splits, rows, out_idx, out_val, index_offset);
  return launch_check("argmax_rows", 2);
}

extern "C" int nfn_argmax_merge(const float* vals, const int* idx, int world, int rows, int* out_idx, float* out_val,
                                nfn_stream_t stream) {
  if (rows <= 0) return 0;
  if (!vals || !idx || !out_idx || world <= 0) return fail(-1, "argmax_merge: bad arguments");
  argmax_merge_kernel<<<(rows + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(vals, idx, world, rows, out_idx, out_val);
  return launch_check("argmax_merge", 1);
}

extern "C" int nfn_sample_rows(const void* logits, int is_fp32, long long ld, int rows, int V, int* out_idx, float* out_logprob,
                               float temperature, int top_k, float top_p, const float* row_params, unsigned long long seed,
                               unsigned long long offset, const unsigned long long* offset_dev, int index_offset,
                               nfn_stream_t stream) {
  if (rows <= 0) return 0;
  if (!logits || !out_idx || V <= 0 || ld < V) return fail(-1, "sample_rows: bad arguments");
  if (top_p < 0.f || top_p > 1.f || top_k < 0) return fail(-1, "sample_rows: top_p must be in [0, 1] and top_k >= 0");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_fp32)
    sample_rows_kernel<float><<<rows, 1024, 0, st>>>(static_cast<const float*>(logits), ld, V, rows, out_idx, out_logprob, temperature,
                                                     top_k, top_p, row_params, seed, offset, offset_dev, index_offset);
  else
    sample_rows_kernel<__nv_bfloat16><<<rows, 1024, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), ld, V, rows, out_idx, out_logprob,
                                                             temperature, top_k, top_p, row_params, seed, offset, offset_dev, index_offset);
  return launch_check("sample_rows", 1);
}
