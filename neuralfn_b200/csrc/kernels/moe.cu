// Mixture-of-experts routing around the grouped tcgen05 GEMM (NFN_TP_GROUPED):
//
//   route    router logits [T, E] (fp32) -> softmax (or sigmoid) scores -> top-k experts and
//            weights per token, per-expert token counts (one warp per token, E <= 256, k <= 8);
//   plan     counts -> 128-row-padded expert offsets, the tile -> expert table and the live
//            tile count the grouped GEMM reads from device memory (no host round trip);
//   permute  token rows -> expert-sorted, tile-padded buffer; remembers where each
//            (token, slot) went;
//   combine  out[token] = sum_slot weight * expert_out[row(token, slot)] (+ residual).
//
// Everything stays on the device and on one stream: route -> plan -> permute -> grouped GEMM
// (gate|up) -> SwiGLU -> grouped GEMM (down) -> combine.
// Reference kernels: kernels.cu:12612-12862 (top-k routing, permute), 15028-15072, 22194-22237.
#include <cfloat>

#include "common.h"
#include "nfn_kernels.h"
#include "sm100_ptx.cuh"

namespace nfn {

constexpr int MOE_MAX_E = 256, MOE_MAX_K = 8, MOE_TILE = 128;

__global__ void __launch_bounds__(256)
moe_route_kernel(const float* __restrict__ logits, int ld, int T, int E, int k, int score_fn, int norm_topk, float route_scale,
                 int* __restrict__ topk_idx, float* __restrict__ topk_w, int* __restrict__ counts) {
  const int tok = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (tok >= T) return;
  constexpr int PER = MOE_MAX_E / 32;
  float v[PER];
  float mx = -FLT_MAX;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < E ? logits[(long long)tok * ld + e] : -FLT_MAX;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = i * 32 + lane;
    if (e < E) {
      v[i] = score_fn == 1 ? 1.f / (1.f + __expf(-v[i])) : __expf(v[i] - mx);
      sum += v[i];
    } else {
      v[i] = -1.f;  // scores are >= 0: never selected
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = score_fn == 1 ? 1.f : 1.f / sum;
  float wsel[MOE_MAX_K];
  int isel[MOE_MAX_K];
  float wsum = 0.f;
  for (int j = 0; j < k; ++j) {
    float best = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = i * 32 + lane;
      if (v[i] > best) { best = v[i]; bi = e; }  // lowest index wins ties within a lane
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    wsel[j] = best * inv;
    isel[j] = bi;
    wsum += wsel[j];
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if (i * 32 + lane == bi) v[i] = -1.f;
  }
  if (lane == 0) {
    const float norm = (norm_topk && wsum > 0.f) ? route_scale / wsum : route_scale;
    for (int j = 0; j < k; ++j) {
      topk_idx[(long long)tok * k + j] = isel[j];
      topk_w[(long long)tok * k + j] = wsel[j] * norm;
      atomicAdd(&counts[isel[j]], 1);
    }
  }
}

// plan[0] = live m tiles, plan[1] = padded rows; offsets[e] = first row of expert e
__global__ void moe_plan_kernel(const int* __restrict__ counts, int E, int max_tiles, int* __restrict__ offsets, int* __restrict__ cursor,
                                int* __restrict__ tile_expert, int* __restrict__ plan) {
  __shared__ int sh_off[MOE_MAX_E + 1];
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      sh_off[e] = run;
      run += (counts[e] + MOE_TILE - 1) / MOE_TILE * MOE_TILE;
    }
    sh_off[E] = run;
    plan[0] = min(run / MOE_TILE, max_tiles);
    plan[1] = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    offsets[e] = sh_off[e];
    cursor[e] = 0;
    for (int t = sh_off[e] / MOE_TILE; t < sh_off[e + 1] / MOE_TILE && t < max_tiles; ++t) tile_expert[t] = e;
  }
  if (threadIdx.x == 0) offsets[E] = sh_off[E];
}

// one warp per (token, slot): claims a row of its expert and copies the token's features there
__global__ void __launch_bounds__(256)
moe_permute_kernel(const __nv_bfloat16* __restrict__ x, int ldx, int T, int k, int d, const int* __restrict__ topk_idx,
                   const int* __restrict__ offsets, int* __restrict__ cursor, int capacity_rows, __nv_bfloat16* __restrict__ xs,
                   int* __restrict__ row_of) {
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= (long long)T * k) return;
  const int tok = (int)(item / k);
  int row = 0;
  if (lane == 0) {
    const int e = topk_idx[item];
    row = offsets[e] + atomicAdd(&cursor[e], 1);
    if (row >= capacity_rows) row = -1;  // cannot happen with a worst-case buffer; dropped if it does
    row_of[item] = row;
  }
  row = __shfl_sync(0xffffffffu, row, 0);
  if (row < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)tok * ldx);
  uint4* dst = reinterpret_cast<uint4*>(xs + (long long)row * d);
  for (int i = lane; i < d / 8; i += 32) dst[i] = src[i];
}

__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ ys, int d, int T, int k, const int* __restrict__ row_of,
                   const float* __restrict__ topk_w, const __nv_bfloat16* __restrict__ resid, int ld_resid,
                   __nv_bfloat16* __restrict__ out, int ld_out) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int vecs = d / 8;
  if (idx >= (long long)T * vecs) return;
  const int tok = (int)(idx / vecs), c = (int)(idx % vecs) * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < k; ++j) {
    const int row = row_of[(long long)tok * k + j];
    if (row < 0) continue;
    const float w = topk_w[(long long)tok * k + j];
    const uint4 u = *reinterpret_cast<const uint4*>(ys + (long long)row * d + c);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), dd = unpack_bf16x2(u.w);
    acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * b.x; acc[3] += w * b.y;
    acc[4] += w * cc.x; acc[5] += w * cc.y; acc[6] += w * dd.x; acc[7] += w * dd.y;
  }
  if (resid) {
    const uint4 u = *reinterpret_cast<const uint4*>(resid + (long long)tok * ld_resid + c);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), dd = unpack_bf16x2(u.w);
    acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += cc.x; acc[5] += cc.y; acc[6] += dd.x; acc[7] += dd.y;
  }
  uint4 o;
  o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]); o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
  *reinterpret_cast<uint4*>(out + (long long)tok * ld_out + c) = o;
}

}  // namespace nfn

using namespace nfn;

// score_fn: 0 softmax, 1 sigmoid. counts must be zero on entry (nfn_moe_plan consumes them; zero
// them again before the next route call, e.g. with cudaMemsetAsync).
extern "C" int nfn_moe_route(const float* logits, int ld, int T, int E, int k, int score_fn, int norm_topk, float route_scale,
                             int* topk_idx, float* topk_w, int* counts, nfn_stream_t stream) {
  if (T <= 0) return 0;
  if (!logits || !topk_idx || !topk_w || !counts) return fail(-1, "moe_route: null operand");
  if (E <= 0 || E > MOE_MAX_E || k <= 0 || k > MOE_MAX_K || k > E || ld < E) return fail(-1, "moe_route: need 1 <= k <= 8, k <= E <= 256, ld >= E");
  moe_route_kernel<<<(T + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(logits, ld, T, E, k, score_fn, norm_topk, route_scale, topk_idx,
                                                                               topk_w, counts);
  return launch_check("moe_route", 1);
}

// offsets: E + 1 ints, cursor: E ints, tile_expert: max_tiles ints, plan: 2 ints.
extern "C" int nfn_moe_plan(const int* counts, int E, int max_tiles, int* offsets, int* cursor, int* tile_expert, int* plan,
                            nfn_stream_t stream) {
  if (!counts || !offsets || !cursor || !tile_expert || !plan || E <= 0 || E > MOE_MAX_E || max_tiles <= 0) return fail(-1, "moe_plan: bad arguments");
  moe_plan_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(counts, E, max_tiles, offsets, cursor, tile_expert, plan);
  return launch_check("moe_plan", 1);
}

extern "C" int nfn_moe_permute(const void* x, int ldx, int T, int k, int d, const int* topk_idx, const int* offsets, int* cursor,
                               int capacity_rows, void* xs, int* row_of, nfn_stream_t stream) {
  if (T <= 0) return 0;
  if (!x || !topk_idx || !offsets || !cursor || !xs || !row_of || (d & 7) || (ldx & 7) || ldx < d || capacity_rows <= 0) return fail(-1, "moe_permute: bad arguments");
  const long long items = (long long)T * k, grid = (items + 7) / 8;
  if (grid > 0x7fffffffLL) return fail(-1, "moe_permute: too many rows for one launch");
  moe_permute_kernel<<<(unsigned)grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, T, k, d, topk_idx, offsets, cursor, capacity_rows, static_cast<__nv_bfloat16*>(xs), row_of);
  return launch_check("moe_permute", 1);
}

extern "C" int nfn_moe_combine(const void* ys, int d, int T, int k, const int* row_of, const float* topk_w, const void* resid,
                               int ld_resid, void* out, int ld_out, nfn_stream_t stream) {
  if (T <= 0) return 0;
  if (!ys || !row_of || !topk_w || !out || (d & 7) || (ld_out & 7) || (resid && (ld_resid & 7))) return fail(-1, "moe_combine: bad arguments");
  const long long total = (long long)T * (d / 8), grid = (total + 255) / 256;
  if (grid > 0x7fffffffLL) return fail(-1, "moe_combine: too large for one launch");
  moe_combine_kernel<<<(unsigned)grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(ys), d, T, k, row_of, topk_w, static_cast<const __nv_bfloat16*>(resid), ld_resid,
      static_cast<__nv_bfloat16*>(out), ld_out);
  return launch_check("moe_combine", 1);
}
