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

// ---- expert parallelism over peer memory --------------------------------------------------------
// Experts are split across `world` ranks (El = E / world each). Every rank routes its own
// tokens, sorts them by (global) expert into a symmetric send buffer and publishes its
// per-expert counts to all peers. From the full count table every rank derives, without
// any further communication, (a) where each (expert, source rank) segment sits in the
// owner's receive buffer and (b) where the rows it sent will be found again. Dispatch is a
// PULL: the owner copies the segments out of the peers' send buffers (plain 16-byte loads
// over NVLink). After the expert FFN (grouped GEMMs) the combine is a pull as well: each
// source reads its rows out of the owners' output buffers and applies the routing weights.
// Nothing is sent back explicitly and no rank writes another rank's memory except flags and
// the count table.
namespace nfn {

constexpr int EP_MAX_WORLD = 8;

struct EpPeers {
  const void* p[EP_MAX_WORLD];
};
struct EpPeersMut {
  int* p[EP_MAX_WORLD];
};

__device__ __forceinline__ void ep_st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ep_ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// counts[E] of this rank -> row `rank` of every rank's table [world][E]; then flag; then wait
// for every rank's row to arrive here. One block.
__global__ void moe_ep_exchange_counts_kernel(const int* __restrict__ counts, int E, EpPeersMut tables, EpPeersMut flags, int* my_flags,
                                              int rank, int world, int epoch, const int* epoch_dev, int* status) {
  const int ep = epoch + (epoch_dev ? *epoch_dev : 0);
  for (int r = 0; r < world; ++r)
    for (int e = threadIdx.x; e < E; e += blockDim.x) tables.p[r][rank * E + e] = counts[e];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) ep_st_release_sys(flags.p[threadIdx.x] + rank, ep);
  if (threadIdx.x < world) {
    const unsigned long long t0 = global_timer_ns();
    while (ep_ld_acquire_sys(my_flags + threadIdx.x) - ep < 0) {
      if (global_timer_ns() - t0 > 10ull * kWaitLimitNs) {
        if (status) atomicCAS(status, 0, NFN_ERR_WAIT_PEER);
        break;
      }
      __nanosleep(64);
    }
  }
}

// From the count table [world][E]:
//   src_off[e]            first row of expert e in THIS rank's send buffer (tight packing)
//   recv_off[le]          first row of local expert le in this rank's receive buffer (128-row padded)
//   seg_src_row[le*W+s]   first row of segment (le, s) inside rank s's send buffer
//   seg_dst_row[le*W+s]   first row of that segment in this rank's receive buffer
//   seg_rows[le*W+s]      rows of the segment
//   home_row[e]           where THIS rank's rows for expert e start in the owner's receive buffer
//   tile_expert / plan    as in moe_plan_kernel, for the local experts
__global__ void moe_ep_plan_kernel(const int* __restrict__ table, int E, int world, int rank, int max_tiles, int* __restrict__ src_off,
                                   int* __restrict__ cursor, int* __restrict__ recv_off, int* __restrict__ seg_src_row,
                                   int* __restrict__ seg_dst_row, int* __restrict__ seg_rows, int* __restrict__ home_row,
                                   int* __restrict__ tile_expert, int* __restrict__ plan) {
  if (threadIdx.x != 0) return;
  const int El = E / world;
  int run = 0;
  for (int e = 0; e < E; ++e) {
    src_off[e] = run;
    cursor[e] = 0;
    run += table[rank * E + e];
  }
  src_off[E] = run;
  for (int owner = 0; owner < world; ++owner) {
    int roff = 0;
    for (int le = 0; le < El; ++le) {
      const int e = owner * El + le;
      int tot = 0;
      for (int s = 0; s < world; ++s) {
        if (owner == rank) {
          int pre = 0;
          for (int e2 = 0; e2 < e; ++e2) pre += table[s * E + e2];
          seg_src_row[le * world + s] = pre;
          seg_dst_row[le * world + s] = roff + tot;
          seg_rows[le * world + s] = table[s * E + e];
        }
        if (s == rank) home_row[e] = roff + tot;
        tot += table[s * E + e];
      }
      if (owner == rank) {
        recv_off[le] = roff;
        for (int t = roff / MOE_TILE; t < (roff + (tot + MOE_TILE - 1) / MOE_TILE * MOE_TILE) / MOE_TILE && t < max_tiles; ++t) tile_expert[t] = le;
      }
      roff += (tot + MOE_TILE - 1) / MOE_TILE * MOE_TILE;
    }
    if (owner == rank) {
      recv_off[El] = roff;
      plan[0] = min(roff / MOE_TILE, max_tiles);
      plan[1] = roff;
    }
  }
}

// grid (segments, row chunks): copies segment rows from the source rank's send buffer
__global__ void __launch_bounds__(256)
moe_ep_pull_kernel(EpPeers send_bufs, const int* __restrict__ seg_src_row, const int* __restrict__ seg_dst_row, const int* __restrict__ seg_rows,
                   int world, int d, int capacity_rows, __nv_bfloat16* __restrict__ xs) {
  const int seg = blockIdx.x, s = seg % world;
  const int rows = seg_rows[seg];
  const long long src0 = seg_src_row[seg], dst0 = seg_dst_row[seg];
  const int vecs = d / 8;
  const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(send_bufs.p[s]) + src0 * d);
  uint4* dst = reinterpret_cast<uint4*>(xs + dst0 * d);
  const long long total = (long long)rows * vecs;
  for (long long i = (long long)blockIdx.y * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.y * blockDim.x) {
    if (dst0 + i / vecs >= capacity_rows) break;
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src + i) : "memory");
    dst[i] = v;
  }
}

__global__ void __launch_bounds__(256)
moe_ep_combine_kernel(EpPeers ys_bufs, int d, int T, int k, int E, int world, const int* __restrict__ topk_idx, const int* __restrict__ row_of,
                      const int* __restrict__ src_off, const int* __restrict__ home_row, const float* __restrict__ topk_w,
                      const __nv_bfloat16* __restrict__ resid, int ld_resid, __nv_bfloat16* __restrict__ out, int ld_out) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int vecs = d / 8, El = E / world;
  if (idx >= (long long)T * vecs) return;
  const int tok = (int)(idx / vecs), c = (int)(idx % vecs) * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < k; ++j) {
    const long long item = (long long)tok * k + j;
    const int e = topk_idx[item], local_row = row_of[item];
    if (local_row < 0) continue;
    const long long row = (long long)home_row[e] + (local_row - src_off[e]);
    const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(ys_bufs.p[e / El]);
    uint4 u;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(base + row * d + c) : "memory");
    const float w = topk_w[item];
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

// tables[r] / flags[r]: rank r's count table [world][E] and flag array [world] (symmetric memory).
extern "C" int nfn_moe_ep_exchange_counts(const int* counts, int E, int* const* tables, int* const* flags, int rank, int world, int epoch,
                                          const int* epoch_dev, nfn_stream_t stream) {
  using namespace nfn;
  if (!counts || !tables || !flags || E <= 0 || E > MOE_MAX_E || world < 1 || world > EP_MAX_WORLD || rank < 0 || rank >= world || E % world)
    return fail(-1, "moe_ep_exchange_counts: bad arguments (E must be a multiple of world <= 8)");
  EpPeersMut t{}, f{};
  for (int r = 0; r < world; ++r) {
    if (!tables[r] || !flags[r]) return fail(-1, "moe_ep_exchange_counts: missing peer pointer");
    t.p[r] = tables[r];
    f.p[r] = flags[r];
  }
  moe_ep_exchange_counts_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(counts, E, t, f, flags[rank], rank, world, epoch, epoch_dev, status_ptr());
  return launch_check("moe_ep_exchange_counts", 1);
}

// Sizes: src_off E+1, cursor E, recv_off E/world+1, seg_* (E/world)*world, home_row E, tile_expert max_tiles, plan 2.
extern "C" int nfn_moe_ep_plan(const int* table, int E, int world, int rank, int max_tiles, int* src_off, int* cursor, int* recv_off,
                               int* seg_src_row, int* seg_dst_row, int* seg_rows, int* home_row, int* tile_expert, int* plan,
                               nfn_stream_t stream) {
  using namespace nfn;
  if (!table || !src_off || !cursor || !recv_off || !seg_src_row || !seg_dst_row || !seg_rows || !home_row || !tile_expert || !plan ||
      E <= 0 || E > MOE_MAX_E || world < 1 || world > EP_MAX_WORLD || E % world || max_tiles <= 0)
    return fail(-1, "moe_ep_plan: bad arguments");
  moe_ep_plan_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(table, E, world, rank, max_tiles, src_off, cursor, recv_off, seg_src_row,
                                                                      seg_dst_row, seg_rows, home_row, tile_expert, plan);
  return launch_check("moe_ep_plan", 1);
}

extern "C" int nfn_moe_ep_pull(const void* const* send_bufs, const int* seg_src_row, const int* seg_dst_row, const int* seg_rows,
                               int n_local_experts, int world, int d, int capacity_rows, void* xs, nfn_stream_t stream) {
  using namespace nfn;
  if (!send_bufs || !seg_src_row || !seg_dst_row || !seg_rows || !xs || (d & 7) || world < 1 || world > EP_MAX_WORLD || n_local_experts <= 0)
    return fail(-1, "moe_ep_pull: bad arguments");
  EpPeers s{};
  for (int r = 0; r < world; ++r) {
    if (!send_bufs[r]) return fail(-1, "moe_ep_pull: missing peer pointer");
    s.p[r] = send_bufs[r];
  }
  const dim3 grid(n_local_experts * world, 16);
  moe_ep_pull_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(s, seg_src_row, seg_dst_row, seg_rows, world, d, capacity_rows,
                                                                         static_cast<__nv_bfloat16*>(xs));
  return launch_check("moe_ep_pull", 1);
}

extern "C" int nfn_moe_ep_combine(const void* const* ys_bufs, int d, int T, int k, int E, int world, const int* topk_idx, const int* row_of,
                                  const int* src_off, const int* home_row, const float* topk_w, const void* resid, int ld_resid, void* out,
                                  int ld_out, nfn_stream_t stream) {
  using namespace nfn;
  if (T <= 0) return 0;
  if (!ys_bufs || !topk_idx || !row_of || !src_off || !home_row || !topk_w || !out || (d & 7) || (ld_out & 7) || world < 1 || world > EP_MAX_WORLD || E % world)
    return fail(-1, "moe_ep_combine: bad arguments");
  EpPeers y{};
  for (int r = 0; r < world; ++r) {
    if (!ys_bufs[r]) return fail(-1, "moe_ep_combine: missing peer pointer");
    y.p[r] = ys_bufs[r];
  }
  const long long total = (long long)T * (d / 8), grid = (total + 255) / 256;
  if (grid > 0x7fffffffLL) return fail(-1, "moe_ep_combine: too large for one launch");
  moe_ep_combine_kernel<<<(unsigned)grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      y, d, T, k, E, world, topk_idx, row_of, src_off, home_row, topk_w, static_cast<const __nv_bfloat16*>(resid), ld_resid,
      static_cast<__nv_bfloat16*>(out), ld_out);
  return launch_check("moe_ep_combine", 1);
}

// ------------------------------------------------------------------------------------------------
// Training side of the expert-parallel exchange. The backward pass sends the upstream gradient of
// every (token, slot) to the owner of its expert along the route of the forward pass, so the rows
// have to land where the forward pass put them: the sources scatter by the saved `row_of` instead of
// claiming rows again. Per-row scalars travel both ways too: the routing weight to the owner (it
// scales the row gradients that feed the expert weight gradients) and <upstream, expert output>
// back to the source (the gradient of the routing weight).
namespace nfn {

// one warp per (token, slot): send[row_of[item]] = src[token]
__global__ void __launch_bounds__(256)
moe_scatter_rows_kernel(const __nv_bfloat16* __restrict__ src, int ld, int T, int k, int d, const int* __restrict__ row_of, int capacity_rows,
                        __nv_bfloat16* __restrict__ send) {
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= (long long)T * k) return;
  const int row = row_of[item];
  if (row < 0 || row >= capacity_rows) return;
  const uint4* s = reinterpret_cast<const uint4*>(src + (item / k) * ld);
  uint4* o = reinterpret_cast<uint4*>(send + (long long)row * d);
  for (int i = lane; i < d / 8; i += 32) o[i] = s[i];
}

// grid (segments): copies each segment's fp32 scalars from the source rank's buffer
__global__ void __launch_bounds__(256)
moe_ep_pull_f32_kernel(EpPeers send_bufs, const int* __restrict__ seg_src_row, const int* __restrict__ seg_dst_row, const int* __restrict__ seg_rows,
                       int world, int capacity_rows, float* __restrict__ out) {
  const int seg = blockIdx.x, s = seg % world;
  const int rows = seg_rows[seg];
  const long long src0 = seg_src_row[seg], dst0 = seg_dst_row[seg];
  const float* src = static_cast<const float*>(send_bufs.p[s]) + src0;
  for (int i = threadIdx.x; i < rows && dst0 + i < capacity_rows; i += blockDim.x) {
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(src + i) : "memory");
    out[dst0 + i] = v;
  }
}

// one thread per (token, slot): reads the scalar of its row from the owner's buffer
__global__ void __launch_bounds__(256)
moe_ep_gather_f32_kernel(EpPeers bufs, int T, int k, int E, int world, const int* __restrict__ topk_idx, const int* __restrict__ row_of,
                         const int* __restrict__ src_off, const int* __restrict__ home_row, float* __restrict__ out) {
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= (long long)T * k) return;
  const int e = topk_idx[item], local_row = row_of[item], El = E / world;
  float v = 0.f;
  if (local_row >= 0 && e >= 0 && e < E) {
    const float* p = static_cast<const float*>(bufs.p[e / El]) + (long long)home_row[e] + (local_row - src_off[e]);
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  }
  out[item] = v;
}

}  // namespace nfn

// send[row_of[t * k + j]] = src[t] for every (token, slot); rows of `send` are d wide.
extern "C" int nfn_moe_scatter_rows(const void* src, int ld, int T, int k, int d, const int* row_of, int capacity_rows, void* send,
                                    nfn_stream_t stream) {
  using namespace nfn;
  if (T <= 0) return 0;
  if (!src || !row_of || !send || (d & 7) || (ld & 7) || k <= 0 || capacity_rows <= 0) return fail(-1, "moe_scatter_rows: bad arguments");
  const long long items = (long long)T * k, grid = (items + 7) / 8;
  if (grid > 0x7fffffffLL) return fail(-1, "moe_scatter_rows: too large for one launch");
  moe_scatter_rows_kernel<<<(unsigned)grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(src), ld, T, k, d, row_of,
                                                                                         capacity_rows, static_cast<__nv_bfloat16*>(send));
  return launch_check("moe_scatter_rows", 1);
}

// The fp32 counterpart of nfn_moe_ep_pull for one scalar per row (same segment tables).
extern "C" int nfn_moe_ep_pull_f32(const void* const* send_bufs, const int* seg_src_row, const int* seg_dst_row, const int* seg_rows,
                                   int n_local_experts, int world, int capacity_rows, float* out, nfn_stream_t stream) {
  using namespace nfn;
  if (!send_bufs || !seg_src_row || !seg_dst_row || !seg_rows || !out || world < 1 || world > EP_MAX_WORLD || n_local_experts <= 0)
    return fail(-1, "moe_ep_pull_f32: bad arguments");
  EpPeers s{};
  for (int r = 0; r < world; ++r) {
    if (!send_bufs[r]) return fail(-1, "moe_ep_pull_f32: missing peer pointer");
    s.p[r] = send_bufs[r];
  }
  moe_ep_pull_f32_kernel<<<n_local_experts * world, 256, 0, static_cast<cudaStream_t>(stream)>>>(s, seg_src_row, seg_dst_row, seg_rows, world,
                                                                                                 capacity_rows, out);
  return launch_check("moe_ep_pull_f32", 1);
}

// out[t * k + j] = the owner's scalar of the row that (token t, slot j) was sent to.
extern "C" int nfn_moe_ep_gather_f32(const void* const* bufs, int T, int k, int E, int world, const int* topk_idx, const int* row_of,
                                     const int* src_off, const int* home_row, float* out, nfn_stream_t stream) {
  using namespace nfn;
  if (T <= 0) return 0;
  if (!bufs || !topk_idx || !row_of || !src_off || !home_row || !out || world < 1 || world > EP_MAX_WORLD || E <= 0 || E % world)
    return fail(-1, "moe_ep_gather_f32: bad arguments");
  EpPeers b{};
  for (int r = 0; r < world; ++r) {
    if (!bufs[r]) return fail(-1, "moe_ep_gather_f32: missing peer pointer");
    b.p[r] = bufs[r];
  }
  const long long items = (long long)T * k, grid = (items + 255) / 256;
  if (grid > 0x7fffffffLL) return fail(-1, "moe_ep_gather_f32: too large for one launch");
  moe_ep_gather_f32_kernel<<<(unsigned)grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(b, T, k, E, world, topk_idx, row_of, src_off, home_row, out);
  return launch_check("moe_ep_gather_f32", 1);
}
