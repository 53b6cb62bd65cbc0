// Single-token (decode) attention over a bf16 KV cache, split along the context so that a
// batch of a few dozen sequences still fills 148 SMs. The step is bound by reading K and V
// once; everything else is fused around that read:
//
//   * prologue: per-head RMS norm of the new q and k (optional weights), rotary embedding
//     at position len-1, query scaling - straight from the packed QKV row of the new token;
//   * cache append: the new k/v row is written to its slot by exactly one CTA, while every
//     CTA treats that row as a register-resident extra position, so no CTA waits on another;
//   * hybrid cache: `cap` is either the full context (global layers) or the window size of
//     a ring buffer (local layers): slot = position % cap, and once the ring is full every
//     slot is live (softmax does not care about order);
//   * grouped-query attention: one CTA serves up to four query heads of one KV head, so K
//     and V rows are read once per group;
//   * combine: partial (max, sum, output) per split go to a workspace; the last CTA to
//     finish a (sequence, head group) - found with a self-resetting ticket - merges them
//     and writes the bf16 output. One launch, no second kernel.
//
// Thread mapping: 128 threads = 16 sub-groups of 8 lanes; a sub-group owns one cache
// position at a time, each lane two contiguous chunks of head_dim/16 elements (one in each
// rotary half, so a rotation pair lives in one lane). Dot products reduce over 8 lanes.
//
// Behavioural counterpart in the reference: kernels.cu:2475-2880 (decode attention with
// local ring / global caches and fused QK-norm + RoPE + append).
#include <algorithm>
#include <cfloat>

#include "common.h"
#include "nfn_kernels.h"
#include "sm100_ptx.cuh"

namespace nfn {

struct DecodeParams {
  const __nv_bfloat16* qkv;
  int ld;
  __nv_bfloat16* kc;
  __nv_bfloat16* vc;
  long long batch_stride;  // elements between sequences in the cache
  const int* lengths;
  __nv_bfloat16* out;
  int B, Hq, Hkv, cap, splits, gtiles;
  const __nv_bfloat16* qw;
  const __nv_bfloat16* kw;
  int qk_norm;
  float eps;
  const float* cosT;
  const float* sinT;
  int max_pos;
  float sign, scale;
  int* tickets;
  float* part_ml;
  float* part_o;
  int* status;
};

constexpr int DEC_TILE = 32;    // cache positions per shared-memory stage
constexpr int DEC_STAGES = 4;   // stages in flight per CTA

__device__ __forceinline__ void dec_bulk_g2s(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar)
               : "memory");
}

template <int HD, int G>
constexpr size_t decode_smem_bytes() {
  const size_t ring = (size_t)DEC_STAGES * 2 * DEC_TILE * HD * 2, merge = (size_t)16 * G * (HD + 2) * sizeof(float);
  return ring > merge ? ring : merge;
}

template <int CH>
__device__ __forceinline__ void load_chunk(const __nv_bfloat16* p, float* dst) {
  if constexpr (CH == 8) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = unpack_bf16x2(w[i]);
      dst[2 * i] = f.x;
      dst[2 * i + 1] = f.y;
    }
  } else {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
    dst[0] = a.x; dst[1] = a.y; dst[2] = b.x; dst[3] = b.y;
  }
}
template <int CH>
__device__ __forceinline__ void store_chunk(__nv_bfloat16* p, const float* src) {
  if constexpr (CH == 8) {
    uint4 u;
    u.x = pack_bf16x2(src[0], src[1]); u.y = pack_bf16x2(src[2], src[3]);
    u.z = pack_bf16x2(src[4], src[5]); u.w = pack_bf16x2(src[6], src[7]);
    *reinterpret_cast<uint4*>(p) = u;
  } else {
    uint2 u;
    u.x = pack_bf16x2(src[0], src[1]); u.y = pack_bf16x2(src[2], src[3]);
    *reinterpret_cast<uint2*>(p) = u;
  }
}
__device__ __forceinline__ float sum8(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  return x;
}

// loads one head vector in the lane layout, applies norm (+weights), rotation and scale
template <int HD>
__device__ __forceinline__ void load_head(const __nv_bfloat16* src, const __nv_bfloat16* w, bool norm, float eps, const float* cosr,
                                          const float* sinr, float sign, float scale, int sub, float* v /* HD/8 */) {
  constexpr int CH = HD / 16, HALF = HD / 2;
  load_chunk<CH>(src + sub * CH, v);
  load_chunk<CH>(src + HALF + sub * CH, v + CH);
  if (norm) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 2 * CH; ++i) ss += v[i] * v[i];
    ss = sum8(ss);
    const float r = rsqrtf(ss / (float)HD + eps);
    float wv[2 * CH];
    if (w) {
      load_chunk<CH>(w + sub * CH, wv);
      load_chunk<CH>(w + HALF + sub * CH, wv + CH);
    }
#pragma unroll
    for (int i = 0; i < 2 * CH; ++i) v[i] *= w ? r * wv[i] : r;
  }
  if (sign != 0.f) {
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const float c = cosr[sub * CH + i], s = sinr[sub * CH + i], lo = v[i], hi = v[CH + i];
      v[i] = lo * c - sign * hi * s;
      v[CH + i] = hi * c + sign * lo * s;
    }
  }
#pragma unroll
  for (int i = 0; i < 2 * CH; ++i) v[i] *= scale;
}

template <int HD, int G>
__global__ void __launch_bounds__(128)
decode_attention_kernel(const DecodeParams p) {
  constexpr int CH = HD / 16, EPL = HD / 8, HALF = HD / 2, NGRP = 16;
  extern __shared__ __align__(128) float smem[];  // stage ring, later [NGRP][G][HD] acc + [NGRP][G][2] (m, l)
  float* sm_acc = smem;
  float* sm_ml = smem + NGRP * G * HD;
  __shared__ int sh_last;
  __shared__ int sh_abort_store;
  __shared__ __align__(8) uint64_t sh_full[DEC_STAGES];
  volatile int* sh_abort_ptr = &sh_abort_store;

  const int split = blockIdx.x, b = blockIdx.z;
  const int kvh = blockIdx.y / p.gtiles, gt = blockIdx.y % p.gtiles;
  const int group = p.Hq / p.Hkv;          // query heads per kv head
  const int g0 = gt * G;                   // first query head (within the group) of this CTA
  const int gcount = min(G, group - g0);
  const int grp = threadIdx.x >> 3, sub = threadIdx.x & 7;

  const int len = p.lengths[b];
  if (len <= 0) return;  // uniform per CTA: empty sequence slot, nothing to do and no ticket needed
  if (threadIdx.x == 0) {
    sh_abort_store = 0;
    for (int s = 0; s < DEC_STAGES; ++s) mbar_init(smem_u32(&sh_full[s]), 1);
    fence_mbar_init();
  }
  __syncthreads();
  const int pos = len - 1;
  const int slot_new = pos % p.cap;
  const int n_slots = min(len, p.cap);
  const int tpos = min(pos, p.max_pos - 1);
  const float* cosr = p.cosT ? p.cosT + (long long)tpos * HALF : nullptr;
  const float* sinr = p.sinT ? p.sinT + (long long)tpos * HALF : nullptr;
  const float sign = cosr ? p.sign : 0.f;

  const __nv_bfloat16* row = p.qkv + (long long)b * p.ld;
  float q[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (g < gcount)
      load_head<HD>(row + (long long)(kvh * group + g0 + g) * HD, p.qw, p.qk_norm, p.eps, cosr, sinr, sign, p.scale, sub, q[g]);
    else
#pragma unroll
      for (int i = 0; i < EPL; ++i) q[g][i] = 0.f;
  }

  float m[G], l[G], acc[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -FLT_MAX;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) acc[g][i] = 0.f;
  }

  // Every lane of the warp calls this together (the reductions use full-warp shuffles);
  // `valid` says whether this sub-group's position counts.
  auto absorb = [&](const float* kv, const float* vv, bool valid) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) d += q[g][i] * kv[i];
      d = sum8(d);
      if (!valid) continue;
      const float mn = fmaxf(m[g], d);
      const float corr = __expf(m[g] - mn), w = __expf(d - mn);
      l[g] = l[g] * corr + w;
#pragma unroll
      for (int i = 0; i < EPL; ++i) acc[g][i] = acc[g][i] * corr + w * vv[i];
      m[g] = mn;
    }
  };

  __nv_bfloat16* kbase = p.kc + (long long)b * p.batch_stride + (long long)kvh * p.cap * HD;
  __nv_bfloat16* vbase = p.vc + (long long)b * p.batch_stride + (long long)kvh * p.cap * HD;

  // the new token: from registers, by sub-group 0 of split 0; that sub-group of query tile 0
  // also appends it to the cache
  if (split == 0 && threadIdx.x < 32) {  // whole warp 0: its four sub-groups compute the same row
    float kn[EPL], vn[EPL];
    load_head<HD>(row + (long long)(p.Hq + kvh) * HD, p.kw, p.qk_norm, p.eps, cosr, sinr, sign, 1.f, sub, kn);
    const __nv_bfloat16* vsrc = row + (long long)(p.Hq + p.Hkv + kvh) * HD;
    load_chunk<CH>(vsrc + sub * CH, vn);
    load_chunk<CH>(vsrc + HALF + sub * CH, vn + CH);
    if (gt == 0 && grp == 0) {
      store_chunk<CH>(kbase + (long long)slot_new * HD + sub * CH, kn);
      store_chunk<CH>(kbase + (long long)slot_new * HD + HALF + sub * CH, kn + CH);
      store_chunk<CH>(vbase + (long long)slot_new * HD + sub * CH, vn);
      store_chunk<CH>(vbase + (long long)slot_new * HD + HALF + sub * CH, vn + CH);
    }
    // attend to the values the cache will hold (bf16-rounded), as later steps will see them
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      kn[i] = __bfloat162float(__float2bfloat16(kn[i]));
      vn[i] = __bfloat162float(__float2bfloat16(vn[i]));
    }
    absorb(kn, vn, grp == 0);
  }

  // The cache rows of this split stream through a ring of shared-memory stages filled by
  // bulk async copies (a tile of DEC_TILE positions of one head is one contiguous run of
  // the cache), several tiles ahead of the arithmetic: enough bytes in flight per SM to
  // cover HBM latency, which per-thread loads at this register budget cannot provide.
  const int per = (n_slots + p.splits - 1) / p.splits;
  const int s_lo = split * per, s_hi = min(n_slots, s_lo + per);
  const int ntiles = s_hi > s_lo ? (s_hi - s_lo + DEC_TILE - 1) / DEC_TILE : 0;
  constexpr uint32_t ROW = HD * 2, STAGE = 2 * DEC_TILE * ROW;  // K tile then V tile
  uint8_t* stage_base = reinterpret_cast<uint8_t*>(smem);
  auto issue = [&](int t) {  // thread 0 only
    const int st = t % DEC_STAGES;
    const int s0 = s_lo + t * DEC_TILE, n = min(DEC_TILE, s_hi - s0);
    const uint32_t bytes = (uint32_t)n * ROW, bar = smem_u32(&sh_full[st]);
    mbar_expect_tx(bar, 2 * bytes);
    dec_bulk_g2s(smem_u32(stage_base + st * STAGE), kbase + (long long)s0 * HD, bytes, bar);
    dec_bulk_g2s(smem_u32(stage_base + st * STAGE + DEC_TILE * ROW), vbase + (long long)s0 * HD, bytes, bar);
  };
  if (threadIdx.x == 0)
    for (int t = 0; t < min(DEC_STAGES, ntiles); ++t) issue(t);
  bool alive = true;
  for (int t = 0; t < ntiles; ++t) {
    const int st = t % DEC_STAGES;
    alive = mbar_wait_bounded(smem_u32(&sh_full[st]), (t / DEC_STAGES) & 1, sh_abort_ptr, p.status, NFN_ERR_WAIT_FULL);
    alive = __syncthreads_and(alive);
    if (!alive) break;
    const int s0 = s_lo + t * DEC_TILE;
    const uint8_t* kt = stage_base + st * STAGE;
    const uint8_t* vt = kt + DEC_TILE * ROW;
#pragma unroll
    for (int r = 0; r < DEC_TILE / NGRP; ++r) {  // trip count is the same for every thread
      const int row = r * NGRP + grp, s = s0 + row;
      const bool valid = s < s_hi && s != slot_new;
      float kv[EPL], vv[EPL];
      const __nv_bfloat16* kr = reinterpret_cast<const __nv_bfloat16*>(kt + row * ROW);
      const __nv_bfloat16* vr = reinterpret_cast<const __nv_bfloat16*>(vt + row * ROW);
      load_chunk<CH>(kr + sub * CH, kv);  // rows past the tile's end hold stale data: masked by `valid`
      load_chunk<CH>(kr + HALF + sub * CH, kv + CH);
      load_chunk<CH>(vr + sub * CH, vv);
      load_chunk<CH>(vr + HALF + sub * CH, vv + CH);
      absorb(kv, vv, valid);
    }
    __syncthreads();  // everyone is done with this stage
    if (threadIdx.x == 0 && t + DEC_STAGES < ntiles) issue(t + DEC_STAGES);
  }
  if (!alive) {
    // a copy never arrived: leave without touching the workspace; give copies still in
    // flight time to land before this CTA's shared memory is handed to another CTA
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    return;
  }
  __syncthreads();  // the stage ring is reused below as the merge buffer

  // ---- merge the 16 sub-groups of this CTA -------------------------------------------------
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      sm_acc[(grp * G + g) * HD + sub * CH + i] = acc[g][i];
      sm_acc[(grp * G + g) * HD + HALF + sub * CH + i] = acc[g][CH + i];
    }
    if (sub == 0) {
      sm_ml[(grp * G + g) * 2] = m[g];
      sm_ml[(grp * G + g) * 2 + 1] = l[g];
    }
  }
  __syncthreads();
  const long long unit = ((long long)b * p.Hkv + kvh) * p.gtiles + gt;
  float* po = p.part_o + (unit * p.splits + split) * (long long)(G * HD);
  float* pml = p.part_ml + (unit * p.splits + split) * (long long)(G * 2);
  for (int e = threadIdx.x; e < G * HD; e += blockDim.x) {
    const int g = e / HD, d = e % HD;
    float mx = -FLT_MAX;
#pragma unroll
    for (int r = 0; r < NGRP; ++r) mx = fmaxf(mx, sm_ml[(r * G + g) * 2]);
    float o = 0.f, ls = 0.f;
#pragma unroll
    for (int r = 0; r < NGRP; ++r) {
      const float w = __expf(sm_ml[(r * G + g) * 2] - mx);
      o += w * sm_acc[(r * G + g) * HD + d];
      ls += w * sm_ml[(r * G + g) * 2 + 1];
    }
    po[e] = o;
    if (d == 0) {
      pml[g * 2] = mx;
      pml[g * 2 + 1] = ls;
    }
  }

  // ---- ticket: the last split to finish merges all splits -----------------------------------
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int t = atomicAdd(&p.tickets[unit], 1);
    sh_last = (t == p.splits - 1);
    if (sh_last) p.tickets[unit] = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!sh_last) return;
  __threadfence();
  const float* ao = p.part_o + unit * p.splits * (long long)(G * HD);
  const float* aml = p.part_ml + unit * p.splits * (long long)(G * 2);
  for (int e = threadIdx.x; e < gcount * HD; e += blockDim.x) {
    const int g = e / HD, d = e % HD;
    float mx = -FLT_MAX;
    for (int s = 0; s < p.splits; ++s) mx = fmaxf(mx, __ldcg(aml + (s * G + g) * 2));
    float o = 0.f, ls = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const float w = __expf(__ldcg(aml + (s * G + g) * 2) - mx);
      o += w * __ldcg(ao + (long long)(s * G + g) * HD + d);
      ls += w * __ldcg(aml + (s * G + g) * 2 + 1);
    }
    p.out[(long long)b * p.Hq * HD + (long long)(kvh * group + g0 + g) * HD + d] = __float2bfloat16(ls > 0.f ? o / ls : 0.f);
  }
}

// ---------------------------------------------------------------------------------------------
// Tensor-core variant. One token against thousands of cached positions is bound by reading K
// and V once, but the SIMT kernel above spends ~75 warp instructions per position on dot
// products, reductions and exponentials and ends up latency-bound at a fifth of the HBM rate.
// Here the query heads that share a KV head form the (padded) 16-row A operand of
// mma.sync.m16n8k16 - the right-sized tensor instruction for 1..16 rows; a tcgen05 tile would
// start at 64 or 128 rows - and a warp consumes 16 cache positions per step:
//   S = Q K^T   2 n-tiles x HD/16 MMAs, K rows loaded straight from global memory as 16-byte
//               chunks (the contraction index is permuted identically in Q and K, so every
//               lane's B fragment is a run of contiguous bytes of one cache row);
//   softmax     on the accumulator fragment (row max / sum over 4 lanes), one rescale per step;
//   O += P V    HD/8 n-tiles x 1 MMA, V rows again as 16-byte chunks, two rows interleaved
//               into a B register with one byte-permute; the output columns are permuted
//               the same way and un-permuted once at the end.
// About 10 warp instructions per position instead of 75; no shared memory in the main loop.
// The four warps of a CTA take alternate steps of the CTA's position range and merge at the
// end; splits merge through the same workspace + ticket scheme as above.
constexpr int MMA_WARPS = 4;
constexpr int MMA_STEP = 16;  // positions per warp step

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t word_of(const uint4& u, int i) { return i == 0 ? u.x : (i == 1 ? u.y : (i == 2 ? u.z : u.w)); }

template <int HD, bool WIDE>
constexpr size_t decode_mma_smem_bytes() {
  constexpr int ROWS = WIDE ? 16 : 8;
  return (size_t)(MMA_WARPS + 1) * ROWS * (HD + 2) * sizeof(float) + (size_t)(16 + 2) * HD * 2;
}

template <int HD, bool WIDE>
__global__ void __launch_bounds__(MMA_WARPS * 32, 3)
decode_attention_mma_kernel(const DecodeParams p) {
  constexpr int ROWS = WIDE ? 16 : 8;          // query-head rows kept per CTA
  constexpr int KCH = HD / 32;                 // 16-byte chunks of a K row per lane
  constexpr int KB = HD / 16;                  // k-blocks of the S product
  constexpr int NT = HD / 8;                   // n-tiles of the O product
  constexpr int VCH = HD / 64;                 // 16-byte chunks of a V row per lane
  constexpr int CH = HD / 16, HALF = HD / 2, NPART = MMA_WARPS + 1;
  extern __shared__ __align__(128) float smem[];
  float* sm_o = smem;                                         // [NPART][ROWS][HD]
  float* sm_ml = smem + NPART * ROWS * HD;                    // [NPART][ROWS][2]
  __nv_bfloat16* sm_q = reinterpret_cast<__nv_bfloat16*>(sm_ml + NPART * ROWS * 2);  // [16][HD]
  __nv_bfloat16* sm_kn = sm_q + 16 * HD;                      // [HD] new k (rotated), then [HD] new v
  __nv_bfloat16* sm_vn = sm_kn + HD;
  __shared__ int sh_last;

  const int split = blockIdx.x, b = blockIdx.z;
  const int kvh = blockIdx.y / p.gtiles, gt = blockIdx.y % p.gtiles;
  const int group = p.Hq / p.Hkv;
  const int g0 = gt * ROWS;
  const int gcount = min(ROWS, group - g0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 2, j = lane & 3;

  const int len = p.lengths[b];
  if (len <= 0) return;  // uniform per CTA
  const int pos = len - 1;
  const int slot_new = pos % p.cap;
  const int n_slots = min(len, p.cap);
  const int tpos = min(pos, p.max_pos - 1);
  const float* cosr = p.cosT ? p.cosT + (long long)tpos * HALF : nullptr;
  const float* sinr = p.sinT ? p.sinT + (long long)tpos * HALF : nullptr;
  const float sign = cosr ? p.sign : 0.f;
  const __nv_bfloat16* row = p.qkv + (long long)b * p.ld;
  __nv_bfloat16* kbase = p.kc + (long long)b * p.batch_stride + (long long)kvh * p.cap * HD;
  __nv_bfloat16* vbase = p.vc + (long long)b * p.batch_stride + (long long)kvh * p.cap * HD;

  // ---- prologue: the 16 sub-groups of 8 lanes prepare one query head each (norm, rotary, scale)
  {
    const int sg = threadIdx.x >> 3, sub = threadIdx.x & 7;
    float v[2 * CH];
    // every lane runs load_head (its reductions are full-warp shuffles); rows past the group are zeroed
    load_head<HD>(row + (long long)(kvh * group + g0 + min(sg, gcount - 1)) * HD, p.qw, p.qk_norm, p.eps, cosr, sinr, sign, p.scale, sub, v);
    if (sg >= gcount) {
#pragma unroll
      for (int i = 0; i < 2 * CH; ++i) v[i] = 0.f;
    }
    store_chunk<CH>(sm_q + sg * HD + sub * CH, v);
    store_chunk<CH>(sm_q + sg * HD + HALF + sub * CH, v + CH);
    if (split == 0 && warp == 0) {  // the new token's k and v (all four sub-groups compute it, the first one stores)
      float kn[2 * CH], vn[2 * CH];
      load_head<HD>(row + (long long)(p.Hq + kvh) * HD, p.kw, p.qk_norm, p.eps, cosr, sinr, sign, 1.f, sub, kn);
      const __nv_bfloat16* vsrc = row + (long long)(p.Hq + p.Hkv + kvh) * HD;
      load_chunk<CH>(vsrc + sub * CH, vn);
      load_chunk<CH>(vsrc + HALF + sub * CH, vn + CH);
      if (sg == 0) {
        store_chunk<CH>(sm_kn + sub * CH, kn);
        store_chunk<CH>(sm_kn + HALF + sub * CH, kn + CH);
        store_chunk<CH>(sm_vn + sub * CH, vn);
        store_chunk<CH>(sm_vn + HALF + sub * CH, vn + CH);
      }
      if (sg == 0 && gt == 0) {  // exactly one CTA appends the row; nobody uses that slot's old content in this launch
        store_chunk<CH>(kbase + (long long)slot_new * HD + sub * CH, kn);
        store_chunk<CH>(kbase + (long long)slot_new * HD + HALF + sub * CH, kn + CH);
        store_chunk<CH>(vbase + (long long)slot_new * HD + sub * CH, vn);
        store_chunk<CH>(vbase + (long long)slot_new * HD + HALF + sub * CH, vn + CH);
      }
    }
  }
  __syncthreads();

  // A fragments of Q: lane (r, j) holds, for k-block kb, the dims of ITS OWN K chunks:
  // pair e = 2 kb (+1) -> chunk c = e / 4, pair i = e % 4 -> dims c * 32 + j * 8 + 2 i (+1)
  uint32_t qa[KB][4];
#pragma unroll
  for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int e = 2 * kb + h, d = (e >> 2) * 32 + j * 8 + 2 * (e & 3);
      qa[kb][2 * h] = *reinterpret_cast<const uint32_t*>(sm_q + r * HD + d);
      qa[kb][2 * h + 1] = WIDE ? *reinterpret_cast<const uint32_t*>(sm_q + (r + 8) * HD + d) : 0u;
    }
  }

  float o[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[t][i] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};  // rows r and r + 8; l is this lane's share

  const int per = (n_slots + p.splits - 1) / p.splits;
  const int s_lo = split * per, s_hi = min(n_slots, s_lo + per);
  const int nsteps = s_hi > s_lo ? (s_hi - s_lo + MMA_STEP - 1) / MMA_STEP : 0;
  const int last_row = max(s_hi - 1, 0);

  for (int st = warp; st < nsteps; st += MMA_WARPS) {
    const int s0 = s_lo + st * MMA_STEP;
    // K rows s0 + r and s0 + 8 + r, V rows s0 + 2j, +1, +8, +9 (clamped: masked below)
    uint4 kq[2][KCH], vq[4][VCH];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const __nv_bfloat16* kr = kbase + (long long)min(s0 + 8 * h + r, last_row) * HD + j * 8;
#pragma unroll
      for (int c = 0; c < KCH; ++c) kq[h][c] = ldg_stream16(kr + c * 32);
    }
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      const int rr = s0 + (q4 >> 1) * 8 + 2 * j + (q4 & 1);
      const __nv_bfloat16* vr = vbase + (long long)min(rr, last_row) * HD + r * 8;
#pragma unroll
      for (int c = 0; c < VCH; ++c) vq[q4][c] = ldg_stream16(vr + c * 64);
    }
    // S = Q K^T for the two groups of 8 positions
    float s[2][4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int i = 0; i < 4; ++i) s[h][i] = 0.f;
#pragma unroll
      for (int kb = 0; kb < KB; ++kb) {
        const int e = 2 * kb;
        mma_bf16_16816(s[h], qa[kb], word_of(kq[h][e >> 2], e & 3), word_of(kq[h][(e + 1) >> 2], (e + 1) & 3));
      }
    }
    // mask: columns 2j, 2j+1 of each group
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int sp = s0 + 8 * h + 2 * j + i;
        if (sp >= s_hi || sp == slot_new) { s[h][i] = -INFINITY; s[h][2 + i] = -INFINITY; }
      }
    // online softmax per row (rows r: elements 0,1; rows r + 8: elements 2,3)
    uint32_t pa[4];
#pragma unroll
    for (int hr = 0; hr < (WIDE ? 2 : 1); ++hr) {
      float mx = fmaxf(fmaxf(s[0][2 * hr], s[0][2 * hr + 1]), fmaxf(s[1][2 * hr], s[1][2 * hr + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float mn = fmaxf(m_run[hr], mx);
      const float mu = mn == -INFINITY ? 0.f : mn;
      const float corr = __expf(m_run[hr] - mu);
      const float p00 = __expf(s[0][2 * hr] - mu), p01 = __expf(s[0][2 * hr + 1] - mu);
      const float p10 = __expf(s[1][2 * hr] - mu), p11 = __expf(s[1][2 * hr + 1] - mu);
      l_run[hr] = l_run[hr] * corr + (p00 + p01) + (p10 + p11);
      m_run[hr] = mn;
      pa[hr] = pack_bf16x2(p00, p01);        // a0 / a1: positions 2j, 2j+1 of the first group
      pa[2 + hr] = pack_bf16x2(p10, p11);    // a2 / a3: of the second group
#pragma unroll
      for (int t = 0; t < NT; ++t) { o[t][2 * hr] *= corr; o[t][2 * hr + 1] *= corr; }
    }
    if (!WIDE) { pa[1] = 0u; pa[3] = 0u; }
    // O += P V: n-tile t takes element t % 8 of chunk t / 8 of this lane's V rows
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const int c = t >> 3, x = t & 7;
      const uint32_t sel = (x & 1) ? 0x7632u : 0x5410u;
      const uint32_t b0 = __byte_perm(word_of(vq[0][c], x >> 1), word_of(vq[1][c], x >> 1), sel);
      const uint32_t b1 = __byte_perm(word_of(vq[2][c], x >> 1), word_of(vq[3][c], x >> 1), sel);
      mma_bf16_16816(o[t], pa, b0, b1);
    }
  }

  // ---- partials of this CTA: one per warp + the new token (split 0) ---------------------------
#pragma unroll
  for (int hr = 0; hr < (WIDE ? 2 : 1); ++hr) {
    float l = l_run[hr];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int rowi = r + 8 * hr;
    if (j == 0) {
      sm_ml[(warp * ROWS + rowi) * 2] = m_run[hr];
      sm_ml[(warp * ROWS + rowi) * 2 + 1] = l;
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const int d0 = (t >> 3) * 64 + (2 * j) * 8 + (t & 7);
      sm_o[(warp * ROWS + rowi) * HD + d0] = o[t][2 * hr];
      sm_o[(warp * ROWS + rowi) * HD + d0 + 8] = o[t][2 * hr + 1];
    }
  }
  if (warp == 0) {  // slot MMA_WARPS: the new token (weight exp(q.k), value v), present in split 0 only
    for (int g = 0; g < ROWS; ++g) {
      float d = 0.f;
      if (split == 0 && g < gcount)
        for (int e = lane; e < HD; e += 32) d += __bfloat162float(sm_q[g * HD + e]) * __bfloat162float(sm_kn[e]);
#pragma unroll
      for (int sft = 16; sft > 0; sft >>= 1) d += __shfl_xor_sync(0xffffffffu, d, sft);
      const bool live = split == 0 && g < gcount;
      if (lane == 0) {
        sm_ml[(MMA_WARPS * ROWS + g) * 2] = live ? d : -INFINITY;
        sm_ml[(MMA_WARPS * ROWS + g) * 2 + 1] = live ? 1.f : 0.f;
      }
      for (int e = lane; e < HD; e += 32) sm_o[(MMA_WARPS * ROWS + g) * HD + e] = live ? __bfloat162float(sm_vn[e]) : 0.f;
    }
  }
  __syncthreads();
  const long long unit = ((long long)b * p.Hkv + kvh) * p.gtiles + gt;
  float* po = p.part_o + (unit * p.splits + split) * (long long)(ROWS * HD);
  float* pml = p.part_ml + (unit * p.splits + split) * (long long)(ROWS * 2);
  for (int e = threadIdx.x; e < ROWS * HD; e += blockDim.x) {
    const int g = e / HD, d = e % HD;
    float mx = -INFINITY;
#pragma unroll
    for (int q = 0; q < NPART; ++q) mx = fmaxf(mx, sm_ml[(q * ROWS + g) * 2]);
    float acc = 0.f, ls = 0.f;
    if (mx != -INFINITY) {
#pragma unroll
      for (int q = 0; q < NPART; ++q) {
        const float w = __expf(sm_ml[(q * ROWS + g) * 2] - mx);
        acc += w * sm_o[(q * ROWS + g) * HD + d];
        ls += w * sm_ml[(q * ROWS + g) * 2 + 1];
      }
    }
    po[e] = acc;
    if (d == 0) {
      pml[g * 2] = mx;
      pml[g * 2 + 1] = ls;
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int t = atomicAdd(&p.tickets[unit], 1);
    sh_last = (t == p.splits - 1);
    if (sh_last) p.tickets[unit] = 0;
  }
  __syncthreads();
  if (!sh_last) return;
  __threadfence();
  const float* ao = p.part_o + unit * p.splits * (long long)(ROWS * HD);
  const float* aml = p.part_ml + unit * p.splits * (long long)(ROWS * 2);
  for (int e = threadIdx.x; e < gcount * HD; e += blockDim.x) {
    const int g = e / HD, d = e % HD;
    float mx = -INFINITY;
    for (int s = 0; s < p.splits; ++s) mx = fmaxf(mx, __ldcg(aml + (s * ROWS + g) * 2));
    float acc = 0.f, ls = 0.f;
    if (mx != -INFINITY)
      for (int s = 0; s < p.splits; ++s) {
        const float w = __expf(__ldcg(aml + (s * ROWS + g) * 2) - mx);
        acc += w * __ldcg(ao + (long long)(s * ROWS + g) * HD + d);
        ls += w * __ldcg(aml + (s * ROWS + g) * 2 + 1);
      }
    p.out[(long long)b * p.Hq * HD + (long long)(kvh * group + g0 + g) * HD + d] = __float2bfloat16(ls > 0.f ? acc / ls : 0.f);
  }
}

template <int HD, bool WIDE>
static int launch_decode_mma(const DecodeParams& p, cudaStream_t st) {
  constexpr size_t smem = decode_mma_smem_bytes<HD, WIDE>();
  static_assert(smem <= 48 * 1024, "decode_attention_mma: static budget");
  dim3 grid(p.splits, p.Hkv * p.gtiles, p.B);
  decode_attention_mma_kernel<HD, WIDE><<<grid, MMA_WARPS * 32, smem, st>>>(p);
  return launch_check("decode_attention_mma", 1);
}

template <int HD, int G>
static int launch_decode(const DecodeParams& p, cudaStream_t st) {
  constexpr size_t smem = decode_smem_bytes<HD, G>();
  auto kern = decode_attention_kernel<HD, G>;
  if (smem > 48 * 1024) {
    static bool done[64] = {};  // per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (!done[dev & 63]) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return fail(-2, "decode_attention: cannot raise the dynamic shared memory limit");
      done[dev & 63] = true;
    }
  }
  dim3 grid(p.splits, p.Hkv * p.gtiles, p.B);
  kern<<<grid, 128, smem, st>>>(p);
  return launch_check("decode_attention", 1);
}

}  // namespace nfn

using namespace nfn;

namespace nfn {
static int g_decode_impl = 1;  // 1: tensor-core kernel, 0: SIMT kernel
}

// Selects the kernel behind nfn_decode_attention (1 = mma.sync variant, the default; 0 = SIMT). Returns the old value.
extern "C" int nfn_decode_attention_set_impl(int impl) {
  const int old = nfn::g_decode_impl;
  nfn::g_decode_impl = impl ? 1 : 0;
  return old;
}

extern "C" long long nfn_decode_attention_workspace_bytes(int B, int n_q_heads, int n_kv_heads, int head_dim, int max_splits) {
  if (B <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads || max_splits <= 0) return -1;
  const int group = n_q_heads / n_kv_heads, G = group >= 4 ? 4 : (group >= 2 ? 2 : 1), gtiles = (group + G - 1) / G;
  const long long units = (long long)B * n_kv_heads * gtiles;
  const long long simt = ((units * 4 + 255) / 256) * 256 + units * max_splits * (long long)G * (head_dim + 2) * 4;
  // the tensor-core kernel keeps 8 or 16 head rows per CTA
  const int rows = group > 8 ? 16 : 8, mtiles = (group + rows - 1) / rows;
  const long long munits = (long long)B * n_kv_heads * mtiles;
  const long long mma = ((munits * 4 + 255) / 256) * 256 + munits * max_splits * (long long)rows * (head_dim + 2) * 4;
  return 256 + std::max(simt, mma);
}

extern "C" int nfn_decode_attention(const void* qkv, int ld, void* k_cache, void* v_cache, long long cache_batch_stride,
                                    const int* lengths, void* out, int B, int n_q_heads, int n_kv_heads, int head_dim, int cap,
                                    const void* q_norm_weight, const void* k_norm_weight, int qk_norm, float eps,
                                    const float* cos_table, const float* sin_table, int max_pos, float rope_sign, float scale,
                                    void* workspace, long long workspace_bytes, int splits, nfn_stream_t stream) {
  if (B <= 0) return 0;
  if (!qkv || !k_cache || !v_cache || !lengths || !out || !workspace) return fail(-1, "decode_attention: null operand");
  if (head_dim != 64 && head_dim != 128) return fail(-1, "decode_attention: head_dim must be 64 or 128");
  if (n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads) return fail(-1, "decode_attention: n_q_heads must be a multiple of n_kv_heads");
  if (cap <= 0 || cache_batch_stride < (long long)n_kv_heads * cap * head_dim) return fail(-1, "decode_attention: cache stride smaller than heads * cap * head_dim");
  if (ld < (n_q_heads + 2 * n_kv_heads) * head_dim || ld % 8) return fail(-1, "decode_attention: qkv row stride too small or not a multiple of 8");
  if ((cos_table == nullptr) != (sin_table == nullptr) || (cos_table && max_pos <= 0)) return fail(-1, "decode_attention: cos/sin tables must come together");
  if (cos_table && rope_sign != 1.f && rope_sign != -1.f) return fail(-1, "decode_attention: rope_sign must be +1 or -1");
  const bool use_mma = g_decode_impl == 1;
  const int group = n_q_heads / n_kv_heads;
  const int G = use_mma ? (group > 8 ? 16 : 8) : (group >= 4 ? 4 : (group >= 2 ? 2 : 1)), gtiles = (group + G - 1) / G;
  const long long units = (long long)B * n_kv_heads * gtiles;
  if (splits <= 0) {
    // one full wave at two (SIMT) or three (tensor-core kernel) resident CTAs per SM (rounding
    // down, so no straggler wave), and at least 128 cache positions per split
    const long long want = ((use_mma ? 3LL : 2LL) * sm_count()) / units;
    splits = (int)std::max<long long>(1, std::min<long long>(want, (cap + 127) / 128));
  }
  splits = min(splits, 64);
  const long long ticket_bytes = ((units * 4 + 255) / 256) * 256;
  const long long need = ticket_bytes + units * splits * (long long)G * (head_dim + 2) * 4;
  if (workspace_bytes < need) return fail(-1, "decode_attention: workspace too small (see nfn_decode_attention_workspace_bytes)");
  if (reinterpret_cast<uintptr_t>(workspace) % 16) return fail(-1, "decode_attention: workspace must be 16-byte aligned");
  DecodeParams p;
  p.qkv = static_cast<const __nv_bfloat16*>(qkv);
  p.ld = ld;
  p.kc = static_cast<__nv_bfloat16*>(k_cache);
  p.vc = static_cast<__nv_bfloat16*>(v_cache);
  p.batch_stride = cache_batch_stride;
  p.lengths = lengths;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.B = B; p.Hq = n_q_heads; p.Hkv = n_kv_heads; p.cap = cap; p.splits = splits; p.gtiles = gtiles;
  p.qw = static_cast<const __nv_bfloat16*>(q_norm_weight);
  p.kw = static_cast<const __nv_bfloat16*>(k_norm_weight);
  p.qk_norm = qk_norm; p.eps = eps;
  p.cosT = cos_table; p.sinT = sin_table; p.max_pos = max_pos; p.sign = rope_sign; p.scale = scale;
  char* ws = static_cast<char*>(workspace);
  p.tickets = reinterpret_cast<int*>(ws);
  p.part_ml = reinterpret_cast<float*>(ws + ticket_bytes);
  p.part_o = p.part_ml + units * splits * (long long)G * 2;
  p.status = status_ptr();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (use_mma) {
    if (head_dim == 128) return G == 16 ? launch_decode_mma<128, true>(p, st) : launch_decode_mma<128, false>(p, st);
    return G == 16 ? launch_decode_mma<64, true>(p, st) : launch_decode_mma<64, false>(p, st);
  }
  if (head_dim == 128) return G == 4 ? launch_decode<128, 4>(p, st) : (G == 2 ? launch_decode<128, 2>(p, st) : launch_decode<128, 1>(p, st));
  return G == 4 ? launch_decode<64, 4>(p, st) : (G == 2 ? launch_decode<64, 2>(p, st) : launch_decode<64, 1>(p, st));
}
