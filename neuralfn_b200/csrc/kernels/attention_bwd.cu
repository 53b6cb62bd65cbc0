// Flash-attention backward on tcgen05 (sm_100a).
//
// One CTA owns a 128-key block of one (batch, kv-head) and walks over every query
// tile (and every query head of the GQA group) that can see it. K_j and V_j stay
// resident in shared memory; per query tile five tensor-core products run, all with
// TMEM accumulators:
//     S^T  = K_j Q_i^T          (keys x queries)      -> TMEM [0,128)
//     dP^T = V_j dO_i^T         (keys x queries)      -> TMEM [128,256)
//     dV  += P^T dO_i           (keys x D, accumulated over all steps in TMEM)
//     dK  += dS^T Q_i           (keys x D, accumulated over all steps in TMEM)
//     dQ_i = dS K_j             (queries x D)         -> TMEM [0,D) (re-uses the S columns)
// 512 softmax threads (four per key row, each taking a quarter of the query columns; the backward
// has no row reductions, and one warp per scheduler leaves most issue slots empty) turn S^T/dP^T into P^T and dS^T = P^T o (dP^T - delta) and write both as bf16 into 128-byte-swizzled shared tiles; the same dS^T tile serves
// as K-major A operand for dK and as MN-major A operand for dQ, and the Q/dO/K tiles
// serve as K-major or MN-major B operands, so nothing is ever transposed in memory.
// dQ partial tiles are added into an fp32 accumulator with vector reductions; dK/dV
// leave TMEM once at the end. Because a CTA loops over the whole GQA group, dK/dV need
// no atomics.
//
// Reference counterparts: ThunderKittens launch_backward_causal call sites, dprep and
// the scalar backward kernels (neuralfn/csrc/tile_cuda/kernels.cu:5280-5838, 22456-23182,
// 3345-3450).
#include "common.h"
#include "sm100_ptx.cuh"

namespace nfn {

constexpr int AB_BLK = 128;
constexpr int AB_SPLIT = 4;                        // warps per TMEM lane quarter; each takes 128 / AB_SPLIT columns
constexpr int AB_COLS = 128 / AB_SPLIT;
constexpr int AB_SOFTMAX_WARPS = 4 * AB_SPLIT;
constexpr int AB_CTRL_WARP = AB_SOFTMAX_WARPS;
constexpr int AB_THREADS = (AB_SOFTMAX_WARPS + 1) * 32;

struct AttnBwdParams {
  const float* lse;    // [B, Hq, T]
  const float* delta;  // [B, Hq, T]
  float* dq_accum;     // fp32 [B*T, Hq*D]
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int ld_dk, ld_dv;
  int B, T, Hq, Hkv;
  int causal, window;
  float scale, scale_log2;
  int* status;
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

template <int D, int STAGES>
__global__ void __launch_bounds__(AB_THREADS)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                const AttnBwdParams p) {
  constexpr uint32_t TILE = AB_BLK * D * 2;         // one [128 x D] bf16 tile
  constexpr uint32_t PT = AB_BLK * AB_BLK * 2;      // one [128 x 128] bf16 tile
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DV = 256, COL_DK = 256 + D, COL_DQ = 0;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE;
  uint8_t* sQdO = sV + TILE;                 // STAGES x (Q tile, dO tile)
  uint8_t* sP = sQdO + STAGES * 2 * TILE;
  uint8_t* sdS = sP + PT;
  float* s_lse = reinterpret_cast<float*>(sdS + PT);  // [softmax warps][columns per warp]
  float* s_delta = s_lse + 4 * AB_BLK;                // likewise
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_delta + 4 * AB_BLK);
  uint64_t* bar_kv = bars;            // 1
  uint64_t* bar_qdo = bars + 1;       // STAGES (<= 2)
  uint64_t* bar_sdp = bars + 3;       // S^T and dP^T complete
  uint64_t* bar_pds = bars + 4;       // one arrival per softmax warp: P^T and dS^T in shared memory
  uint64_t* bar_out = bars + 5;       // dV/dK/dQ products retired
  uint64_t* bar_dqfree = bars + 6;    // one arrival per softmax warp: dQ tile read out of TMEM
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jb = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int k0 = jb * AB_BLK;
  const int nQ = (p.T + AB_BLK - 1) / AB_BLK;

  // query tiles that can see this key block
  int i_lo = 0, i_hi = nQ;
  if (p.causal) {
    i_lo = jb;
    if (p.window > 0) i_hi = min(nQ, (k0 + AB_BLK - 1 + p.window - 1) / AB_BLK + 1);
  } else if (p.window > 0) {
    i_lo = max(0, (k0 - p.window + 1) / AB_BLK);
    i_hi = min(nQ, (k0 + AB_BLK - 1 + p.window - 1) / AB_BLK + 1);
  }
  const int nqb = max(0, i_hi - i_lo);
  const int nsteps = nqb * G;

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    mbar_init(smem_u32(bar_kv), 1);
    mbar_init(smem_u32(&bar_qdo[0]), 1);
    mbar_init(smem_u32(&bar_qdo[1]), 1);
    mbar_init(smem_u32(bar_sdp), 1);
    mbar_init(smem_u32(bar_pds), AB_SOFTMAX_WARPS);  // one arrival per softmax warp
    mbar_init(smem_u32(bar_out), 1);
    mbar_init(smem_u32(bar_dqfree), AB_SOFTMAX_WARPS);  // one arrival per softmax warp
    fence_mbar_init();
  }
  if (warp == AB_CTRL_WARP) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int row0 = b * p.T;

  if (warp == AB_CTRL_WARP) {
    if (lane == 0 && nsteps > 0) {
      // ------------------------------------------------------ control thread --
      auto load_qdo = [&](int s) {
        const int stage = s % STAGES;
        const int hq = hk * G + s / nqb;
        const int i = i_lo + s % nqb;
        const uint32_t fb = smem_u32(&bar_qdo[stage]);
        const uint32_t sq = smem_u32(sQdO + stage * 2 * TILE);
        const uint32_t sdo = sq + TILE;
        mbar_expect_tx(fb, 2 * TILE);
#pragma unroll
        for (int d = 0; d < D / 64; ++d) {
          tma_load_2d(sq + d * (AB_BLK * 128), &tm_q, fb, hq * D + d * 64, row0 + i * AB_BLK);
          tma_load_2d(sdo + d * (AB_BLK * 128), &tm_do, fb, hq * D + d * 64, row0 + i * AB_BLK);
        }
      };
      mbar_expect_tx(smem_u32(bar_kv), 2 * TILE);
#pragma unroll
      for (int d = 0; d < D / 64; ++d) {
        tma_load_2d(smem_u32(sK) + d * (AB_BLK * 128), &tm_k, smem_u32(bar_kv), hk * D + d * 64, row0 + k0);
        tma_load_2d(smem_u32(sV) + d * (AB_BLK * 128), &tm_v, smem_u32(bar_kv), hk * D + d * 64, row0 + k0);
      }
      load_qdo(0);
      bool ok = mbar_wait_bounded(smem_u32(bar_kv), 0, cta_abort, p.status, NFN_ERR_WAIT_FULL);

      constexpr uint32_t idesc_kk = make_idesc_bf16(128, 128, 0, 0);  // S^T, dP^T
      constexpr uint32_t idesc_kn = make_idesc_bf16(128, D, 0, 1);    // dV, dK: A K-major, B MN-major
      constexpr uint32_t idesc_nn = make_idesc_bf16(128, D, 1, 1);    // dQ: A MN-major, B MN-major
      for (int s = 0; s < nsteps && ok; ++s) {
        const int stage = s % STAGES;
        if (STAGES == 2 && s + 1 < nsteps) {
          if (s >= 1) {
            ok = mbar_wait_bounded(smem_u32(bar_out), (s - 1) & 1, cta_abort, p.status, NFN_ERR_WAIT_MISC);
            if (!ok) break;
          }
          load_qdo(s + 1);
        }
        ok = mbar_wait_bounded(smem_u32(&bar_qdo[stage]), (s / STAGES) & 1, cta_abort, p.status,
                               NFN_ERR_WAIT_FULL);
        if (!ok) break;
        if (s >= 1) {
          ok = mbar_wait_bounded(smem_u32(bar_dqfree), (s - 1) & 1, cta_abort, p.status,
                                 NFN_ERR_WAIT_TMEM_EMPTY);
          if (!ok) break;
        }
        tc_fence_after();
        const uint32_t sq = smem_u32(sQdO + stage * 2 * TILE);
        const uint32_t sdo = sq + TILE;
        const uint32_t sk = smem_u32(sK), sv = smem_u32(sV);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * (AB_BLK * 128) + (kk % 4) * 32;
          umma_bf16_ss(tmem_base + COL_S, make_smem_desc_sw128(sk + off, 16, 1024),
                       make_smem_desc_sw128(sq + off, 16, 1024), idesc_kk, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * (AB_BLK * 128) + (kk % 4) * 32;
          umma_bf16_ss(tmem_base + COL_DP, make_smem_desc_sw128(sv + off, 16, 1024),
                       make_smem_desc_sw128(sdo + off, 16, 1024), idesc_kk, kk != 0);
        }
        umma_commit(smem_u32(bar_sdp));
        ok = mbar_wait_bounded(smem_u32(bar_pds), s & 1, cta_abort, p.status, NFN_ERR_WAIT_MISC);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sp = smem_u32(sP), sds = smem_u32(sdS);
#pragma unroll
        for (int kk = 0; kk < AB_BLK / 16; ++kk) {  // contraction over the 128 queries
          const uint32_t a_off = (kk / 4) * (AB_BLK * 128) + (kk % 4) * 32;
          const uint32_t b_off = kk * (16 * 128);
          umma_bf16_ss(tmem_base + COL_DV, make_smem_desc_sw128(sp + a_off, 16, 1024),
                       make_smem_desc_sw128(sdo + b_off, AB_BLK * 128, 1024), idesc_kn,
                       (s | kk) != 0);
        }
#pragma unroll
        for (int kk = 0; kk < AB_BLK / 16; ++kk) {
          const uint32_t a_off = (kk / 4) * (AB_BLK * 128) + (kk % 4) * 32;
          const uint32_t b_off = kk * (16 * 128);
          umma_bf16_ss(tmem_base + COL_DK, make_smem_desc_sw128(sds + a_off, 16, 1024),
                       make_smem_desc_sw128(sq + b_off, AB_BLK * 128, 1024), idesc_kn,
                       (s | kk) != 0);
        }
#pragma unroll
        for (int kk = 0; kk < AB_BLK / 16; ++kk) {  // contraction over the 128 keys
          const uint32_t off = kk * (16 * 128);
          umma_bf16_ss(tmem_base + COL_DQ, make_smem_desc_sw128(sds + off, AB_BLK * 128, 1024),
                       make_smem_desc_sw128(sk + off, AB_BLK * 128, 1024), idesc_nn, kk != 0);
        }
        umma_commit(smem_u32(bar_out));
        if (STAGES == 1 && s + 1 < nsteps) {
          ok = mbar_wait_bounded(smem_u32(bar_out), s & 1, cta_abort, p.status, NFN_ERR_WAIT_MISC);
          if (!ok) break;
          load_qdo(s + 1);
        }
      }
    }
  } else {
    // ------------------------------------------------------ softmax threads --
    // warp w owns TMEM lanes 32 (w & 3) ... and, of every 128-column tile, the half (w >> 2): the
    // backward pass has no row reductions (P and dS are element-wise given lse and delta), so two
    // warps can share a row without talking to each other
    const int quarter = warp & 3, half = warp >> 2;  // `half`: which column slice (0 .. AB_SPLIT - 1)
    const int r = quarter * 32 + lane;  // key row within the block == TMEM lane; also query row for dQ
    const int kidx = k0 + r;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const float LOG2E = 1.4426950408889634f;
    bool ok = true;
    float nx_lse[AB_COLS / 32], nx_dlt[AB_COLS / 32];
    auto fetch_stats = [&](int s2) {  // lse (in log2 units) and delta of this warp's query columns at step s2
      const int hq2 = hk * G + s2 / nqb;
      const int q02 = (i_lo + s2 % nqb) * AB_BLK;
#pragma unroll
      for (int e = 0; e < AB_COLS / 32; ++e) {
        const int q = q02 + half * AB_COLS + e * 32 + lane;
        const size_t idx = ((size_t)b * p.Hq + hq2) * p.T + q;
        nx_lse[e] = q < p.T ? __ldg(p.lse + idx) * LOG2E : INFINITY;
        nx_dlt[e] = q < p.T ? __ldg(p.delta + idx) : 0.f;
      }
    };
    for (int s = 0; s < nsteps; ++s) {
      const int hq = hk * G + s / nqb;
      const int i = i_lo + s % nqb;
      const int q0 = i * AB_BLK;
      // stage lse / delta of this query tile: every warp keeps a private copy of the 128
      // values, so only warp-level synchronisation is needed (no CTA barrier that a
      // timed-out warp could leave the others stuck on)
      // (the values were fetched into registers during the previous step's dQ phase, so their
      // latency is off the critical path)
      float* lse2 = s_lse + warp * AB_COLS;   // this warp's query columns
      float* dlt = s_delta + warp * AB_COLS;
      if (s == 0) fetch_stats(0);
      __syncwarp();
#pragma unroll
      for (int e = 0; e < AB_COLS / 32; ++e) {
        lse2[e * 32 + lane] = nx_lse[e];
        dlt[e * 32 + lane] = nx_dlt[e];
      }
      __syncwarp();
      ok = mbar_wait_bounded(smem_u32(bar_sdp), s & 1, cta_abort, p.status, NFN_ERR_WAIT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      bool need_mask = (k0 + AB_BLK > p.T);
      if (p.causal) need_mask |= (k0 + AB_BLK - 1 > q0);
      if (p.window > 0) {
        need_mask |= (q0 + AB_BLK - 1 >= k0 + p.window);
        if (!p.causal) need_mask |= (k0 + AB_BLK - 1 >= q0 + p.window);
      }
      auto visible = [&](int q) -> bool {
        if (kidx >= p.T) return false;
        if (p.causal) {
          if (kidx > q) return false;
          if (p.window > 0 && kidx <= q - p.window) return false;
        } else if (p.window > 0) {
          if (kidx <= q - p.window || kidx >= q + p.window) return false;
        }
        return true;
      };
#pragma unroll 1
      for (int c = half * (AB_COLS / 32); c < (half + 1) * (AB_COLS / 32); ++c) {
        uint32_t sv_[32], dp_[32];
        tmem_ld_32x32(t_row + COL_S + c * 32, sv_);
        tmem_ld_32x32(t_row + COL_DP + c * 32, dp_);
        tmem_ld_wait();
        uint32_t pk[16], dk_[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const int qa = c * 32 + 2 * e, ql = qa - half * AB_COLS;
          float p0 = fast_exp2(__uint_as_float(sv_[2 * e]) * p.scale_log2 - lse2[ql]);
          float p1 = fast_exp2(__uint_as_float(sv_[2 * e + 1]) * p.scale_log2 - lse2[ql + 1]);
          if (need_mask) {
            if (!visible(q0 + qa)) p0 = 0.f;
            if (!visible(q0 + qa + 1)) p1 = 0.f;
          }
          const float d0 = p0 * (__uint_as_float(dp_[2 * e]) - dlt[ql]);
          const float d1 = p1 * (__uint_as_float(dp_[2 * e + 1]) - dlt[ql + 1]);
          pk[e] = pack_bf16x2(p0, p1);
          dk_[e] = pack_bf16x2(d0, d1);
        }
        uint8_t* prow = sP + (c / 2) * (AB_BLK * 128) + r * 128;
        uint8_t* drow = sdS + (c / 2) * (AB_BLK * 128) + r * 128;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int chunk = ((c & 1) * 4 + ch) ^ (r & 7);
          *reinterpret_cast<uint4*>(prow + chunk * 16) =
              make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
          *reinterpret_cast<uint4*>(drow + chunk * 16) =
              make_uint4(dk_[ch * 4], dk_[ch * 4 + 1], dk_[ch * 4 + 2], dk_[ch * 4 + 3]);
        }
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(bar_pds));
      if (s + 1 < nsteps) fetch_stats(s + 1);
      // dQ tile: lane r == query row q0 + r
      ok = mbar_wait_bounded(smem_u32(bar_out), s & 1, cta_abort, p.status, NFN_ERR_WAIT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      {
        const int q = q0 + r;
        float* dst = p.dq_accum + (size_t)(row0 + q) * (p.Hq * D) + hq * D;
#pragma unroll
        for (int c = half; c < D / 32; c += AB_SPLIT) {
          uint32_t v[32];
          tmem_ld_32x32(t_row + COL_DQ + c * 32, v);
          tmem_ld_wait();
          if (q < p.T) {
#pragma unroll
            for (int e = 0; e < 8; ++e)
              red_add_v4(dst + c * 32 + e * 4, __uint_as_float(v[4 * e]), __uint_as_float(v[4 * e + 1]),
                         __uint_as_float(v[4 * e + 2]), __uint_as_float(v[4 * e + 3]));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(bar_dqfree));
    }
    // dK / dV leave TMEM once
    if (ok && nsteps > 0) {
      // the last bar_out wait above already covers every product issued before it.
      // tcgen05.ld is warp-collective: every lane issues the loads, only rows inside
      // the sequence store.
      const bool row_ok = kidx < p.T;
      {
        __nv_bfloat16* dkrow = p.dk + (size_t)(row0 + kidx) * p.ld_dk + hk * D;
        __nv_bfloat16* dvrow = p.dv + (size_t)(row0 + kidx) * p.ld_dv + hk * D;
#pragma unroll
        for (int c = half; c < D / 32; c += AB_SPLIT) {
          uint32_t v[32];
          tmem_ld_32x32(t_row + COL_DV + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(v[8 * e]), __uint_as_float(v[8 * e + 1]));
            u.y = pack_bf16x2(__uint_as_float(v[8 * e + 2]), __uint_as_float(v[8 * e + 3]));
            u.z = pack_bf16x2(__uint_as_float(v[8 * e + 4]), __uint_as_float(v[8 * e + 5]));
            u.w = pack_bf16x2(__uint_as_float(v[8 * e + 6]), __uint_as_float(v[8 * e + 7]));
            if (row_ok) reinterpret_cast<uint4*>(dvrow + c * 32)[e] = u;
          }
          tmem_ld_32x32(t_row + COL_DK + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(v[8 * e]) * p.scale, __uint_as_float(v[8 * e + 1]) * p.scale);
            u.y = pack_bf16x2(__uint_as_float(v[8 * e + 2]) * p.scale, __uint_as_float(v[8 * e + 3]) * p.scale);
            u.z = pack_bf16x2(__uint_as_float(v[8 * e + 4]) * p.scale, __uint_as_float(v[8 * e + 5]) * p.scale);
            u.w = pack_bf16x2(__uint_as_float(v[8 * e + 6]) * p.scale, __uint_as_float(v[8 * e + 7]) * p.scale);
            if (row_ok) reinterpret_cast<uint4*>(dkrow + c * 32)[e] = u;
          }
        }
      }
    } else if (nsteps == 0 && kidx < p.T && half == 0) {
      // no query sees these keys: zero gradients
      __nv_bfloat16* dkrow = p.dk + (size_t)(row0 + kidx) * p.ld_dk + hk * D;
      __nv_bfloat16* dvrow = p.dv + (size_t)(row0 + kidx) * p.ld_dv + hk * D;
      for (int e = 0; e < D / 8; ++e) {
        reinterpret_cast<uint4*>(dkrow)[e] = make_uint4(0, 0, 0, 0);
        reinterpret_cast<uint4*>(dvrow)[e] = make_uint4(0, 0, 0, 0);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*cta_abort) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == AB_CTRL_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// delta[b, h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (token, head)
template <int D>
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                  float* __restrict__ delta, int B, int T, int Hq, int ld_do, int ld_o) {
  const long long w = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= (long long)B * T * Hq) return;
  const int h = (int)(w % Hq);
  const long long tok = w / Hq;
  constexpr int PER = D / 32;
  const __nv_bfloat16* a = dout + tok * ld_do + h * D + lane * PER;
  const __nv_bfloat16* c = out + tok * ld_o + h * D + lane * PER;
  float s = 0.f;
#pragma unroll
  for (int e = 0; e < PER; e += 2) {
    float2 x = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(a + e));
    float2 y = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(c + e));
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) {
    const int bi = (int)(tok / T), t = (int)(tok % T);
    delta[((size_t)bi * Hq + h) * T + t] = s;
  }
}

// dq = bf16(dq_accum * scale)
__global__ void __launch_bounds__(256)
attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long rows,
                       int width, int ld_dq, float scale) {
  const int vec_per_row = width / 8;
  const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
  if (idx >= rows * vec_per_row) return;
  const long long row = idx / vec_per_row;
  const int v = (int)(idx % vec_per_row);
  const float4 a = reinterpret_cast<const float4*>(acc + row * width)[2 * v];
  const float4 c = reinterpret_cast<const float4*>(acc + row * width)[2 * v + 1];
  uint4 u;
  u.x = pack_bf16x2(a.x * scale, a.y * scale); u.y = pack_bf16x2(a.z * scale, a.w * scale);
  u.z = pack_bf16x2(c.x * scale, c.y * scale); u.w = pack_bf16x2(c.z * scale, c.w * scale);
  reinterpret_cast<uint4*>(dq + row * ld_dq)[v] = u;
}

template <int D, int STAGES>
static int launch_attn_bwd(const void* dout, const void* q, const void* k, const void* v,
                           const void* o, const float* lse, float* delta, float* dq_accum, void* dq,
                           void* dk, void* dv, int B, int T, int Hq, int Hkv, int ld_do, int ld_q,
                           int ld_k, int ld_v, int ld_o, int ld_dq, int ld_dk, int ld_dv, int causal,
                           int window, float scale, cudaStream_t st) {
  constexpr size_t TILE = AB_BLK * D * 2, PT = AB_BLK * AB_BLK * 2;
  constexpr size_t SMEM = 2 * TILE + STAGES * 2 * TILE + 2 * PT + 8 * AB_BLK * 4 + 128 + 1024;
  auto kern = attn_bwd_kernel<D, STAGES>;
  static bool attr[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess)
      return launch_check("attn_bwd attr");
    attr[dev & 63] = true;
  }
  const long long rows = (long long)B * T;
  {
    const long long warps = rows * Hq;
    attn_delta_kernel<D><<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(
        (const __nv_bfloat16*)dout, (const __nv_bfloat16*)o, delta, B, T, Hq, ld_do, ld_o);
  }
  cudaMemsetAsync(dq_accum, 0, (size_t)rows * Hq * D * sizeof(float), st);
  CUtensorMap tq, tk, tv, tdo;
  if (!make_tmap_2d(&tq, q, 2, (uint64_t)Hq * D, rows, ld_q, 64, AB_BLK, 128)) return -3;
  if (!make_tmap_2d(&tk, k, 2, (uint64_t)Hkv * D, rows, ld_k, 64, AB_BLK, 128)) return -3;
  if (!make_tmap_2d(&tv, v, 2, (uint64_t)Hkv * D, rows, ld_v, 64, AB_BLK, 128)) return -3;
  if (!make_tmap_2d(&tdo, dout, 2, (uint64_t)Hq * D, rows, ld_do, 64, AB_BLK, 128)) return -3;
  AttnBwdParams p;
  p.lse = lse; p.delta = delta; p.dq_accum = dq_accum;
  p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv; p.ld_dk = ld_dk; p.ld_dv = ld_dv;
  p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal; p.window = window;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status_ptr();
  dim3 grid(ceil_div(T, AB_BLK), Hkv, B);
  kern<<<grid, AB_THREADS, SMEM, st>>>(tq, tk, tv, tdo, p);
  {
    const long long total = rows * (Hq * D / 8);
    attn_dq_convert_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        dq_accum, (__nv_bfloat16*)dq, rows, Hq * D, ld_dq, scale);
  }
  return launch_check("attn_bwd", 3);
}

}  // namespace nfn

using namespace nfn;

extern "C" int nfn_attention_backward_v1(const void* dout, const void* q, const void* k, const void* v,
                                      const void* o, const float* lse, float* delta, float* dq_accum,
                                      void* dq, void* dk, void* dv, int B, int T, int Hq, int Hkv,
                                      int D, int ld_do, int ld_q, int ld_k, int ld_v, int ld_o,
                                      int ld_dq, int ld_dk, int ld_dv, int causal, int window,
                                      float scale, nfn_stream_t stream) {
  if (B <= 0 || T <= 0) return 0;
  if (Hq % Hkv) return fail(-1, "attention_backward: Hq must be a multiple of Hkv");
  if ((ld_do | ld_q | ld_k | ld_v | ld_o | ld_dq | ld_dk | ld_dv) & 7)
    return fail(-1, "attention_backward: row strides must be multiples of 8");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (D == 64)
    return launch_attn_bwd<64, 2>(dout, q, k, v, o, lse, delta, dq_accum, dq, dk, dv, B, T, Hq, Hkv,
                                  ld_do, ld_q, ld_k, ld_v, ld_o, ld_dq, ld_dk, ld_dv, causal, window,
                                  scale, st);
  if (D == 128)
    return launch_attn_bwd<128, 1>(dout, q, k, v, o, lse, delta, dq_accum, dq, dk, dv, B, T, Hq, Hkv,
                                   ld_do, ld_q, ld_k, ld_v, ld_o, ld_dq, ld_dk, ld_dv, causal, window,
                                   scale, st);
  return fail(-1, "attention_backward: head_dim must be 64 or 128");
}
