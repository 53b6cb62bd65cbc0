// Flash-attention backward on tcgen05 (sm_100a), pipelined version: two kernels, no atomics.
//
//   attn_bwd_dkv_kernel  one CTA owns a 128-key block of one (batch, kv head) and walks over the
//                        64-query tiles (of every query head of the GQA group) that can see it:
//                            S^T  = K Q_i^T     dP^T = V dO_i^T            (keys x queries, TMEM)
//                            P^T  = exp2(S^T c - lse),  dS^T = P^T o (dP^T - delta)   (registers)
//                            dV  += P^T dO_i    dK  += dS^T Q_i            (keys x D, TMEM)
//   attn_bwd_dq_kernel   one CTA owns a 128-query tile of one (batch, head) and walks over the
//                        64-key blocks it can see:
//                            S = Q K_j^T   dP = dO V_j^T   dS = P o (dP - delta)   dQ += dS K_j
// Recomputing S and dP in the second kernel costs two extra products per tile pair, but every
// gradient then has exactly one owner: dQ needs no fp32 accumulation buffer, no memset, no
// conversion pass and no reduction traffic through L2, and all three gradients are deterministic.
//
// Both kernels use the role layout of the forward kernel (attention_fwd2.cu): four math warps with
// one thread per TMEM lane, one MMA warp, one TMA warp, two CTAs per SM at head_dim 64. A math thread
// pulls its rows of S and dP out of TMEM in one go and releases the columns at once, so the products
// of the next step run under the exponentials of this one.
//
// Mask options as in the forward pass: causal, sliding / bidirectional window, packed-sequence ids,
// score soft-cap. `delta` = rowsum(dO o O) comes from a small pre-pass kernel.
//
// Reference counterparts: ThunderKittens launch_backward_causal call sites, dprep and the scalar
// backward kernels (neuralfn/csrc/tile_cuda/kernels.cu:5280-5838, 22456-23182, 3345-3450).
#include "attention_v2.cuh"
#include "kernel_timers.cuh"

namespace nfn {

constexpr int AB2_SEQ = 1;      // packed-sequence ids
constexpr int AB2_SOFTCAP = 2;  // score soft-cap

struct AttnBwd2Params {
  const float* lse;    // [B, Hq, T] natural log
  const float* delta;  // [B, Hq, T]
  __nv_bfloat16* dq; __nv_bfloat16* dk; __nv_bfloat16* dv;
  int ld_dq, ld_dk, ld_dv;
  int B, Hq, Hkv;
  AttnMask mask;
  float scale, softcap;
  int* status;
};

// delta[b, h, t] = sum_d dO[t, h, d] * O[t, h, d]. One thread per 16-byte piece of a token row
// (8 elements); the D / 8 neighbouring lanes that share a head add up with shuffles.
template <int D>
__global__ void __launch_bounds__(256)
attn_delta2_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                   float* __restrict__ delta, int B, int T, int Hq, int ld_do, int ld_o) {
  constexpr int LANES = D / 8;  // lanes per (token, head): 8 or 16
  const int per_row = Hq * LANES;
  const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
  const long long tok = idx / per_row;
  const int piece = (int)(idx % per_row);
  float s = 0.f;
  const bool live = tok < (long long)B * T;
  if (live) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(dout + tok * ld_do) + piece);
    const uint4 c = __ldg(reinterpret_cast<const uint4*>(out + tok * ld_o) + piece);
    const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
    const float2 c0 = unpack_bf16x2(c.x), c1 = unpack_bf16x2(c.y), c2 = unpack_bf16x2(c.z), c3 = unpack_bf16x2(c.w);
    s = (a0.x * c0.x + a0.y * c0.y) + (a1.x * c1.x + a1.y * c1.y) + (a2.x * c2.x + a2.y * c2.y) + (a3.x * c3.x + a3.y * c3.y);
  }
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (live && (piece % LANES) == 0) {
    const int h = piece / LANES;
    const int bi = (int)(tok / T), t = (int)(tok % T);
    delta[((size_t)bi * Hq + h) * T + t] = s;
  }
}

// One row of the transposed-or-not score tile: p = exp2(c_mul * f(s) - lse2[i]) and
// ds = p * (dp - delta[i]) [* (1 - tanh^2)] for the 64 columns of this thread, in place
// (s <- p, dp <- ds as fp32 bit patterns). `col_lse2` / `col_delta` index by column when
// PER_COLUMN (dK/dV kernel: statistics belong to the query = column), else they are this row's.
template <int N, bool CAPPED>
__device__ __forceinline__ void bwd_p_ds_row(uint32_t (&s)[N], uint32_t (&dp)[N], float c_mul, float cap_in,
                                             float row_lse2, float row_delta) {
  // separate passes (exponent, ex2, product) so that neighbouring instructions are independent
  uint32_t t[CAPPED ? N : 2];  // tanh values, needed again for the soft-cap derivative
  if (CAPPED) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      t[i] = __float_as_uint(fast_tanh(__uint_as_float(s[i]) * cap_in));
      s[i] = t[i];
    }
  }
#pragma unroll
  for (int i = 0; i < N; i += 2) {
    float x0, x1;
    fma2_bcast(x0, x1, __uint_as_float(s[i]), __uint_as_float(s[i + 1]), c_mul, -row_lse2);
    s[i] = __float_as_uint(x0);
    s[i + 1] = __float_as_uint(x1);
  }
#pragma unroll
  for (int i = 0; i < N; ++i) s[i] = __float_as_uint(fast_exp2(__uint_as_float(s[i])));
#pragma unroll
  for (int i = 0; i < N; ++i) {
    float d = (__uint_as_float(dp[i]) - row_delta) * __uint_as_float(s[i]);
    if (CAPPED) d *= 1.f - __uint_as_float(t[i]) * __uint_as_float(t[i]);
    dp[i] = __float_as_uint(d);
  }
}

// ------------------------------------------------------------------------------------- dQ --
template <int D>
struct AttnDqCfg {
  static constexpr int BM = 128, BN = 64;
  static constexpr uint32_t QD_BYTES = BM * D * 2;       // Q tile, dO tile
  static constexpr uint32_t KV_BYTES = BN * D * 2;       // one K or V block
  static constexpr uint32_t DS_BYTES = BM * BN * 2;
  static constexpr uint32_t SMEM = 2 * QD_BYTES + 2 * 2 * KV_BYTES + DS_BYTES + 256;
  static constexpr uint32_t COL_S = 0, COL_DP = BN, COL_DQ = 2 * BN;
  static constexpr uint32_t TMEM_COLS = 256;
  static constexpr int CTAS_PER_SM = (SMEM <= 112 * 1024) ? 2 : 1;
};

template <int D, int FEAT>
__global__ void __launch_bounds__(AV2_THREADS, (AttnDqCfg<D>::CTAS_PER_SM))
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                   const AttnBwd2Params p) {
  using C = AttnDqCfg<D>;
  constexpr int BM = C::BM, BN = C::BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  {
    uint32_t dyn;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
    if (static_cast<uint32_t>(smem - smem_raw) + C::SMEM > dyn) {
      if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, NFN_ERR_WAIT_MISC);
      return;
    }
  }
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + C::QD_BYTES;
  uint8_t* sK = sdO + C::QD_BYTES;                 // [2] stages
  uint8_t* sV = sK + 2 * C::KV_BYTES;              // [2] stages
  uint8_t* sdS = sV + 2 * C::KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + C::DS_BYTES);
  uint64_t* bar_qdo = bars;         // TMA: Q and dO landed
  uint64_t* bar_k = bars + 1;       // [2] TMA: K stage landed
  uint64_t* bar_v = bars + 3;       // [2] TMA: V stage landed
  uint64_t* bar_kfree = bars + 5;   // [2] MMA: dQ += dS_j K_j retired (K stage free); producer only
  uint64_t* bar_vfree = bars + 7;   // [2] MMA: dP_j retired (V stage free); producer only
  uint64_t* bar_s = bars + 9;       // MMA: S_j and dP_j complete
  uint64_t* bar_sfree = bars + 10;  // 4 arrivals: S_j / dP_j are in registers
  uint64_t* bar_ds = bars + 11;     // 4 arrivals: dS_j is in shared memory
  uint64_t* bar_dq = bars + 12;     // MMA: dQ += dS_j K_j retired (dS tile free)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = gridDim.x - 1 - blockIdx.x;  // heavy (late) tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qb * BM;
  const int T = p.mask.T;
  int k_lo, k_hi;
  attn_key_range(p.mask, q0, BM, k_lo, k_hi);
  const int jb_lo = k_lo / BN;
  const int nblk = max(0, (k_hi + BN - 1) / BN - jb_lo);

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    mbar_init(smem_u32(bar_qdo), 1);
    for (int s2 = 0; s2 < 2; ++s2) {
      mbar_init(smem_u32(&bar_k[s2]), 1);
      mbar_init(smem_u32(&bar_v[s2]), 1);
      mbar_init(smem_u32(&bar_kfree[s2]), 1);
      mbar_init(smem_u32(&bar_vfree[s2]), 1);
    }
    mbar_init(smem_u32(bar_s), 1);
    mbar_init(smem_u32(bar_sfree), AV2_MATH_WARPS);
    mbar_init(smem_u32(bar_ds), AV2_MATH_WARPS);
    mbar_init(smem_u32(bar_dq), 1);
    fence_mbar_init();
  }
  if (warp == AV2_MMA_WARP) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int row0 = b * T;

  if (warp == AV2_TMA_WARP) {
    if (lane == 0 && nblk > 0) {
      auto load_k = [&](int j, int stage) {
        const uint32_t fb = smem_u32(&bar_k[stage]);
        mbar_expect_tx(fb, C::KV_BYTES);
#pragma unroll
        for (int d = 0; d < D / 64; ++d)
          tma_load_2d(smem_u32(sK + stage * C::KV_BYTES) + d * (BN * 128), &tm_k, fb, hk * D + d * 64, row0 + (jb_lo + j) * BN);
      };
      auto load_v = [&](int j, int stage) {
        const uint32_t fb = smem_u32(&bar_v[stage]);
        mbar_expect_tx(fb, C::KV_BYTES);
#pragma unroll
        for (int d = 0; d < D / 64; ++d)
          tma_load_2d(smem_u32(sV + stage * C::KV_BYTES) + d * (BN * 128), &tm_v, fb, hk * D + d * 64, row0 + (jb_lo + j) * BN);
      };
      mbar_expect_tx(smem_u32(bar_qdo), 2 * C::QD_BYTES);
#pragma unroll
      for (int d = 0; d < D / 64; ++d) {
        tma_load_2d(smem_u32(sQ) + d * (BM * 128), &tm_q, smem_u32(bar_qdo), h * D + d * 64, row0 + q0);
        tma_load_2d(smem_u32(sdO) + d * (BM * 128), &tm_do, smem_u32(bar_qdo), h * D + d * 64, row0 + q0);
      }
      load_k(0, 0);
      load_v(0, 0);
      if (nblk > 1) { load_k(1, 1); load_v(1, 1); }
      for (int j = 0; j + 2 < nblk; ++j) {
        if (!mbar_wait_bounded(smem_u32(&bar_vfree[j & 1]), (j >> 1) & 1, cta_abort, p.status, 0x200 + 1)) break;
        load_v(j + 2, j & 1);
        if (!mbar_wait_bounded(smem_u32(&bar_kfree[j & 1]), (j >> 1) & 1, cta_abort, p.status, 0x200 + 2)) break;
        load_k(j + 2, j & 1);
      }
    }
  } else if (warp == AV2_MMA_WARP) {
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BM, BN, 0, 0);
      constexpr uint32_t idesc_dq = make_idesc_bf16(BM, D, 0, 1);
      auto issue_s_dp = [&](int stage) {
        const uint32_t sq = smem_u32(sQ), sdo = smem_u32(sdO);
        const uint32_t sk = smem_u32(sK + stage * C::KV_BYTES), sv = smem_u32(sV + stage * C::KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t a_off = (kk / 4) * (BM * 128) + (kk % 4) * 32;
          const uint32_t b_off = (kk / 4) * (BN * 128) + (kk % 4) * 32;
          umma_bf16_ss(tmem_base + C::COL_S, make_smem_desc_sw128(sq + a_off, 16, 1024),
                       make_smem_desc_sw128(sk + b_off, 16, 1024), idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t a_off = (kk / 4) * (BM * 128) + (kk % 4) * 32;
          const uint32_t b_off = (kk / 4) * (BN * 128) + (kk % 4) * 32;
          umma_bf16_ss(tmem_base + C::COL_DP, make_smem_desc_sw128(sdo + a_off, 16, 1024),
                       make_smem_desc_sw128(sv + b_off, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(smem_u32(bar_s));
        umma_commit(smem_u32(&bar_vfree[stage]));
      };
      bool ok = mbar_wait_bounded(smem_u32(bar_qdo), 0, cta_abort, p.status, 0x200 + 3);
      ok = ok && mbar_wait_bounded(smem_u32(&bar_k[0]), 0, cta_abort, p.status, 0x200 + 4);
      ok = ok && mbar_wait_bounded(smem_u32(&bar_v[0]), 0, cta_abort, p.status, 0x200 + 5);
      if (ok) { tc_fence_after(); issue_s_dp(0); }
      for (int j = 0; j < nblk && ok; ++j) {
        if (j + 1 < nblk) {
          const int ns = (j + 1) & 1, ph = ((j + 1) >> 1) & 1;
          ok = mbar_wait_bounded(smem_u32(bar_sfree), j & 1, cta_abort, p.status, 0x200 + 6);
          ok = ok && mbar_wait_bounded(smem_u32(&bar_k[ns]), ph, cta_abort, p.status, 0x200 + 7);
          ok = ok && mbar_wait_bounded(smem_u32(&bar_v[ns]), ph, cta_abort, p.status, 0x200 + 8);
          if (!ok) break;
          tc_fence_after();
          issue_s_dp(ns);
        }
        ok = mbar_wait_bounded(smem_u32(bar_ds), j & 1, cta_abort, p.status, 0x200 + 9);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sds = smem_u32(sdS), sk = smem_u32(sK + (j & 1) * C::KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {  // contraction over the BN keys
          const uint32_t a_off = (kk / 4) * (BM * 128) + (kk % 4) * 32;
          umma_bf16_ss(tmem_base + C::COL_DQ, make_smem_desc_sw128(sds + a_off, 16, 1024),
                       make_smem_desc_sw128(sk + kk * (16 * 128), BN * 128, 1024), idesc_dq, (j | kk) != 0);
        }
        umma_commit(smem_u32(bar_dq));
        umma_commit(smem_u32(&bar_kfree[j & 1]));
      }
    }
  } else {
    // ------------------------------------------------------------ math threads --
    const int r = warp * 32 + lane;
    const int q = q0 + r;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    const float LOG2E = 1.4426950408889634f;
    constexpr bool capped = (FEAT & AB2_SOFTCAP) != 0;
    const float cap_in = capped ? p.scale / p.softcap : 0.f;
    const float c_mul = capped ? p.softcap * LOG2E : p.scale * LOG2E;
    const bool row_ok = q < T;
    const size_t stat = ((size_t)b * p.Hq + h) * T + (row_ok ? q : 0);
    const float lse2 = row_ok ? __ldg(p.lse + stat) * LOG2E : INFINITY;  // +inf: p = 0 for rows outside the sequence
    const float dlt = row_ok ? __ldg(p.delta + stat) : 0.f;
    const int my_seq = ((FEAT & AB2_SEQ) && row_ok) ? __ldg(p.mask.seq_ids + row0 + q) : 0;
    int v_lo = 0, v_hi = T;
    if (p.mask.causal) {
      v_hi = min(T, q + 1);
      if (p.mask.window > 0) v_lo = max(0, q - p.mask.window + 1);
    } else if (p.mask.window > 0) {
      v_lo = max(0, q - p.mask.window + 1);
      v_hi = min(T, q + p.mask.window);
    }
    bool ok = true;
    for (int j = 0; j < nblk; ++j) {
      ok = mbar_wait_bounded(smem_u32(bar_s), j & 1, cta_abort, p.status, 0x200 + 10);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t s[BN], dp[BN];
      tmem_ld_row<BN>(t_row + C::COL_S, s);
      tmem_ld_row<BN>(t_row + C::COL_DP, dp);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(bar_sfree));
      bwd_p_ds_row<BN, capped>(s, dp, c_mul, cap_in, lse2, dlt);
      const int kbase = (jb_lo + j) * BN;
      if (attn_block_needs_mask(p.mask, q0, BM, kbase, BN)) {
        const int lo_rel = v_lo - kbase;
        const unsigned span = (unsigned)max(0, v_hi - v_lo);
#pragma unroll
        for (int i = 0; i < BN; ++i)
          if ((unsigned)(i - lo_rel) >= span) dp[i] = 0u;
        if (FEAT & AB2_SEQ) {
#pragma unroll
          for (int i = 0; i < BN; ++i)
            if (__ldg(p.mask.seq_ids + row0 + min(kbase + i, T - 1)) != my_seq) dp[i] = 0u;
        }
      }
      if (j > 0) {  // the previous dQ product must have finished reading the dS tile
        ok = mbar_wait_bounded(smem_u32(bar_dq), (j - 1) & 1, cta_abort, p.status, 0x200 + 11);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
#pragma unroll
      for (int c = 0; c < BN / 8; ++c) {
        const uint32_t* e = &dp[c * 8];
        st_swizzled_row_chunk(sdS, BM, r, c,
                              make_uint4(pack_bf16x2(__uint_as_float(e[0]), __uint_as_float(e[1])),
                                         pack_bf16x2(__uint_as_float(e[2]), __uint_as_float(e[3])),
                                         pack_bf16x2(__uint_as_float(e[4]), __uint_as_float(e[5])),
                                         pack_bf16x2(__uint_as_float(e[6]), __uint_as_float(e[7]))));
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(bar_ds));
    }
    if (ok && nblk > 0) {
      ok = mbar_wait_bounded(smem_u32(bar_dq), (nblk - 1) & 1, cta_abort, p.status, 0x200 + 12);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* drow = p.dq + (size_t)(row0 + q) * p.ld_dq + h * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        if (nblk > 0) {
          tmem_ld_32x32(t_row + C::COL_DQ + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(o[g * 8]) * p.scale, __uint_as_float(o[g * 8 + 1]) * p.scale);
            u.y = pack_bf16x2(__uint_as_float(o[g * 8 + 2]) * p.scale, __uint_as_float(o[g * 8 + 3]) * p.scale);
            u.z = pack_bf16x2(__uint_as_float(o[g * 8 + 4]) * p.scale, __uint_as_float(o[g * 8 + 5]) * p.scale);
            u.w = pack_bf16x2(__uint_as_float(o[g * 8 + 6]) * p.scale, __uint_as_float(o[g * 8 + 7]) * p.scale);
            *reinterpret_cast<uint4*>(drow + c * 32 + g * 8) = u;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*cta_abort) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == AV2_MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------- dK, dV --
template <int D>
struct AttnDkvCfg {
  static constexpr int BK = 128, BQ = 64;                // keys per CTA, queries per step
  static constexpr uint32_t KV_BYTES = BK * D * 2;       // K tile, V tile (resident)
  static constexpr uint32_t QD_BYTES = BQ * D * 2;       // one Q or dO tile
  static constexpr uint32_t PT_BYTES = BK * BQ * 2;      // P^T tile, dS^T tile
  static constexpr uint32_t STAT_BYTES = 4 * 3 * BQ * 4; // per math warp: lse, delta, sequence id of the step's queries
  static constexpr uint32_t SMEM = 2 * KV_BYTES + 2 * 2 * QD_BYTES + 2 * PT_BYTES + STAT_BYTES + 256;
  static constexpr uint32_t COL_S = 0, COL_DP = BQ, COL_DV = 2 * BQ, COL_DK = 2 * BQ + D;
  static constexpr uint32_t TMEM_COLS = (2 * BQ + 2 * D <= 256) ? 256 : 512;
  static constexpr int CTAS_PER_SM = (SMEM <= 112 * 1024 && TMEM_COLS == 256) ? 2 : 1;
};

template <int D, int FEAT>
__global__ void __launch_bounds__(AV2_THREADS, (AttnDkvCfg<D>::CTAS_PER_SM))
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                    const AttnBwd2Params p) {
  using C = AttnDkvCfg<D>;
  constexpr int BK = C::BK, BQ = C::BQ;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  {
    uint32_t dyn;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
    if (static_cast<uint32_t>(smem - smem_raw) + C::SMEM > dyn) {
      if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, NFN_ERR_WAIT_MISC);
      return;
    }
  }
  uint8_t* sK = smem;
  uint8_t* sV = sK + C::KV_BYTES;
  uint8_t* sQ = sV + C::KV_BYTES;                  // [2] stages
  uint8_t* sdO = sQ + 2 * C::QD_BYTES;             // [2] stages
  uint8_t* sP = sdO + 2 * C::QD_BYTES;
  uint8_t* sdS = sP + C::PT_BYTES;
  float* s_stat = reinterpret_cast<float*>(sdS + C::PT_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(s_stat) + C::STAT_BYTES);
  uint64_t* bar_kv = bars;          // TMA: K and V landed
  uint64_t* bar_qdo = bars + 1;     // [2] TMA: Q / dO stage landed
  uint64_t* bar_qfree = bars + 3;   // [2] MMA: dV / dK of the step retired (stage free); producer only
  uint64_t* bar_s = bars + 5;       // MMA: S^T and dP^T complete
  uint64_t* bar_sfree = bars + 6;   // 4 arrivals: S^T / dP^T are in registers
  uint64_t* bar_pds = bars + 7;     // 4 arrivals: P^T and dS^T are in shared memory
  uint64_t* bar_out = bars + 8;     // MMA: dV / dK of the step retired (P^T / dS^T tiles free)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jb = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int k0 = jb * BK;
  const int T = p.mask.T;
  int q_lo, q_hi;
  attn_query_range(p.mask, k0, BK, q_lo, q_hi);
  const int i_lo = q_lo / BQ;
  const int nqb = max(0, (q_hi + BQ - 1) / BQ - i_lo);   // query tiles per head
  const int nsteps = nqb * G;

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    mbar_init(smem_u32(bar_kv), 1);
    for (int s2 = 0; s2 < 2; ++s2) {
      mbar_init(smem_u32(&bar_qdo[s2]), 1);
      mbar_init(smem_u32(&bar_qfree[s2]), 1);
    }
    mbar_init(smem_u32(bar_s), 1);
    mbar_init(smem_u32(bar_sfree), AV2_MATH_WARPS);
    mbar_init(smem_u32(bar_pds), AV2_MATH_WARPS);
    mbar_init(smem_u32(bar_out), 1);
    fence_mbar_init();
  }
  if (warp == AV2_MMA_WARP) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int row0 = b * T;

  if (warp == AV2_TMA_WARP) {
    if (lane == 0 && nsteps > 0) {
      auto load_qdo = [&](int s, int stage) {
        const int hq = hk * G + s / nqb;
        const int qrow = row0 + (i_lo + s % nqb) * BQ;
        const uint32_t fb = smem_u32(&bar_qdo[stage]);
        mbar_expect_tx(fb, 2 * C::QD_BYTES);
#pragma unroll
        for (int d = 0; d < D / 64; ++d) {
          tma_load_2d(smem_u32(sQ + stage * C::QD_BYTES) + d * (BQ * 128), &tm_q, fb, hq * D + d * 64, qrow);
          tma_load_2d(smem_u32(sdO + stage * C::QD_BYTES) + d * (BQ * 128), &tm_do, fb, hq * D + d * 64, qrow);
        }
      };
      mbar_expect_tx(smem_u32(bar_kv), 2 * C::KV_BYTES);
#pragma unroll
      for (int d = 0; d < D / 64; ++d) {
        tma_load_2d(smem_u32(sK) + d * (BK * 128), &tm_k, smem_u32(bar_kv), hk * D + d * 64, row0 + k0);
        tma_load_2d(smem_u32(sV) + d * (BK * 128), &tm_v, smem_u32(bar_kv), hk * D + d * 64, row0 + k0);
      }
      load_qdo(0, 0);
      if (nsteps > 1) load_qdo(1, 1);
      for (int s = 0; s + 2 < nsteps; ++s) {
        if (!mbar_wait_bounded(smem_u32(&bar_qfree[s & 1]), (s >> 1) & 1, cta_abort, p.status, 0x300 + 1)) break;
        load_qdo(s + 2, s & 1);
      }
    }
  } else if (warp == AV2_MMA_WARP) {
    if (lane == 0 && nsteps > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BK, BQ, 0, 0);   // S^T, dP^T
      constexpr uint32_t idesc_g = make_idesc_bf16(BK, D, 0, 1);    // dV, dK: A K-major, B MN-major
      auto issue_s_dp = [&](int stage) {
        const uint32_t sk = smem_u32(sK), sv = smem_u32(sV);
        const uint32_t sq = smem_u32(sQ + stage * C::QD_BYTES), sdo = smem_u32(sdO + stage * C::QD_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t a_off = (kk / 4) * (BK * 128) + (kk % 4) * 32;
          const uint32_t b_off = (kk / 4) * (BQ * 128) + (kk % 4) * 32;
          umma_bf16_ss(tmem_base + C::COL_S, make_smem_desc_sw128(sk + a_off, 16, 1024),
                       make_smem_desc_sw128(sq + b_off, 16, 1024), idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t a_off = (kk / 4) * (BK * 128) + (kk % 4) * 32;
          const uint32_t b_off = (kk / 4) * (BQ * 128) + (kk % 4) * 32;
          umma_bf16_ss(tmem_base + C::COL_DP, make_smem_desc_sw128(sv + a_off, 16, 1024),
                       make_smem_desc_sw128(sdo + b_off, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(smem_u32(bar_s));
      };
      bool ok = mbar_wait_bounded(smem_u32(bar_kv), 0, cta_abort, p.status, 0x300 + 2);
      ok = ok && mbar_wait_bounded(smem_u32(&bar_qdo[0]), 0, cta_abort, p.status, 0x300 + 3);
      if (ok) { tc_fence_after(); issue_s_dp(0); }
      for (int s = 0; s < nsteps && ok; ++s) {
        if (s + 1 < nsteps) {
          const int ns = (s + 1) & 1;
          ok = mbar_wait_bounded(smem_u32(bar_sfree), s & 1, cta_abort, p.status, 0x300 + 4);
          ok = ok && mbar_wait_bounded(smem_u32(&bar_qdo[ns]), ((s + 1) >> 1) & 1, cta_abort, p.status, 0x300 + 5);
          if (!ok) break;
          tc_fence_after();
          issue_s_dp(ns);
        }
        ok = mbar_wait_bounded(smem_u32(bar_pds), s & 1, cta_abort, p.status, 0x300 + 6);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sp = smem_u32(sP), sds = smem_u32(sdS);
        const uint32_t sq = smem_u32(sQ + (s & 1) * C::QD_BYTES), sdo = smem_u32(sdO + (s & 1) * C::QD_BYTES);
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk) {  // contraction over the BQ queries
          const uint32_t a_off = (kk / 4) * (BK * 128) + (kk % 4) * 32;
          umma_bf16_ss(tmem_base + C::COL_DV, make_smem_desc_sw128(sp + a_off, 16, 1024),
                       make_smem_desc_sw128(sdo + kk * (16 * 128), BQ * 128, 1024), idesc_g, (s | kk) != 0);
        }
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk) {
          const uint32_t a_off = (kk / 4) * (BK * 128) + (kk % 4) * 32;
          umma_bf16_ss(tmem_base + C::COL_DK, make_smem_desc_sw128(sds + a_off, 16, 1024),
                       make_smem_desc_sw128(sq + kk * (16 * 128), BQ * 128, 1024), idesc_g, (s | kk) != 0);
        }
        umma_commit(smem_u32(bar_out));
        umma_commit(smem_u32(&bar_qfree[s & 1]));
      }
    }
  } else {
    // ------------------------------------------------------------ math threads --
    const int r = warp * 32 + lane;      // key row within the block == TMEM lane
    const int kidx = k0 + r;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    const float LOG2E = 1.4426950408889634f;
    constexpr bool capped = (FEAT & AB2_SOFTCAP) != 0;
    const float cap_in = capped ? p.scale / p.softcap : 0.f;
    const float c_mul = capped ? p.softcap * LOG2E : p.scale * LOG2E;
    const bool row_ok = kidx < T;
    const int my_seq = ((FEAT & AB2_SEQ) && row_ok) ? __ldg(p.mask.seq_ids + row0 + kidx) : 0;
    // queries that can see this key form one interval [v_lo, v_hi)
    int v_lo = 0, v_hi = row_ok ? T : 0;
    if (row_ok) {
      if (p.mask.causal) {
        v_lo = kidx;
        if (p.mask.window > 0) v_hi = min(T, kidx + p.mask.window);
      } else if (p.mask.window > 0) {
        v_lo = max(0, kidx - p.mask.window + 1);
        v_hi = min(T, kidx + p.mask.window);
      }
    }
    // every warp keeps a private copy of the step's per-query statistics (warp-level sync only)
    float* st_lse = s_stat + warp * (3 * BQ);
    float* st_dlt = st_lse + BQ;
    int* st_seq = reinterpret_cast<int*>(st_dlt + BQ);
    float nx_lse[BQ / 32], nx_dlt[BQ / 32];
    int nx_seq[BQ / 32];
    auto fetch_stats = [&](int s2) {
      const int hq2 = hk * G + s2 / nqb;
      const int q02 = (i_lo + s2 % nqb) * BQ;
#pragma unroll
      for (int e = 0; e < BQ / 32; ++e) {
        const int q = q02 + e * 32 + lane;
        const size_t idx = ((size_t)b * p.Hq + hq2) * T + q;
        nx_lse[e] = q < T ? __ldg(p.lse + idx) * LOG2E : INFINITY;
        nx_dlt[e] = q < T ? __ldg(p.delta + idx) : 0.f;
        nx_seq[e] = ((FEAT & AB2_SEQ) && q < T) ? __ldg(p.mask.seq_ids + row0 + q) : -1;
      }
    };
    bool ok = true;
    if (nsteps > 0) fetch_stats(0);
    for (int s = 0; s < nsteps; ++s) {
      const int q0 = (i_lo + s % nqb) * BQ;
      __syncwarp();  // every lane finished reading the previous step's statistics
#pragma unroll
      for (int e = 0; e < BQ / 32; ++e) {
        st_lse[e * 32 + lane] = nx_lse[e];
        st_dlt[e * 32 + lane] = nx_dlt[e];
        if (FEAT & AB2_SEQ) st_seq[e * 32 + lane] = nx_seq[e];
      }
      __syncwarp();
      ok = mbar_wait_bounded(smem_u32(bar_s), s & 1, cta_abort, p.status, 0x300 + 7);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sv_[BQ], dp[BQ];
      tmem_ld_row<BQ>(t_row + C::COL_S, sv_);
      tmem_ld_row<BQ>(t_row + C::COL_DP, dp);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(bar_sfree));
      if (s + 1 < nsteps) fetch_stats(s + 1);  // latency hidden behind the exponentials
      uint32_t th[capped ? BQ : 2];
      if (capped) {
#pragma unroll
        for (int i = 0; i < BQ; ++i) {
          th[i] = __float_as_uint(fast_tanh(__uint_as_float(sv_[i]) * cap_in));
          sv_[i] = th[i];
        }
      }
      // separate passes (exponent, ex2, product): neighbouring instructions are independent
#pragma unroll
      for (int i = 0; i < BQ; i += 4) {
        const float4 l4 = *reinterpret_cast<const float4*>(st_lse + i);
        sv_[i] = __float_as_uint(fmaf(__uint_as_float(sv_[i]), c_mul, -l4.x));
        sv_[i + 1] = __float_as_uint(fmaf(__uint_as_float(sv_[i + 1]), c_mul, -l4.y));
        sv_[i + 2] = __float_as_uint(fmaf(__uint_as_float(sv_[i + 2]), c_mul, -l4.z));
        sv_[i + 3] = __float_as_uint(fmaf(__uint_as_float(sv_[i + 3]), c_mul, -l4.w));
      }
#pragma unroll
      for (int i = 0; i < BQ; ++i) sv_[i] = __float_as_uint(fast_exp2(__uint_as_float(sv_[i])));
#pragma unroll
      for (int i = 0; i < BQ; i += 4) {
        const float4 d4 = *reinterpret_cast<const float4*>(st_dlt + i);
        const float dv[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float de = (__uint_as_float(dp[i + e]) - dv[e]) * __uint_as_float(sv_[i + e]);
          if (capped) de *= 1.f - __uint_as_float(th[i + e]) * __uint_as_float(th[i + e]);
          dp[i + e] = __float_as_uint(de);
        }
      }
      if (attn_block_needs_mask(p.mask, q0, BQ, k0, BK)) {
        const int lo_rel = v_lo - q0;
        const unsigned span = (unsigned)max(0, v_hi - v_lo);
#pragma unroll
        for (int i = 0; i < BQ; ++i)
          if ((unsigned)(i - lo_rel) >= span) { sv_[i] = 0u; dp[i] = 0u; }
        if (FEAT & AB2_SEQ) {
#pragma unroll
          for (int i = 0; i < BQ; ++i)
            if (st_seq[i] != my_seq) { sv_[i] = 0u; dp[i] = 0u; }
        }
      }
      if (s > 0) {  // the previous step's dV / dK products must have finished reading the tiles
        ok = mbar_wait_bounded(smem_u32(bar_out), (s - 1) & 1, cta_abort, p.status, 0x300 + 8);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
#pragma unroll
      for (int c = 0; c < BQ / 8; ++c) {
        const uint32_t* e = &sv_[c * 8];
        const uint32_t* f = &dp[c * 8];
        st_swizzled_row_chunk(sP, BK, r, c,
                              make_uint4(pack_bf16x2(__uint_as_float(e[0]), __uint_as_float(e[1])),
                                         pack_bf16x2(__uint_as_float(e[2]), __uint_as_float(e[3])),
                                         pack_bf16x2(__uint_as_float(e[4]), __uint_as_float(e[5])),
                                         pack_bf16x2(__uint_as_float(e[6]), __uint_as_float(e[7]))));
        st_swizzled_row_chunk(sdS, BK, r, c,
                              make_uint4(pack_bf16x2(__uint_as_float(f[0]), __uint_as_float(f[1])),
                                         pack_bf16x2(__uint_as_float(f[2]), __uint_as_float(f[3])),
                                         pack_bf16x2(__uint_as_float(f[4]), __uint_as_float(f[5])),
                                         pack_bf16x2(__uint_as_float(f[6]), __uint_as_float(f[7]))));
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(bar_pds));
    }
    if (ok && nsteps > 0) {
      ok = mbar_wait_bounded(smem_u32(bar_out), (nsteps - 1) & 1, cta_abort, p.status, 0x300 + 9);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* dkrow = p.dk + (size_t)(row0 + kidx) * p.ld_dk + hk * D;
      __nv_bfloat16* dvrow = p.dv + (size_t)(row0 + kidx) * p.ld_dv + hk * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t a[32], g[32];
        if (nsteps > 0) {
          tmem_ld_32x32(t_row + C::COL_DV + c * 32, a);
          tmem_ld_32x32(t_row + C::COL_DK + c * 32, g);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) { a[i] = 0u; g[i] = 0u; }
        }
        if (row_ok) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint4 u, w;
            u.x = pack_bf16x2(__uint_as_float(a[8 * e]), __uint_as_float(a[8 * e + 1]));
            u.y = pack_bf16x2(__uint_as_float(a[8 * e + 2]), __uint_as_float(a[8 * e + 3]));
            u.z = pack_bf16x2(__uint_as_float(a[8 * e + 4]), __uint_as_float(a[8 * e + 5]));
            u.w = pack_bf16x2(__uint_as_float(a[8 * e + 6]), __uint_as_float(a[8 * e + 7]));
            w.x = pack_bf16x2(__uint_as_float(g[8 * e]) * p.scale, __uint_as_float(g[8 * e + 1]) * p.scale);
            w.y = pack_bf16x2(__uint_as_float(g[8 * e + 2]) * p.scale, __uint_as_float(g[8 * e + 3]) * p.scale);
            w.z = pack_bf16x2(__uint_as_float(g[8 * e + 4]) * p.scale, __uint_as_float(g[8 * e + 5]) * p.scale);
            w.w = pack_bf16x2(__uint_as_float(g[8 * e + 6]) * p.scale, __uint_as_float(g[8 * e + 7]) * p.scale);
            reinterpret_cast<uint4*>(dvrow + c * 32)[e] = u;
            reinterpret_cast<uint4*>(dkrow + c * 32)[e] = w;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*cta_abort) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == AV2_MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

int attention_impl();  // attention_fwd2.cu

template <typename Kern>
static int set_smem_attr(Kern kern, size_t smem, bool* done) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (!done[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -1;
    done[dev & 63] = true;
  }
  return 0;
}

template <int D, int FEAT>
static int launch_attn_bwd2(const nfn_attention_args& a, cudaStream_t st) {
  using CQ = AttnDqCfg<D>;
  using CK = AttnDkvCfg<D>;
  auto kern_dkv = attn_bwd_dkv_kernel<D, FEAT>;
  auto kern_dq = attn_bwd_dq_kernel<D, FEAT>;
  static bool attr_dkv[64] = {}, attr_dq[64] = {};
  if (set_smem_attr(kern_dkv, CK::SMEM, attr_dkv) != 0) return launch_check("attn_bwd_dkv attr", 0);
  if (set_smem_attr(kern_dq, CQ::SMEM, attr_dq) != 0) return launch_check("attn_bwd_dq attr", 0);
  const long long rows = (long long)a.B * a.T;
  {
    const long long threads = rows * a.Hq * (D / 8);
    attn_delta2_kernel<D><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(
        (const __nv_bfloat16*)a.d_o, (const __nv_bfloat16*)a.o, a.delta, a.B, a.T, a.Hq, a.ld_do, a.ld_o);
  }
  AttnBwd2Params p;
  p.lse = a.lse; p.delta = a.delta;
  p.dq = (__nv_bfloat16*)a.dq; p.dk = (__nv_bfloat16*)a.dk; p.dv = (__nv_bfloat16*)a.dv;
  p.ld_dq = a.ld_dq; p.ld_dk = a.ld_dk; p.ld_dv = a.ld_dv;
  p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv;
  p.mask.T = a.T; p.mask.causal = a.causal; p.mask.window = a.window; p.mask.seq_ids = a.seq_ids;
  p.scale = a.scale; p.softcap = a.softcap;
  p.status = status_ptr();
  {
    // dK / dV: resident K, V tiles of 128 keys; Q / dO stream in 64-row tiles
    CUtensorMap tq, tk, tv, tdo;
    if (!make_tmap_2d(&tq, a.q, 2, (uint64_t)a.Hq * D, rows, a.ld_q, 64, CK::BQ, 128)) return -3;
    if (!make_tmap_2d(&tdo, a.d_o, 2, (uint64_t)a.Hq * D, rows, a.ld_do, 64, CK::BQ, 128)) return -3;
    if (!make_tmap_2d(&tk, a.k, 2, (uint64_t)a.Hkv * D, rows, a.ld_k, 64, CK::BK, 128)) return -3;
    if (!make_tmap_2d(&tv, a.v, 2, (uint64_t)a.Hkv * D, rows, a.ld_v, 64, CK::BK, 128)) return -3;
    dim3 grid(ceil_div(a.T, CK::BK), a.Hkv, a.B);
    kern_dkv<<<grid, AV2_THREADS, CK::SMEM, st>>>(tq, tk, tv, tdo, p);
  }
  {
    // dQ: resident Q, dO tiles of 128 queries; K / V stream in 64-row blocks
    CUtensorMap tq, tk, tv, tdo;
    if (!make_tmap_2d(&tq, a.q, 2, (uint64_t)a.Hq * D, rows, a.ld_q, 64, CQ::BM, 128)) return -3;
    if (!make_tmap_2d(&tdo, a.d_o, 2, (uint64_t)a.Hq * D, rows, a.ld_do, 64, CQ::BM, 128)) return -3;
    if (!make_tmap_2d(&tk, a.k, 2, (uint64_t)a.Hkv * D, rows, a.ld_k, 64, CQ::BN, 128)) return -3;
    if (!make_tmap_2d(&tv, a.v, 2, (uint64_t)a.Hkv * D, rows, a.ld_v, 64, CQ::BN, 128)) return -3;
    dim3 grid(ceil_div(a.T, CQ::BM), a.Hq, a.B);
    kern_dq<<<grid, AV2_THREADS, CQ::SMEM, st>>>(tq, tk, tv, tdo, p);
  }
  return launch_check("attn_bwd2", 3);
}

template <int D>
static int dispatch_attn_bwd2(const nfn_attention_args& a, cudaStream_t st) {
  const int feat = (a.seq_ids ? AB2_SEQ : 0) | (a.softcap > 0.f ? AB2_SOFTCAP : 0);
  switch (feat) {
    case 0: return launch_attn_bwd2<D, 0>(a, st);
    case AB2_SEQ: return launch_attn_bwd2<D, AB2_SEQ>(a, st);
    case AB2_SOFTCAP: return launch_attn_bwd2<D, AB2_SOFTCAP>(a, st);
    default: return launch_attn_bwd2<D, AB2_SEQ | AB2_SOFTCAP>(a, st);
  }
}

}  // namespace nfn

using namespace nfn;

extern "C" int nfn_attention_backward_v1(const void* dout, const void* q, const void* k, const void* v,
                                         const void* o, const float* lse, float* delta, float* dq_accum,
                                         void* dq, void* dk, void* dv, int B, int T, int Hq, int Hkv,
                                         int D, int ld_do, int ld_q, int ld_k, int ld_v, int ld_o,
                                         int ld_dq, int ld_dk, int ld_dv, int causal, int window,
                                         float scale, nfn_stream_t stream);

extern "C" int nfn_attention_backward_ex(const nfn_attention_args* args, nfn_stream_t stream) {
  if (!args) return fail(-1, "attention_backward: null args");
  const nfn_attention_args& a = *args;
  if (a.B <= 0 || a.T <= 0) return 0;
  if (a.Hkv <= 0 || a.Hq % a.Hkv) return fail(-1, "attention_backward: Hq must be a multiple of Hkv");
  if ((a.ld_do | a.ld_q | a.ld_k | a.ld_v | a.ld_o | a.ld_dq | a.ld_dk | a.ld_dv) & 7)
    return fail(-1, "attention_backward: row strides must be multiples of 8");
  if (!a.d_o || !a.q || !a.k || !a.v || !a.o || !a.lse || !a.delta || !a.dq || !a.dk || !a.dv)
    return fail(-1, "attention_backward: null operand");
  if ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) | reinterpret_cast<uintptr_t>(a.v) |
       reinterpret_cast<uintptr_t>(a.d_o) | reinterpret_cast<uintptr_t>(a.dq) | reinterpret_cast<uintptr_t>(a.dk) |
       reinterpret_cast<uintptr_t>(a.dv)) & 15)
    return fail(-1, "attention_backward: operands must be 16-byte aligned");
  if (a.gate) return fail(-1, "attention_backward: the output gate is a forward-only epilogue");
  if (a.softcap < 0.f) return fail(-1, "attention_backward: softcap must be >= 0");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a.D == 64) return dispatch_attn_bwd2<64>(a, st);
  if (a.D == 128) return dispatch_attn_bwd2<128>(a, st);
  return fail(-1, "attention_backward: head_dim must be 64 or 128");
}

// dq_accum (fp32 [B*T, Hq*D]) is only used by the first-generation kernel.
extern "C" int nfn_attention_backward(const void* dout, const void* q, const void* k, const void* v,
                                      const void* o, const float* lse, float* delta, float* dq_accum,
                                      void* dq, void* dk, void* dv, int B, int T, int Hq, int Hkv,
                                      int D, int ld_do, int ld_q, int ld_k, int ld_v, int ld_o,
                                      int ld_dq, int ld_dk, int ld_dv, int causal, int window,
                                      float scale, nfn_stream_t stream) {
  if (attention_impl() == 1 && dq_accum)
    return nfn_attention_backward_v1(dout, q, k, v, o, lse, delta, dq_accum, dq, dk, dv, B, T, Hq, Hkv, D, ld_do, ld_q,
                                     ld_k, ld_v, ld_o, ld_dq, ld_dk, ld_dv, causal, window, scale, stream);
  nfn_attention_args a = {};
  a.q = q; a.k = k; a.v = v; a.o = const_cast<void*>(o); a.lse = const_cast<float*>(lse);
  a.B = B; a.T = T; a.Hq = Hq; a.Hkv = Hkv; a.D = D;
  a.ld_q = ld_q; a.ld_k = ld_k; a.ld_v = ld_v; a.ld_o = ld_o;
  a.causal = causal; a.window = window; a.scale = scale;
  a.d_o = dout; a.ld_do = ld_do; a.delta = delta;
  a.dq = dq; a.dk = dk; a.dv = dv; a.ld_dq = ld_dq; a.ld_dk = ld_dk; a.ld_dv = ld_dv;
  return nfn_attention_backward_ex(&a, stream);
}
