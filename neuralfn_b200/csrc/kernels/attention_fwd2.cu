// Flash-attention forward on tcgen05 (sm_100a), pipelined version.
//
// One CTA handles a 128-query tile of one (batch, head); two CTAs share an SM. Roles:
//   warps 0-3  softmax: one thread per query row (== TMEM lane). The thread reads its whole row of
//              S out of TMEM at once, hands the S columns back to the MMA warp straight away, and
//              then computes max / exp2 / sum in registers and writes P (bf16) into a swizzled
//              shared-memory tile.
//   warp 4     MMA issuer:  S_{j+1} = Q K_{j+1}^T as soon as S_j has been read (so it runs under the
//              exponentials of block j), then O += P_j V_j once P_j is in shared memory.
//   warp 5     TMA producer: Q once, K/V through a two-stage ring.
// The running output stays in TMEM. It is rescaled only when some row's maximum grew by more than
// 2^8 since the last rescale (the reference maximum may lag behind the true one; the final division
// by the row sum, kept under the same lagging maximum, makes the result exact), so the common
// iteration has no read-modify-write of O at all.
//
// Mask options: causal, sliding window, bidirectional window, packed-sequence ids; optional score
// soft-cap cap * tanh(s * scale / cap); optional sigmoid output gate; grouped-query heads; head_dim
// 64 (128 keys per iteration) and 128 (64 keys per iteration); arbitrary row strides (packed QKV).
// Writes O (bf16) and the log-sum-exp per row (fp32) for the backward pass.
//
// Reference counterparts: ThunderKittens launch_forward_causal call sites and the scalar attention
// kernels (neuralfn/csrc/tile_cuda/kernels.cu:5649-5838, 22305-22402, 3266-3344; sequence-id mask
// :3299-3301).
#include "attention_v2.cuh"
#include "kernel_timers.cuh"

namespace nfn {

struct AttnFwd2Params {
  __nv_bfloat16* o;
  float* lse;
  const __nv_bfloat16* gate;  // optional [rows, Hq*D]: o *= sigmoid(gate)
  int ld_o, ld_gate;
  int B, Hq, Hkv;
  AttnMask mask;
  float scale;       // softmax scale
  float softcap;     // 0: off
  int* status;
};

// FEAT bits: compiled-in options, so that the plain causal kernel carries no code for them
constexpr int AF_SEQ = 1;      // packed-sequence ids
constexpr int AF_SOFTCAP = 2;  // score soft-cap

template <int D, int BN_, bool P_TMEM_>
struct AttnFwd2Cfg {
  static constexpr int BM = 128;
  static constexpr int BN = BN_;
  static constexpr uint32_t Q_BYTES = BM * D * 2;
  static constexpr uint32_t K_BYTES = BN * D * 2;
  static constexpr uint32_t KV_STAGE = 2 * K_BYTES;
  // P (bf16 probabilities) is handed to the second product either through a swizzled
  // shared-memory tile (P_TMEM = false) or through TMEM columns as the A operand of a
  // TMEM-sourced MMA (P_TMEM = true: no shared-memory store, no proxy fence, and the product
  // reads only V from shared memory)
  static constexpr bool P_TMEM = P_TMEM_;
  static constexpr uint32_t P_BYTES = P_TMEM ? 0 : BM * BN * 2;
  static constexpr uint32_t SMEM = Q_BYTES + 2 * KV_STAGE + P_BYTES + 128;
  static constexpr uint32_t P_COL = BN;                                   // bf16 pairs: BN / 2 columns
  static constexpr uint32_t O_COL = P_TMEM ? BN + BN / 2 : BN;
  static constexpr uint32_t TMEM_COLS = (O_COL + D <= 128) ? 128 : 256;   // S: [0, BN)  [P]  O
  // CTAs per SM the kernel is compiled for: bounded by shared memory (227 KB), TMEM (512 columns)
  // and the register file (192 threads x 112 registers x 3)
  static constexpr int CTAS_PER_SM = (SMEM <= 72 * 1024 && TMEM_COLS == 128) ? 3 : 2;
};

template <int D, int BN_, int FEAT, bool P_TMEM_>
__global__ void __launch_bounds__(AV2_THREADS, (AttnFwd2Cfg<D, BN_, P_TMEM_>::CTAS_PER_SM))
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const AttnFwd2Params p) {
  using C = AttnFwd2Cfg<D, BN_, P_TMEM_>;
  constexpr int BM = C::BM, BN = C::BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  {
    uint32_t dyn;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
    if (static_cast<uint32_t>(smem - smem_raw) + C::SMEM > dyn) {
      if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, NFN_ERR_WAIT_MISC);
      return;
    }
  }
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + C::Q_BYTES;
  uint8_t* sP = sKV + 2 * C::KV_STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + C::P_BYTES);
  uint64_t* bar_q = bars;          // TMA: Q landed
  uint64_t* bar_k = bars + 1;      // [2] TMA: K stage landed
  uint64_t* bar_v = bars + 3;      // [2] TMA: V stage landed
  uint64_t* bar_s = bars + 5;      // MMA: S_j complete (frees K stage j & 1)
  uint64_t* bar_sfree = bars + 6;  // 4 arrivals: S_j is in registers, its TMEM columns are free
  uint64_t* bar_p = bars + 7;      // 4 arrivals: P_j in shared memory (and O rescaled if needed)
  uint64_t* bar_o = bars + 8;      // MMA: O += P_j V_j retired (frees V stage j & 1)
  uint64_t* bar_kfree = bars + 9;  // [2] MMA: the product that read K stage s retired (only the producer waits on these,
  uint64_t* bar_vfree = bars + 11; // [2]      per stage, so it can never fall a whole phase behind)
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
  const int jb_hi = (k_hi + BN - 1) / BN;
  const int nblk = max(0, jb_hi - jb_lo);

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    mbar_init(smem_u32(bar_q), 1);
    for (int s2 = 0; s2 < 2; ++s2) {
      mbar_init(smem_u32(&bar_k[s2]), 1);
      mbar_init(smem_u32(&bar_v[s2]), 1);
      mbar_init(smem_u32(&bar_kfree[s2]), 1);
      mbar_init(smem_u32(&bar_vfree[s2]), 1);
    }
    mbar_init(smem_u32(bar_s), 1);
    mbar_init(smem_u32(bar_sfree), AV2_MATH_WARPS);
    mbar_init(smem_u32(bar_p), AV2_MATH_WARPS);
    mbar_init(smem_u32(bar_o), 1);
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
  const int row0 = b * T;  // first token row of this batch in the [B*T, width] views

  if (warp == AV2_TMA_WARP) {
    // ------------------------------------------------------------ TMA producer --
    if (lane == 0 && nblk > 0) {
      // K and V have their own barriers: the K slot of block j is free as soon as S_j retired,
      // long before O += P_j V_j releases the V slot, so the next K can be in flight earlier
      auto load_k = [&](int j, int stage) {
        const uint32_t fb = smem_u32(&bar_k[stage]);
        const uint32_t sk = smem_u32(sKV + stage * C::KV_STAGE);
        mbar_expect_tx(fb, C::K_BYTES);
#pragma unroll
        for (int d = 0; d < D / 64; ++d)
          tma_load_2d(sk + d * (BN * 128), &tm_k, fb, hk * D + d * 64, row0 + (jb_lo + j) * BN);
      };
      auto load_v = [&](int j, int stage) {
        const uint32_t fb = smem_u32(&bar_v[stage]);
        const uint32_t sv = smem_u32(sKV + stage * C::KV_STAGE + C::K_BYTES);
        mbar_expect_tx(fb, C::K_BYTES);
#pragma unroll
        for (int d = 0; d < D / 64; ++d)
          tma_load_2d(sv + d * (BN * 128), &tm_v, fb, hk * D + d * 64, row0 + (jb_lo + j) * BN);
      };
      mbar_expect_tx(smem_u32(bar_q), C::Q_BYTES);
#pragma unroll
      for (int d = 0; d < D / 64; ++d)
        tma_load_2d(smem_u32(sQ) + d * (BM * 128), &tm_q, smem_u32(bar_q), h * D + d * 64, row0 + q0);
      load_k(0, 0);
      load_v(0, 0);
      if (nblk > 1) { load_k(1, 1); load_v(1, 1); }
      for (int j = 0; j + 2 < nblk; ++j) {
        if (!mbar_wait_bounded(smem_u32(&bar_kfree[j & 1]), (j >> 1) & 1, cta_abort, p.status, 0x100 + 1)) break;
        load_k(j + 2, j & 1);
        if (!mbar_wait_bounded(smem_u32(&bar_vfree[j & 1]), (j >> 1) & 1, cta_abort, p.status, 0x100 + 2)) break;
        load_v(j + 2, j & 1);
      }
    }
  } else if (warp == AV2_MMA_WARP) {
    // -------------------------------------------------------------- MMA issuer --
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BM, BN, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(BM, D, 0, 1);
      auto issue_s = [&](int stage) {
        const uint32_t sq = smem_u32(sQ);
        const uint32_t sk = smem_u32(sKV + stage * C::KV_STAGE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t a_off = (kk / 4) * (BM * 128) + (kk % 4) * 32;
          const uint32_t b_off = (kk / 4) * (BN * 128) + (kk % 4) * 32;
          umma_bf16_ss(tmem_base, make_smem_desc_sw128(sq + a_off, 16, 1024),
                       make_smem_desc_sw128(sk + b_off, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(smem_u32(bar_s));
        umma_commit(smem_u32(&bar_kfree[stage]));
      };
      bool ok = mbar_wait_bounded(smem_u32(bar_q), 0, cta_abort, p.status, 0x100 + 3);
      ok = ok && mbar_wait_bounded(smem_u32(&bar_k[0]), 0, cta_abort, p.status, 0x100 + 4);
      if (ok) { tc_fence_after(); issue_s(0); }
      for (int j = 0; j < nblk && ok; ++j) {
        if (j + 1 < nblk) {
          const int ns = (j + 1) & 1;
          ok = mbar_wait_bounded(smem_u32(bar_sfree), j & 1, cta_abort, p.status, 0x100 + 5);
          ok = ok && mbar_wait_bounded(smem_u32(&bar_k[ns]), ((j + 1) >> 1) & 1, cta_abort, p.status,
                                       0x100 + 6);
          if (!ok) break;
          tc_fence_after();
          issue_s(ns);
        }
        ok = mbar_wait_bounded(smem_u32(bar_p), j & 1, cta_abort, p.status, 0x100 + 7);
        ok = ok && mbar_wait_bounded(smem_u32(&bar_v[j & 1]), (j >> 1) & 1, cta_abort, p.status, 0x100 + 8);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sp = smem_u32(sP);
        const uint32_t sv = smem_u32(sKV + (j & 1) * C::KV_STAGE + C::K_BYTES);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint32_t a_off = (kk / 4) * (BM * 128) + (kk % 4) * 32;
          const uint32_t b_off = kk * (16 * 128);
          if (C::P_TMEM)  // 16 keys of P = 8 TMEM columns of bf16 pairs
            umma_bf16_ts(tmem_base + C::O_COL, tmem_base + C::P_COL + kk * 8,
                         make_smem_desc_sw128(sv + b_off, BN * 128, 1024), idesc_o, (j | kk) != 0);
          else
            umma_bf16_ss(tmem_base + C::O_COL, make_smem_desc_sw128(sp + a_off, 16, 1024),
                         make_smem_desc_sw128(sv + b_off, BN * 128, 1024), idesc_o, (j | kk) != 0);
        }
        umma_commit(smem_u32(bar_o));
        umma_commit(smem_u32(&bar_vfree[j & 1]));
      }
    }
  } else {
    // --------------------------------------------------------- softmax threads --
    const int r = warp * 32 + lane;  // row within the tile == TMEM lane
    const int q = q0 + r;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    const float LOG2E = 1.4426950408889634f;
    // exponent = c_mul * f(s) with f = identity (c_mul = scale * log2 e) or tanh(s * cap_in) (c_mul = cap * log2 e)
    constexpr bool capped = (FEAT & AF_SOFTCAP) != 0;
    const float cap_in = capped ? p.scale / p.softcap : 0.f;
    const float c_mul = capped ? p.softcap * LOG2E : p.scale * LOG2E;
    const int my_seq = ((FEAT & AF_SEQ) && q < T) ? __ldg(p.mask.seq_ids + row0 + q) : 0;
    // visible keys of this row form one interval [v_lo, v_hi)
    int v_lo = 0, v_hi = T;
    if (p.mask.causal) {
      v_hi = min(T, q + 1);
      if (p.mask.window > 0) v_lo = max(0, q - p.mask.window + 1);
    } else if (p.mask.window > 0) {
      v_lo = max(0, q - p.mask.window + 1);
      v_hi = min(T, q + p.mask.window);
    }
    float m_run = -INFINITY, l_run = 0.f;  // m_run in units of f(s)
    bool ok = true;
    NFN_TIMER_DECL(8)
    for (int j = 0; j < nblk; ++j) {
      ok = mbar_wait_bounded(smem_u32(bar_s), j & 1, cta_abort, p.status, 0x100 + 9);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      NFN_TIMER_LAP(0)  // waiting for S
      uint32_t s[BN];
      tmem_ld_row<BN>(t_row, s);
      tmem_ld_wait();
      NFN_TIMER_LAP(1)  // TMEM load
      // the S columns can be overwritten by the next product from here on
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(bar_sfree));

      const int kbase = (jb_lo + j) * BN;
      if (capped) {
#pragma unroll
        for (int i = 0; i < BN; ++i) s[i] = __float_as_uint(fast_tanh(__uint_as_float(s[i]) * cap_in));
      }
      if (attn_block_needs_mask(p.mask, q0, BM, kbase, BN)) {
        const int lo_rel = v_lo - kbase;
        const unsigned span = (unsigned)max(0, v_hi - v_lo);
#pragma unroll
        for (int i = 0; i < BN; ++i)
          if ((unsigned)(i - lo_rel) >= span) s[i] = 0xff800000u;  // -inf
        if (FEAT & AF_SEQ) {
#pragma unroll
          for (int i = 0; i < BN; ++i) {
            const int k = min(kbase + i, T - 1);
            if (__ldg(p.mask.seq_ids + row0 + k) != my_seq) s[i] = 0xff800000u;
          }
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < BN; i += 8) {
        mx0 = fmax3(mx0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
        mx1 = fmax3(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
        mx2 = fmax3(mx2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
        mx3 = fmax3(mx3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
      }
      const float m_new = fmaxf(fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)), m_run);
      NFN_TIMER_LAP(2)  // mask + max
      // rescale only when some row of this warp moved its maximum by more than 2^8
      const bool grow = (m_new - m_run) * c_mul > 8.f;  // also true for -inf -> finite, false for -inf -> -inf
      const bool rescale = __any_sync(0xffffffffu, grow);
      float alpha = 1.f;
      if (rescale) {
        alpha = (m_run == -INFINITY) ? 0.f : fast_exp2((m_run - m_new) * c_mul);
        l_run *= alpha;
        m_run = m_new;
      }
      const float moff = (m_run == -INFINITY) ? 0.f : m_run * c_mul;
      // exponentials in place (fp32), row sum
      float l0 = 0.f, l1 = 0.f;
#pragma unroll
      // three passes over the row instead of one fused loop: within a pass every instruction is
      // independent of its neighbours, so a warp keeps the exponential unit fed back to back
      // instead of stalling on each ex2 result (there are only two such warps per scheduler)
      for (int i = 0; i < BN; i += 2) {
        float x0, x1;
        fma2_bcast(x0, x1, __uint_as_float(s[i]), __uint_as_float(s[i + 1]), c_mul, -moff);
        s[i] = __float_as_uint(x0);
        s[i + 1] = __float_as_uint(x1);
      }
#pragma unroll
      for (int i = 0; i < BN; ++i) s[i] = __float_as_uint(fast_exp2(__uint_as_float(s[i])));
      float l2 = 0.f, l3 = 0.f;
#pragma unroll
      for (int i = 0; i < BN; i += 4) {
        add2(l0, l1, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
        add2(l2, l3, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
      }
      l_run += (l0 + l1) + (l2 + l3);
      NFN_TIMER_LAP(3)  // exponentials
      if (j > 0) {
        // O += P_{j-1} V_{j-1} must have retired before P's tile is overwritten and before O is
        // rescaled; it was issued a whole block of exponentials ago, so this rarely waits
        ok = mbar_wait_bounded(smem_u32(bar_o), (j - 1) & 1, cta_abort, p.status, 0x100 + 10);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (rescale) {
#pragma unroll 1
          for (int c = 0; c < D / 16; ++c) {
            uint32_t o[16];
            tmem_ld_32x16(t_row + C::O_COL + c * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x16(t_row + C::O_COL + c * 16, o);
          }
          tmem_st_wait();
        }
      }
      NFN_TIMER_LAP(4)  // waiting for the previous PV (+ rescale)
      if (C::P_TMEM) {
        // pack in place: s[i] <- bf16x2(e[2i], e[2i+1]), then BN / 2 columns straight into TMEM
#pragma unroll
        for (int i = 0; i < BN / 2; ++i) s[i] = pack_bf16x2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1]));
#pragma unroll
        for (int c = 0; c < BN / 64; ++c)
          tmem_st_32x32(t_row + C::P_COL + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
        tmem_st_wait();
      } else {
#pragma unroll
        for (int c = 0; c < BN / 8; ++c) {
          const uint32_t* e = &s[c * 8];
          st_swizzled_row_chunk(sP, BM, r, c,
                                make_uint4(pack_bf16x2(__uint_as_float(e[0]), __uint_as_float(e[1])),
                                           pack_bf16x2(__uint_as_float(e[2]), __uint_as_float(e[3])),
                                           pack_bf16x2(__uint_as_float(e[4]), __uint_as_float(e[5])),
                                           pack_bf16x2(__uint_as_float(e[6]), __uint_as_float(e[7]))));
        }
        fence_proxy_async();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(bar_p));
      NFN_TIMER_LAP(5)  // P stores + fences
    }
    if (threadIdx.x == 0) { NFN_TIMER_FLUSH(0, 6) }
    // ---- epilogue: O / l -> global, log-sum-exp ----
    if (ok && nblk > 0) {
      ok = mbar_wait_bounded(smem_u32(bar_o), (nblk - 1) & 1, cta_abort, p.status, 0x100 + 11);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const bool row_ok = q < T;
      __nv_bfloat16* orow = p.o + (size_t)(row0 + q) * p.ld_o + h * D;
      const __nv_bfloat16* grow_ = p.gate ? p.gate + (size_t)(row0 + q) * p.ld_gate + h * D : nullptr;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        if (nblk > 0) {
          tmem_ld_32x32(t_row + C::O_COL + c * 32, o);  // warp-collective: every lane issues it
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(o[g * 8 + i]) * inv;
            if (grow_) {
              const uint4 gu = *reinterpret_cast<const uint4*>(grow_ + c * 32 + g * 8);
              const float2 g0 = unpack_bf16x2(gu.x), g1 = unpack_bf16x2(gu.y), g2 = unpack_bf16x2(gu.z), g3 = unpack_bf16x2(gu.w);
              const float gv[8] = {g0.x, g0.y, g1.x, g1.y, g2.x, g2.y, g3.x, g3.y};
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] *= 1.f / (1.f + __expf(-gv[i]));
            }
            uint4 u;
            u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]);
            u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
            *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = u;
          }
        }
      }
      if (p.lse && row_ok) {
        // natural-log units of the (capped, scaled) scores: m * c_mul / log2 e + log l
        const float mnat = (m_run == -INFINITY) ? 0.f : m_run * (c_mul / LOG2E);
        p.lse[((size_t)b * p.Hq + h) * T + q] = l_run > 0.f ? mnat + logf(l_run) : -INFINITY;
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

template <int D, int BN, int FEAT, bool P_TMEM>
static int launch_attn_fwd2(const nfn_attention_args& a, cudaStream_t st) {
  using C = AttnFwd2Cfg<D, BN, P_TMEM>;
  constexpr size_t SMEM = C::SMEM;
  auto kern = attn_fwd2_kernel<D, BN, FEAT, P_TMEM>;
  static bool attr[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess)
      return launch_check("attn_fwd2 attr", 0);
    attr[dev & 63] = true;
  }
  CUtensorMap tq, tk, tv;
  const uint64_t rows = (uint64_t)a.B * a.T;
  if (!make_tmap_2d(&tq, a.q, 2, (uint64_t)a.Hq * D, rows, a.ld_q, 64, C::BM, 128)) return -3;
  if (!make_tmap_2d(&tk, a.k, 2, (uint64_t)a.Hkv * D, rows, a.ld_k, 64, C::BN, 128)) return -3;
  if (!make_tmap_2d(&tv, a.v, 2, (uint64_t)a.Hkv * D, rows, a.ld_v, 64, C::BN, 128)) return -3;
  AttnFwd2Params p;
  p.o = (__nv_bfloat16*)a.o; p.lse = a.lse; p.ld_o = a.ld_o;
  p.gate = (const __nv_bfloat16*)a.gate; p.ld_gate = a.ld_gate;
  p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv;
  p.mask.T = a.T; p.mask.causal = a.causal; p.mask.window = a.window; p.mask.seq_ids = a.seq_ids;
  p.scale = a.scale; p.softcap = a.softcap;
  p.status = status_ptr();
  dim3 grid(ceil_div(a.T, C::BM), a.Hq, a.B);
  kern<<<grid, AV2_THREADS, SMEM, st>>>(tq, tk, tv, p);
  return launch_check("attn_fwd2");
}

static int g_attn_p_tmem = -1;  // NFN_ATTENTION_P_TMEM=1: P through TMEM (TMEM-sourced MMA) in the plain kernel
template <int D, int BN>
static int dispatch_attn_fwd2(const nfn_attention_args& a, cudaStream_t st) {
  if (g_attn_p_tmem < 0) { const char* e = getenv("NFN_ATTENTION_P_TMEM"); g_attn_p_tmem = (e && e[0] == '1') ? 1 : 0; }
  const int feat = (a.seq_ids ? AF_SEQ : 0) | (a.softcap > 0.f ? AF_SOFTCAP : 0);
  switch (feat) {
    case 0: return g_attn_p_tmem ? launch_attn_fwd2<D, BN, 0, true>(a, st) : launch_attn_fwd2<D, BN, 0, false>(a, st);
    case AF_SEQ: return launch_attn_fwd2<D, BN, AF_SEQ, false>(a, st);
    case AF_SOFTCAP: return launch_attn_fwd2<D, BN, AF_SOFTCAP, false>(a, st);
    default: return launch_attn_fwd2<D, BN, AF_SEQ | AF_SOFTCAP, false>(a, st);
  }
}

NFN_TIMER_EXPORT(nfn_attention_fwd_timers)

}  // namespace nfn
namespace nfn {

static int g_attn_impl = -1;  // 2 = pipelined kernels (default), 1 = first-generation kernels
int attention_impl() {
  if (g_attn_impl < 0) {
    const char* e = getenv("NFN_ATTENTION_IMPL");
    g_attn_impl = (e && e[0] == '1') ? 1 : 2;
  }
  return g_attn_impl;
}

}  // namespace nfn

using namespace nfn;

extern "C" int nfn_attention_forward_v1(const void* q, const void* k, const void* v, void* o, float* lse,
                                        int B, int T, int Hq, int Hkv, int D, int ld_q, int ld_k,
                                        int ld_v, int ld_o, int causal, int window, float scale,
                                        nfn_stream_t stream);

extern "C" int nfn_attention_set_impl(int impl) {
  const int old = attention_impl();
  g_attn_impl = (impl == 1) ? 1 : 2;
  return old;
}

extern "C" int nfn_attention_forward_ex(const nfn_attention_args* args, nfn_stream_t stream) {
  if (!args) return fail(-1, "attention: null args");
  const nfn_attention_args& a = *args;
  if (a.B <= 0 || a.T <= 0) return 0;
  if (a.Hkv <= 0 || a.Hq % a.Hkv) return fail(-1, "attention: Hq must be a multiple of Hkv");
  if ((a.ld_q | a.ld_k | a.ld_v | a.ld_o) & 7) return fail(-1, "attention: row strides must be multiples of 8");
  if ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) | reinterpret_cast<uintptr_t>(a.v) |
       reinterpret_cast<uintptr_t>(a.o)) & 15)
    return fail(-1, "attention: operands must be 16-byte aligned");
  if (a.gate && ((a.ld_gate & 7) || (reinterpret_cast<uintptr_t>(a.gate) & 15)))
    return fail(-1, "attention: gate must be 16-byte aligned with a row stride multiple of 8");
  if (a.softcap < 0.f) return fail(-1, "attention: softcap must be >= 0");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool plain = !a.seq_ids && a.softcap == 0.f && !a.gate;
  if (attention_impl() == 1 && plain)
    return nfn_attention_forward_v1(a.q, a.k, a.v, a.o, a.lse, a.B, a.T, a.Hq, a.Hkv, a.D, a.ld_q, a.ld_k, a.ld_v,
                                    a.ld_o, a.causal, a.window, a.scale, stream);
  if (a.D == 64) {
    static int bn = 0;  // keys per iteration at head_dim 64: 64 (default) or 128 (NFN_ATTENTION_BN=128)
    if (!bn) { const char* e = getenv("NFN_ATTENTION_BN"); bn = (e && atoi(e) == 128) ? 128 : 64; }
    return bn == 128 ? dispatch_attn_fwd2<64, 128>(a, st) : dispatch_attn_fwd2<64, 64>(a, st);
  }
  if (a.D == 128) return dispatch_attn_fwd2<128, 64>(a, st);
  return fail(-1, "attention: head_dim must be 64 or 128");
}

// q: bf16 rows [B*T] x (Hq*D) with row stride ld_q; k, v: rows x (Hkv*D); o: rows x (Hq*D).
// lse: optional fp32 [B, Hq, T].
extern "C" int nfn_attention_forward(const void* q, const void* k, const void* v, void* o, float* lse,
                                     int B, int T, int Hq, int Hkv, int D, int ld_q, int ld_k,
                                     int ld_v, int ld_o, int causal, int window, float scale,
                                     nfn_stream_t stream) {
  nfn_attention_args a = {};
  a.q = q; a.k = k; a.v = v; a.o = o; a.lse = lse;
  a.B = B; a.T = T; a.Hq = Hq; a.Hkv = Hkv; a.D = D;
  a.ld_q = ld_q; a.ld_k = ld_k; a.ld_v = ld_v; a.ld_o = ld_o;
  a.causal = causal; a.window = window; a.scale = scale;
  return nfn_attention_forward_ex(&a, stream);
}
