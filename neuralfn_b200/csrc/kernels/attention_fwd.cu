// Flash-attention forward on tcgen05 (sm_100a).
//
// One CTA handles a 128-query tile of one (batch, head). Warps 0-7 run the online softmax: two
// threads per query row (warps w and w + 4 share TMEM lane quarter w & 3), each taking half of the
// key columns of S and half of the output columns, so that every scheduler has two warps to
// interleave; the pair exchanges its half-row maxima (and, at the end, its half-row sums) through
// four spare TMEM columns behind a two-arrival mbarrier. Warp 8 is the control warp whose lane 0
// issues the TMA loads (Q once, K/V through a two-stage ring) and the two tensor-core
// products per key block:
//     S = Q K^T   (128 x 128 x D, accumulator in TMEM columns [0,128))
//     O_j = P V   (128 x D x 128, accumulator in TMEM columns [128,128+D))
// The softmax threads read S straight out of TMEM (two passes of 32-column slices:
// row max, then exp/sum), write P as bf16 into a 128-byte-swizzled shared tile that
// the second MMA consumes, and keep the running output in registers (rescaled by the
// usual exp(m_old - m_new) factor). Supports causal and bidirectional masks, sliding
// windows, grouped-query heads, head_dim 64 and 128, and arbitrary row strides
// (packed QKV). Writes O (bf16) and the log-sum-exp per row (fp32) for the backward.
//
// Reference counterparts: ThunderKittens launch_forward_causal call sites and the
// scalar attention kernels (neuralfn/csrc/tile_cuda/kernels.cu:5649-5838, 22305-22402,
// 3266-3344).
#include "common.h"
#include "sm100_ptx.cuh"

namespace nfn {

constexpr int ATT_BM = 128;  // queries per CTA
constexpr int ATT_BN = 128;  // keys per iteration
constexpr int ATT_SOFTMAX_WARPS = 8;
constexpr int ATT_CTRL_WARP = ATT_SOFTMAX_WARPS;
constexpr int ATT_THREADS = (ATT_SOFTMAX_WARPS + 1) * 32;

struct AttnFwdParams {
  __nv_bfloat16* o;
  float* lse;
  int ld_o;
  int B, T, Hq, Hkv;
  int causal;      // 1: keys <= query
  int window;      // 0: unlimited; W: causal keys in (q-W, q]; bidirectional |q-k| < W
  float scale_log2;  // softmax scale * log2(e)
  float scale;
  int* status;
};

// Shared memory one CTA needs (tiles + barriers). With head_dim 64 this is 112 KB + 128 B, so
// two CTAs share an SM (and its 512 TMEM columns, 256 each): while one CTA's softmax warps
// work on their S tile the other CTA's MMAs run, which hides most of the QK -> softmax -> PV
// dependency chain that a single resident CTA exposes.
template <int D>
__host__ __device__ constexpr uint32_t attn_fwd_smem_bytes() {
  return ATT_BM * D * 2 + 2 * (2 * ATT_BN * D * 2) + ATT_BM * ATT_BN * 2 + 128;
}

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, (D == 64 ? 2 : 1))
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const AttnFwdParams p) {
  constexpr uint32_t Q_BYTES = ATT_BM * D * 2;
  constexpr uint32_t K_BYTES = ATT_BN * D * 2;
  constexpr uint32_t V_BYTES = ATT_BN * D * 2;
  constexpr uint32_t P_BYTES = ATT_BM * ATT_BN * 2;
  constexpr uint32_t KV_STAGE = K_BYTES + V_BYTES;
  constexpr uint32_t TMEM_COLS = (D == 64) ? 256 : 512;  // S | O | four mailbox columns
  constexpr uint32_t O_COL = 128;
  constexpr uint32_t XCHG_COL = O_COL + D;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  {
    // The launch asks for exactly attn_fwd_smem_bytes<D>(): the dynamic window starts
    // 1024-aligned on this architecture. Should it ever not, give up cleanly (status word)
    // rather than run past the allocation.
    uint32_t dyn;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
    if (static_cast<uint32_t>(smem - smem_raw) + attn_fwd_smem_bytes<D>() > dyn) {
      if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, NFN_ERR_WAIT_MISC);
      return;
    }
  }
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + Q_BYTES;
  uint8_t* sP = sKV + 2 * KV_STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);
  uint64_t* bar_q = bars;          // 1
  uint64_t* bar_kv = bars + 1;     // 2
  uint64_t* bar_s = bars + 3;      // 1
  uint64_t* bar_p = bars + 4;      // 4 arrivals (one per softmax warp)
  uint64_t* bar_o = bars + 5;      // 1
  uint64_t* bar_pair = bars + 6;   // 4 (one per lane quarter), 2 arrivals each
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = gridDim.x - 1 - blockIdx.x;  // heavy (late) tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qb * ATT_BM;

  // key-block range visible to this query tile
  int k_lo = 0, k_hi = p.T;  // [k_lo, k_hi)
  if (p.causal) {
    k_hi = min(p.T, q0 + ATT_BM);
    if (p.window > 0) k_lo = max(0, q0 - p.window + 1);
  } else if (p.window > 0) {
    k_lo = max(0, q0 - p.window + 1);
    k_hi = min(p.T, q0 + ATT_BM - 1 + p.window);
  }
  const int jb_lo = k_lo / ATT_BN;
  const int jb_hi = (k_hi + ATT_BN - 1) / ATT_BN;
  const int nblk = jb_hi - jb_lo;

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    mbar_init(smem_u32(bar_q), 1);
    mbar_init(smem_u32(&bar_kv[0]), 1);
    mbar_init(smem_u32(&bar_kv[1]), 1);
    mbar_init(smem_u32(bar_s), 1);
    mbar_init(smem_u32(bar_p), ATT_SOFTMAX_WARPS);  // one arrival per softmax warp
    for (int qd = 0; qd < 4; ++qd) mbar_init(smem_u32(&bar_pair[qd]), 2);
    mbar_init(smem_u32(bar_o), 1);
    fence_mbar_init();
  }
  if (warp == ATT_CTRL_WARP) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == ATT_CTRL_WARP) {
    if (lane == 0) {
      // ------------------------------------------------------ control thread --
      const int row0 = b * p.T;  // first token row of this batch in the [B*T, width] views
      auto load_kv = [&](int j, int stage) {
        const uint32_t fb = smem_u32(&bar_kv[stage]);
        const uint32_t sk = smem_u32(sKV + stage * KV_STAGE);
        const uint32_t sv = sk + K_BYTES;
        mbar_expect_tx(fb, KV_STAGE);
        const int krow = row0 + (jb_lo + j) * ATT_BN;
#pragma unroll
        for (int d = 0; d < D / 64; ++d) {
          tma_load_2d(sk + d * (ATT_BN * 128), &tm_k, fb, hk * D + d * 64, krow);
          tma_load_2d(sv + d * (ATT_BN * 128), &tm_v, fb, hk * D + d * 64, krow);
        }
      };
      mbar_expect_tx(smem_u32(bar_q), Q_BYTES);
#pragma unroll
      for (int d = 0; d < D / 64; ++d)
        tma_load_2d(smem_u32(sQ) + d * (ATT_BM * 128), &tm_q, smem_u32(bar_q), h * D + d * 64,
                    row0 + q0);
      if (nblk > 0) load_kv(0, 0);
      if (nblk > 1) load_kv(1, 1);

      constexpr uint32_t idesc_s = make_idesc_bf16(ATT_BM, ATT_BN, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(ATT_BM, D, 0, 1);
      bool ok = mbar_wait_bounded(smem_u32(bar_q), 0, cta_abort, p.status, NFN_ERR_WAIT_FULL);
      auto issue_s = [&](int stage) {
        const uint32_t sq = smem_u32(sQ);
        const uint32_t sk = smem_u32(sKV + stage * KV_STAGE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * (128 * 128) + (kk % 4) * 32;
          umma_bf16_ss(tmem_base, make_smem_desc_sw128(sq + off, 16, 1024),
                       make_smem_desc_sw128(sk + off, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(smem_u32(bar_s));
      };
      uint32_t kv_phase[2] = {0, 0};
      if (ok && nblk > 0) {
        ok = mbar_wait_bounded(smem_u32(&bar_kv[0]), kv_phase[0], cta_abort, p.status,
                               NFN_ERR_WAIT_FULL);
        kv_phase[0] ^= 1;
        if (ok) { tc_fence_after(); issue_s(0); }
      }
      for (int j = 0; j < nblk && ok; ++j) {
        const int stage = j & 1;
        // P_j ready (and S_j fully read)
        ok = mbar_wait_bounded(smem_u32(bar_p), j & 1, cta_abort, p.status, NFN_ERR_WAIT_MISC);
        if (!ok) break;
        tc_fence_after();
        {
          const uint32_t sp = smem_u32(sP);
          const uint32_t sv = smem_u32(sKV + stage * KV_STAGE + K_BYTES);
#pragma unroll
          for (int kk = 0; kk < ATT_BN / 16; ++kk) {
            const uint32_t a_off = (kk / 4) * (128 * 128) + (kk % 4) * 32;
            const uint32_t b_off = kk * (16 * 128);
            umma_bf16_ss(tmem_base + O_COL, make_smem_desc_sw128(sp + a_off, 16, 1024),
                         make_smem_desc_sw128(sv + b_off, ATT_BN * 128, 1024), idesc_o, kk != 0);
          }
          umma_commit(smem_u32(bar_o));
        }
        if (j + 1 < nblk) {
          const int ns = (j + 1) & 1;
          ok = mbar_wait_bounded(smem_u32(&bar_kv[ns]), kv_phase[ns], cta_abort, p.status,
                                 NFN_ERR_WAIT_FULL);
          kv_phase[ns] ^= 1;
          if (!ok) break;
          tc_fence_after();
          issue_s(ns);
        }
        if (j + 2 < nblk) {
          // stage `stage` is free once O_j retired
          ok = mbar_wait_bounded(smem_u32(bar_o), j & 1, cta_abort, p.status, NFN_ERR_WAIT_MISC);
          if (!ok) break;
          load_kv(j + 2, stage);
        }
      }
    }
  } else {
    // ------------------------------------------------------ softmax threads --
    const int quarter = warp & 3, half = warp >> 2;
    const int r = quarter * 32 + lane;  // row within the tile == TMEM lane
    const int q = q0 + r;
    constexpr int DH = D / 2;           // output columns this thread accumulates
    constexpr int CH = ATT_BN / 64;     // 32-column slices of S per thread (its half of the keys)
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    float m_run = -INFINITY, l_run = 0.f;  // l_run covers this thread's key columns only
    float acc[DH];
#pragma unroll
    for (int i = 0; i < DH; ++i) acc[i] = 0.f;
    bool ok = true;
    uint32_t pair_phase = 0;
    // hand `mine` to the other thread of this row and return its value
    auto exchange = [&](float mine, int slot) -> float {
      tmem_st_col(t_row + XCHG_COL + slot * 2 + half, __float_as_uint(mine));
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_pair[quarter]));
      bool w = mbar_wait_bounded(smem_u32(&bar_pair[quarter]), pair_phase, cta_abort, p.status, NFN_ERR_WAIT_MISC);
      pair_phase ^= 1;
      w = __all_sync(0xffffffffu, w);
      if (!w) ok = false;
      tc_fence_after();
      const uint32_t other = tmem_ld_col(t_row + XCHG_COL + slot * 2 + (half ^ 1));
      tmem_ld_wait();
      return __uint_as_float(other);
    };
    for (int j = 0; j < nblk; ++j) {
      ok = mbar_wait_bounded(smem_u32(bar_s), j & 1, cta_abort, p.status, NFN_ERR_WAIT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int kbase = (jb_lo + j) * ATT_BN;
      // does this block need element masks?
      bool need_mask = (kbase + ATT_BN > p.T);
      if (p.causal) need_mask |= (kbase + ATT_BN - 1 > q0);
      if (p.window > 0) {
        need_mask |= (kbase < q0 + ATT_BM - p.window);             // lower window edge
        if (!p.causal) need_mask |= (kbase + ATT_BN - 1 >= q0 + p.window);
      }
      auto visible = [&](int k) -> bool {
        if (k >= p.T) return false;
        if (p.causal) {
          if (k > q) return false;
          if (p.window > 0 && k <= q - p.window) return false;
        } else if (p.window > 0) {
          if (k <= q - p.window || k >= q + p.window) return false;
        }
        return true;
      };
      // pass 1: maximum over this thread's half of the keys, then over the pair
      float m_blk = -INFINITY;
#pragma unroll 1
      for (int c = half * CH; c < (half + 1) * CH; ++c) {
        uint32_t s[32];
        tmem_ld_32x32(t_row + c * 32, s);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (visible(kbase + c * 32 + i)) m_blk = fmaxf(m_blk, __uint_as_float(s[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) m_blk = fmaxf(m_blk, __uint_as_float(s[i]));
        }
      }
      m_blk = fmaxf(m_blk, exchange(m_blk, j & 1));
      if (!ok) break;
      const float m_new = fmaxf(m_run, m_blk);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = fast_exp2((m_run - m_use) * p.scale_log2);  // m_run = -inf -> 0
      const float moff = m_use * p.scale_log2;
      // pass 2: p = exp2(s*scale - m*scale), row sum, bf16 P into swizzled smem
      float l_blk = 0.f;
#pragma unroll 1
      for (int c = half * CH; c < (half + 1) * CH; ++c) {
        uint32_t s[32];
        tmem_ld_32x32(t_row + c * 32, s);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = fast_exp2(__uint_as_float(s[2 * i]) * p.scale_log2 - moff);
          float p1 = fast_exp2(__uint_as_float(s[2 * i + 1]) * p.scale_log2 - moff);
          if (need_mask) {
            if (!visible(kbase + c * 32 + 2 * i)) p0 = 0.f;
            if (!visible(kbase + c * 32 + 2 * i + 1)) p1 = 0.f;
          }
          // sum what the MMA will actually see (bf16-rounded probabilities)
          const uint32_t w = pack_bf16x2(p0, p1);
          const float2 back = unpack_bf16x2(w);
          l_blk += back.x + back.y;
          pk[i] = w;
        }
        // 32 keys = 64 bytes = 4 chunks of 16 B; key half = c / 2, chunk base = (c % 2) * 4
        uint8_t* prow = sP + (c / 2) * (ATT_BM * 128) + r * 128;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int chunk = ((c & 1) * 4 + ch) ^ (r & 7);
          *reinterpret_cast<uint4*>(prow + chunk * 16) =
              make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
        }
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(bar_p));
      // rescale the running state while the PV product runs
      l_run = l_run * alpha + l_blk;
      m_run = m_new;
#pragma unroll
      for (int i = 0; i < DH; ++i) acc[i] *= alpha;
      ok = mbar_wait_bounded(smem_u32(bar_o), j & 1, cta_abort, p.status, NFN_ERR_WAIT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(t_row + O_COL + half * DH + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[c * 32 + i] += __uint_as_float(o[i]);
      }
      tc_fence_before();
    }
    if (ok) l_run += exchange(l_run, nblk & 1);  // both halves of the row sum
    if (ok && q < p.T) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* orow = p.o + (size_t)(b * p.T + q) * p.ld_o + h * D + half * DH;
#pragma unroll
      for (int i = 0; i < DH / 8; ++i) {
        uint4 u;
        u.x = pack_bf16x2(acc[8 * i] * inv, acc[8 * i + 1] * inv);
        u.y = pack_bf16x2(acc[8 * i + 2] * inv, acc[8 * i + 3] * inv);
        u.z = pack_bf16x2(acc[8 * i + 4] * inv, acc[8 * i + 5] * inv);
        u.w = pack_bf16x2(acc[8 * i + 6] * inv, acc[8 * i + 7] * inv);
        reinterpret_cast<uint4*>(orow)[i] = u;
      }
      if (p.lse && half == 0)
        p.lse[((size_t)b * p.Hq + h) * p.T + q] =
            l_run > 0.f ? m_run * p.scale + logf(l_run) : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*cta_abort) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == ATT_CTRL_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int D>
static int launch_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B,
                           int T, int Hq, int Hkv, int ld_q, int ld_k, int ld_v, int ld_o,
                           int causal, int window, float scale, cudaStream_t st) {
  constexpr size_t SMEM = attn_fwd_smem_bytes<D>();
  auto kern = attn_fwd_kernel<D>;
  static bool attr[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess)
      return launch_check("attn_fwd attr");
    attr[dev & 63] = true;
  }
  CUtensorMap tq, tk, tv;
  const uint64_t rows = (uint64_t)B * T;
  if (!make_tmap_2d(&tq, q, 2, (uint64_t)Hq * D, rows, ld_q, 64, ATT_BM, 128)) return -3;
  if (!make_tmap_2d(&tk, k, 2, (uint64_t)Hkv * D, rows, ld_k, 64, ATT_BN, 128)) return -3;
  if (!make_tmap_2d(&tv, v, 2, (uint64_t)Hkv * D, rows, ld_v, 64, ATT_BN, 128)) return -3;
  AttnFwdParams p;
  p.o = (__nv_bfloat16*)o; p.lse = lse; p.ld_o = ld_o;
  p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
  p.causal = causal; p.window = window;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status_ptr();
  dim3 grid(ceil_div(T, ATT_BM), Hq, B);
  kern<<<grid, ATT_THREADS, SMEM, st>>>(tq, tk, tv, p);
  return launch_check("attn_fwd");
}

}  // namespace nfn

using namespace nfn;

// q: bf16 rows [B*T] x (Hq*D) with row stride ld_q; k, v: rows x (Hkv*D); o: rows x (Hq*D).
// lse: optional fp32 [B, Hq, T].
extern "C" int nfn_attention_forward_v1(const void* q, const void* k, const void* v, void* o, float* lse,
                                     int B, int T, int Hq, int Hkv, int D, int ld_q, int ld_k,
                                     int ld_v, int ld_o, int causal, int window, float scale,
                                     nfn_stream_t stream) {
  if (B <= 0 || T <= 0) return 0;
  if (Hq % Hkv) return fail(-1, "attention: Hq must be a multiple of Hkv");
  if ((ld_q | ld_k | ld_v | ld_o) & 7) return fail(-1, "attention: row strides must be multiples of 8");
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(o)) & 15)
    return fail(-1, "attention: operands must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (D == 64)
    return launch_attn_fwd<64>(q, k, v, o, lse, B, T, Hq, Hkv, ld_q, ld_k, ld_v, ld_o, causal, window, scale, st);
  if (D == 128)
    return launch_attn_fwd<128>(q, k, v, o, lse, B, T, Hq, Hkv, ld_q, ld_k, ld_v, ld_o, causal, window, scale, st);
  return fail(-1, "attention: head_dim must be 64 or 128");
}
