// Block attention over a KV cache on tcgen05 (sm_100a): R new rows per sequence (a speculative
// verification block, a draft block, or a chunk of a continued prefill) attend to the sequence's
// cached keys plus the block's own keys, WITHOUT touching the cache. The block's K/V rows are
// optionally copied to a staging buffer from which a separate commit kernel appends only the
// accepted prefix, so a rejected row never has to be rolled back.
//
// One CTA handles one (sequence, kv head, chunk of the head group, KV split). The 128 MMA rows
// are (query head of the group) x (block row): with R <= 16 eight query heads share one pass over
// the keys, which is what makes the pass HBM-bound rather than FLOP-bound. Structure as in the
// training forward kernel: warps 0-7 run the online softmax out of TMEM, two threads per row (each
// half of the key columns and of the output columns; they swap half-row maxima and sums through
// spare TMEM columns), P goes as bf16 into a swizzled tile; warp 8 issues TMA loads of 128-key cache tiles (two-stage ring)
// and the two products S = Q K^T and O_j = P V.
//
// Cache layout [sequence][kv head][cap][D] bf16; a ring (local layer) stores position p in row
// p % cap. Tiles walk PHYSICAL rows, so `cap` needs no alignment and a tile never wraps; each
// key's age (distance behind the newest cached position) is recovered from its row index for
// the window mask. The block's own keys are the first tile; the softmax threads place them
// (and Q) into shared memory with plain loads.
//
// KV splits write unnormalised partials; the last CTA of a (sequence, head chunk) - found with
// a self-resetting ticket - merges them.
//
// Reference counterparts: the DFlash block attention descriptor and its "short split" variant
// (neuralfn/csrc/tile_cuda/resident_glimmer_cuda.cpp:3753-3791, kernels.cu:2904-3057) and the
// all-layer cache commit (resident_glimmer_cuda.cpp:3956-4041).
#include <algorithm>

#include "common.h"
#include "sm100_ptx.cuh"

namespace nfn {

constexpr int BA_M = 128;
constexpr int BA_N = 128;
constexpr int BA_SOFTMAX_WARPS = 8;  // two per TMEM lane quarter: each takes half of the key columns and half of the output columns
constexpr int BA_CTRL_WARP = BA_SOFTMAX_WARPS;
constexpr int BA_THREADS = (BA_SOFTMAX_WARPS + 1) * 32;

struct BlockAttnParams {
  const __nv_bfloat16* qkv;
  int ld;
  __nv_bfloat16* out;
  int ld_o;
  __nv_bfloat16 *stage_k, *stage_v;  // optional [B*R, Hkv*D]
  const int* lengths;
  const int* n_rows;
  int B, R, RP, Hq, Hkv, G, GC, gchunks, cap, window, causal, splits;
  float scale_log2;
  float* part;   // [B][Hkv*gchunks][splits][128][D+4]: max, sum, 2 pad words, D outputs (rows stay 16-byte aligned)
  int* tickets;  // [B][Hkv*gchunks]
  int* status;
};

template <int D>
__host__ __device__ constexpr uint32_t block_attn_smem_bytes() {
  return BA_M * D * 2 + 2 * (2 * BA_N * D * 2) + BA_M * BA_N * 2 + 128;
}

// 16-byte chunk `chunk` (of D/8) of row `row` inside a [128 x D] tile stored as D/64 panels of
// 128 rows x 128 bytes with the 128-byte swizzle that TMA and the UMMA descriptors use
__device__ __forceinline__ uint8_t* sw128_chunk(uint8_t* tile, int row, int chunk) {
  return tile + (chunk >> 3) * (128 * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

template <int D>
__global__ void __launch_bounds__(BA_THREADS, (D == 64 ? 2 : 1))
block_attn_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const BlockAttnParams p) {
  constexpr uint32_t Q_BYTES = BA_M * D * 2, K_BYTES = BA_N * D * 2, P_BYTES = BA_M * BA_N * 2;
  constexpr uint32_t KV_STAGE = 2 * K_BYTES;
  constexpr uint32_t TMEM_COLS = (D == 64) ? 256 : 512, O_COL = 128, XCHG_COL = O_COL + D;  // S | O | four mailbox columns
  constexpr int CH = D / 8;  // 16-byte chunks per row

  const int s = blockIdx.x, y = blockIdx.y, b = blockIdx.z;
  const int nrows = p.n_rows ? min(p.n_rows[b], p.R) : p.R;
  if (nrows <= 0) return;  // uniform for every CTA of this sequence: nobody takes a ticket
  const int pos0 = p.lengths[b];
  const int hk = y / p.gchunks, g0 = (y % p.gchunks) * p.GC;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  {
    uint32_t dyn;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
    if (static_cast<uint32_t>(smem - smem_raw) + block_attn_smem_bytes<D>() > dyn) {
      if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, NFN_ERR_WAIT_MISC);
      return;
    }
  }
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + Q_BYTES;
  uint8_t* sP = sKV + 2 * KV_STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);
  uint64_t* bar_q = bars;       // 4 arrivals (one per softmax warp): Q (and the block's own K/V tile) are in shared memory
  uint64_t* bar_kv = bars + 1;  // 2
  uint64_t* bar_s = bars + 3;
  uint64_t* bar_p = bars + 4;   // 4 arrivals
  uint64_t* bar_o = bars + 5;
  uint64_t* bar_pair = bars + 6;  // 4 (one per lane quarter), 2 arrivals each
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* sh_last = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // physical cache tiles of this split; split 0 also takes the block's own keys as its first tile
  const int n_valid = min(pos0, p.cap);
  const int ntiles_c = (n_valid + BA_N - 1) / BA_N;
  const int chunk_t = (ntiles_c + p.splits - 1) / p.splits;
  const int t_lo = min(ntiles_c, s * chunk_t), t_hi = min(ntiles_c, t_lo + chunk_t);
  const int staged = (s == 0) ? 1 : 0;
  const int nblk = staged + (t_hi - t_lo);

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    *sh_last = 0;
    mbar_init(smem_u32(bar_q), BA_SOFTMAX_WARPS);  // one arrival per softmax warp
    for (int qd = 0; qd < 4; ++qd) mbar_init(smem_u32(&bar_pair[qd]), 2);
    mbar_init(smem_u32(&bar_kv[0]), 1);
    mbar_init(smem_u32(&bar_kv[1]), 1);
    mbar_init(smem_u32(bar_s), 1);
    mbar_init(smem_u32(bar_p), BA_SOFTMAX_WARPS);  // one arrival per softmax warp
    mbar_init(smem_u32(bar_o), 1);
    fence_mbar_init();
  }
  if (warp == BA_CTRL_WARP) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == BA_CTRL_WARP) {
    if (lane == 0 && nblk > 0) {
      // ------------------------------------------------------ control thread --
      const int crow0 = (b * p.Hkv + hk) * p.cap;  // first cache row of this (sequence, kv head)
      auto load_kv = [&](int j, int stage) {        // j: tile index of this CTA, j >= staged
        const uint32_t fb = smem_u32(&bar_kv[stage]);
        const uint32_t sk = smem_u32(sKV + stage * KV_STAGE);
        const uint32_t sv = sk + K_BYTES;
        mbar_expect_tx(fb, KV_STAGE);
        const int krow = crow0 + (t_lo + j - staged) * BA_N;
#pragma unroll
        for (int d = 0; d < D / 64; ++d) {
          tma_load_2d(sk + d * (BA_N * 128), &tm_k, fb, d * 64, krow);
          tma_load_2d(sv + d * (BA_N * 128), &tm_v, fb, d * 64, krow);
        }
      };
      if (!staged) load_kv(0, 0);
      if (nblk > 1) load_kv(1, 1);
      constexpr uint32_t idesc_s = make_idesc_bf16(BA_M, BA_N, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(BA_M, D, 0, 1);
      bool ok = mbar_wait_bounded(smem_u32(bar_q), 0, cta_abort, p.status, NFN_ERR_WAIT_FULL);
      auto issue_s = [&](int stage) {
        const uint32_t sq = smem_u32(sQ);
        const uint32_t sk = smem_u32(sKV + stage * KV_STAGE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * (128 * 128) + (kk % 4) * 32;
          umma_bf16_ss(tmem_base, make_smem_desc_sw128(sq + off, 16, 1024), make_smem_desc_sw128(sk + off, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(smem_u32(bar_s));
      };
      uint32_t kv_phase[2] = {0, 0};
      auto wait_tile = [&](int j) -> bool {  // tile j's K/V are in stage j & 1
        if (j == 0 && staged) return true;   // covered by bar_q
        const int st = j & 1;
        const bool w = mbar_wait_bounded(smem_u32(&bar_kv[st]), kv_phase[st], cta_abort, p.status, NFN_ERR_WAIT_FULL);
        kv_phase[st] ^= 1;
        return w;
      };
      if (ok) {
        ok = wait_tile(0);
        if (ok) { tc_fence_after(); issue_s(0); }
      }
      for (int j = 0; j < nblk && ok; ++j) {
        const int stage = j & 1;
        ok = mbar_wait_bounded(smem_u32(bar_p), j & 1, cta_abort, p.status, NFN_ERR_WAIT_MISC);
        if (!ok) break;
        tc_fence_after();
        {
          const uint32_t sp = smem_u32(sP);
          const uint32_t sv = smem_u32(sKV + stage * KV_STAGE + K_BYTES);
#pragma unroll
          for (int kk = 0; kk < BA_N / 16; ++kk) {
            const uint32_t a_off = (kk / 4) * (128 * 128) + (kk % 4) * 32;
            const uint32_t b_off = kk * (16 * 128);
            umma_bf16_ss(tmem_base + O_COL, make_smem_desc_sw128(sp + a_off, 16, 1024),
                         make_smem_desc_sw128(sv + b_off, BA_N * 128, 1024), idesc_o, kk != 0);
          }
          umma_commit(smem_u32(bar_o));
        }
        if (j + 1 < nblk) {
          ok = wait_tile(j + 1);
          if (!ok) break;
          tc_fence_after();
          issue_s((j + 1) & 1);
        }
        if (j + 2 < nblk) {
          ok = mbar_wait_bounded(smem_u32(bar_o), j & 1, cta_abort, p.status, NFN_ERR_WAIT_MISC);
          if (!ok) break;
          load_kv(j + 2, stage);
        }
      }
    }
  } else {
    // ------------------------------------------------------ softmax threads --
    const int quarter = warp & 3, half = warp >> 2;
    const int m = quarter * 32 + lane;       // MMA row == TMEM lane
    constexpr int DH = D / 2;                // output columns this thread accumulates
    const int gl = m / p.RP, r = m % p.RP;   // head inside the chunk, row inside the block
    const int g = g0 + gl;
    const bool row_valid = gl < p.GC && g < p.G && r < nrows;
    const int head = hk * p.G + g;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    float m_run = -INFINITY, l_run = 0.f;  // l_run: this thread's key columns only until the final exchange
    float acc[DH];
#pragma unroll
    for (int i = 0; i < DH; ++i) acc[i] = 0.f;
    bool ok = true;
    uint32_t pair_phase = 0;
    auto exchange = [&](float mine, int slot) -> float {  // swap a value with the other thread of this row
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

    if (nblk > 0) {
      // Q row (zeros for padding rows) and, in split 0, key/value row m of the block itself
      const uint4 zero = make_uint4(0, 0, 0, 0);
      const uint4* qsrc = reinterpret_cast<const uint4*>(p.qkv + (size_t)(b * p.R + r) * p.ld + (size_t)head * D);
#pragma unroll
      for (int c = half * (CH / 2); c < (half + 1) * (CH / 2); ++c) *reinterpret_cast<uint4*>(sw128_chunk(sQ, m, c)) = row_valid ? qsrc[c] : zero;
      if (staged) {
        const bool kv_valid = m < nrows;
        const __nv_bfloat16* rowp = p.qkv + (size_t)(b * p.R + (kv_valid ? m : 0)) * p.ld;
        const uint4* ksrc = reinterpret_cast<const uint4*>(rowp + (size_t)(p.Hq + hk) * D);
        const uint4* vsrc = reinterpret_cast<const uint4*>(rowp + (size_t)(p.Hq + p.Hkv + hk) * D);
        const bool copy_out = kv_valid && p.stage_k && (y % p.gchunks) == 0;
        uint4* ko = copy_out ? reinterpret_cast<uint4*>(p.stage_k + ((size_t)(b * p.R + m) * p.Hkv + hk) * D) : nullptr;
        uint4* vo = copy_out ? reinterpret_cast<uint4*>(p.stage_v + ((size_t)(b * p.R + m) * p.Hkv + hk) * D) : nullptr;
#pragma unroll
        for (int c = half * (CH / 2); c < (half + 1) * (CH / 2); ++c) {
          const uint4 kq = kv_valid ? ksrc[c] : zero, vq = kv_valid ? vsrc[c] : zero;
          *reinterpret_cast<uint4*>(sw128_chunk(sKV, m, c)) = kq;
          *reinterpret_cast<uint4*>(sw128_chunk(sKV + K_BYTES, m, c)) = vq;
          if (copy_out) { ko[c] = kq; vo[c] = vq; }
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(bar_q));
    }

    // window bookkeeping: a cached key of age a (a = 0 is position pos0 - 1) is visible to block
    // row r when a < window - 1 - r ... i.e. its position is inside (q - window, q]
    const int age_lim = p.window > 0 ? p.window - 1 - r : 0x7fffffff;
    for (int j = 0; j < nblk; ++j) {
      ok = mbar_wait_bounded(smem_u32(bar_s), j & 1, cta_abort, p.status, NFN_ERR_WAIT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool own = staged && j == 0;
      // cache tile: physical rows [row_base, +128); age of physical row x is (pos0 - 1 - x) mod cap
      const int row_base = own ? 0 : (t_lo + j - staged) * BA_N;
      const int age0 = own ? 0 : (pos0 - 1 - row_base) % p.cap;  // pos0 >= 1 whenever a cache tile exists
      auto visible = [&](int e) -> bool {
        if (own) return e < nrows && (!p.causal || e <= r);
        if (row_base + e >= n_valid) return false;
        int age = age0 - e;
        if (age < 0) age += p.cap;
        return age < age_lim;
      };
      float m_blk = -INFINITY;
#pragma unroll 1
      for (int c = 2 * half; c < 2 * half + 2; ++c) {
        uint32_t sv[32];
        tmem_ld_32x32(t_row + c * 32, sv);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (visible(c * 32 + i)) m_blk = fmaxf(m_blk, __uint_as_float(sv[i]));
      }
      m_blk = fmaxf(m_blk, exchange(m_blk, j & 1));
      if (!ok) break;
      const float m_new = fmaxf(m_run, m_blk);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = fast_exp2((m_run - m_use) * p.scale_log2);
      const float moff = m_use * p.scale_log2;
      float l_blk = 0.f;
#pragma unroll 1
      for (int c = 2 * half; c < 2 * half + 2; ++c) {
        uint32_t sv[32];
        tmem_ld_32x32(t_row + c * 32, sv);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = fast_exp2(__uint_as_float(sv[2 * i]) * p.scale_log2 - moff);
          float p1 = fast_exp2(__uint_as_float(sv[2 * i + 1]) * p.scale_log2 - moff);
          if (!visible(c * 32 + 2 * i)) p0 = 0.f;
          if (!visible(c * 32 + 2 * i + 1)) p1 = 0.f;
          const uint32_t w = pack_bf16x2(p0, p1);
          const float2 back = unpack_bf16x2(w);
          l_blk += back.x + back.y;
          pk[i] = w;
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
          *reinterpret_cast<uint4*>(sw128_chunk(sP, m, c * 4 + ch)) = make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(bar_p));
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

    // ---- combine -------------------------------------------------------------------------
    if (ok && nblk > 0) l_run += exchange(l_run, nblk & 1);  // the whole row's sum in both threads
    const bool failed = !__all_sync(0xffffffffu, ok);
    if (p.splits > 1) {
      float* mine = p.part + ((((size_t)b * gridDim.y + y) * p.splits + s) * BA_M + m) * (D + 4);
      if (row_valid) {
        if (half == 0) {
          mine[0] = failed ? -INFINITY : m_run;
          mine[1] = failed ? 0.f : l_run;
        }
#pragma unroll
        for (int i = 0; i < DH / 4; ++i)
          reinterpret_cast<float4*>(mine + 4 + half * DH)[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
      }
      __threadfence();
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (threadIdx.x == 0) {
        const int t = atomicAdd(&p.tickets[b * gridDim.y + y], 1);
        const int last = (t == p.splits - 1);
        if (last) p.tickets[b * gridDim.y + y] = 0;  // ready for the next launch
        *sh_last = last;
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (*sh_last && row_valid) {
        __threadfence();
        const float* base = p.part + (((size_t)b * gridDim.y + y) * p.splits * BA_M + m) * (D + 4);
        const size_t sstride = (size_t)BA_M * (D + 4);
        float M = -INFINITY;
        for (int i = 0; i < p.splits; ++i) M = fmaxf(M, __ldcg(base + i * sstride));
        const float Mu = (M == -INFINITY) ? 0.f : M;
        float L = 0.f;
#pragma unroll
        for (int i = 0; i < DH; ++i) acc[i] = 0.f;
        for (int i = 0; i < p.splits; ++i) {
          const float* ps = base + i * sstride;
          const float w = fast_exp2((__ldcg(ps) - Mu) * p.scale_log2);
          L += w * __ldcg(ps + 1);
#pragma unroll
          for (int d4 = 0; d4 < DH / 4; ++d4) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(ps + 4 + half * DH) + d4);
            acc[4 * d4] += w * v.x; acc[4 * d4 + 1] += w * v.y; acc[4 * d4 + 2] += w * v.z; acc[4 * d4 + 3] += w * v.w;
          }
        }
        l_run = L;
      }
    }
    if ((p.splits == 1 || *sh_last) && row_valid && !failed) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      uint4* orow = reinterpret_cast<uint4*>(p.out + (size_t)(b * p.R + r) * p.ld_o + (size_t)head * D + half * DH);
#pragma unroll
      for (int i = 0; i < DH / 8; ++i) {
        uint4 u;
        u.x = pack_bf16x2(acc[8 * i] * inv, acc[8 * i + 1] * inv);
        u.y = pack_bf16x2(acc[8 * i + 2] * inv, acc[8 * i + 3] * inv);
        u.z = pack_bf16x2(acc[8 * i + 4] * inv, acc[8 * i + 5] * inv);
        u.w = pack_bf16x2(acc[8 * i + 6] * inv, acc[8 * i + 7] * inv);
        orow[i] = u;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*cta_abort) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == BA_CTRL_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Appends the first accepted[b] staged rows of every layer to that layer's cache (ring rows
// (pos0 + i) % cap). One launch for all layers: grid (layer, sequence).
struct CommitParams {
  const void* const* stage_k;
  const void* const* stage_v;
  void* const* kc;
  void* const* vc;
  const int* caps;
  const int* lengths;
  const int* accepted;
  int R, Hkv, D;
};

__global__ void kv_commit_layers_kernel(const CommitParams p) {
  const int l = blockIdx.x, b = blockIdx.y;
  const int n = min(p.accepted[b], p.R);
  if (n <= 0) return;
  const int cap = p.caps[l], pos0 = p.lengths[b];
  const int chunks = p.D / 8, per_row = p.Hkv * chunks;
  const uint4* sk = static_cast<const uint4*>(p.stage_k[l]) + (size_t)b * p.R * per_row;
  const uint4* sv = static_cast<const uint4*>(p.stage_v[l]) + (size_t)b * p.R * per_row;
  uint4* kc = static_cast<uint4*>(p.kc[l]) + (size_t)b * p.Hkv * cap * chunks;
  uint4* vc = static_cast<uint4*>(p.vc[l]) + (size_t)b * p.Hkv * cap * chunks;
  const int first = n > cap ? n - cap : 0;  // earlier rows would be overwritten by later ones
  for (int i = first * per_row + threadIdx.x; i < n * per_row; i += blockDim.x) {
    const int row = i / per_row, rem = i - row * per_row, h = rem / chunks, c = rem - h * chunks;
    const size_t dst = ((size_t)h * cap + (pos0 + row) % cap) * chunks + c;
    kc[dst] = sk[i];
    vc[dst] = sv[i];
  }
}

template <int D>
static int launch_block_attn(const BlockAttnParams& p, const void* kc, const void* vc, int Y, cudaStream_t st) {
  constexpr size_t SMEM = block_attn_smem_bytes<D>();
  auto kern = block_attn_kernel<D>;
  static bool attr[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess) return launch_check("block_attn attr", 0);
    attr[dev & 63] = true;
  }
  CUtensorMap tk, tv;
  const uint64_t rows = (uint64_t)p.B * p.Hkv * p.cap;
  if (!make_tmap_2d(&tk, kc, 2, (uint64_t)D, rows, D, 64, BA_N, 128)) return -3;
  if (!make_tmap_2d(&tv, vc, 2, (uint64_t)D, rows, D, 64, BA_N, 128)) return -3;
  dim3 grid(p.splits, Y, p.B);
  kern<<<grid, BA_THREADS, SMEM, st>>>(tk, tv, p);
  return launch_check("block_attn");
}

static int block_attn_geometry(int R, int Hq, int Hkv, int* RP, int* GC, int* gchunks) {
  if (R < 1 || R > BA_M || Hkv < 1 || Hq % Hkv) return -1;
  int rp = 1;
  while (rp < R) rp <<= 1;
  const int G = Hq / Hkv;
  *RP = rp;
  *GC = std::min(G, BA_M / rp);
  *gchunks = (G + *GC - 1) / *GC;
  return 0;
}

}  // namespace nfn

using namespace nfn;

extern "C" long long nfn_block_attention_workspace_bytes(int B, int rows, int n_q_heads, int n_kv_heads, int head_dim, int max_splits) {
  int RP, GC, gch;
  if (B < 1 || max_splits < 1 || block_attn_geometry(rows, n_q_heads, n_kv_heads, &RP, &GC, &gch)) return -1;
  const long long units = (long long)B * n_kv_heads * gch;
  return ((units * 4 + 255) / 256) * 256 + units * max_splits * BA_M * (long long)(head_dim + 4) * 4;
}

extern "C" int nfn_block_attention(const void* qkv, int ld, const void* k_cache, const void* v_cache, const int* lengths, const int* n_rows,
                                   void* out, int ld_o, void* stage_k, void* stage_v, int B, int rows, int n_q_heads, int n_kv_heads,
                                   int head_dim, int cap, int window, int causal, float scale, void* workspace, long long workspace_bytes,
                                   int splits, nfn_stream_t stream) {
  if (B <= 0) return 0;
  if (!qkv || !k_cache || !v_cache || !lengths || !out || !workspace) return fail(-1, "block_attention: null operand");
  if ((stage_k == nullptr) != (stage_v == nullptr)) return fail(-1, "block_attention: give both staging buffers or none");
  BlockAttnParams p{};
  if (block_attn_geometry(rows, n_q_heads, n_kv_heads, &p.RP, &p.GC, &p.gchunks)) return fail(-1, "block_attention: 1 <= rows <= 128 and Hq % Hkv == 0 required");
  if (head_dim != 64 && head_dim != 128) return fail(-1, "block_attention: head_dim must be 64 or 128");
  if ((ld & 7) || (ld_o & 7) || ld < (n_q_heads + 2 * n_kv_heads) * head_dim) return fail(-1, "block_attention: bad row strides");
  if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(stage_k) | reinterpret_cast<uintptr_t>(stage_v) | reinterpret_cast<uintptr_t>(workspace)) & 15)
    return fail(-1, "block_attention: operands must be 16-byte aligned");
  if (cap <= 0 || window < 0 || (window > 0 && window > cap)) return fail(-1, "block_attention: the window must fit in the cache rows");
  const int Y = n_kv_heads * p.gchunks;
  const long long units = (long long)B * Y;
  if (splits <= 0) {
    const long long want = (2LL * sm_count() + units - 1) / units;
    splits = (int)std::max<long long>(1, std::min<long long>(want, (cap + BA_N - 1) / BA_N));
  }
  const long long ticket_bytes = ((units * 4 + 255) / 256) * 256;
  if (splits > 1) {
    const long long per_split = units * BA_M * (long long)(head_dim + 4) * 4;
    const long long fit = (workspace_bytes - ticket_bytes) / per_split;
    splits = fit < 1 ? 1 : (int)std::min<long long>(splits, fit);  // a single split needs no workspace
  }
  p.qkv = static_cast<const __nv_bfloat16*>(qkv); p.ld = ld;
  p.out = static_cast<__nv_bfloat16*>(out); p.ld_o = ld_o;
  p.stage_k = static_cast<__nv_bfloat16*>(stage_k); p.stage_v = static_cast<__nv_bfloat16*>(stage_v);
  p.lengths = lengths; p.n_rows = n_rows;
  p.B = B; p.R = rows; p.Hq = n_q_heads; p.Hkv = n_kv_heads; p.G = n_q_heads / n_kv_heads;
  p.cap = cap; p.window = window; p.causal = causal; p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.tickets = static_cast<int*>(workspace);
  p.part = reinterpret_cast<float*>(static_cast<char*>(workspace) + ticket_bytes);
  p.status = status_ptr();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return head_dim == 64 ? launch_block_attn<64>(p, k_cache, v_cache, Y, st) : launch_block_attn<128>(p, k_cache, v_cache, Y, st);
}

extern "C" int nfn_kv_commit_layers(const void* const* stage_k, const void* const* stage_v, void* const* k_caches, void* const* v_caches,
                                    const int* caps, const int* lengths, const int* accepted, int n_layers, int B, int rows, int n_kv_heads,
                                    int head_dim, nfn_stream_t stream) {
  if (n_layers <= 0 || B <= 0) return 0;
  if (!stage_k || !stage_v || !k_caches || !v_caches || !caps || !lengths || !accepted || (head_dim & 7)) return fail(-1, "kv_commit_layers: bad arguments");
  CommitParams p{stage_k, stage_v, k_caches, v_caches, caps, lengths, accepted, rows, n_kv_heads, head_dim};
  kv_commit_layers_kernel<<<dim3(n_layers, B), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return launch_check("kv_commit_layers");
}
