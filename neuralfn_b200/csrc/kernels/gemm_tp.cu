// Tensor-parallel / sharded-parameter GEMMs that carry their collective inside the kernel.
//
// Three modes of one persistent tcgen05 kernel (K-major bf16 operands, fp32 TMEM accumulator,
// same pipeline as the plain GEMM: TMA producer warp, MMA issuer warp, four epilogue warps):
//
//  AG_A  all-gather -> GEMM (column-parallel linear on sequence-sharded activations):
//        C[M, N] = gather(A)[M, K] . B[N, K]^T. Every rank owns rows_per_rank rows of A inside
//        a symmetric buffer of the full [M, K]. A few "copy CTAs" of the same launch pull the
//        peers' row blocks into the local buffer with bulk async copies (global -> shared ->
//        global, ~190 KB in flight per CTA, enough to keep NVLink busy) and raise one flag per
//        128-row block; the GEMM CTAs start on the local rows and only wait, per tile, for
//        the block they are about to read. The remote rows cross NVLink exactly once and are
//        then read by TMA from local memory.
//  AG_B  the same with the gathered operand on the B side: the weight shards of a
//        parameter-sharded (ZeRO-3 style) layer are gathered into the first GEMM that uses them.
//  RS    GEMM -> reduce-scatter (row-parallel linear): each rank multiplies its K-shard and
//        its epilogue TMA-stores every bf16 partial tile straight into the slot the owning
//        rank keeps for it (owner order is rotated so all links are busy at once). The last
//        CTA to finish signals the peers; then, still in the same launch, every CTA sums the
//        `world` slots of the locally owned rows (+ bias + residual) into the bf16 result.
//
// Signals are epochs (never reset): flag >= epoch means "done for this call"; the epoch is
// epoch + *epoch_dev so a captured CUDA graph produces fresh values on replay. Cross-GPU
// flags use release/acquire at system scope, local block flags at device scope. Every wait
// is bounded by wall-clock time; on expiry the CTA records a code in the status word, stops
// issuing work, drains and frees its TMEM.
//
// Hazards the caller owns: the gathered buffer (AG) and the slot buffer (RS) are reused
// by the next call, so alternate two of each (or make sure an exchange in the opposite
// direction separates two uses, as attention/MLP blocks naturally do).
// No load in this file uses cluster multicast.
#include <algorithm>

#include "gemm_epilogue.cuh"
#include "nfn_kernels.h"

namespace nfn {

constexpr int TP_BM = 128, TP_BK = 64, TP_UMMA_K = 16, TP_THREADS = 192, TP_MAX_WORLD = 8;
constexpr uint32_t EPI_TILE_BYTES_TP = TP_BM * 64 * 2;  // one 128 x 64 bf16 staging tile
constexpr uint32_t TP_PIECE = 32 * 1024;  // bytes per bulk copy of the gather
constexpr int CTRL_TICKET = 16, CTRL_CHUNKS = 32;  // int offsets inside a rank's control block

struct TpMaps {
  CUtensorMap m[TP_MAX_WORLD];
};

struct TpParams {
  int mode;  // NFN_TP_AG_A / NFN_TP_AG_B / NFN_TP_RS
  int m, n, k, tiles_m, tiles_n;
  int rank, world, epoch;
  const int* epoch_dev;
  int n_copy, rows_per_rank;
  int flags;
  float act_param;
  const __nv_bfloat16* bias;
  const unsigned char* peer_src[TP_MAX_WORLD];  // AG: start of peer r's own row slice in ITS buffer
  unsigned char* local_buf;                     // AG: local gathered buffer
  int* ctrl;                                    // local control block
  int* peer_ctrl[TP_MAX_WORLD];
  const __nv_bfloat16* slots;                   // RS: local slots [world, rows_per_rank, n]
  __nv_bfloat16* out;
  int ld_out;
  const __nv_bfloat16* resid;
  int ld_resid;
  // GROUPED: m tile -> group (expert) table and the number of live m tiles, both written by
  // an earlier kernel on the stream; B is a [groups, N, K] stack read through a 3-D map
  const int* tile_group;
  const int* num_m_tiles_dev;
  int* status;
};

__device__ __forceinline__ void st_release_sys_i32(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys_i32(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_i32(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu_i32(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Polls *p until it reaches `want`; gives up after kWaitLimitNs (ten times that for flags
// another GPU writes: ranks may enter the call some time apart), raising the CTA abort flag.
template <bool SYS>
__device__ __forceinline__ bool flag_wait_bounded(const int* p, int want, volatile int* cta_abort, int* status, int code) {
  const unsigned long long t0 = global_timer_ns();
  const unsigned long long limit = SYS ? 10ull * kWaitLimitNs : kWaitLimitNs;
#pragma unroll 1
  for (uint32_t it = 0;; ++it) {
    const int v = SYS ? ld_acquire_sys_i32(p) : ld_acquire_gpu_i32(p);
    if (v - want >= 0) return true;
    if ((it & 7u) == 7u) {
      if (*cta_abort) return false;
      if (global_timer_ns() - t0 > limit) break;
      __nanosleep(64);
    }
  }
  *cta_abort = 1;
  if (status) atomicCAS(status, 0, code);
  return false;
}

__device__ __forceinline__ void bulk_g2s(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_src), "r"(bytes) : "memory");
}

// logical tile -> (m tile, n tile, owner of the gathered / scattered block)
struct TileCoord {
  int mt, nt, owner;
};
__device__ __forceinline__ TileCoord tile_coord(const TpParams& p, int t, int BN) {
  TileCoord c;
  if (p.mode == NFN_TP_GROUPED) {
    c.mt = t / p.tiles_n;
    c.nt = t % p.tiles_n;
    c.owner = p.rank;
    return c;
  }
  if (p.mode == NFN_TP_AG_B) {
    const int per = p.rows_per_rank / BN;  // n tiles per rank
    const int ln = t / p.tiles_m;
    c.owner = (p.rank + ln / per) % p.world;
    c.nt = c.owner * per + ln % per;
    c.mt = t % p.tiles_m;
  } else {
    const int per = p.rows_per_rank / TP_BM;  // m tiles per rank
    const int lm = t / p.tiles_n;
    const int j = lm / per;
    c.owner = (p.mode == NFN_TP_RS) ? (p.rank + 1 + j) % p.world : (p.rank + j) % p.world;
    c.mt = c.owner * per + lm % per;
    c.nt = t % p.tiles_n;
  }
  return c;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(TP_THREADS, 1)
gemm_tp_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
               const __grid_constant__ TpMaps tma_c, const TpParams p) {
  constexpr uint32_t A_BYTES = TP_BM * TP_BK * 2, B_BYTES = BN * TP_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + 2 * EPI_TILE_BYTES_TP);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint64_t* epi_bar = bars + 2 * STAGES + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 5);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* sh_flag = cta_abort + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int epoch = p.epoch + (p.epoch_dev ? *p.epoch_dev : 0);
  const bool is_copy_cta = (int)blockIdx.x < p.n_copy;

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    *sh_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&tfull_bar[b]), 1);
      mbar_init(smem_u32(&tempty_bar[b]), 4);
    }
    mbar_init(smem_u32(epi_bar), 4);  // one arrival per epilogue warp
    fence_mbar_init();
  }
  if (!is_copy_cta && warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  // ======================================================================= gather CTAs ==
  if (is_copy_cta) {
    if (threadIdx.x == 0) {
      if (blockIdx.x == 0) {
        // this rank's own rows were written by earlier work on this stream: tell the peers
        __threadfence_system();
        for (int r = 0; r < p.world; ++r)
          if (r != p.rank) st_release_sys_i32(p.peer_ctrl[r] + p.rank, epoch);
      }
      const long long chunk_bytes = (long long)TP_BM * p.k * 2;
      const int per = p.rows_per_rank / TP_BM;  // 128-row blocks per rank
      const int n_remote = per * (p.world - 1);
      uint32_t phase_bits = 0;  // one phase bit per stage
      bool ok = true;
      for (int c = blockIdx.x; c < n_remote && ok; c += p.n_copy) {
        const int owner = (p.rank + 1 + c / per) % p.world;
        const int blk = c % per;
        if (!flag_wait_bounded<true>(p.ctrl + owner, epoch, cta_abort, p.status, NFN_ERR_WAIT_PEER)) break;
        const unsigned char* src = p.peer_src[owner] + (long long)blk * chunk_bytes;
        unsigned char* dst = p.local_buf + ((long long)owner * per + blk) * chunk_bytes;
        const int pieces = (int)((chunk_bytes + TP_PIECE - 1) / TP_PIECE);
        auto piece_bytes = [&](int i) { return (uint32_t)min((long long)TP_PIECE, chunk_bytes - (long long)i * TP_PIECE); };
        // ring of TP_PIECE-byte slots over the (otherwise unused) operand stages, one
        // mbarrier per slot
        const int slots = min((int)(STAGES * STAGE_BYTES / TP_PIECE), STAGES);
        int issued = 0;
        for (; issued < min(slots, pieces); ++issued) {
          const uint32_t bar = smem_u32(&full_bar[issued]);
          mbar_expect_tx(bar, piece_bytes(issued));
          bulk_g2s(smem_u32(smem + (size_t)issued * TP_PIECE), src + (long long)issued * TP_PIECE, piece_bytes(issued), bar);
        }
        for (int i = 0; i < pieces; ++i) {
          const int s = i % slots;
          if (!mbar_wait_bounded(smem_u32(&full_bar[s]), (phase_bits >> s) & 1u, cta_abort, p.status, NFN_ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          phase_bits ^= 1u << s;
          bulk_s2g(dst + (long long)i * TP_PIECE, smem_u32(smem + (size_t)s * TP_PIECE), piece_bytes(i));
          bulk_commit();
          if (issued < pieces) {
            bulk_wait_read<0>();  // the slot's bytes have left shared memory
            const uint32_t bar = smem_u32(&full_bar[s]);
            mbar_expect_tx(bar, piece_bytes(issued));
            bulk_g2s(smem_u32(smem + (size_t)s * TP_PIECE), src + (long long)issued * TP_PIECE, piece_bytes(issued), bar);
            ++issued;
          }
        }
        if (!ok) break;
        bulk_wait_all();       // the block is in local memory
        fence_proxy_async();
        __threadfence();
        st_release_gpu_i32(p.ctrl + CTRL_CHUNKS + owner * per + blk, epoch);
      }
      bulk_wait_all();
    }
    __syncthreads();
    return;  // copy CTAs own no TMEM
  }

  // ========================================================================= GEMM CTAs ==
  const uint32_t tmem_base = *tmem_slot;
  const int live_m_tiles = (p.mode == NFN_TP_GROUPED) ? min(p.tiles_m, max(0, *p.num_m_tiles_dev)) : p.tiles_m;
  const int num_tiles = live_m_tiles * p.tiles_n;
  const int total_kb = (p.k + TP_BK - 1) / TP_BK;
  const int first = (int)blockIdx.x - p.n_copy, stride = (int)gridDim.x - p.n_copy;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int t = first; t < num_tiles && ok; t += stride) {
        const TileCoord tc = tile_coord(p, t, BN);
        const int group = (p.mode == NFN_TP_GROUPED) ? p.tile_group[tc.mt] : 0;
        if (p.mode != NFN_TP_RS && tc.owner != p.rank) {
          // wait for the gathered block(s) this tile reads
          const int blocks = (p.mode == NFN_TP_AG_B) ? BN / TP_BM : 1;
          const int b0 = (p.mode == NFN_TP_AG_B) ? tc.nt * (BN / TP_BM) : tc.mt;
          for (int b = 0; b < blocks && ok; ++b)
            ok = flag_wait_bounded<false>(p.ctrl + CTRL_CHUNKS + b0 + b, epoch, cta_abort, p.status, NFN_ERR_WAIT_PEER);
          if (!ok) break;
          fence_proxy_async();  // generic-proxy flag read -> async-proxy (TMA) data reads
        }
        for (int kb = 0; kb < total_kb; ++kb) {
          if (!mbar_wait_bounded(smem_u32(&empty_bar[stage]), phase ^ 1, cta_abort, p.status, NFN_ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t fb = smem_u32(&full_bar[stage]);
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          mbar_expect_tx(fb, STAGE_BYTES);
          tma_load_2d(sa, &tma_a, fb, kb * TP_BK, tc.mt * TP_BM);
          if (p.mode == NFN_TP_GROUPED) tma_load_3d(sa + A_BYTES, &tma_b, fb, kb * TP_BK, tc.nt * BN, group);
          else tma_load_2d(sa + A_BYTES, &tma_b, fb, kb * TP_BK, tc.nt * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TP_BM, BN, 0, 0);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int t = first; t < num_tiles && ok; t += stride) {
        if (!mbar_wait_bounded(smem_u32(&tempty_bar[acc]), acc_phase ^ 1, cta_abort, p.status, NFN_ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < total_kb; ++kb) {
          if (!mbar_wait_bounded(smem_u32(&full_bar[stage]), phase, cta_abort, p.status, NFN_ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint64_t da = make_smem_desc_sw128(sa, 16, 1024), db = make_smem_desc_sw128(sa + A_BYTES, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < TP_BK / TP_UMMA_K; ++kk) {
            const uint64_t adv = (uint64_t)((TP_UMMA_K * 2) >> 4) * kk;
            umma_bf16_ss(tmem_d, da + adv, db + adv, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&empty_bar[stage]));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(smem_u32(&tfull_bar[acc]));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------------- epilogue --
    const int q = warp & 3, trow = q * 32 + lane;
    const bool issuer = (warp == 2 && lane == 0);
    const int act = (p.flags >> NFN_EPI_ACT_SHIFT) & 0xF;
    const bool has_bias = (p.flags & NFN_EPI_BIAS) && p.mode != NFN_TP_RS;  // RS adds the bias once, in the reduction
    uint32_t acc = 0, acc_phase = 0, chunk_ctr = 0, epi_phase = 0;
    bool epi_ok = true;
    auto epi_sync = [&]() {
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(epi_bar));
      bool w = mbar_wait_bounded(smem_u32(epi_bar), epi_phase, cta_abort, p.status, NFN_ERR_WAIT_MISC);
      epi_phase ^= 1;
      w = __all_sync(0xffffffffu, w);
      if (!w) epi_ok = false;
    };
    for (int t = first; t < num_tiles; t += stride) {
      const TileCoord tc = tile_coord(p, t, BN);
      const int m0 = tc.mt * TP_BM, n0 = tc.nt * BN;
      bool ok = mbar_wait_bounded(smem_u32(&tfull_bar[acc]), acc_phase, cta_abort, p.status, NFN_ERR_WAIT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      const CUtensorMap* cmap = (p.mode == NFN_TP_RS) ? &tma_c.m[tc.owner] : &tma_c.m[0];
      const int store_row = (p.mode == NFN_TP_RS) ? m0 - tc.owner * p.rows_per_rank : m0;
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        const int nc = n0 + c * 64;
        if (nc >= p.n) break;
        if (issuer) bulk_wait_read<1>();
        uint8_t* tile_c = epi_smem + (chunk_ctr & 1) * EPI_TILE_BYTES_TP;
        epi_sync();
        if (!epi_ok) break;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 64 + half * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int ng = nc + half * 32 + g * 8;
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[g * 8 + j]);
            if (has_bias && ng < p.n) {
              float b8[8];
              unpack8_bf16(__ldg(reinterpret_cast<const uint4*>(p.bias + ng)), b8);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] += b8[j];
            }
            if (p.mode != NFN_TP_RS) act8(v, act, p.act_param);
            stage_store8(tile_c, trow, half * 4 + g, pack8_bf16(v));
          }
        }
        fence_proxy_async();
        epi_sync();
        if (!epi_ok) break;
        if (issuer) {
          tma_store_2d(cmap, smem_u32(tile_c), nc, store_row);
          bulk_commit();
        }
        __syncwarp();
        ++chunk_ctr;
      }
      if (!epi_ok) break;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (issuer) {
      bulk_wait_all();  // every tile this CTA produced has landed (locally or at its owner)
      fence_proxy_async();
      __threadfence_system();
    }
  }

  // -------------------------------------------------------------------------- teardown --
  tc_fence_before();
  __syncthreads();
  if (*cta_abort) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (p.mode != NFN_TP_RS || *cta_abort) return;

  // ================================================= RS: signal, wait, reduce the slots ==
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int n_gemm = (int)gridDim.x - p.n_copy;
    const int t = atomicAdd(p.ctrl + CTRL_TICKET, 1);
    if (t == n_gemm - 1) {
      p.ctrl[CTRL_TICKET] = 0;
      __threadfence_system();
      for (int r = 0; r < p.world; ++r)
        if (r != p.rank) st_release_sys_i32(p.peer_ctrl[r] + p.rank, epoch);
      st_release_gpu_i32(p.ctrl + p.rank, epoch);  // our own slot is complete too
    }
    bool ok = true;
    for (int r = 0; r < p.world && ok; ++r)
      ok = flag_wait_bounded<true>(p.ctrl + r, epoch, cta_abort, p.status, NFN_ERR_WAIT_PEER);
    *sh_flag = ok ? 1 : 0;
  }
  __syncthreads();
  if (!*sh_flag) return;
  const long long vecs = (long long)p.rows_per_rank * (p.n / 8);
  const long long slot_stride = (long long)p.rows_per_rank * p.n;
  const bool add_bias = p.flags & NFN_EPI_BIAS;
  for (long long i = (long long)blockIdx.x * TP_THREADS + threadIdx.x; i < vecs; i += (long long)gridDim.x * TP_THREADS) {
    const int row = (int)(i / (p.n / 8)), col = (int)(i % (p.n / 8)) * 8;
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < p.world; ++r) {
      float x8[8];
      // peers wrote these through NVLink: read around L1
      const uint4 u = __ldcg(reinterpret_cast<const uint4*>(p.slots + r * slot_stride + (long long)row * p.n + col));
      unpack8_bf16(u, x8);
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j] += x8[j];
    }
    if (add_bias) {
      float b8[8];
      unpack8_bf16(__ldg(reinterpret_cast<const uint4*>(p.bias + col)), b8);
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j] += b8[j];
    }
    if (p.resid) {
      float x8[8];
      unpack8_bf16(*reinterpret_cast<const uint4*>(p.resid + (long long)row * p.ld_resid + col), x8);
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j] += x8[j];
    }
    *reinterpret_cast<uint4*>(p.out + (long long)row * p.ld_out + col) = pack8_bf16(s);
  }
}

template <int BN, int STAGES>
static int launch_tp(const nfn_gemm_tp_args& a, cudaStream_t stream) {
  constexpr size_t SMEM = 1024 + (size_t)STAGES * (TP_BM * TP_BK * 2 + BN * TP_BK * 2) + 2 * EPI_TILE_BYTES_TP + 256;
  auto kern = gemm_tp_kernel<BN, STAGES>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess)
      return launch_check("gemm_tp attr", 0);
    attr_set[dev & 63] = true;
  }
  TpParams p{};
  p.mode = a.mode;
  p.m = a.m; p.n = a.n; p.k = a.k;
  p.tiles_m = ceil_div(a.m, TP_BM);
  p.tiles_n = ceil_div(a.n, BN);
  p.rank = a.rank; p.world = a.world; p.epoch = a.epoch; p.epoch_dev = a.epoch_dev;
  p.rows_per_rank = a.rows_per_rank;
  p.flags = a.flags; p.act_param = a.act_param;
  p.bias = static_cast<const __nv_bfloat16*>(a.bias);
  p.ctrl = a.ctrl_local;
  for (int r = 0; r < a.world; ++r) p.peer_ctrl[r] = a.ctrl_peer[r];
  p.status = status_ptr();
  const int sms = sm_count();
  const int tiles = p.tiles_m * p.tiles_n;
  p.n_copy = 0;
  CUtensorMap ta, tb;
  TpMaps maps;
  if (!make_tmap_2d(&ta, a.a, 2, (uint64_t)a.k, (uint64_t)a.m, (uint64_t)a.lda, TP_BK, TP_BM, 128)) return -3;
  if (a.mode == NFN_TP_GROUPED) {
    if (!make_tmap_3d(&tb, a.b, 2, (uint64_t)a.k, (uint64_t)a.n, (uint64_t)a.groups, (uint64_t)a.ldb, (uint64_t)a.ldb * a.n, TP_BK, BN, 1, 128)) return -3;
    p.tile_group = a.tile_group;
    p.num_m_tiles_dev = a.num_m_tiles_dev;
  } else if (!make_tmap_2d(&tb, a.b, 2, (uint64_t)a.k, (uint64_t)a.n, (uint64_t)a.ldb, TP_BK, BN, 128)) {
    return -3;
  }
  if (a.mode == NFN_TP_RS) {
    const long long slot_elems = (long long)a.rows_per_rank * a.n;
    for (int r = 0; r < a.world; ++r) {
      // owner r keeps slot [rank] for us inside its slot buffer
      const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(a.peer_bufs[r]) + (long long)a.rank * slot_elems;
      if (!make_tmap_2d(&maps.m[r], base, 2, (uint64_t)a.n, (uint64_t)a.rows_per_rank, (uint64_t)a.n, 64, TP_BM, 128)) return -3;
    }
    for (int r = a.world; r < TP_MAX_WORLD; ++r) maps.m[r] = maps.m[0];
    p.slots = static_cast<const __nv_bfloat16*>(a.peer_bufs[a.rank]);
    p.out = static_cast<__nv_bfloat16*>(a.out);
    p.ld_out = a.ld_out;
    p.resid = static_cast<const __nv_bfloat16*>(a.resid);
    p.ld_resid = a.ld_resid;
  } else {
    if (!make_tmap_2d(&maps.m[0], a.c, 2, (uint64_t)a.n, (uint64_t)a.m, (uint64_t)a.ldc, 64, TP_BM, 128)) return -3;
    for (int r = 1; r < TP_MAX_WORLD; ++r) maps.m[r] = maps.m[0];
    const int gathered_ld = (a.mode == NFN_TP_AG_A) ? a.lda : a.ldb;
    unsigned char* local = const_cast<unsigned char*>(static_cast<const unsigned char*>(a.mode == NFN_TP_AG_A ? a.a : a.b));
    p.local_buf = local;
    for (int r = 0; r < a.world; ++r)
      p.peer_src[r] = static_cast<const unsigned char*>(a.peer_bufs[r]) + (long long)r * a.rows_per_rank * gathered_ld * 2;
    if (a.world > 1 && a.mode != NFN_TP_GROUPED) p.n_copy = a.n_copy > 0 ? a.n_copy : 16;
  }
  int grid = std::min(sms, tiles + p.n_copy);
  if (grid <= p.n_copy) grid = p.n_copy + 1;
  kern<<<grid, TP_THREADS, SMEM, stream>>>(ta, tb, maps, p);
  return launch_check("gemm_tp", 1);
}

}  // namespace nfn

using namespace nfn;

extern "C" int nfn_gemm_tp(const nfn_gemm_tp_args* args, nfn_stream_t stream_) {
  if (!args) return fail(-1, "gemm_tp: null args");
  const nfn_gemm_tp_args& a = *args;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a.mode != NFN_TP_AG_A && a.mode != NFN_TP_AG_B && a.mode != NFN_TP_RS && a.mode != NFN_TP_GROUPED) return fail(-1, "gemm_tp: unknown mode");
  if (a.mode == NFN_TP_GROUPED) {
    // grouped GEMM: rows of A are sorted by group and padded to whole 128-row tiles; tile t
    // multiplies with B[tile_group[t]]. Single rank, no flags.
    if (a.m <= 0 || a.n <= 0 || a.k <= 0 || (a.k & 7) || (a.n & 7) || (a.lda & 7) || (a.ldb & 7) || (a.ldc & 7)) return fail(-1, "gemm_tp: grouped sizes and leading dimensions must be multiples of 8");
    if (!a.a || !a.b || !a.c || !a.tile_group || !a.num_m_tiles_dev || a.groups <= 0) return fail(-1, "gemm_tp: grouped mode needs a, b, c, tile_group, num_m_tiles_dev and groups");
    if (a.m % TP_BM) return fail(-1, "gemm_tp: grouped row capacity must be a multiple of 128");
    return (a.n >= 2048) ? launch_tp<256, 4>(a, stream) : launch_tp<128, 6>(a, stream);
  }
  if (a.m <= 0 || a.n <= 0 || a.k <= 0) return fail(-1, "gemm_tp: empty problem");
  if (a.world < 1 || a.world > TP_MAX_WORLD || a.rank < 0 || a.rank >= a.world) return fail(-1, "gemm_tp: bad rank / world (at most 8 ranks)");
  if ((a.k & 7) || (a.n & 7) || (a.lda & 7) || (a.ldb & 7)) return fail(-1, "gemm_tp: K, N and leading dimensions must be multiples of 8");
  if (!a.a || !a.b || !a.ctrl_local) return fail(-1, "gemm_tp: null operand");
  for (int r = 0; r < a.world; ++r)
    if (!a.peer_bufs[r] || !a.ctrl_peer[r]) return fail(-1, "gemm_tp: missing peer buffer or control pointer");
  const bool wide = a.n >= 2048 && (a.mode != NFN_TP_AG_B || a.rows_per_rank % 256 == 0);
  const int BN = wide ? 256 : 128;
  if (a.mode == NFN_TP_AG_A) {
    if (a.lda != a.k) return fail(-1, "gemm_tp: the gathered A buffer must be contiguous (lda == K)");
    if (a.rows_per_rank * a.world != a.m || a.rows_per_rank % TP_BM) return fail(-1, "gemm_tp: M must be world * rows_per_rank with rows_per_rank a multiple of 128");
    if (!a.c || (a.ldc & 7)) return fail(-1, "gemm_tp: bad output");
    if (CTRL_CHUNKS + a.m / TP_BM > a.ctrl_ints) return fail(-1, "gemm_tp: control block too small for M / 128 block flags");
  } else if (a.mode == NFN_TP_AG_B) {
    if (a.ldb != a.k) return fail(-1, "gemm_tp: the gathered B buffer must be contiguous (ldb == K)");
    if (a.rows_per_rank * a.world != a.n || a.rows_per_rank % BN) return fail(-1, "gemm_tp: N must be world * rows_per_rank with rows_per_rank a multiple of the N tile (128; 256 when N >= 2048)");
    if (!a.c || (a.ldc & 7)) return fail(-1, "gemm_tp: bad output");
    if (CTRL_CHUNKS + a.n / TP_BM > a.ctrl_ints) return fail(-1, "gemm_tp: control block too small for N / 128 block flags");
  } else {
    if (a.rows_per_rank * a.world != a.m || a.rows_per_rank % TP_BM) return fail(-1, "gemm_tp: M must be world * rows_per_rank with rows_per_rank a multiple of 128");
    if (!a.out || (a.ld_out & 7) || (a.resid && (a.ld_resid & 7))) return fail(-1, "gemm_tp: bad reduce-scatter output / residual");
    if (a.ctrl_ints < CTRL_CHUNKS) return fail(-1, "gemm_tp: control block too small");
  }
  return wide ? launch_tp<256, 4>(a, stream) : launch_tp<128, 6>(a, stream);
}
