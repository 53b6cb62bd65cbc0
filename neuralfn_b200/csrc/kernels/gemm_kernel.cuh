// Device side of the persistent, warp-specialised BF16 GEMM for sm_100a.
//
//   warp 0      : TMA producer   (one lane issues cp.async.bulk.tensor tile loads)
//   warp 1      : MMA issuer     (one lane issues tcgen05.mma; owns the TMEM allocation)
//   warps 2..9  : epilogue       (tcgen05.ld accumulator -> fused epilogue -> global)
//
// Tiles are 128 x BN x 64 with a STAGES-deep shared-memory ring (128-byte swizzle,
// filled by TMA, consumed by tcgen05.mma through shared-memory matrix descriptors).
// The fp32 accumulator lives in TMEM and is double-buffered, so the epilogue of tile
// i overlaps the main loop of tile i+1. bf16 outputs leave through a swizzled
// shared-memory staging tile and TMA bulk stores (fully coalesced, clipped at the
// matrix edge by the hardware); fp32 / accumulating / split-K outputs use direct
// bounds-checked stores.
#pragma once
#include "gemm_epilogue.cuh"

namespace nfn {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 320;
constexpr int EPI_CHUNK = 64;                       // columns per staged chunk
constexpr uint32_t EPI_TILE_BYTES = BM * EPI_CHUNK * 2;  // 16 KB

template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ CUtensorMap tma_aux,
                 const GemmParams p) {
  constexpr uint32_t A_BYTES = BM * BK * 2;
  constexpr uint32_t B_BYTES = BN * BK * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulator buffers
  static_assert(TMEM_COLS == 256 || TMEM_COLS == 512, "TMEM columns must be a power of two");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;  // 2 staging tiles, 1024-aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + 2 * EPI_TILE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint64_t* epi_bar = bars + 2 * STAGES + 4;  // 8 arrivals (one per epilogue warp): epilogue-wide sync with a bounded wait
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 5);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&tfull_bar[b]), 1);
      mbar_init(smem_u32(&tempty_bar[b]), 8);
    }
    mbar_init(smem_u32(epi_bar), 8);
    fence_mbar_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_mn = p.tiles_m * p.tiles_n;
  const int num_tiles = tiles_mn * p.split_k;
  const int total_kb = (p.k + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int sp = tile / tiles_mn, t2 = tile % tiles_mn;
        int tm, tn;
        tile_mn(p, t2, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        const int kb_lo = p.group_rows ? p.group_rows[sp] / BK : sp * p.kb_per_split;
        const int kb_hi = p.group_rows ? min(total_kb, p.group_rows[sp + 1] / BK) : min(total_kb, kb_lo + p.kb_per_split);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait_bounded(smem_u32(&empty_bar[stage]), phase ^ 1, cta_abort, p.status,
                                 NFN_ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t fb = smem_u32(&full_bar[stage]);
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
          mbar_expect_tx(fb, STAGE_BYTES);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d(sa, &tma_a, fb, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, &tma_a, fb, m0 + 64 * j, k0);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tma_b, fb, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &tma_b, fb, n0 + 64 * j, k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t stage = 0, phase = 0;
      uint32_t acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int sp = tile / tiles_mn;
        const int kb_lo = p.group_rows ? p.group_rows[sp] / BK : sp * p.kb_per_split;
        const int kb_hi = p.group_rows ? min(total_kb, p.group_rows[sp + 1] / BK) : min(total_kb, kb_lo + p.kb_per_split);
        if (!mbar_wait_bounded(smem_u32(&tempty_bar[acc]), acc_phase ^ 1, cta_abort, p.status,
                               NFN_ERR_WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait_bounded(smem_u32(&full_bar[stage]), phase, cta_abort, p.status,
                                 NFN_ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
          const uint64_t da = A_MN ? make_smem_desc_sw128(sa, 8192, 1024)
                                   : make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t db = B_MN ? make_smem_desc_sw128(sb, 8192, 1024)
                                   : make_smem_desc_sw128(sb, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // advance the start address by one UMMA_K slice (encoded in 16-byte units)
            const uint64_t a_adv = A_MN ? (uint64_t)((UMMA_K * 128) >> 4) * kk
                                        : (uint64_t)((UMMA_K * 2) >> 4) * kk;
            const uint64_t b_adv = B_MN ? (uint64_t)((UMMA_K * 128) >> 4) * kk
                                        : (uint64_t)((UMMA_K * 2) >> 4) * kk;
            umma_bf16_ss(tmem_d, da + a_adv, db + b_adv, idesc, (kb > kb_lo || kk > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&empty_bar[stage]));  // frees the smem stage when MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(smem_u32(&tfull_bar[acc]));  // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
#define EPI_TILE_FIRST ((int)blockIdx.x)
#define EPI_TILE_STEP ((int)gridDim.x)
#define EPI_TILE_M0(tm) ((tm) * BM)
#define EPI_RELEASE_ACC(acc) mbar_arrive(smem_u32(&tempty_bar[acc]))
#include "gemm_epilogue_body.inc"
#undef EPI_TILE_FIRST
#undef EPI_TILE_STEP
#undef EPI_TILE_M0
#undef EPI_RELEASE_ACC
  }

  // ---------------------------------------------------------------- teardown --
  tc_fence_before();
  __syncthreads();
  if (*cta_abort) {
    // give any copy or MMA still in flight time to land before shared memory and
    // TMEM are released
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace nfn
