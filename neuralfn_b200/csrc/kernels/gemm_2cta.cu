// BF16 GEMM on CTA pairs (tcgen05 cta_group::2): two CTAs of a 2-CTA cluster share one
// 256 x 256 output tile. Each CTA stages its own 128 rows of A and its own 128 rows of B
// per k-block; the pair's single MMA (M = 256, N = 256, issued by the leader CTA) reads both
// CTAs' shared memory and leaves each CTA's 128 x 256 half of the accumulator in that CTA's
// TMEM. Per output element this halves the B-operand bytes that cross the L2 -> SM fabric,
// which is what bounds the 1-CTA kernel at K = 768 (each 128 x 256 tile pulls 590 KB for
// 50 MFLOP there; the pair pulls 393 KB per CTA for the same work).
//
//   warp 0 (each CTA)   TMA producer: A rows [m0 + 128 r, +128), B rows [n0 + 128 r, +128) with
//                       cta_group::2 loads whose transaction bytes count on the LEADER's barrier
//   warp 1 (leader)     MMA issuer; commits are multicast to both CTAs' barriers
//   warps 2..9 (each)   epilogue of the CTA's own 128 rows (same fused epilogue / TMA-store
//                       path as the 1-CTA kernel); the peer releases the accumulator with a
//                       remote mbarrier arrive on the leader's barrier
//
// A is K-major; B is K-major (forward products X W^T) or MN-major (input gradients dY W, template
// parameter B_MN: each CTA then stages its 128 columns of B as two 64-column panels of BK rows).
// MN-major A, split-K and fp32 / accumulating outputs stay on the 1-CTA kernel. No load in this
// file uses cluster multicast.
#include <algorithm>

#include "gemm_epilogue.cuh"
#include "nfn_kernels.h"

namespace nfn {

int epi_direct_flag();  // gemm_tcgen05.cu

constexpr int P2_BM = 128;          // rows per CTA (256 per pair)
constexpr int P2_BN = 256;          // columns per pair tile; each CTA stages 128 of the B rows
constexpr int P2_BK = 64;
constexpr int P2_THREADS = 320;
constexpr int P2_STAGES = 6;
constexpr uint32_t P2_EPI_TILE = 128 * 64 * 2;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_2cta(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2cta() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc_2cta(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// tile load into THIS CTA's shared memory; the bytes are counted on the barrier at `bar_cluster`
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const void* tmap, uint32_t bar_cluster, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(tmap), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  const uint32_t z = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t"
      "}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(z)
      : "memory");
}
// arrive on the barrier at the same shared-memory offset in both CTAs of the pair once the
// MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(mask)
               : "memory");
}

template <bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P2_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ CUtensorMap tma_aux, const GemmParams p) {
  constexpr int BM = P2_BM, BN = P2_BN, BK = P2_BK, STAGES = P2_STAGES, UMMA_K = 16, EPI_CHUNK = 64;
  constexpr uint32_t EPI_TILE_BYTES = P2_EPI_TILE;
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + 2 * EPI_TILE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint64_t* epi_bar = bars + 2 * STAGES + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 5);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);   // leader's copy is the live one: one expect_tx arrive + both CTAs' bytes
      mbar_init(smem_u32(&empty_bar[s]), 1);  // one multicast commit per phase, in each CTA
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&tfull_bar[b]), 1);   // multicast commit, in each CTA
      mbar_init(smem_u32(&tempty_bar[b]), 16);  // leader's copy: 8 epilogue warps of each CTA
    }
    mbar_init(smem_u32(epi_bar), 8);
    fence_mbar_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc_2cta(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish_2cta();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_mn = p.tiles_m * p.tiles_n;  // pair tiles: 256 x 256
  const int num_tiles = tiles_mn;
  const int total_kb = (p.k + BK - 1) / BK;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        int tm, tn;
        tile_mn(p, tile, tm, tn);
        const int m0 = tm * (2 * BM) + (int)rank * BM;
        const int nb0 = tn * BN + (int)rank * (BN / 2);
        for (int kb = 0; kb < total_kb; ++kb) {
          if (!mbar_wait_bounded(smem_u32(&empty_bar[stage]), phase ^ 1, cta_abort, p.status, NFN_ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t fb_leader = mapa_shared(smem_u32(&full_bar[stage]), 0);
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          if (leader) mbar_expect_tx(smem_u32(&full_bar[stage]), 2 * STAGE_BYTES);
          tma_load_2d_pair(sa, &tma_a, fb_leader, kb * BK, m0);
          if (!B_MN) {
            tma_load_2d_pair(sa + A_BYTES, &tma_b, fb_leader, kb * BK, nb0);
          } else {
#pragma unroll
            for (int j = 0; j < (BN / 2) / 64; ++j) tma_load_2d_pair(sa + A_BYTES + j * 8192, &tma_b, fb_leader, nb0 + 64 * j, kb * BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, 0, B_MN ? 1 : 0);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
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
          const uint64_t da = make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t db = B_MN ? make_smem_desc_sw128(sa + A_BYTES, 8192, 1024) : make_smem_desc_sw128(sa + A_BYTES, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t a_adv = (uint64_t)((UMMA_K * 2) >> 4) * kk;
            const uint64_t b_adv = B_MN ? (uint64_t)((UMMA_K * 128) >> 4) * kk : a_adv;
            umma_bf16_ss_pair(tmem_d, da + a_adv, db + b_adv, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit_pair(smem_u32(&empty_bar[stage]));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(smem_u32(&tfull_bar[acc]));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    const uint32_t tempty_leader0 = mapa_shared(smem_u32(&tempty_bar[0]), 0);
    const uint32_t tempty_leader1 = mapa_shared(smem_u32(&tempty_bar[1]), 0);
#define EPI_TILE_FIRST pair
#define EPI_TILE_STEP n_pairs
#define EPI_TILE_M0(tm) ((tm) * (2 * BM) + (int)rank * BM)
#define EPI_RELEASE_ACC(acc) mbar_arrive_cluster((acc) ? tempty_leader1 : tempty_leader0)
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
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  cluster_sync_all();  // neither CTA leaves (or frees TMEM) while its partner may still touch it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2cta(tmem_base, TMEM_COLS);
  }
}

}  // namespace nfn

namespace nfn {

template <bool B_MN>
static int launch_gemm_pair(const nfn_gemm_args& a, cudaStream_t stream) {
  constexpr size_t SMEM = 1024 + (size_t)P2_STAGES * (P2_BM * P2_BK * 2 + (P2_BN / 2) * P2_BK * 2) + 2 * P2_EPI_TILE + 256;
  // per device: opt in to the shared-memory size once and ask how many 2-CTA clusters can be
  // resident at the same time (GPCs with an odd number of free SMs leave one SM without a partner)
  static int max_pairs[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = gemm_bf16_pair_kernel<B_MN>;
  if (!max_pairs[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess)
      return launch_check("gemm_pair attr", 0);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count() & ~1, 1, 1);
    cfg.blockDim = dim3(P2_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / 2;
    }
    max_pairs[dev & 63] = std::min(n, sm_count() / 2);
  }
  CUtensorMap ta, tb, tc, tx;
  if (!make_tmap_2d(&ta, a.a, 2, (uint64_t)a.k, (uint64_t)a.m, (uint64_t)a.lda, P2_BK, P2_BM, 128)) return -3;
  if (!B_MN) {
    if (!make_tmap_2d(&tb, a.b, 2, (uint64_t)a.k, (uint64_t)a.n, (uint64_t)a.ldb, P2_BK, P2_BN / 2, 128)) return -3;
  } else {
    if (!make_tmap_2d(&tb, a.b, 2, (uint64_t)a.n, (uint64_t)a.k, (uint64_t)a.ldb, 64, P2_BK, 128)) return -3;
  }
  if (!make_tmap_2d(&tc, a.c, 2, (uint64_t)a.n, (uint64_t)a.m, (uint64_t)a.ldc, 64, P2_BM, 128)) return -3;
  tx = tc;
  if ((a.flags & NFN_EPI_SAVE_PRE) &&
      !make_tmap_2d(&tx, a.aux_out, 2, (uint64_t)a.n, (uint64_t)a.m, (uint64_t)a.ld_aux_out, 64, P2_BM, 128))
    return -3;
  GemmParams p;
  p.c = a.c;
  p.bias = static_cast<const __nv_bfloat16*>(a.bias);
  p.aux_in = static_cast<const __nv_bfloat16*>(a.aux_in);
  p.aux_out = static_cast<__nv_bfloat16*>(a.aux_out);
  p.m = a.m; p.n = a.n; p.k = a.k;
  p.ldc = a.ldc; p.ld_aux_in = a.ld_aux_in; p.ld_aux_out = a.ld_aux_out;
  p.flags = a.flags | epi_direct_flag(); p.alpha = a.alpha; p.act_param = a.act_param;
  p.tiles_m = ceil_div(a.m, 2 * P2_BM);
  p.tiles_n = ceil_div(a.n, P2_BN);
  p.split_k = 1;
  p.kb_per_split = ceil_div(a.k, P2_BK);
  p.split_stride = 0;
  p.status = status_ptr();
  p.raster_gw = pick_raster_gw(a.m, a.k, p.tiles_n);
  const int tiles = p.tiles_m * p.tiles_n;
  const int pairs = std::min(max_pairs[dev & 63], tiles);
  kern<<<2 * pairs, P2_THREADS, SMEM, stream>>>(ta, tb, tc, tx, p);
  const int rc = launch_check("gemm_pair", 1);
  return rc < 0 ? rc : 1;
}

// Returns 1 when the problem was launched on CTA pairs, 0 when it is not eligible, < 0 on error.
int try_launch_gemm_pair(const nfn_gemm_args& a, cudaStream_t stream) {
  const bool out_f32 = a.flags & NFN_EPI_OUT_F32, accum = a.flags & NFN_EPI_ACCUM;
  if (a.a_mn || out_f32 || accum || a.split_k > 1) return 0;
  if (a.m < 512 || a.n < 256 || a.k < 256) return 0;
  return a.b_mn ? launch_gemm_pair<true>(a, stream) : launch_gemm_pair<false>(a, stream);
}

}  // namespace nfn
