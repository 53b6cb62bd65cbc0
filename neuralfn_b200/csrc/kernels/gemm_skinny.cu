// Products with 3 to 64 rows (batched decode, verification blocks): C[M, N] = A[M, K] . B[N, K]^T with the GEMM family's
// epilogue. Like the one- and two-row case this only streams the weight matrix once, so it is an HBM-bandwidth problem;
// unlike it there are enough rows for the tensor cores to do the arithmetic, but far too few for a tcgen05 tile (128 rows
// of A, of which at most half would be real). So: mma.sync.m16n8k16 with the token rows as the 16-row operand and eight
// weight rows as the 8-column operand, every operand fragment fetched from global memory as ONE 16-byte load per lane.
//
// That works because a contraction does not care about the order of k. Inside a chunk of 32 k-values lane (g, j) - g = lane / 4,
// j = lane % 4 - loads k = 8 j .. 8 j + 7 of weight row g (and of token rows g, g + 8): the four 32-bit words of that
// load are exactly the fragment registers of two k16 steps (words 0 / 1 = the two k-pairs of step 0, words 2 / 3 = step 1),
// with A and B using the same assignment. A warp's 32 lanes thus read 8 weight rows x 64 contiguous bytes per load.
//
// A CTA owns SK_NT * 8 weight rows; its eight warps split K between them (so a row's whole K range is in flight at
// once and even narrow products fill the GPU), keep SK_UNROLL chunks of loads in flight each, and add their partial
// tiles through shared memory; the last step applies alpha, bias, activation, residual and accumulate and stores bf16. The
// token rows (M x K, a few hundred KB at most) are read by every CTA and stay in L1 / L2.
//
// Counterpart in the reference: the small-M tiles of its quantised decode path (`glimmer_k_mmq.cu:48-60`, mmvq / mmq
// selection by row count); this kernel is the bf16-weight equivalent.
#include <algorithm>
#include <cstdint>

#include "common.h"
#include "nfn_kernels.h"
#include "sm100_ptx.cuh"

namespace nfn {

constexpr int SK_WARPS = 8, SK_THREADS = SK_WARPS * 32, SK_NT = 4, SK_ROWS = SK_NT * 8;

struct SkinnyParams {
  const __nv_bfloat16* a;
  const __nv_bfloat16* b;
  __nv_bfloat16* c;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* resid;
  int m, n, k, lda, ldb, ldc, ld_resid;
  int act, accum;
  float alpha, act_param;
};

__device__ __forceinline__ uint4 sk_ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void sk_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float sk_act(float v, int act, float prm) {
  switch (act) {
    case NFN_ACT_GELU_TANH: return gelu_tanh_f(v);
    case NFN_ACT_GELU_ERF: return gelu_erf_f(v);
    case NFN_ACT_SILU: return silu_f(v);
    case NFN_ACT_RELU2: { const float r = fmaxf(v, 0.f); return r * r; }
    case NFN_ACT_RELU: return fmaxf(v, 0.f);
    case NFN_ACT_TANH_CAP: return prm * fast_tanh(v / prm);
    default: return v;
  }
}

// MT = 16-row tiles of A (M <= 16 MT).
template <int MT>
__global__ void __launch_bounds__(SK_THREADS, MT <= 2 ? 2 : 1)
gemm_skinny_kernel(const SkinnyParams p) {
  constexpr int SK_UNROLL = MT <= 2 ? 4 : 2;  // chunks of weight loads in flight per warp (registers: 16 per chunk)
  extern __shared__ float sk_part[];  // [SK_WARPS][MT * 16][SK_ROWS + 1]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, j = lane & 3;
  const int n0 = blockIdx.x * SK_ROWS;
  // this warp's share of the 32-wide k chunks
  const int chunks = p.k / 32;
  const int c_lo = (int)((long long)chunks * warp / SK_WARPS), c_hi = (int)((long long)chunks * (warp + 1) / SK_WARPS);

  float acc[MT][SK_NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < SK_NT; ++nt)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[mt][nt][q] = 0.f;

  // weight rows of this lane (one per n-tile), clamped at the edge: a clamped row is computed twice and stored once
  const __nv_bfloat16* wrow[SK_NT];
#pragma unroll
  for (int nt = 0; nt < SK_NT; ++nt) wrow[nt] = p.b + (size_t)min(n0 + nt * 8 + g, p.n - 1) * p.ldb + 8 * j;
  // token rows g and g + 8 of every m-tile, clamped likewise (rows past M are never stored)
  const __nv_bfloat16* arow[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    arow[mt][0] = p.a + (size_t)min(mt * 16 + g, p.m - 1) * p.lda + 8 * j;
    arow[mt][1] = p.a + (size_t)min(mt * 16 + g + 8, p.m - 1) * p.lda + 8 * j;
  }

  for (int c0 = c_lo; c0 < c_hi; c0 += SK_UNROLL) {
    uint4 w[SK_UNROLL][SK_NT];
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u) {
      const bool ok = c0 + u < c_hi;
#pragma unroll
      for (int nt = 0; nt < SK_NT; ++nt) w[u][nt] = ok ? sk_ld_stream(wrow[nt] + (size_t)(c0 + u) * 32) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u) {
      if (c0 + u >= c_hi) break;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const uint4 x0 = __ldg(reinterpret_cast<const uint4*>(arow[mt][0] + (size_t)(c0 + u) * 32));
        const uint4 x1 = __ldg(reinterpret_cast<const uint4*>(arow[mt][1] + (size_t)(c0 + u) * 32));
#pragma unroll
        for (int nt = 0; nt < SK_NT; ++nt) {
          sk_mma(acc[mt][nt], x0.x, x1.x, x0.y, x1.y, w[u][nt].x, w[u][nt].y);
          sk_mma(acc[mt][nt], x0.z, x1.z, x0.w, x1.w, w[u][nt].z, w[u][nt].w);
        }
      }
    }
  }

  // partial tiles -> shared memory: accumulator (row g / g + 8, columns 2 j, 2 j + 1 of the n-tile)
  constexpr int LD = SK_ROWS + 1;
  float* mine = sk_part + (size_t)warp * (MT * 16) * LD;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < SK_NT; ++nt) {
      const int col = nt * 8 + 2 * j;
      mine[(mt * 16 + g) * LD + col] = acc[mt][nt][0];
      mine[(mt * 16 + g) * LD + col + 1] = acc[mt][nt][1];
      mine[(mt * 16 + g + 8) * LD + col] = acc[mt][nt][2];
      mine[(mt * 16 + g + 8) * LD + col + 1] = acc[mt][nt][3];
    }
  __syncthreads();
  // sum over the K slices and finish: alpha, bias, activation, residual, accumulate (the order of the tcgen05 kernels)
  for (int i = threadIdx.x; i < p.m * SK_ROWS; i += SK_THREADS) {
    const int r = i / SK_ROWS, col = i % SK_ROWS, n = n0 + col;
    if (n >= p.n) continue;
    float v = 0.f;
#pragma unroll
    for (int w8 = 0; w8 < SK_WARPS; ++w8) v += sk_part[((size_t)w8 * (MT * 16) + r) * LD + col];
    v *= p.alpha;
    if (p.bias) v += __bfloat162float(p.bias[n]);
    v = sk_act(v, p.act, p.act_param);
    if (p.resid) v += __bfloat162float(p.resid[(size_t)r * p.ld_resid + n]);
    __nv_bfloat16* cp = p.c + (size_t)r * p.ldc + n;
    if (p.accum) v += __bfloat162float(*cp);
    *cp = __float2bfloat16(v);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Up to 32 rows (opt-in, mode 3): token fragments in REGISTERS for the whole kernel, weights through a ring of bulk async copies.
//
// Why the kernel above stalls with two row tiles: it re-reads the token rows from L2 for every eight weight rows, and its
// loads in flight are bounded by registers (tens of KB per SM; the DRAM latency needs more than a hundred). Here
//  * a warp (sixteen per CTA) owns a fixed k range of at most UMAX chunks and loads its token fragments once (8 * MT * UMAX
//    registers);
//  * warp 0 streams the weights: per group of sixteen weight rows one bulk async copy per row (lane r copies row r: the CTA's
//    whole k range, a few KB contiguous) into a ring of shared-memory stages, completion counted on an mbarrier;
//  * the warps read their weight fragments from the stage (conflict-free 16-byte loads: the row pitch is 64 mod 128 bytes),
//    run 8 * MT mma per chunk in 2 * MT independent chains, and add their partial tiles through shared memory into the CTA's
//    fp32 strip [rows, columns of this pass]; the block barrier of that sum is also what frees the stage for the next copy.
// Measured steps on the way (32 x 12288 x 6656, L2 flushed): loads into registers one group ahead 65.5 us; eight warps and a
// ring of six 8-row stages filled by one thread 82 us (barrier and fixed-latency stalls: two warps per scheduler walking one
// dependent mma chain each, and the copy-issuing thread on the critical path); this form 55.4 us.
//
// K is longer than 8 warps x UMAX chunks, so S CTAs split it: they form a thread-block cluster, each fills its strip for the
// same weight rows, and after a cluster barrier CTA r sums column share r of all S strips over distributed shared memory in
// rank order (deterministic), applies the epilogue and stores bf16. No workspace, no second launch.
constexpr int RS_MAX_COLS = 256;       // most columns (weight rows) per pass of a cluster: strip = MT * 16 x 256 fp32
constexpr int RS_STAGES = 6;

__device__ __forceinline__ uint32_t rs_cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void rs_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float rs_ld_peer(const float* local, uint32_t rank) {
  uint32_t a = (uint32_t)__cvta_generic_to_shared(local), ra;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
  return v;
}
__device__ __forceinline__ void rs_bulk_g2s(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar)
               : "memory");
}

constexpr int RS_WARPS = 16, RS_THREADS = RS_WARPS * 32, RS_GROUP_ROWS = 16;   // weight rows per ring stage: two mma column tiles

template <int MT, int UMAX>
struct ResidentLayout {
  static constexpr int ROWS = MT * 16;
  static constexpr int PITCH = RS_WARPS * UMAX * 64 + 64;          // bytes per weight row in a stage: 64 mod 128
  static constexpr int STAGE = RS_GROUP_ROWS * PITCH;
  static constexpr int PART_BYTES = 2 * RS_WARPS * ROWS * RS_GROUP_ROWS * 4;   // two buffers of every warp's partial tile
  static constexpr int STRIP_BYTES = ROWS * RS_MAX_COLS * 4;
  static constexpr int STAGES = (227 * 1024 - 256 - PART_BYTES - STRIP_BYTES) / STAGE;
  static constexpr int TOTAL = PART_BYTES + STRIP_BYTES + STAGES * STAGE;
  static_assert(STAGES >= 2 && STAGES <= RS_STAGES, "ring depth");
};

template <int MT, int UMAX>
__global__ void __launch_bounds__(RS_THREADS, 1)
gemm_skinny_resident_kernel(const SkinnyParams p, const int S, const int pass_cols, const int passes_total, int* status) {
  using Lay = ResidentLayout<MT, UMAX>;
  constexpr int ROWS = Lay::ROWS, PITCH = Lay::PITCH, STAGE = Lay::STAGE, NS = Lay::STAGES, GR = RS_GROUP_ROWS;
  extern __shared__ __align__(128) unsigned char rs_smem[];
  __shared__ __align__(8) uint64_t full[RS_STAGES];
  __shared__ int sh_abort;
  float* part = reinterpret_cast<float*>(rs_smem);                                   // [2][RS_WARPS][ROWS][GR]
  float* strip = reinterpret_cast<float*>(rs_smem + Lay::PART_BYTES);                // [ROWS][pass_cols]
  unsigned char* ring = rs_smem + Lay::PART_BYTES + Lay::STRIP_BYTES;               // [NS][GR][PITCH]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, j = lane & 3;
  const uint32_t ks = rs_cluster_ctarank();
  const int cluster = blockIdx.x / S, n_clusters = gridDim.x / S;
  // chunks of 32 k-values: this CTA's share of K, and this warp's share of that
  const int chunks = p.k / 32;
  const int cta_lo = (int)((long long)chunks * ks / S), cta_cnt = (int)((long long)chunks * (ks + 1) / S) - cta_lo;
  const int w_lo = cta_cnt * warp / RS_WARPS, cnt = cta_cnt * (warp + 1) / RS_WARPS - w_lo;

  if (threadIdx.x == 0) {
    sh_abort = 0;
    for (int s2 = 0; s2 < NS; ++s2) mbar_init(smem_u32(&full[s2]), 1);
    fence_mbar_init();
  }
  __syncthreads();

  // the groups of sixteen weight rows this cluster works through, pass after pass (pass_cols is a multiple of 16)
  auto groups_of = [&](int pass) { return (min(pass_cols, p.n - pass * pass_cols) + GR - 1) / GR; };
  int total = 0;
  for (int pass = cluster; pass < passes_total; pass += n_clusters) total += groups_of(pass);
  int prod_pass = cluster, prod_grp = 0;                                             // warp 0 (uniform)
  const uint32_t slice_bytes = (uint32_t)cta_cnt * 64u;
  auto issue = [&](int seq) {                                                        // warp 0: lane r copies weight row r of the group
    const int st = seq % NS, n0 = prod_pass * pass_cols + prod_grp * GR;
    const uint32_t bar = smem_u32(&full[st]);
    if (lane == 0) mbar_expect_tx(bar, (uint32_t)GR * slice_bytes);
    if (lane < GR)
      rs_bulk_g2s(smem_u32(ring + (size_t)st * STAGE + (size_t)lane * PITCH), p.b + (size_t)min(n0 + lane, p.n - 1) * p.ldb + (size_t)cta_lo * 32,
                  slice_bytes, bar);
    if (++prod_grp == groups_of(prod_pass)) { prod_grp = 0; prod_pass += n_clusters; }
  };
  if (warp == 0)
    for (int seq = 0; seq < min(NS, total); ++seq) issue(seq);

  uint4 xa[UMAX][MT][2];
#pragma unroll
  for (int u = 0; u < UMAX; ++u)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = mt * 16 + g + 8 * h;
        xa[u][mt][h] = (u < cnt && r < p.m) ? __ldg(reinterpret_cast<const uint4*>(p.a + (size_t)r * p.lda + (size_t)(cta_lo + w_lo + u) * 32 + 8 * j))
                                             : make_uint4(0u, 0u, 0u, 0u);
      }

  bool dead = false;      // a wait ran out: keep walking (the cluster's barriers still need this CTA) without touching the ring
  int seq = 0;
  for (int pass = cluster; pass < passes_total; pass += n_clusters) {     // the same trip count in every CTA of a cluster
    const int n_pass = pass * pass_cols;
    const int cols = min(pass_cols, p.n - n_pass), groups = (cols + GR - 1) / GR;
    for (int gi = 0; gi < groups; ++gi, ++seq) {
      const int st = seq % NS, buf = seq & 1;
      bool ok = dead ? false : mbar_wait_bounded(smem_u32(&full[st]), (uint32_t)(seq / NS) & 1u, &sh_abort, status, NFN_ERR_WAIT_FULL);
      float acc[MT][2][4];                                                // [row tile][column tile of eight weight rows]
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int q = 0; q < 4; ++q) acc[mt][nt][q] = 0.f;
      if (ok) {
        const unsigned char* wrow = ring + (size_t)st * STAGE + (size_t)g * PITCH + (size_t)w_lo * 64 + j * 16;
#pragma unroll
        for (int u = 0; u < UMAX; ++u)
          if (u < cnt) {
            const uint4 w0 = *reinterpret_cast<const uint4*>(wrow + u * 64);
            const uint4 w1 = *reinterpret_cast<const uint4*>(wrow + 8 * PITCH + u * 64);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              sk_mma(acc[mt][0], xa[u][mt][0].x, xa[u][mt][1].x, xa[u][mt][0].y, xa[u][mt][1].y, w0.x, w0.y);
              sk_mma(acc[mt][1], xa[u][mt][0].x, xa[u][mt][1].x, xa[u][mt][0].y, xa[u][mt][1].y, w1.x, w1.y);
              sk_mma(acc[mt][0], xa[u][mt][0].z, xa[u][mt][1].z, xa[u][mt][0].w, xa[u][mt][1].w, w0.z, w0.w);
              sk_mma(acc[mt][1], xa[u][mt][0].z, xa[u][mt][1].z, xa[u][mt][0].w, xa[u][mt][1].w, w1.z, w1.w);
            }
          }
      }
      float* mine = part + ((size_t)(buf * RS_WARPS + warp) * ROWS) * GR;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          *reinterpret_cast<float2*>(mine + (mt * 16 + g) * GR + nt * 8 + 2 * j) = make_float2(acc[mt][nt][0], acc[mt][nt][1]);
          *reinterpret_cast<float2*>(mine + (mt * 16 + g + 8) * GR + nt * 8 + 2 * j) = make_float2(acc[mt][nt][2], acc[mt][nt][3]);
        }
      ok = __syncthreads_and(ok);                                        // every warp is done with stage st and with its partial tile
      if (!ok) dead = true;
      if (warp == 0 && !dead && seq + NS < total) issue(seq + NS);
      for (int i = threadIdx.x; i < ROWS * GR; i += RS_THREADS) {
        float v = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < RS_WARPS; ++w8) v += part[((size_t)(buf * RS_WARPS + w8) * ROWS) * GR + i];
        strip[(i / GR) * pass_cols + gi * GR + (i % GR)] = v;
      }
    }
    rs_cluster_sync();                                                    // every strip of the cluster is complete
    // CTA ks finishes columns [share_lo, share_hi) of the pass
    const int share_lo = (int)((long long)cols * ks / S), share_hi = (int)((long long)cols * (ks + 1) / S), width = share_hi - share_lo;
    for (int i = threadIdx.x; i < p.m * width; i += RS_THREADS) {
      const int r = i / width, c = share_lo + i % width, n = n_pass + c;
      float v = 0.f;
      for (int s2 = 0; s2 < S; ++s2) v += rs_ld_peer(&strip[r * pass_cols + c], (uint32_t)s2);
      v *= p.alpha;
      if (p.bias) v += __bfloat162float(p.bias[n]);
      v = sk_act(v, p.act, p.act_param);
      if (p.resid) v += __bfloat162float(p.resid[(size_t)r * p.ld_resid + n]);
      __nv_bfloat16* cp = p.c + (size_t)r * p.ldc + n;
      if (p.accum) v += __bfloat162float(*cp);
      *cp = __float2bfloat16(v);
    }
    rs_cluster_sync();                                                    // nobody overwrites a strip a peer still reads
  }
  if (dead)
    for (int i = 0; i < 64; ++i) __nanosleep(1000);                       // let copies in flight land before the CTA goes away
}

template <int MT, int UMAX>
static int launch_skinny_resident(const SkinnyParams& p, cudaStream_t stream) {
  using Lay = ResidentLayout<MT, UMAX>;
  auto kern = gemm_skinny_resident_kernel<MT, UMAX>;
  const int chunks = p.k / 32;
  const int S = (chunks + RS_WARPS * UMAX - 1) / (RS_WARPS * UMAX);
  if (S > 8) return 0;                                                   // portable cluster size
  const size_t smem = Lay::TOTAL;
  static int max_clusters[64][9] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = S;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.blockDim = dim3(RS_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int& mc = max_clusters[dev & 63][S];
  if (!mc) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      cudaGetLastError();
      mc = -1;
      return 0;
    }
    cfg.gridDim = dim3(sm_count() / S * S, 1, 1);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      mc = -1;
    } else {
      mc = std::min(n, sm_count() / S);
    }
  }
  if (mc <= 0) return 0;
  // passes of equal width, a whole number of them per cluster: groups of sixteen weight rows, at most RS_MAX_COLS columns per pass
  const int groups = (p.n + RS_GROUP_ROWS - 1) / RS_GROUP_ROWS, max_groups = RS_MAX_COLS / RS_GROUP_ROWS;
  const int clusters = std::min(mc, groups);
  const int per_cluster = (groups + clusters - 1) / clusters;                       // groups one cluster works through
  const int passes_per_cluster = (per_cluster + max_groups - 1) / max_groups;
  const int pass_cols = (per_cluster + passes_per_cluster - 1) / passes_per_cluster * RS_GROUP_ROWS;
  const int passes = (p.n + pass_cols - 1) / pass_cols;
  cfg.gridDim = dim3(std::min(clusters, passes) * S, 1, 1);
  if (cudaLaunchKernelEx(&cfg, kern, p, S, pass_cols, passes, status_ptr()) != cudaSuccess) return launch_check("gemm_skinny_resident", 0);
  const int rc = launch_check("gemm_skinny_resident", 1);
  return rc == 0 ? 1 : rc;
}

static int g_skinny_mode = 1;

// Returns 1 when it launched, 0 when the product is not one of its cases (the caller continues with the tcgen05 path),
// negative on a launch error.
int try_launch_skinny(const nfn_gemm_args& a, cudaStream_t stream) {
  const int unsupported = NFN_EPI_SAVE_PRE | NFN_EPI_DACT | NFN_EPI_OUT_F32;
  if (!g_skinny_mode || a.m < 3 || a.m > 64 || a.a_mn || a.b_mn || (a.flags & unsupported) || (a.k & 31) || a.k < 256 || (a.lda & 7) || (a.ldb & 7))
    return 0;
  // measured (12288 x 6656 weights, L2 flushed): 8 rows 49 us against 52 us on the tcgen05 split-K path, 32 rows 65 against
  // 50 us, 64 rows 81 against 50 us - with more than one 16-row tile the token fragments, which every warp fetches from L2
  // right before use, become the bottleneck. So by default only up to 16 rows come here; mode 2 forces every eligible product.
  // The register-resident cluster form (mode 3) removes those re-reads: 55.4 us at 32 rows (tcgen05 split-K: 50.1), 47.1 us at
  // 8 rows (49.2 here, 52 - 54 on tcgen05). It stays opt-in: clusters of four fill only 132 of the 148 SMs, and its ring holds
  // two 16-row stages (the partial tiles of sixteen warps take 64 KB), which is less in flight than the DRAM latency asks for.
  // the weights must dominate the traffic for this to be the right kernel: N x K well above the token rows
  if ((long long)a.n * a.k < (1LL << 20)) return 0;
  const bool aligned = ((reinterpret_cast<uintptr_t>(a.a) | reinterpret_cast<uintptr_t>(a.b)) & 15) == 0;
  if (!aligned) return 0;
  SkinnyParams p;
  p.a = static_cast<const __nv_bfloat16*>(a.a);
  p.b = static_cast<const __nv_bfloat16*>(a.b);
  p.c = static_cast<__nv_bfloat16*>(a.c);
  p.bias = (a.flags & NFN_EPI_BIAS) ? static_cast<const __nv_bfloat16*>(a.bias) : nullptr;
  p.resid = (a.flags & NFN_EPI_RESID) ? static_cast<const __nv_bfloat16*>(a.aux_in) : nullptr;
  p.m = a.m; p.n = a.n; p.k = a.k; p.lda = a.lda; p.ldb = a.ldb; p.ldc = a.ldc; p.ld_resid = a.ld_aux_in;
  p.act = (a.flags >> NFN_EPI_ACT_SHIFT) & 0xF;
  p.accum = (a.flags & NFN_EPI_ACCUM) ? 1 : 0;
  p.alpha = a.alpha; p.act_param = a.act_param;
  const int mt = (a.m + 15) / 16;
  // mode 3: the register-resident cluster form for every product up to 32 rows (measured slower than both other paths, see above)
  if (g_skinny_mode == 3 && mt <= 2) {
    const int rc = mt == 2 ? launch_skinny_resident<2, 4>(p, stream) : launch_skinny_resident<1, 4>(p, stream);
    if (rc != 0) return rc;
  }
  if (a.m > 16 && g_skinny_mode != 2) return 0;
  const int grid = (a.n + SK_ROWS - 1) / SK_ROWS;
  const size_t smem = (size_t)SK_WARPS * (mt <= 1 ? 16 : (mt <= 2 ? 32 : 64)) * (SK_ROWS + 1) * sizeof(float);
  cudaError_t e = cudaSuccess;
  if (mt <= 1) {
    gemm_skinny_kernel<1><<<grid, SK_THREADS, smem, stream>>>(p);
  } else if (mt <= 2) {
    gemm_skinny_kernel<2><<<grid, SK_THREADS, smem, stream>>>(p);
  } else {
    static bool raised = false;
    if (!raised) {
      e = cudaFuncSetAttribute(gemm_skinny_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      raised = e == cudaSuccess;
    }
    if (e != cudaSuccess) return fail(-2, "gemm_skinny: cannot raise the dynamic shared memory limit");
    gemm_skinny_kernel<4><<<grid, SK_THREADS, smem, stream>>>(p);
  }
  const int rc = launch_check("gemm_skinny", 1);
  return rc == 0 ? 1 : rc;
}

}  // namespace nfn

// 1 (default): products with 3 - 16 rows over K-major operands take the mma.sync weight-streaming kernel; 2: up to 64 rows
// do; 3: products up to 32 rows take its register-resident cluster form; 0: none (the tcgen05 split-K path). Returns the
// previous setting.
extern "C" int nfn_gemm_skinny_set_impl(int mode) {
  const int prev = nfn::g_skinny_mode;
  nfn::g_skinny_mode = mode < 0 ? 0 : (mode > 3 ? 3 : mode);
  return prev;
}
