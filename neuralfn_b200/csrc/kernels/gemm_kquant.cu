// Prefill GEMM over K-quant weights with the dequantisation fused into the operand pipeline:
// C[M, N] = A[M, K] . dequant(W)[N, K]^T, W stored as Q4_K / Q5_K / Q6_K super-blocks (256
// weights each, GGUF layouts). The bf16 weight matrix is never written to memory: four producer
// warps decode each 128 x 64 weight tile straight into the 128-byte-swizzled shared-memory
// layout that tcgen05.mma reads, while one TMA thread streams the activation tiles; the
// accumulator lives in TMEM and leaves through the same fused epilogue as the bf16 GEMM (bias,
// activation, residual, TMA store).
//
//   warp 0        TMA producer (A tiles)
//   warp 1        MMA issuer
//   warps 2..9    epilogue
//   warps 10..13  weight decoders: thread r decodes row r of the tile (64 weights per k-block =
//                 a quarter of one super-block) and writes eight 16-byte chunks
//
// Per stage the full barrier collects five arrivals: the TMA thread's expect_tx and one elected
// lane of every decoder warp (after its writes were fenced into the async proxy).
//
// The same pipeline serves NF4 base weights (4-bit codes, one fp32 absmax per 64 weights) and a
// fused LoRA branch: the rank-r update s * (x A^T) B^T rides along as ONE extra k-block whose A
// tile is the pre-computed T = s * x A^T (bf16 [M, 64], zero-padded beyond r) and whose B tile
// is the adapter's B matrix (bf16 [N, 64]), both fetched by TMA, so base product and adapter
// accumulate in the same TMEM tile and leave through one epilogue.
//
// Reference counterpart: the grouped MMQ prefill path (neuralfn/csrc/tile_cuda/glimmer_k_mmq.cu,
// kernels.cu:1324-2015), which runs llama.cpp's int8 mma.sync tiles; this kernel keeps the
// weights in their GGUF bytes and feeds the 5th-generation tensor cores in bf16 instead.
#include "gemm_kernel.cuh"
#include "nfn_kernels.h"

namespace nfn {

constexpr int KQ_BN = 128;
constexpr int KQ_STAGES = 6;
constexpr int KQ_THREADS = 14 * 32;
constexpr int KQ_DEC_WARP0 = 10;

__device__ __forceinline__ float kq_half(const uint8_t* p) {
  return __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(p)));
}
__device__ __forceinline__ void kq_scale_min(int j, const uint8_t* q, float* sc, float* mn) {
  if (j < 4) {
    *sc = (float)(q[j] & 63);
    *mn = (float)(q[j + 4] & 63);
  } else {
    *sc = (float)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
    *mn = (float)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}
__device__ __forceinline__ void kq_store8(uint8_t* tile, int row, int chunk, const float (&v)[8]) {
  *reinterpret_cast<uint4*>(tile + row * 128 + ((chunk ^ (row & 7)) << 4)) = pack8_bf16(v);
}

constexpr int NFN_QTYPE_NF4_ = NFN_QTYPE_NF4;
__constant__ float kq_nf4[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                                 -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                                 0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                                 0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};

// 64 NF4 weights (32 code bytes, low nibble = even element) times their group's absmax
__device__ __forceinline__ void kq_decode_nf4(const uint8_t* codes, float absmax, uint8_t* tile, int row) {
  const uint4* q = reinterpret_cast<const uint4*>(codes);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint4 u = __ldg(q + h);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int c = 0; c < 4; ++c) {  // 4 bytes -> 8 weights
      float v[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t byte = (w[c] >> (8 * e)) & 0xFF;
        v[2 * e] = kq_nf4[byte & 0xF] * absmax;
        v[2 * e + 1] = kq_nf4[byte >> 4] * absmax;
      }
      kq_store8(tile, row, 4 * h + c, v);
    }
  }
}

// 64 weights [64 j, 64 j + 64) of one super-block -> row `row` of the shared tile.
template <int QT>
__device__ __forceinline__ void kq_decode_quarter(const uint8_t* blk, int j, uint8_t* tile, int row);

template <>
__device__ __forceinline__ void kq_decode_quarter<NFN_QTYPE_Q4_K>(const uint8_t* blk, int j, uint8_t* tile, int row) {
  const float d = kq_half(blk), dmin = kq_half(blk + 2);
  float s1, m1, s2, m2;
  kq_scale_min(2 * j, blk + 4, &s1, &m1);
  kq_scale_min(2 * j + 1, blk + 4, &s2, &m2);
  const float a1 = d * s1, b1 = dmin * m1, a2 = d * s2, b2 = dmin * m2;
  const uint4* qs = reinterpret_cast<const uint4*>(blk + 16 + 32 * j);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint4 u = __ldg(qs + h);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int c = 0; c < 2; ++c) {  // 8 bytes -> 8 low-nibble weights and 8 high-nibble weights
      float lo[8], hi[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const uint32_t byte = (w[2 * c + (e >> 2)] >> (8 * (e & 3))) & 0xFF;
        lo[e] = a1 * (float)(byte & 0xF) - b1;
        hi[e] = a2 * (float)(byte >> 4) - b2;
      }
      kq_store8(tile, row, 2 * h + c, lo);      // weights 16 h + 8 c ...
      kq_store8(tile, row, 4 + 2 * h + c, hi);  // weights 32 + 16 h + 8 c ...
    }
  }
}

template <>
__device__ __forceinline__ void kq_decode_quarter<NFN_QTYPE_Q5_K>(const uint8_t* blk, int j, uint8_t* tile, int row) {
  const float d = kq_half(blk), dmin = kq_half(blk + 2);
  float s1, m1, s2, m2;
  kq_scale_min(2 * j, blk + 4, &s1, &m1);
  kq_scale_min(2 * j + 1, blk + 4, &s2, &m2);
  const float a1 = d * s1, b1 = dmin * m1, a2 = d * s2, b2 = dmin * m2;
  const uint4* qh = reinterpret_cast<const uint4*>(blk + 16);
  const uint4* qs = reinterpret_cast<const uint4*>(blk + 48 + 32 * j);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint4 u = __ldg(qs + h), g = __ldg(qh + h);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w}, hb[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      float lo[8], hi[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int wi = 2 * c + (e >> 2), sh = 8 * (e & 3);
        const uint32_t byte = (w[wi] >> sh) & 0xFF, high = (hb[wi] >> sh) & 0xFF;
        lo[e] = a1 * (float)((byte & 0xF) + (((high >> (2 * j)) & 1) << 4)) - b1;
        hi[e] = a2 * (float)((byte >> 4) + (((high >> (2 * j + 1)) & 1) << 4)) - b2;
      }
      kq_store8(tile, row, 2 * h + c, lo);
      kq_store8(tile, row, 4 + 2 * h + c, hi);
    }
  }
}

template <>
__device__ __forceinline__ void kq_decode_quarter<NFN_QTYPE_Q6_K>(const uint8_t* blk, int j, uint8_t* tile, int row) {
  // super-block: ql[128] | qh[64] | scales int8[16] | d f16 ; two halves of 128 weights
  const int n = j >> 1, part = j & 1;
  const unsigned short* ql = reinterpret_cast<const unsigned short*>(blk + 64 * n);
  const unsigned short* qh = reinterpret_cast<const unsigned short*>(blk + 128 + 32 * n);
  const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192 + 8 * n);
  const float d = kq_half(blk + 208);
  const int nib = part ? 4 : 0;            // which nibble of ql
  const int hs_a = part ? 4 : 0, hs_b = part ? 6 : 2;  // which 2 bits of qh
  const int sa = part ? 4 : 0, sb = part ? 6 : 2;      // scale index base
#pragma unroll
  for (int c = 0; c < 4; ++c) {  // 8 weights of the first run (l = 8 c ...) and of the second run
    float va[8], vb[8];
    const float da = d * (float)sc[sa + (c >> 1)], db = d * (float)sc[sb + (c >> 1)];
#pragma unroll
    for (int e2 = 0; e2 < 4; ++e2) {
      const unsigned short la = __ldg(ql + 4 * c + e2), lb = __ldg(ql + 16 + 4 * c + e2), h = __ldg(qh + 4 * c + e2);
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        const int qa = ((la >> (8 * b + nib)) & 0xF) | (((h >> (8 * b + hs_a)) & 3) << 4);
        const int qb = ((lb >> (8 * b + nib)) & 0xF) | (((h >> (8 * b + hs_b)) & 3) << 4);
        va[2 * e2 + b] = da * (float)(qa - 32);
        vb[2 * e2 + b] = db * (float)(qb - 32);
      }
    }
    kq_store8(tile, row, c, va);
    kq_store8(tile, row, 4 + c, vb);
  }
}

// Pulls the bytes a later k-block will decode into L1 so that the decode itself does not sit out a
// full L2 / HBM round trip per stage (a decoder thread handles its stages one after another).
__device__ __forceinline__ void kq_prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }

template <int QT>
__device__ __forceinline__ void kq_prefetch(const uint8_t* rowp, int kb, int main_kb) {
  if (kb >= main_kb) return;
  if constexpr (QT == NFN_QTYPE_NF4_) {
    kq_prefetch_l1(rowp + (size_t)kb * 32);
  } else {
    constexpr int BB = QT == NFN_QTYPE_Q4_K ? 144 : (QT == NFN_QTYPE_Q5_K ? 176 : 210);
    const uint8_t* blk = rowp + (size_t)(kb >> 2) * BB;
    const int j = kb & 3;
    if constexpr (QT == NFN_QTYPE_Q4_K) {
      kq_prefetch_l1(blk);
      kq_prefetch_l1(blk + 16 + 32 * j);
    } else if constexpr (QT == NFN_QTYPE_Q5_K) {
      kq_prefetch_l1(blk);
      kq_prefetch_l1(blk + 48 + 32 * j);
    } else {
      kq_prefetch_l1(blk + 64 * (j >> 1));
      kq_prefetch_l1(blk + 128 + 32 * (j >> 1));
      kq_prefetch_l1(blk + 192);
    }
  }
}

template <int QT>
__global__ void __launch_bounds__(KQ_THREADS, 1)
gemm_kquant_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_c,
                   const __grid_constant__ CUtensorMap tma_aux, const __grid_constant__ CUtensorMap tma_lt,
                   const __grid_constant__ CUtensorMap tma_lb, const uint8_t* __restrict__ wq, const float* __restrict__ absmax,
                   const int lora, const GemmParams p) {
  constexpr int BN = KQ_BN, STAGES = KQ_STAGES;
  constexpr bool NF4 = QT == NFN_QTYPE_NF4_;
  constexpr int BLOCK_BYTES = QT == NFN_QTYPE_Q4_K ? 144 : (QT == NFN_QTYPE_Q5_K ? 176 : 210);
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
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
  if (threadIdx.x == 0) {
    *cta_abort = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 5);  // TMA thread + one lane of each decoder warp
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&tfull_bar[b]), 1);
      mbar_init(smem_u32(&tempty_bar[b]), 8);
    }
    mbar_init(smem_u32(epi_bar), 8);
    fence_mbar_init();
    tma_prefetch_desc(&tma_a);
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
  const int num_tiles = tiles_mn;
  const int main_kb = p.k / BK;
  const int total_kb = main_kb + (lora ? 1 : 0);  // the adapter rides along as one more k-block
  const int blocks_per_row = p.k / 256;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_mn(p, tile, tm, tn);
        for (int kb = 0; kb < total_kb; ++kb) {
          if (!mbar_wait_bounded(smem_u32(&empty_bar[stage]), phase ^ 1, cta_abort, p.status, NFN_ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t fb = smem_u32(&full_bar[stage]);
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          if (kb < main_kb) {
            mbar_expect_tx(fb, A_BYTES);
            tma_load_2d(sa, &tma_a, fb, kb * BK, tm * BM);
          } else {
            mbar_expect_tx(fb, A_BYTES + B_BYTES);
            tma_load_2d(sa, &tma_lt, fb, 0, tm * BM);
            tma_load_2d(sa + A_BYTES, &tma_lb, fb, 0, tn * BN);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, 0, 0);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
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
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t adv = (uint64_t)((UMMA_K * 2) >> 4) * kk;
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
  } else if (warp >= KQ_DEC_WARP0) {
    // -------------------------------------------------------- weight decoders --
    const int r = threadIdx.x - KQ_DEC_WARP0 * 32;  // row of the tile
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      tile_mn(p, tile, tm, tn);
      const int n = tn * BN + r;
      const int nc = min(n, p.n - 1);
      const uint8_t* rowp = NF4 ? wq + (size_t)nc * (p.k / 2) : wq + (size_t)nc * blocks_per_row * BLOCK_BYTES;
      const float* absrow = NF4 ? absmax + (size_t)nc * main_kb : nullptr;
      kq_prefetch<QT>(rowp, 0, main_kb);
      kq_prefetch<QT>(rowp, 1, main_kb);
      for (int kb = 0; kb < total_kb; ++kb) {
        kq_prefetch<QT>(rowp, kb + 2, main_kb);
        ok = mbar_wait_bounded(smem_u32(&empty_bar[stage]), phase ^ 1, cta_abort, p.status, NFN_ERR_WAIT_EMPTY);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        uint8_t* tile_b = smem + stage * STAGE_BYTES + A_BYTES;
        if (kb >= main_kb) {
          // adapter block: both tiles come by TMA; only the arrival is owed
        } else if (n < p.n) {
          if constexpr (NF4) kq_decode_nf4(rowp + (size_t)kb * 32, __ldg(absrow + kb), tile_b, r);
          else kq_decode_quarter<(NF4 ? NFN_QTYPE_Q4_K : QT)>(rowp + (size_t)(kb >> 2) * BLOCK_BYTES, kb & 3, tile_b, r);
        } else {
          const float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
          for (int c = 0; c < 8; ++c) kq_store8(tile_b, r, c, z);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&full_bar[stage]));
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
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

  tc_fence_before();
  __syncthreads();
  if (*cta_abort) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int QT>
static int launch_gemm_kquant(const nfn_gemm_args& a, const float* absmax, const void* lora_t, int ld_t, const void* lora_b, int ld_b,
                              cudaStream_t stream) {
  constexpr size_t SMEM = 1024 + (size_t)KQ_STAGES * (BM * BK * 2 + KQ_BN * BK * 2) + 2 * EPI_TILE_BYTES + 256;
  auto kern = gemm_kquant_kernel<QT>;
  static bool attr[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess) return launch_check("gemm_kquant attr", 0);
    attr[dev & 63] = true;
  }
  CUtensorMap ta, tc, tx;
  if (!make_tmap_2d(&ta, a.a, 2, (uint64_t)a.k, (uint64_t)a.m, (uint64_t)a.lda, BK, BM, 128)) return -3;
  if (!make_tmap_2d(&tc, a.c, 2, (uint64_t)a.n, (uint64_t)a.m, (uint64_t)a.ldc, EPI_CHUNK, BM, 128)) return -3;
  tx = tc;
  if ((a.flags & NFN_EPI_SAVE_PRE) && !make_tmap_2d(&tx, a.aux_out, 2, (uint64_t)a.n, (uint64_t)a.m, (uint64_t)a.ld_aux_out, EPI_CHUNK, BM, 128)) return -3;
  CUtensorMap tlt = ta, tlb = ta;
  const int lora = lora_t != nullptr;
  if (lora) {
    if (!make_tmap_2d(&tlt, lora_t, 2, 64, (uint64_t)a.m, (uint64_t)ld_t, BK, BM, 128)) return -3;
    if (!make_tmap_2d(&tlb, lora_b, 2, 64, (uint64_t)a.n, (uint64_t)ld_b, BK, KQ_BN, 128)) return -3;
  }
  GemmParams p;
  p.c = a.c;
  p.bias = static_cast<const __nv_bfloat16*>(a.bias);
  p.aux_in = static_cast<const __nv_bfloat16*>(a.aux_in);
  p.aux_out = static_cast<__nv_bfloat16*>(a.aux_out);
  p.m = a.m; p.n = a.n; p.k = a.k;
  p.ldc = a.ldc; p.ld_aux_in = a.ld_aux_in; p.ld_aux_out = a.ld_aux_out;
  p.flags = a.flags; p.alpha = a.alpha; p.act_param = a.act_param;
  p.tiles_m = ceil_div(a.m, BM);
  p.tiles_n = ceil_div(a.n, KQ_BN);
  p.split_k = 1;
  p.kb_per_split = a.k / BK;
  p.split_stride = 0;
  p.status = status_ptr();
  // consecutive CTAs take consecutive m-tiles of one weight tile: the decoded tile is rebuilt per CTA,
  // the packed bytes behind it stay in L2
  p.raster_gw = 1;
  const int tiles = p.tiles_m * p.tiles_n;
  kern<<<std::min(tiles, sm_count()), KQ_THREADS, SMEM, stream>>>(ta, tc, tx, tlt, tlb, static_cast<const uint8_t*>(a.b), absmax, lora, p);
  return launch_check("gemm_kquant");
}

}  // namespace nfn

using namespace nfn;

extern "C" int nfn_gemm_quant_lora(int qtype, const nfn_gemm_args* args, const float* absmax, const void* lora_t, int ld_t,
                                   const void* lora_b, int ld_b, nfn_stream_t stream_) {
  if (!args) return fail(-1, "gemm_kquant: null args");
  const nfn_gemm_args& a = *args;
  if (a.m <= 0 || a.n <= 0 || a.k <= 0) return fail(-1, "gemm_kquant: empty problem");
  const bool nf4 = qtype == NFN_QTYPE_NF4;
  if (nf4 ? (a.k % 64 != 0 || !absmax) : (a.k % 256 != 0))
    return fail(-1, "gemm_kquant: K must be a multiple of the quantisation group (256; 64 with absmax for NF4)");
  if ((lora_t == nullptr) != (lora_b == nullptr)) return fail(-1, "gemm_kquant: give both adapter operands or none");
  if (lora_t && ((ld_t & 7) || (ld_b & 7) || ld_t < 64 || ld_b < 64 || ((reinterpret_cast<uintptr_t>(lora_t) | reinterpret_cast<uintptr_t>(lora_b)) & 15)))
    return fail(-1, "gemm_kquant: adapter operands are bf16 [M, 64] and [N, 64], 16-byte aligned");
  if ((a.n & 7) || (a.ldc & 7) || (a.lda & 7)) return fail(-1, "gemm_kquant: N, lda and ldc must be multiples of 8");
  if (a.a_mn || a.b_mn || a.split_k > 1 || (a.flags & (NFN_EPI_OUT_F32 | NFN_EPI_ACCUM))) return fail(-1, "gemm_kquant: K-major operands, bf16 output, no split-K");
  if ((reinterpret_cast<uintptr_t>(a.a) | reinterpret_cast<uintptr_t>(a.c)) & 15) return fail(-1, "gemm_kquant: operands must be 16-byte aligned");
  if (reinterpret_cast<uintptr_t>(a.b) & (qtype == NFN_QTYPE_Q6_K ? 1 : 15)) return fail(-1, "gemm_kquant: weight blocks are misaligned");
  if (nf4 && (a.k / 2) % 16) return fail(-1, "gemm_kquant: NF4 rows must be 16-byte multiples (K % 32 == 0)");
  if ((a.flags & NFN_EPI_BIAS) && !a.bias) return fail(-1, "gemm_kquant: bias flag without bias");
  if ((a.flags & (NFN_EPI_RESID | NFN_EPI_DACT)) && (!a.aux_in || (a.ld_aux_in & 7))) return fail(-1, "gemm_kquant: aux_in missing or misaligned");
  if ((a.flags & NFN_EPI_SAVE_PRE) && (!a.aux_out || (a.ld_aux_out & 7))) return fail(-1, "gemm_kquant: aux_out missing or misaligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  switch (qtype) {
    case NFN_QTYPE_Q4_K: return launch_gemm_kquant<NFN_QTYPE_Q4_K>(a, absmax, lora_t, ld_t, lora_b, ld_b, st);
    case NFN_QTYPE_Q5_K: return launch_gemm_kquant<NFN_QTYPE_Q5_K>(a, absmax, lora_t, ld_t, lora_b, ld_b, st);
    case NFN_QTYPE_Q6_K: return launch_gemm_kquant<NFN_QTYPE_Q6_K>(a, absmax, lora_t, ld_t, lora_b, ld_b, st);
    case NFN_QTYPE_NF4: return launch_gemm_kquant<NFN_QTYPE_NF4>(a, absmax, lora_t, ld_t, lora_b, ld_b, st);
  }
  return fail(-1, "gemm_kquant: qtype must be Q4_K, Q5_K, Q6_K or NF4");
}

extern "C" int nfn_gemm_kquant(int qtype, const nfn_gemm_args* args, nfn_stream_t stream) {
  return nfn_gemm_quant_lora(qtype, args, nullptr, nullptr, 0, nullptr, 0, stream);
}
