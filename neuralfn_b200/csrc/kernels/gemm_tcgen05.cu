// Persistent, warp-specialised BF16 GEMM for sm_100a.
//
//   warp 0      : TMA producer   (one lane issues cp.async.bulk.tensor tile loads)
//   warp 1      : MMA issuer     (one lane issues tcgen05.mma; owns the TMEM allocation)
//   warps 2..5  : epilogue       (tcgen05.ld accumulator -> fused epilogue -> global)
//
// Tiles are 128 x BN x 64 with a STAGES-deep shared-memory ring (128-byte swizzle,
// filled by TMA, consumed straight by tcgen05.mma through shared-memory matrix
// descriptors). The fp32 accumulator lives in TMEM and is double-buffered so the
// epilogue of tile i overlaps the main loop of tile i+1. Either operand may be
// K-major or MN-major, which gives the forward (X W^T), input-gradient (dY W) and
// weight-gradient (dY^T X) products without any transposes in memory.
//
// Covers the role of the reference's linear kernels and library GEMM call sites
// (neuralfn/csrc/tile_cuda/kernels.cu:16746-17574 and its cuBLASLt wrappers) with
// the bias / GELU / residual / dGELU / accumulate epilogues fused.
#include "common.h"
#include "sm100_ptx.cuh"

namespace nfn {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;

struct GemmParams {
  void* c;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* aux_in;
  __nv_bfloat16* aux_out;
  int m, n, k;
  int ldc, ld_aux_in, ld_aux_out;
  int flags;
  float alpha, act_param;
  int tiles_m, tiles_n;
  int* status;
};

__device__ __forceinline__ float apply_act(float v, int act, float prm) {
  switch (act) {
    case NFN_ACT_GELU_TANH: return gelu_tanh_f(v);
    case NFN_ACT_GELU_ERF: return gelu_erf_f(v);
    case NFN_ACT_SILU: return silu_f(v);
    case NFN_ACT_RELU2: { float r = fmaxf(v, 0.f); return r * r; }
    case NFN_ACT_TANH_CAP: return prm * tanhf(v / prm);
    default: return v;
  }
}
__device__ __forceinline__ float apply_dact(float pre, int act, float prm) {
  switch (act) {
    case NFN_ACT_GELU_TANH: return dgelu_tanh_f(pre);
    case NFN_ACT_GELU_ERF: return dgelu_erf_f(pre);
    case NFN_ACT_SILU: return dsilu_f(pre);
    case NFN_ACT_RELU2: return pre > 0.f ? 2.f * pre : 0.f;
    case NFN_ACT_TANH_CAP: { float t = tanhf(pre / prm); return 1.f - t * t; }
    default: return 1.f;
  }
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a,
                 const __grid_constant__ CUtensorMap tma_b, const GemmParams p) {
  constexpr uint32_t A_BYTES = BM * BK * 2;
  constexpr uint32_t B_BYTES = BN * BK * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulator buffers
  static_assert(TMEM_COLS == 256 || TMEM_COLS == 512, "TMEM columns must be a power of two");

  extern __shared__ uint8_t smem_raw[];
  // 128B swizzle wants 1024-byte aligned tiles.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                  // [STAGES]
  uint64_t* empty_bar = bars + STAGES;        // [STAGES]
  uint64_t* tfull_bar = bars + 2 * STAGES;    // [2]
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
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
      mbar_init(smem_u32(&tempty_bar[b]), 4);
    }
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

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.k + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % p.tiles_m) * BM;
        const int n0 = (tile / p.tiles_m) * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
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
        if (!mbar_wait_bounded(smem_u32(&tempty_bar[acc]), acc_phase ^ 1, cta_abort, p.status,
                               NFN_ERR_WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
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
            umma_bf16_ss(tmem_d, da + a_adv, db + b_adv, idesc, (kb | kk) != 0 ? 1u : 0u);
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
    // ------------------------------------------------------------ epilogue --
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const int act = (p.flags >> NFN_EPI_ACT_SHIFT) & 0xF;
    const bool has_bias = p.flags & NFN_EPI_BIAS;
    const bool save_pre = p.flags & NFN_EPI_SAVE_PRE;
    const bool resid = p.flags & NFN_EPI_RESID;
    const bool dact = p.flags & NFN_EPI_DACT;
    const bool accum = p.flags & NFN_EPI_ACCUM;
    const bool out_f32 = p.flags & NFN_EPI_OUT_F32;
    uint32_t acc = 0, acc_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int m0 = (tile % p.tiles_m) * BM;
      const int n0 = (tile / p.tiles_m) * BN;
      bool ok = mbar_wait_bounded(smem_u32(&tfull_bar[acc]), acc_phase, cta_abort, p.status,
                                  NFN_ERR_WAIT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.m;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int nc = n0 + c * 32;
        if (nc >= p.n) break;  // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int ng = nc + g * 8;
            if (ng < p.n) {
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[g * 8 + j]) * p.alpha;
              if (has_bias) {
                const uint4 bb = __ldg(reinterpret_cast<const uint4*>(p.bias + ng));
                const uint32_t bw[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float2 f = unpack_bf16x2(bw[j]);
                  v[2 * j] += f.x;
                  v[2 * j + 1] += f.y;
                }
              }
              if (save_pre) {
                uint4 o;
                o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
                o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
                *reinterpret_cast<uint4*>(p.aux_out + (size_t)row * p.ld_aux_out + ng) = o;
              }
              if (act != NFN_ACT_NONE && !dact) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = apply_act(v[j], act, p.act_param);
              }
              if (dact || resid) {
                const uint4 xx =
                    *reinterpret_cast<const uint4*>(p.aux_in + (size_t)row * p.ld_aux_in + ng);
                const uint32_t xw[4] = {xx.x, xx.y, xx.z, xx.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float2 f = unpack_bf16x2(xw[j]);
                  if (dact) {
                    v[2 * j] *= apply_dact(f.x, act, p.act_param);
                    v[2 * j + 1] *= apply_dact(f.y, act, p.act_param);
                  } else {
                    v[2 * j] += f.x;
                    v[2 * j + 1] += f.y;
                  }
                }
              }
              if (out_f32) {
                float* cp = reinterpret_cast<float*>(p.c) + (size_t)row * p.ldc + ng;
                if (accum) {
                  const float4 c0 = *reinterpret_cast<const float4*>(cp);
                  const float4 c1 = *reinterpret_cast<const float4*>(cp + 4);
                  v[0] += c0.x; v[1] += c0.y; v[2] += c0.z; v[3] += c0.w;
                  v[4] += c1.x; v[5] += c1.y; v[6] += c1.z; v[7] += c1.w;
                }
                *reinterpret_cast<float4*>(cp) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4*>(cp + 4) = make_float4(v[4], v[5], v[6], v[7]);
              } else {
                __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.c) + (size_t)row * p.ldc + ng;
                if (accum) {
                  const uint4 cc = *reinterpret_cast<const uint4*>(cp);
                  const uint32_t cw[4] = {cc.x, cc.y, cc.z, cc.w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    float2 f = unpack_bf16x2(cw[j]);
                    v[2 * j] += f.x;
                    v[2 * j + 1] += f.y;
                  }
                }
                uint4 o;
                o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
                o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
                *reinterpret_cast<uint4*>(cp) = o;
              }
            }
          }
        }
      }
      // hand the accumulator buffer back to the MMA issuer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
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

template <int BN, int STAGES, bool A_MN, bool B_MN>
static int launch_gemm(const nfn_gemm_args& a, cudaStream_t stream) {
  constexpr size_t SMEM = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 1024 + 256;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN>;
  if (!attr_set[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) !=
        cudaSuccess)
      return launch_check("gemm attr");
    attr_set[dev & 63] = true;
  }
  CUtensorMap ta, tb;
  bool ok;
  if (!A_MN) ok = make_tmap_2d(&ta, a.a, 2, (uint64_t)a.k, (uint64_t)a.m, (uint64_t)a.lda, BK, BM, 128);
  else       ok = make_tmap_2d(&ta, a.a, 2, (uint64_t)a.m, (uint64_t)a.k, (uint64_t)a.lda, 64, BK, 128);
  if (!ok) return -3;
  if (!B_MN) ok = make_tmap_2d(&tb, a.b, 2, (uint64_t)a.k, (uint64_t)a.n, (uint64_t)a.ldb, BK, BN, 128);
  else       ok = make_tmap_2d(&tb, a.b, 2, (uint64_t)a.n, (uint64_t)a.k, (uint64_t)a.ldb, 64, BK, 128);
  if (!ok) return -3;

  GemmParams p;
  p.c = a.c;
  p.bias = static_cast<const __nv_bfloat16*>(a.bias);
  p.aux_in = static_cast<const __nv_bfloat16*>(a.aux_in);
  p.aux_out = static_cast<__nv_bfloat16*>(a.aux_out);
  p.m = a.m; p.n = a.n; p.k = a.k;
  p.ldc = a.ldc; p.ld_aux_in = a.ld_aux_in; p.ld_aux_out = a.ld_aux_out;
  p.flags = a.flags; p.alpha = a.alpha; p.act_param = a.act_param;
  p.tiles_m = ceil_div(a.m, BM);
  p.tiles_n = ceil_div(a.n, BN);
  p.status = status_ptr();
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, GEMM_THREADS, SMEM, stream>>>(ta, tb, p);
  return launch_check("gemm");
}

}  // namespace nfn

extern "C" int nfn_gemm_bf16(const nfn_gemm_args* args, nfn_stream_t stream_) {
  using namespace nfn;
  if (!args) return fail(-1, "null args");
  const nfn_gemm_args& a = *args;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a.m <= 0 || a.n <= 0 || a.k <= 0) return fail(-1, "gemm: empty problem");
  if ((a.n & 7) || (a.ldc & 7)) return fail(-1, "gemm: N and ldc must be multiples of 8");
  if ((a.lda & 7) || (a.ldb & 7)) return fail(-1, "gemm: lda/ldb must be multiples of 8");
  if ((reinterpret_cast<uintptr_t>(a.a) | reinterpret_cast<uintptr_t>(a.b) |
       reinterpret_cast<uintptr_t>(a.c)) & 15)
    return fail(-1, "gemm: operands must be 16-byte aligned");
  if ((a.flags & NFN_EPI_BIAS) && !a.bias) return fail(-1, "gemm: bias flag without bias");
  if ((a.flags & (NFN_EPI_RESID | NFN_EPI_DACT)) && (!a.aux_in || (a.ld_aux_in & 7)))
    return fail(-1, "gemm: aux_in missing or misaligned");
  if ((a.flags & NFN_EPI_RESID) && (a.flags & NFN_EPI_DACT))
    return fail(-1, "gemm: RESID and DACT both read aux_in");
  if ((a.flags & NFN_EPI_SAVE_PRE) && (!a.aux_out || (a.ld_aux_out & 7)))
    return fail(-1, "gemm: aux_out missing or misaligned");

  const int tiles256 = ceil_div(a.m, BM) * ceil_div(a.n, 256);
  const bool wide = tiles256 >= sm_count() && (a.n % 256 == 0 || a.n >= 1024);
#define NFN_DISPATCH(AMN, BMN)                                              \
  return wide ? launch_gemm<256, 4, AMN, BMN>(a, stream)                    \
              : launch_gemm<128, 6, AMN, BMN>(a, stream)
  if (!a.a_mn && !a.b_mn) { NFN_DISPATCH(false, false); }
  if (!a.a_mn && a.b_mn) { NFN_DISPATCH(false, true); }
  if (a.a_mn && !a.b_mn) { NFN_DISPATCH(true, false); }
  NFN_DISPATCH(true, true);
#undef NFN_DISPATCH
}
