// Products with one to four rows (single-stream decode: the "matrix" A is a handful of token
// vectors): C[M, N] = A[M, K] . B[N, K]^T with the GEMM family's epilogue. Such a product only
// streams the weight matrix once, so it is a pure HBM-bandwidth problem and a tensor-core tile
// (64 or 128 rows at least) has nothing to contribute: every warp takes one weight row at a
// time, its 32 lanes read the row as 16-byte chunks (four in flight per lane) with streaming
// loads, multiply with the matching chunks of the token vectors (which stay in L1), and reduce
// with shuffles. Epilogue order as in the tcgen05 kernels: alpha, bias, activation, residual,
// accumulate.
//
// Counterpart in the reference: the decode-time `linear_*` kernels of kernels.cu:16746-16840
// (one thread-tile per output element).
#include "common.h"
#include "nfn_kernels.h"
#include "sm100_ptx.cuh"

namespace nfn {

struct GemvParams {
  const __nv_bfloat16* a;
  const __nv_bfloat16* b;
  __nv_bfloat16* c;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* resid;
  int n, k, lda, ldb, ldc, ld_resid;
  int act, accum;
  float alpha, act_param;
};

__device__ __forceinline__ uint4 gemv_ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ float gemv_act(float v, int act, float prm) {
  switch (act) {
    case NFN_ACT_GELU_TANH: return gelu_tanh_f(v);
    case NFN_ACT_GELU_ERF: return gelu_erf_f(v);
    case NFN_ACT_SILU: return silu_f(v);
    case NFN_ACT_RELU2: { const float r = fmaxf(v, 0.f); return r * r; }
    case NFN_ACT_TANH_CAP: return prm * fast_tanh(v / prm);
    default: return v;
  }
}

constexpr int GEMV_THREADS = 256, GEMV_UNROLL = 4;

template <int M>
__global__ void __launch_bounds__(GEMV_THREADS, 4)
gemv_bf16_kernel(const GemvParams p) {
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * (GEMV_THREADS / 32) + (threadIdx.x >> 5), nwarps = gridDim.x * (GEMV_THREADS / 32);
  for (int n = warp; n < p.n; n += nwarps) {
    const __nv_bfloat16* w = p.b + (size_t)n * p.ldb;
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    for (int k0 = lane * 8; k0 < p.k; k0 += 256 * GEMV_UNROLL) {
      uint4 wv[GEMV_UNROLL];
#pragma unroll
      for (int u = 0; u < GEMV_UNROLL; ++u) {
        const int k = k0 + u * 256;
        wv[u] = k < p.k ? gemv_ld_stream(w + k) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < GEMV_UNROLL; ++u) {
        const int k = k0 + u * 256;
        if (k >= p.k) break;
        const float2 w0 = unpack_bf16x2(wv[u].x), w1 = unpack_bf16x2(wv[u].y), w2 = unpack_bf16x2(wv[u].z), w3 = unpack_bf16x2(wv[u].w);
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const uint4 xv = __ldg(reinterpret_cast<const uint4*>(p.a + (size_t)m * p.lda + k));
          const float2 x0 = unpack_bf16x2(xv.x), x1 = unpack_bf16x2(xv.y), x2 = unpack_bf16x2(xv.z), x3 = unpack_bf16x2(xv.w);
          acc[m] += w0.x * x0.x + w0.y * x0.y + w1.x * x1.x + w1.y * x1.y + w2.x * x2.x + w2.y * x2.y + w3.x * x3.x + w3.y * x3.y;
        }
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], s);
    }
    if (lane < M) {
      float v = acc[0];
#pragma unroll
      for (int m = 1; m < M; ++m)
        if (lane == m) v = acc[m];
      v *= p.alpha;
      if (p.bias) v += __bfloat162float(p.bias[n]);
      v = gemv_act(v, p.act, p.act_param);
      if (p.resid) v += __bfloat162float(p.resid[(size_t)lane * p.ld_resid + n]);
      __nv_bfloat16* cp = p.c + (size_t)lane * p.ldc + n;
      if (p.accum) v += __bfloat162float(*cp);
      *cp = __float2bfloat16(v);
    }
  }
}

// Returns 1 when it launched, 0 when the product is not a GEMV case (the caller continues with the
// tensor-core path), negative on a launch error.
int try_launch_gemv(const nfn_gemm_args& a, cudaStream_t stream) {
  const int unsupported = NFN_EPI_SAVE_PRE | NFN_EPI_DACT | NFN_EPI_OUT_F32;
  if (a.m > 4 || a.a_mn || a.b_mn || (a.flags & unsupported) || (a.k & 7) || a.k < 256) return 0;
  GemvParams p;
  p.a = static_cast<const __nv_bfloat16*>(a.a);
  p.b = static_cast<const __nv_bfloat16*>(a.b);
  p.c = static_cast<__nv_bfloat16*>(a.c);
  p.bias = (a.flags & NFN_EPI_BIAS) ? static_cast<const __nv_bfloat16*>(a.bias) : nullptr;
  p.resid = (a.flags & NFN_EPI_RESID) ? static_cast<const __nv_bfloat16*>(a.aux_in) : nullptr;
  p.n = a.n; p.k = a.k; p.lda = a.lda; p.ldb = a.ldb; p.ldc = a.ldc; p.ld_resid = a.ld_aux_in;
  p.act = (a.flags >> NFN_EPI_ACT_SHIFT) & 0xF;
  p.accum = (a.flags & NFN_EPI_ACCUM) ? 1 : 0;
  p.alpha = a.alpha; p.act_param = a.act_param;
  const int warps_per_block = GEMV_THREADS / 32;
  const int grid = std::max(1, std::min(sm_count() * 4, (a.n + warps_per_block - 1) / warps_per_block));
  switch (a.m) {
    case 1: gemv_bf16_kernel<1><<<grid, GEMV_THREADS, 0, stream>>>(p); break;
    case 2: gemv_bf16_kernel<2><<<grid, GEMV_THREADS, 0, stream>>>(p); break;
    case 3: gemv_bf16_kernel<3><<<grid, GEMV_THREADS, 0, stream>>>(p); break;
    default: gemv_bf16_kernel<4><<<grid, GEMV_THREADS, 0, stream>>>(p); break;
  }
  const int rc = launch_check("gemv_bf16", 1);
  return rc == 0 ? 1 : rc;
}

}  // namespace nfn
