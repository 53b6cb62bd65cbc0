// Products with one or two rows (single-stream decode: the "matrix" A is one or two token
// vectors; from three rows on the tensor-core path is faster): C[M, N] = A[M, K] . B[N, K]^T with the GEMM family's epilogue. Such a product only
// streams the weight matrix once, so it is a pure HBM-bandwidth problem and a tensor-core tile
// (64 or 128 rows at least) has nothing to contribute: every warp takes one weight row at a
// time, its 32 lanes read the rows as 16-byte chunks (eight in flight per lane) with streaming
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
    case NFN_ACT_RELU: return fmaxf(v, 0.f);
    case NFN_ACT_TANH_CAP: return prm * fast_tanh(v / prm);
    default: return v;
  }
}

constexpr int GEMV_THREADS = 256, GEMV_UNROLL = 4;

__device__ __forceinline__ float gemv_dot8(const uint4& w, const float (&x)[8]) {
  const float2 w0 = unpack_bf16x2(w.x), w1 = unpack_bf16x2(w.y), w2 = unpack_bf16x2(w.z), w3 = unpack_bf16x2(w.w);
  return w0.x * x[0] + w0.y * x[1] + w1.x * x[2] + w1.y * x[3] + w2.x * x[4] + w2.y * x[5] + w3.x * x[6] + w3.y * x[7];
}

// A warp takes PAIRS of weight rows (n, n + 1): eight independent 16-byte streaming loads per lane
// are in flight per iteration and every chunk of the token vectors is unpacked once for both rows.
// The host picks the number of warps so that every warp gets the same number of pairs.
template <int M>
__global__ void __launch_bounds__(GEMV_THREADS, 3)
gemv_bf16_kernel(const GemvParams p) {
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * (GEMV_THREADS / 32) + (threadIdx.x >> 5), nwarps = gridDim.x * (GEMV_THREADS / 32);
  const int pairs = (p.n + 1) >> 1;
  for (int pr = warp; pr < pairs; pr += nwarps) {
    const int n0 = 2 * pr;
    const bool two = n0 + 1 < p.n;
    const __nv_bfloat16* wa = p.b + (size_t)n0 * p.ldb;
    const __nv_bfloat16* wb = two ? wa + p.ldb : wa;  // an odd last row is read twice, its second result dropped
    float acc[2][M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[0][m] = acc[1][m] = 0.f;
    for (int k0 = lane * 8; k0 < p.k; k0 += 256 * GEMV_UNROLL) {
      uint4 va[GEMV_UNROLL], vb[GEMV_UNROLL];
#pragma unroll
      for (int u = 0; u < GEMV_UNROLL; ++u) {
        const int k = k0 + u * 256;
        const bool ok = k < p.k;
        va[u] = ok ? gemv_ld_stream(wa + k) : make_uint4(0, 0, 0, 0);
        vb[u] = ok ? gemv_ld_stream(wb + k) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < GEMV_UNROLL; ++u) {
        const int k = k0 + u * 256;
        if (k >= p.k) break;
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const uint4 xv = __ldg(reinterpret_cast<const uint4*>(p.a + (size_t)m * p.lda + k));
          const float2 x0 = unpack_bf16x2(xv.x), x1 = unpack_bf16x2(xv.y), x2 = unpack_bf16x2(xv.z), x3 = unpack_bf16x2(xv.w);
          const float x[8] = {x0.x, x0.y, x1.x, x1.y, x2.x, x2.y, x3.x, x3.y};
          acc[0][m] += gemv_dot8(va[u], x);
          acc[1][m] += gemv_dot8(vb[u], x);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m)
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) acc[r][m] += __shfl_xor_sync(0xffffffffu, acc[r][m], s);
    // lane (r * M + m) finishes output (row m, column n0 + r)
    if (lane < 2 * M) {
      const int r = lane / M, m = lane % M, n = n0 + r;
      float v = 0.f;
#pragma unroll
      for (int rr = 0; rr < 2; ++rr)
#pragma unroll
        for (int mm = 0; mm < M; ++mm)
          if (rr == r && mm == m) v = acc[rr][mm];
      if (r == 0 || two) {
        v *= p.alpha;
        if (p.bias) v += __bfloat162float(p.bias[n]);
        v = gemv_act(v, p.act, p.act_param);
        if (p.resid) v += __bfloat162float(p.resid[(size_t)m * p.ld_resid + n]);
        __nv_bfloat16* cp = p.c + (size_t)m * p.ldc + n;
        if (p.accum) v += __bfloat162float(*cp);
        *cp = __float2bfloat16(v);
      }
    }
  }
}

// Returns 1 when it launched, 0 when the product is not a GEMV case (the caller continues with the
// tensor-core path), negative on a launch error.
int try_launch_gemv(const nfn_gemm_args& a, cudaStream_t stream) {
  const int unsupported = NFN_EPI_SAVE_PRE | NFN_EPI_DACT | NFN_EPI_OUT_F32;
  if (a.m > 2 || a.a_mn || a.b_mn || (a.flags & unsupported) || (a.k & 7) || a.k < 256) return 0;
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
  // as many warps as three resident CTAs per SM can hold, trimmed so that every warp takes the same number of row pairs
  const int warps_per_block = GEMV_THREADS / 32;
  const int pairs = (a.n + 1) / 2, max_warps = sm_count() * 3 * warps_per_block;
  const int rounds = (pairs + max_warps - 1) / max_warps;
  const int warps = (pairs + rounds - 1) / rounds;
  const int grid = std::max(1, (warps + warps_per_block - 1) / warps_per_block);
  if (a.m == 1) gemv_bf16_kernel<1><<<grid, GEMV_THREADS, 0, stream>>>(p);
  else gemv_bf16_kernel<2><<<grid, GEMV_THREADS, 0, stream>>>(p);
  const int rc = launch_check("gemv_bf16", 1);
  return rc == 0 ? 1 : rc;
}

}  // namespace nfn
