// Row normalisation kernels (HBM-bound): LayerNorm and RMSNorm forward/backward
// with fp32 statistics, bf16 activations, optional fused residual-gradient add,
// and the per-head weightless QK RMS norm applied to packed QKV.
//
// One warp per row; each lane keeps its slice of the row in registers so the row
// is read from HBM exactly once in the forward and once per operand in the backward.
// Weight/bias gradients use a deterministic two-stage column reduction.
//
// Reference counterparts: neuralfn/csrc/tile_cuda/kernels.cu:13960-14934 (rms/layer norm
// family) and :19111-19155 (qk_rms_norm_packed_bf16 forward/backward).
#include <algorithm>

#include "common.h"
#include "sm100_ptx.cuh"

namespace nfn {

constexpr int NORM_THREADS = 256;  // 8 rows per block

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum across the TPR threads that share a row (TPR = 32: one warp; TPR = 256: whole block).
template <int TPR>
__device__ __forceinline__ float row_sum(float v, float* red) {
  v = warp_sum(v);
  if (TPR == 32) return v;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < TPR / 32; ++i) t += red[i];
  return t;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// ------------------------------------------------------------- forward ------
// mode: 0 = LayerNorm (weight, bias), 1 = RMSNorm (weight optional; centered => scale 1+w)
// VEC = number of 8-element vectors per lane (C <= VEC*256).
template <int VEC, int TPR>
__global__ void __launch_bounds__(NORM_THREADS)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y,
                float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int C,
                float eps, int mode, int centered) {
  __shared__ float red[8];
  const int lane = threadIdx.x % TPR;
  const int row = blockIdx.x * (NORM_THREADS / TPR) + threadIdx.x / TPR;
  if (TPR == 32 && row >= rows) return;  // TPR == 256: one row per block, grid == rows
  const __nv_bfloat16* xr = x + (size_t)row * C;
  float v[VEC][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = (i * TPR + lane) * 8;
    if (c < C) {
      load8(xr + c, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[i][j];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
    }
  }
  float mean = 0.f;
  if (mode == 0) mean = row_sum<TPR>(s, red) / C;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = (i * TPR + lane) * 8;
    if (c < C) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { float d = v[i][j] - mean; sq += d * d; }
    }
  }
  const float rstd = rsqrtf(row_sum<TPR>(sq, red) / C + eps);
  if (lane == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  __nv_bfloat16* yr = y + (size_t)row * C;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = (i * TPR + lane) * 8;
    if (c < C) {
      float o[8], wv[8], bv[8];
      if (w) load8(w + c, wv);
      if (b) load8(b + c, bv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float n = (v[i][j] - mean) * rstd;
        float g = w ? (centered ? 1.f + wv[j] : wv[j]) : 1.f;
        o[j] = n * g + (b ? bv[j] : 0.f);
      }
      store8(yr + c, o);
    }
  }
}

// ------------------------------------------------------------ backward ------
// dx = rstd * (g - mean(g) - n * mean(g*n))   [LayerNorm]   g = dy * w
// dx = rstd * (g - n * mean(g*n))             [RMSNorm]
// optional: dx += dresid (fused residual-stream gradient)
template <int VEC, int TPR>
__global__ void __launch_bounds__(NORM_THREADS)
norm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean_in,
                   const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dresid,
                   __nv_bfloat16* __restrict__ dx, int rows, int C, int mode, int centered) {
  __shared__ float red[8];
  const int lane = threadIdx.x % TPR;
  const int row = blockIdx.x * (NORM_THREADS / TPR) + threadIdx.x / TPR;
  if (TPR == 32 && row >= rows) return;
  const float mean = (mode == 0) ? mean_in[row] : 0.f;
  const float rstd = rstd_in[row];
  const size_t off = (size_t)row * C;
  float g[VEC][8], n[VEC][8];
  float sg = 0.f, sgn = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = (i * TPR + lane) * 8;
    if (c < C) {
      float xv[8], wv[8];
      load8(dy + off + c, g[i]);
      load8(x + off + c, xv);
      if (w) load8(w + c, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        n[i][j] = (xv[j] - mean) * rstd;
        const float gw = w ? (centered ? 1.f + wv[j] : wv[j]) : 1.f;
        g[i][j] *= gw;
        sg += g[i][j];
        sgn += g[i][j] * n[i][j];
      }
    }
  }
  sg = (mode == 0) ? row_sum<TPR>(sg, red) / C : 0.f;
  sgn = row_sum<TPR>(sgn, red) / C;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = (i * TPR + lane) * 8;
    if (c < C) {
      float o[8], r[8];
      if (dresid) load8(dresid + off + c, r);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = rstd * (g[i][j] - sg - n[i][j] * sgn) + (dresid ? r[j] : 0.f);
      }
      store8(dx + off + c, o);
    }
  }
}

// Stage 1 of dweight/dbias: block (cx, ry) reduces rows ry, ry+RY, ... for 64 columns.
// partial layout: [RY][2][C] fp32 (dweight then dbias).
constexpr int WG_COLS = 64;
__global__ void __launch_bounds__(256)
norm_bwd_wb_partial_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                           const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                           float* __restrict__ partial, int rows, int C, int mode) {
  // 256 threads = 4 row-lanes x 64 columns
  const int col = blockIdx.x * WG_COLS + (threadIdx.x & 63);
  const int rlane = threadIdx.x >> 6;
  const int RY = gridDim.y;
  float dw = 0.f, db = 0.f;
  if (col < C) {
    for (int r = blockIdx.y * 4 + rlane; r < rows; r += RY * 4) {
      const float m = (mode == 0) ? mean_in[r] : 0.f;
      const float rs = rstd_in[r];
      const float g = __bfloat162float(dy[(size_t)r * C + col]);
      const float xv = __bfloat162float(x[(size_t)r * C + col]);
      dw += g * (xv - m) * rs;
      db += g;
    }
  }
  __shared__ float sw[4][WG_COLS], sb[4][WG_COLS];
  sw[rlane][threadIdx.x & 63] = dw;
  sb[rlane][threadIdx.x & 63] = db;
  __syncthreads();
  if (rlane == 0 && col < C) {
    const int t = threadIdx.x;
    dw = sw[0][t] + sw[1][t] + sw[2][t] + sw[3][t];
    db = sb[0][t] + sb[1][t] + sb[2][t] + sb[3][t];
    partial[((size_t)blockIdx.y * 2 + 0) * C + col] = dw;
    partial[((size_t)blockIdx.y * 2 + 1) * C + col] = db;
  }
}
// Stage 2: sum partials over RY, write (or accumulate into) bf16 grads.
__global__ void norm_bwd_wb_final_kernel(const float* __restrict__ partial,
                                         __nv_bfloat16* __restrict__ dw,
                                         __nv_bfloat16* __restrict__ db, int RY, int C, int accumulate) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= C) return;
  float a = 0.f, b = 0.f;
  for (int r = 0; r < RY; ++r) {
    a += partial[((size_t)r * 2 + 0) * C + col];
    b += partial[((size_t)r * 2 + 1) * C + col];
  }
  if (dw) dw[col] = __float2bfloat16(a + (accumulate ? __bfloat162float(dw[col]) : 0.f));
  if (db) db[col] = __float2bfloat16(b + (accumulate ? __bfloat162float(db[col]) : 0.f));
}

// Column sum of a bf16 matrix [rows, C] -> bf16 [C] (bias gradients). Same two stages.
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const __nv_bfloat16* __restrict__ dy, int ld, float* __restrict__ partial,
                      int rows, int C) {
  // each thread owns 2 adjacent columns; 4 row-lanes x 64 column-pairs = 128 columns per block
  const int cp = threadIdx.x & 63, rlane = threadIdx.x >> 6;
  const int col = (blockIdx.x * 64 + cp) * 2;
  const int RY = gridDim.y;
  float a = 0.f, b = 0.f;
  if (col < C) {
    for (int r = blockIdx.y * 4 + rlane; r < rows; r += RY * 4) {
      const float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dy + (size_t)r * ld + col));
      a += f.x; b += f.y;
    }
  }
  __shared__ float sa[4][64], sb[4][64];
  sa[rlane][cp] = a; sb[rlane][cp] = b;
  __syncthreads();
  if (rlane == 0 && col < C) {
    a = sa[0][cp] + sa[1][cp] + sa[2][cp] + sa[3][cp];
    b = sb[0][cp] + sb[1][cp] + sb[2][cp] + sb[3][cp];
    partial[(size_t)blockIdx.y * C + col] = a;
    partial[(size_t)blockIdx.y * C + col + 1] = b;
  }
}
__global__ void colsum_final_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                                    int RY, int C, int accumulate) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= C) return;
  float a = 0.f;
  for (int r = 0; r < RY; ++r) a += partial[(size_t)r * C + col];
  out[col] = __float2bfloat16(a + (accumulate ? __bfloat162float(out[col]) : 0.f));
}

template <typename F>
static int dispatch_vec(int C, F&& f) {
  if (C % 8) return fail(-1, "norm: width must be a multiple of 8");
  using std::integral_constant;
  if (C <= 256) return f(integral_constant<int, 1>{}, integral_constant<int, 32>{});
  if (C <= 512) return f(integral_constant<int, 2>{}, integral_constant<int, 32>{});
  if (C <= 768) return f(integral_constant<int, 3>{}, integral_constant<int, 32>{});
  if (C <= 1024) return f(integral_constant<int, 4>{}, integral_constant<int, 32>{});
  if (C <= 2048) return f(integral_constant<int, 1>{}, integral_constant<int, 256>{});
  if (C <= 4096) return f(integral_constant<int, 2>{}, integral_constant<int, 256>{});
  if (C <= 8192) return f(integral_constant<int, 4>{}, integral_constant<int, 256>{});
  return fail(-1, "norm: width above 8192 is not supported");
}

}  // namespace nfn

using namespace nfn;

extern "C" int nfn_norm_forward(const void* x, const void* w, const void* b, void* y, float* mean,
                                float* rstd, int rows, int C, float eps, int mode, int centered,
                                nfn_stream_t stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dispatch_vec(C, [&](auto vec, auto tpr) {
    constexpr int V = decltype(vec)::value;
    constexpr int T = decltype(tpr)::value;
    const int grid = ceil_div(rows, NORM_THREADS / T);
    norm_fwd_kernel<V, T><<<grid, NORM_THREADS, 0, st>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)b,
        (__nv_bfloat16*)y, mean, rstd, rows, C, eps, mode, centered);
    return launch_check("norm_fwd");
  });
}

extern "C" int nfn_norm_backward_dx(const void* dy, const void* x, const void* w, const float* mean,
                                    const float* rstd, const void* dresid, void* dx, int rows, int C,
                                    int mode, int centered, nfn_stream_t stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dispatch_vec(C, [&](auto vec, auto tpr) {
    constexpr int V = decltype(vec)::value;
    constexpr int T = decltype(tpr)::value;
    const int grid = ceil_div(rows, NORM_THREADS / T);
    norm_bwd_dx_kernel<V, T><<<grid, NORM_THREADS, 0, st>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, mean, rstd,
        (const __nv_bfloat16*)dresid, (__nv_bfloat16*)dx, rows, C, mode, centered);
    return launch_check("norm_bwd_dx");
  });
}

// dx, dweight and dbias in ONE pass over dy and x. Each block strides over the rows (one warp
// per row at a time), keeps its column partials of dweight / dbias in registers, folds its eight
// warps through shared memory at the end and writes one partial row; the small final kernel sums
// the partial rows. Compared with separate dx and dweight/dbias kernels this reads dy and x once
// instead of twice and keeps every load a 16-byte vector.
template <int VEC>
__global__ void __launch_bounds__(NORM_THREADS)
norm_bwd_fused_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                      const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean_in,
                      const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dresid,
                      __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int rows, int C, int mode, int centered) {
  constexpr int RPB = NORM_THREADS / 32;
  __shared__ float sacc[RPB][VEC * 256];
  const int lane = threadIdx.x & 31, wrow = threadIdx.x >> 5;
  float aw[VEC][8], ab[VEC][8], wv[VEC][8];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = (i * 32 + lane) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) { aw[i][j] = 0.f; ab[i][j] = 0.f; wv[i][j] = 1.f; }
    if (w && c < C) {
      load8(w + c, wv[i]);
      if (centered) {
#pragma unroll
        for (int j = 0; j < 8; ++j) wv[i][j] += 1.f;
      }
    }
  }
  for (int row = blockIdx.x * RPB + wrow; row < rows; row += gridDim.x * RPB) {
    const float mean = (mode == 0) ? mean_in[row] : 0.f;
    const float rstd = rstd_in[row];
    const size_t off = (size_t)row * C;
    float g[VEC][8], n[VEC][8];
    float sg = 0.f, sgn = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < C) {
        float xv[8];
        load8(dy + off + c, g[i]);
        load8(x + off + c, xv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          n[i][j] = (xv[j] - mean) * rstd;
          aw[i][j] += g[i][j] * n[i][j];
          ab[i][j] += g[i][j];
          g[i][j] *= wv[i][j];
          sg += g[i][j];
          sgn += g[i][j] * n[i][j];
        }
      }
    }
    sg = (mode == 0) ? warp_sum(sg) / C : 0.f;
    sgn = warp_sum(sgn) / C;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < C) {
        float o[8], r[8];
        if (dresid) load8(dresid + off + c, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - sg - n[i][j] * sgn) + (dresid ? r[j] : 0.f);
        store8(dx + off + c, o);
      }
    }
  }
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < VEC; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) sacc[wrow][(i * 32 + lane) * 8 + j] = pass == 0 ? aw[i][j] : ab[i][j];
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += NORM_THREADS) {
      float t = 0.f;
#pragma unroll
      for (int r = 0; r < RPB; ++r) t += sacc[r][c];
      partial[((size_t)blockIdx.x * 2 + pass) * C + c] = t;
    }
  }
}

// scratch: fp32 [ry * 2 * C]; ry = nfn_norm_wb_rows()
extern "C" int nfn_norm_wb_rows(void) { return 64; }

extern "C" int nfn_norm_backward_wb(const void* dy, const void* x, const float* mean,
                                    const float* rstd, void* dw, void* db, float* scratch, int rows,
                                    int C, int mode, int accumulate, nfn_stream_t stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int RY = 64;
  dim3 grid(ceil_div(C, WG_COLS), RY);
  norm_bwd_wb_partial_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)dy,
                                                   (const __nv_bfloat16*)x, mean, rstd, scratch,
                                                   rows, C, mode);
  norm_bwd_wb_final_kernel<<<ceil_div(C, 256), 256, 0, st>>>(scratch, (__nv_bfloat16*)dw,
                                                             (__nv_bfloat16*)db, RY, C, accumulate);
  return launch_check("norm_bwd_wb", 2);
}

// Partial rows the fused backward may write: scratch must hold nfn_norm_fused_rows() * 2 * C floats.
extern "C" int nfn_norm_fused_rows(void) { return 2 * 160; }

extern "C" int nfn_norm_backward(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, const void* dresid,
                                 void* dx, void* dw, void* db, float* scratch, int rows, int C, int mode, int centered, int accumulate,
                                 nfn_stream_t stream) {
  if (rows <= 0) return 0;
  if (C % 8) return fail(-1, "norm_backward: C must be a multiple of 8");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (C > 1024) {  // wide rows: the two-kernel path
    int rc = nfn_norm_backward_dx(dy, x, w, mean, rstd, dresid, dx, rows, C, mode, centered, stream);
    if (rc) return rc;
    return nfn_norm_backward_wb(dy, x, mean, rstd, dw, db, scratch, rows, C, mode, accumulate, stream);
  }
  const int grid = std::min(ceil_div(rows, NORM_THREADS / 32), std::min(2 * sm_count(), nfn_norm_fused_rows()));
#define NFN_FUSED(V)                                                                                                   \
  norm_bwd_fused_kernel<V><<<grid, NORM_THREADS, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,           \
      (const __nv_bfloat16*)w, mean, rstd, (const __nv_bfloat16*)dresid, (__nv_bfloat16*)dx, scratch, rows, C, mode, centered)
  if (C <= 256) NFN_FUSED(1);
  else if (C <= 512) NFN_FUSED(2);
  else if (C <= 768) NFN_FUSED(3);
  else NFN_FUSED(4);
#undef NFN_FUSED
  norm_bwd_wb_final_kernel<<<ceil_div(C, 256), 256, 0, st>>>(scratch, (__nv_bfloat16*)dw, (__nv_bfloat16*)db, grid, C, accumulate);
  return launch_check("norm_backward", 2);
}

// scratch: fp32 [64 * C]
extern "C" int nfn_colsum(const void* dy, int ld, void* out, float* scratch, int rows, int C,
                          int accumulate, nfn_stream_t stream) {
  if (rows <= 0) return 0;
  if (C % 2 || ld % 2) return fail(-1, "colsum: C and ld must be even");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int RY = 64;
  dim3 grid(ceil_div(C, 128), RY);
  colsum_partial_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)dy, ld, scratch, rows, C);
  colsum_final_kernel<<<ceil_div(C, 256), 256, 0, st>>>(scratch, (__nv_bfloat16*)out, RY, C,
                                                        accumulate);
  return launch_check("colsum", 2);
}

