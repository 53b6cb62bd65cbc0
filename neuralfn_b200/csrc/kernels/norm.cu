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

// Column sum of a bf16 matrix [rows, C] -> bf16 [C] (bias gradients). Two stages: block (cx, ry)
// sums its share of the rows for 128 columns with 16-byte loads (16 row lanes x 16 column vectors,
// four rows in flight per thread), then a small kernel folds the RY partial rows.
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const __nv_bfloat16* __restrict__ dy, int ld, float* __restrict__ partial,
                      int rows, int C) {
  const int cv = threadIdx.x & 15, rlane = threadIdx.x >> 4;
  const int col = (blockIdx.x * 16 + cv) * 8;
  const int RY = gridDim.y;
  float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const bool vec_ok = col + 8 <= C && (ld & 7) == 0 && (reinterpret_cast<uintptr_t>(dy) & 15) == 0;
  if (vec_ok) {
    const int stride = RY * 16;
    int r = blockIdx.y * 16 + rlane;
    for (; r + 3 * stride < rows; r += 4 * stride) {
      float f0[8], f1[8], f2[8], f3[8];
      load8(dy + (size_t)r * ld + col, f0);
      load8(dy + (size_t)(r + stride) * ld + col, f1);
      load8(dy + (size_t)(r + 2 * stride) * ld + col, f2);
      load8(dy + (size_t)(r + 3 * stride) * ld + col, f3);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += (f0[j] + f1[j]) + (f2[j] + f3[j]);
    }
    for (; r < rows; r += stride) {
      float f0[8];
      load8(dy + (size_t)r * ld + col, f0);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += f0[j];
    }
  } else if (col < C) {  // ragged edge or unaligned view: element loads
    for (int r = blockIdx.y * 16 + rlane; r < rows; r += RY * 16)
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (col + j < C) a[j] += __bfloat162float(dy[(size_t)r * ld + col + j]);
  }
  __shared__ float sa[16][129];
#pragma unroll
  for (int j = 0; j < 8; ++j) sa[rlane][cv * 8 + j] = a[j];
  __syncthreads();
  if (threadIdx.x < 128) {
    const int c = blockIdx.x * 128 + threadIdx.x;
    if (c < C) {
      float t = 0.f;
#pragma unroll
      for (int r = 0; r < 16; ++r) t += sa[r][threadIdx.x];
      partial[(size_t)blockIdx.y * C + c] = t;
    }
  }
}
// 32 columns per block, 8 row groups: coalesced reads of the partial rows, short dependent chains
__global__ void __launch_bounds__(256)
colsum_final_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, int RY, int C, int accumulate) {
  __shared__ float s[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + cx;
  float a = 0.f;
  if (col < C)
    for (int r = ry; r < RY; r += 8) a += partial[(size_t)r * C + col];
  s[ry][cx] = a;
  __syncthreads();
  if (ry == 0 && col < C) {
    float t = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) t += s[r][cx];
    out[col] = __float2bfloat16(t + (accumulate ? __bfloat162float(out[col]) : 0.f));
  }
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

// ---- one-pass backward, many threads per row -------------------------------------------------
// dx, dweight, dbias and (optionally) the column sum of dx itself in ONE pass over dy and x.
// A row is spread over C / 8 threads (one 16-byte vector each), so a thread carries only
// 3 x 8 column accumulators and the kernel runs at high occupancy; a block handles a few rows at
// a time and strides over the matrix. The row reductions cross warps through a double-buffered
// shared-memory slot (one block barrier per row step). Each block folds its column accumulators
// through shared memory and writes one partial row [3][C]; norm_bwd2_final_kernel sums them.
// The column sum of dx is the bias gradient of the linear layer that produced the residual
// stream this norm reads (dx is d(residual stream)), so that layer needs no separate pass.
constexpr int NB2_MAX_THREADS = 1024;

template <bool LAYER, int MAXT>
__global__ void __launch_bounds__(MAXT)
norm_bwd2_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                 const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean_in,
                 const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dresid,
                 __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int rows, int C, int tpr, int rpb,
                 int centered) {
  extern __shared__ float nb2_smem[];       // [rpb][tpr * 8] column fold buffer, then [2][rpb][wpr][2] row sums
  const int wpr = tpr >> 5;
  float* s_fold = nb2_smem;
  float* s_red = nb2_smem + (size_t)rpb * tpr * 8;
  const int tir = threadIdx.x % tpr, rslot = threadIdx.x / tpr;
  const int lane = threadIdx.x & 31, wir = tir >> 5;
  const int c = tir * 8;
  const bool col_ok = c < C;
  float wv[8], aw[8], ab[8], ac[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { wv[j] = 1.f; aw[j] = 0.f; ab[j] = 0.f; ac[j] = 0.f; }
  if (w && col_ok) {
    load8(w + c, wv);
    if (centered) {
#pragma unroll
      for (int j = 0; j < 8; ++j) wv[j] += 1.f;
    }
  }
  const float inv_c = 1.f / (float)C;
  int it = 0;
  for (int base = blockIdx.x * rpb; base < rows; base += gridDim.x * rpb, ++it) {
    const int row = base + rslot;
    const bool live = row < rows && col_ok;
    const size_t off = (size_t)row * C + c;
    float g[8], n[8], r[8];
    float mean = 0.f, rstd = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { g[j] = 0.f; n[j] = 0.f; r[j] = 0.f; }
    if (live) {
      float xv[8];
      load8(dy + off, g);
      load8(x + off, xv);
      if (dresid) load8(dresid + off, r);
      mean = LAYER ? mean_in[row] : 0.f;
      rstd = rstd_in[row];
#pragma unroll
      for (int j = 0; j < 8; ++j) n[j] = (xv[j] - mean) * rstd;
    }
    float sg = 0.f, sgn = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      aw[j] += g[j] * n[j];
      ab[j] += g[j];
      g[j] *= wv[j];
      sg += g[j];
      sgn += g[j] * n[j];
    }
    sg = warp_sum(sg);
    sgn = warp_sum(sgn);
    if (wpr > 1) {
      float* slot = s_red + ((size_t)((it & 1) * rpb + rslot) * wpr) * 2;
      if (lane == 0) { slot[wir * 2] = sg; slot[wir * 2 + 1] = sgn; }
      // only the threads of this row meet (named barrier 1 + slot; at most 12 rows per block),
      // so the rows of a block do not run in lock step
      asm volatile("bar.sync %0, %1;" ::"r"(1 + rslot), "r"(tpr) : "memory");
      sg = 0.f; sgn = 0.f;
      for (int k2 = 0; k2 < wpr; ++k2) { sg += slot[k2 * 2]; sgn += slot[k2 * 2 + 1]; }
    }
    sg = LAYER ? sg * inv_c : 0.f;
    sgn *= inv_c;
    if (live) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rstd * (g[j] - sg - n[j] * sgn) + r[j];
      uint4 u;
      u.x = pack_bf16x2(o[0], o[1]); u.y = pack_bf16x2(o[2], o[3]);
      u.z = pack_bf16x2(o[4], o[5]); u.w = pack_bf16x2(o[6], o[7]);
      *reinterpret_cast<uint4*>(dx + off) = u;
      // sum what was stored (bf16-rounded), so the result equals a column sum of dx itself
      const float2 q0 = unpack_bf16x2(u.x), q1 = unpack_bf16x2(u.y), q2 = unpack_bf16x2(u.z), q3 = unpack_bf16x2(u.w);
      ac[0] += q0.x; ac[1] += q0.y; ac[2] += q1.x; ac[3] += q1.y;
      ac[4] += q2.x; ac[5] += q2.y; ac[6] += q3.x; ac[7] += q3.y;
    }
  }
  // fold the row slots of this block, one accumulator kind at a time
#pragma unroll
  for (int kind = 0; kind < 3; ++kind) {
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 8; ++j) s_fold[(size_t)rslot * tpr * 8 + c + j] = kind == 0 ? aw[j] : (kind == 1 ? ab[j] : ac[j]);
    __syncthreads();
    for (int cc = threadIdx.x; cc < C; cc += blockDim.x) {
      float t = 0.f;
      for (int r2 = 0; r2 < rpb; ++r2) t += s_fold[(size_t)r2 * tpr * 8 + cc];
      partial[((size_t)blockIdx.x * 3 + kind) * C + cc] = t;
    }
  }
}

// Sums the partial rows [nblk][3][C]: 32 columns per block, 32 row groups per block (the loads
// of one thread are independent, so with few hundred partial rows the chain per thread is short).
__global__ void __launch_bounds__(1024)
norm_bwd2_final_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ dw, __nv_bfloat16* __restrict__ db,
                       __nv_bfloat16* __restrict__ dcol, int nblk, int C, int accumulate) {
  __shared__ float s[3][32][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + cx;
  float a[3] = {0.f, 0.f, 0.f};
  if (col < C) {
#pragma unroll 4
    for (int r = ry; r < nblk; r += 32) {
#pragma unroll
      for (int k = 0; k < 3; ++k) a[k] += partial[((size_t)r * 3 + k) * C + col];
    }
  }
#pragma unroll
  for (int k = 0; k < 3; ++k) s[k][ry][cx] = a[k];
  __syncthreads();
  if (ry < 3 && col < C) {
    float t = 0.f;
#pragma unroll
    for (int r = 0; r < 32; ++r) t += s[ry][r][cx];
    __nv_bfloat16* out = ry == 0 ? dw : (ry == 1 ? db : dcol);
    if (out) out[col] = __float2bfloat16(t + (accumulate ? __bfloat162float(out[col]) : 0.f));
  }
}

// Partial rows the one-pass backward may write: scratch must hold nfn_norm_fused_rows() * 3 * C floats.
extern "C" int nfn_norm_fused_rows(void) { return 640; }

// dx_colsum (optional, bf16 [C]) receives sum over rows of dx.
extern "C" int nfn_norm_backward_ex(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                                    const void* dresid, void* dx, void* dw, void* db, void* dx_colsum, float* scratch,
                                    int rows, int C, int mode, int centered, int accumulate, nfn_stream_t stream) {
  if (rows <= 0) return 0;
  if (C % 8) return fail(-1, "norm_backward: C must be a multiple of 8");
  if (C > 8 * NB2_MAX_THREADS) return fail(-1, "norm_backward: rows wider than 8192 are not supported");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int tpr = ((C / 8) + 31) / 32 * 32;               // threads per row, whole warps
  const int rpb = std::min(12, std::max(1, 384 / tpr));    // rows a block works on at a time (one named barrier each)
  const int threads = tpr * rpb;
  const int per_sm = std::max(1, 1536 / threads);
  const int grid = std::min(ceil_div(rows, rpb), std::min(per_sm * sm_count(), nfn_norm_fused_rows()));
  const size_t smem = ((size_t)rpb * tpr * 8 + (size_t)2 * rpb * (tpr / 32) * 2) * sizeof(float);
#define NFN_NB2(L, M)                                                                                                       \
  norm_bwd2_kernel<L, M><<<grid, threads, smem, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, mean, \
                                                      rstd, (const __nv_bfloat16*)dresid, (__nv_bfloat16*)dx, scratch, rows, C, tpr, rpb, centered)
  if (threads <= 512) {
    if (mode == 0) NFN_NB2(true, 512); else NFN_NB2(false, 512);
  } else {
    if (mode == 0) NFN_NB2(true, 1024); else NFN_NB2(false, 1024);
  }
#undef NFN_NB2
  norm_bwd2_final_kernel<<<ceil_div(C, 32), 1024, 0, st>>>(scratch, (__nv_bfloat16*)dw, (__nv_bfloat16*)db, (__nv_bfloat16*)dx_colsum, grid, C,
                                                          accumulate);
  return launch_check("norm_backward", 2);
}

extern "C" int nfn_norm_backward(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, const void* dresid,
                                 void* dx, void* dw, void* db, float* scratch, int rows, int C, int mode, int centered, int accumulate,
                                 nfn_stream_t stream) {
  return nfn_norm_backward_ex(dy, x, w, mean, rstd, dresid, dx, dw, db, nullptr, scratch, rows, C, mode, centered, accumulate, stream);
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
  colsum_final_kernel<<<ceil_div(C, 32), 256, 0, st>>>(scratch, (__nv_bfloat16*)out, RY, C, accumulate);
  return launch_check("colsum", 2);
}

