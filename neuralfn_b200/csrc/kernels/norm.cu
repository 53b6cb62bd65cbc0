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
                   __nv_bfloat16* __restrict__ dx, int rows, int C, int mode, int centered,
                   float* __restrict__ wb_accum = nullptr) {
  // wb_accum (TPR == 32 only): fp32 [2][C], zeroed by the caller; receives sum_rows dy * n and
  // sum_rows dy. The block's eight rows are folded in shared memory first, so global memory sees
  // one reduction per column and block instead of one per row.
  __shared__ float red[8];
  __shared__ float s_wb[TPR == 32 ? 2 * VEC * 256 : 1];
  const int lane = threadIdx.x % TPR;
  const int row = blockIdx.x * (NORM_THREADS / TPR) + threadIdx.x / TPR;
  if (TPR == 32 && wb_accum) {
    for (int c = threadIdx.x; c < 2 * VEC * 256; c += NORM_THREADS) s_wb[c] = 0.f;
    __syncthreads();
  }
  const bool live = !(TPR == 32 && row >= rows);
  if (TPR == 32 && !live && !wb_accum) return;
  if (live) {
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
        if (TPR == 32 && wb_accum) {
          atomicAdd(&s_wb[c + j], g[i][j] * n[i][j]);
          atomicAdd(&s_wb[VEC * 256 + c + j], g[i][j]);
        }
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
  }  // live
  if (TPR == 32 && wb_accum) {
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += NORM_THREADS) {
      atomicAdd(wb_accum + c, s_wb[c]);
      atomicAdd(wb_accum + C + c, s_wb[VEC * 256 + c]);
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

// Column sum of a bf16 matrix [rows, C] -> bf16 [C] (bias gradients), one launch. A block owns 64
// columns (8 threads x 8 columns, 16-byte loads) and every RY-th group of 32 rows; it writes one
// partial row, takes a ticket, and the last block of its column group to finish adds the partial
// rows up and writes the result. The tickets live in a static device array and reset themselves,
// so calls on one device must not overlap (they are issued on one stream).
constexpr int CS_COLS = 64, CS_MAX_GROUPS = 4096;
constexpr int CS_CG = CS_COLS / 8;   // threads across the columns (8 columns each)
constexpr int CS_RL = 256 / CS_CG;   // row lanes per block
__device__ unsigned int g_colsum_tickets[CS_MAX_GROUPS];

__global__ void __launch_bounds__(256)
colsum_kernel(const __nv_bfloat16* __restrict__ dy, int ld, float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
              int rows, int C, int accumulate) {
  __shared__ float sacc[CS_RL][CS_COLS];
  __shared__ int s_last;
  const int cg = threadIdx.x % CS_CG, rlane = threadIdx.x / CS_CG;
  const int col = blockIdx.x * CS_COLS + cg * 8;
  const int RY = gridDim.y;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col < C) {
    const int step = RY * CS_RL;
    int r = blockIdx.y * CS_RL + rlane;
    for (; r + 3 * step < rows; r += 4 * step) {  // four independent loads in flight
      float f0[8], f1[8], f2[8], f3[8];
      load8(dy + (size_t)r * ld + col, f0);
      load8(dy + (size_t)(r + step) * ld + col, f1);
      load8(dy + (size_t)(r + 2 * step) * ld + col, f2);
      load8(dy + (size_t)(r + 3 * step) * ld + col, f3);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += (f0[k] + f1[k]) + (f2[k] + f3[k]);
    }
    for (; r < rows; r += step) {
      float f0[8];
      load8(dy + (size_t)r * ld + col, f0);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += f0[k];
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) sacc[rlane][cg * 8 + k] = acc[k];
  __syncthreads();
  const int c = blockIdx.x * CS_COLS + threadIdx.x;
  const bool owner = threadIdx.x < CS_COLS && c < C;
  if (owner) {
    float t = 0.f;
#pragma unroll
    for (int r = 0; r < CS_RL; ++r) t += sacc[r][threadIdx.x];
    partial[(size_t)blockIdx.y * C + c] = t;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(&g_colsum_tickets[blockIdx.x], 1u);
    s_last = (t == (unsigned)RY - 1);
    if (s_last) g_colsum_tickets[blockIdx.x] = 0;
  }
  __syncthreads();
  if (s_last && owner) {
    __threadfence();
    float a = 0.f;
    for (int r = 0; r < RY; ++r) a += __ldcg(partial + (size_t)r * C + c);
    out[c] = __float2bfloat16(a + (accumulate ? __bfloat162float(out[c]) : 0.f));
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

// Rows of scratch the fused backward uses: scratch must hold nfn_norm_fused_rows() * 2 * C floats.
extern "C" int nfn_norm_fused_rows(void) { return 1; }

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
  // one row per warp at full occupancy (the dx kernel), with dweight / dbias folded per block in
  // shared memory and reduced into scratch[2][C] (zeroed here) with one atomic per column and block
  if (cudaMemsetAsync(scratch, 0, (size_t)2 * C * sizeof(float), st) != cudaSuccess) return launch_check("norm_backward memset", 0);
  const int grid = ceil_div(rows, NORM_THREADS / 32);
#define NFN_FUSED(V)                                                                                                   \
  norm_bwd_dx_kernel<V, 32><<<grid, NORM_THREADS, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,          \
      (const __nv_bfloat16*)w, mean, rstd, (const __nv_bfloat16*)dresid, (__nv_bfloat16*)dx, rows, C, mode, centered, scratch)
  if (C <= 256) NFN_FUSED(1);
  else if (C <= 512) NFN_FUSED(2);
  else if (C <= 768) NFN_FUSED(3);
  else NFN_FUSED(4);
#undef NFN_FUSED
  norm_bwd_wb_final_kernel<<<ceil_div(C, 256), 256, 0, st>>>(scratch, (__nv_bfloat16*)dw, (__nv_bfloat16*)db, 1, C, accumulate);
  return launch_check("norm_backward", 2);
}

// scratch: fp32 [64 * C]
extern "C" int nfn_colsum(const void* dy, int ld, void* out, float* scratch, int rows, int C,
                          int accumulate, nfn_stream_t stream) {
  if (rows <= 0) return 0;
  if (C % 2 || ld % 2) return fail(-1, "colsum: C and ld must be even");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (C % 8 || ld % 8 || (reinterpret_cast<uintptr_t>(dy) & 15)) return fail(-1, "colsum: C and ld must be multiples of 8 and dy 16-byte aligned");
  const int groups = ceil_div(C, CS_COLS);
  if (groups > CS_MAX_GROUPS) return fail(-1, "colsum: matrix too wide");
  const int RY = std::max(1, std::min(64, 2 * sm_count() / groups));  // scratch holds 64 partial rows
  colsum_kernel<<<dim3(groups, RY), 256, 0, st>>>((const __nv_bfloat16*)dy, ld, scratch, (__nv_bfloat16*)out, rows, C, accumulate);
  return launch_check("colsum", 1);
}

