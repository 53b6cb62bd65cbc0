// Token cross-entropy over bf16 logits with optional logit soft-cap and z-loss,
// forward and backward fused: one block owns one row, stages it once in shared
// memory (rows up to ~100 K vocabulary entries), computes the log-sum-exp, the row
// loss, and overwrites the logits with their gradient. HBM traffic is one read and
// one write of the logits.
//
//   value_j = logits_j (already soft-capped by the producing GEMM epilogue when cap > 0)
//   loss    = lse - value_t + z * lse^2
//   dlogit_j = (p_j - [j == t] + 2 z lse p_j) * (1 - (value_j / cap)^2) * row_scale
//
// Columns >= vocab (padding up to ld) receive zero gradient; rows whose target is
// negative are ignored (zero loss, zero gradient).
//
// Reference counterpart: token_cross_entropy_variant_bf16_u16
// (neuralfn/csrc/tile_cuda/kernels.cu:19018-19108) and TokenCrossEntropyStage
// (neuralfn/torch_backend.py:762-806).
#include "common.h"
#include "sm100_ptx.cuh"

namespace nfn {

constexpr int CE_THREADS = 512;

__device__ __forceinline__ float block_reduce_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = red[0];
  for (int i = 1; i < CE_THREADS / 32; ++i) t = fmaxf(t, red[i]);
  return t;
}
__device__ __forceinline__ float block_reduce_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < CE_THREADS / 32; ++i) t += red[i];
  return t;
}

// STAGE: keep the row in shared memory between the two passes.
template <bool STAGE>
__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const int* __restrict__ targets,
                  const float* __restrict__ row_scale, float* __restrict__ row_loss,
                  float* __restrict__ row_lse, int rows, int vocab, int ld, float cap, float z_coef,
                  float grad_scale, int write_grad) {
  extern __shared__ uint4 ce_smem[];
  __shared__ float red[CE_THREADS / 32];
  const int row = blockIdx.x;
  if (row >= rows) return;
  __nv_bfloat16* g = logits + (size_t)row * ld;
  const int tgt = targets[row];
  const int nvec = ld / 8;       // 16-byte vectors per row (ld % 8 == 0)
  const uint4* gv = reinterpret_cast<const uint4*>(g);

  if (STAGE) {
    // Bring the whole row into shared memory with asynchronous 16-byte copies: every thread has
    // all of its vectors in flight at once instead of one dependent load per loop iteration
    // (which caps a 1024-thread SM at about 16 KB in flight, a third of what HBM can deliver).
    for (int i = threadIdx.x; i < nvec; i += CE_THREADS)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(ce_smem + i)), "l"(gv + i) : "memory");
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
    // each thread only reads back the vectors it copied itself: no barrier needed here
  }

  // pass 1: online max / sum of exp over the valid vocabulary
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    const uint4 u = STAGE ? ce_smem[i] : gv[i];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) { float2 t = unpack_bf16x2(w[j]); f[2 * j] = t.x; f[2 * j + 1] = t.y; }
    const int c0 = i * 8;
    float lm = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) if (c0 + j < vocab) lm = fmaxf(lm, f[j]);
    if (lm > m) { s *= __expf(m - lm); m = lm; }
    if (lm > -INFINITY) {
#pragma unroll
      for (int j = 0; j < 8; ++j) if (c0 + j < vocab) s += __expf(f[j] - m);
    }
  }
  const float gm = block_reduce_max(m, red);
  s = (m > -INFINITY) ? s * __expf(m - gm) : 0.f;
  const float gs = block_reduce_sum(s, red);
  const float lse = gm + logf(gs);
  const bool active = tgt >= 0 && tgt < vocab;
  const float rs = (row_scale ? row_scale[row] : 1.f);
  if (threadIdx.x == 0) {
    float loss = 0.f;
    if (active) {
      const float vt = __bfloat162float(g[tgt]);
      loss = (lse - vt + z_coef * lse * lse) * rs;
    }
    row_loss[row] = loss;
    if (row_lse) row_lse[row] = lse;
  }
  if (!write_grad) return;
  __syncthreads();  // staged row complete; target logit read before overwrite

  // pass 2: gradient in place
  const float coef = active ? grad_scale * rs : 0.f;
  const float zfac = 1.f + 2.f * z_coef * lse;
  const float inv_cap2 = cap > 0.f ? 1.f / (cap * cap) : 0.f;
  uint4* gw = reinterpret_cast<uint4*>(g);
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    const uint4 u = STAGE ? ce_smem[i] : gv[i];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) { float2 t = unpack_bf16x2(w[j]); f[2 * j] = t.x; f[2 * j + 1] = t.y; }
    const int c0 = i * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = c0 + j;
      float d = 0.f;
      if (c < vocab) {
        const float p = __expf(f[j] - lse);
        d = p * zfac - (c == tgt ? 1.f : 0.f);
        d *= (1.f - f[j] * f[j] * inv_cap2) * coef;
      }
      f[j] = d;
    }
    uint4 o;
    o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
    o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
    gw[i] = o;
  }
}

// Deterministic sum of n floats into out[0] (* scale). Single block.
__global__ void __launch_bounds__(1024) sum_rows_kernel(const float* __restrict__ v, float* out,
                                                        int n, float scale, int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += 1024) s += v[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = red[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) out[0] = s * scale + (accumulate ? out[0] : 0.f);
  }
}

}  // namespace nfn

using namespace nfn;

// logits: bf16 [rows, ld] (overwritten with gradients when write_grad != 0)
// targets: int32 [rows] (negative = ignored); row_scale: optional fp32 [rows]
// row_loss: fp32 [rows] out; row_lse: optional fp32 [rows] out
// mean_loss: optional fp32 [1] out = sum(row_loss) * loss_scale
extern "C" int nfn_cross_entropy(void* logits, const int* targets, const float* row_scale,
                                 float* row_loss, float* row_lse, float* mean_loss, int rows,
                                 int vocab, int ld, float cap, float z_coef, float grad_scale,
                                 float loss_scale, int write_grad, nfn_stream_t stream) {
  if (rows <= 0) return 0;
  if (ld % 8 || vocab > ld) return fail(-1, "cross_entropy: ld must be a multiple of 8 and >= vocab");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)ld * 2;
  const bool stage = smem <= 110 * 1024;  // two blocks per SM stay resident
  if (stage) {
    static bool attr[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr[dev & 63]) {
      cudaFuncSetAttribute(ce_fwd_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           110 * 1024);
      attr[dev & 63] = true;
    }
    ce_fwd_bwd_kernel<true><<<rows, CE_THREADS, smem, st>>>(
        (__nv_bfloat16*)logits, targets, row_scale, row_loss, row_lse, rows, vocab, ld, cap, z_coef,
        grad_scale, write_grad);
  } else {
    ce_fwd_bwd_kernel<false><<<rows, CE_THREADS, 0, st>>>(
        (__nv_bfloat16*)logits, targets, row_scale, row_loss, row_lse, rows, vocab, ld, cap, z_coef,
        grad_scale, write_grad);
  }
  if (mean_loss) sum_rows_kernel<<<1, 1024, 0, st>>>(row_loss, mean_loss, rows, loss_scale, 0);
  return launch_check("cross_entropy", mean_loss ? 2 : 1);
}

extern "C" int nfn_sum_f32(const float* v, float* out, int n, float scale, int accumulate,
                           nfn_stream_t stream) {
  sum_rows_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(v, out, n, scale, accumulate);
  return launch_check("sum_f32");
}
