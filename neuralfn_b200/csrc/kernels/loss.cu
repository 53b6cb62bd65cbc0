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

// (d0, d1) = (a0, a1) * (b0, b1) + (c0, c1): one issue slot for two fp32 FMAs (sm_100)
__device__ __forceinline__ void ce_fma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void ce_mul2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmul.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ uint32_t ce_max_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// STAGE: keep the row in shared memory between the passes. CAPPED: the logits are already
// soft-capped to [-cap, cap], so `cap` bounds the row maximum and no maximum pass is needed.
// The kernel is bound by instruction issue, not by HBM, unless the per-element work is kept to a
// handful of instructions: whole 8-element vectors inside the vocabulary take a branch-free path
// with packed two-wide fp32 arithmetic; only the vector that straddles the vocabulary edge is
// handled element by element, and the target column is corrected by one thread afterwards.
template <bool STAGE, bool CAPPED>
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
  const int nvec = ld / 8;            // 16-byte vectors per row (ld % 8 == 0)
  const int nfull = vocab / 8;        // vectors entirely inside the vocabulary
  const int ntail = vocab - nfull * 8;  // valid elements of vector `nfull` (0: none)
  const uint4* gv = reinterpret_cast<const uint4*>(g);
  const float LOG2E = 1.4426950408889634f;

  if (STAGE) {
    // the whole row in flight at once (asynchronous 16-byte copies); each thread reads back only
    // the vectors it copied itself, so no barrier is needed before the first pass
    for (int i = threadIdx.x; i < nvec; i += CE_THREADS)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(ce_smem + i)), "l"(gv + i) : "memory");
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
  }

  // row maximum (skipped when the soft-cap already bounds it)
  // (a large cap would let exp(f - cap) underflow for ordinary logits, so it still takes the pass)
  float gm = cap;
  if (!(CAPPED && cap <= 40.f)) {
    uint32_t mx = 0xff80ff80u;  // (-inf, -inf)
    for (int i = threadIdx.x; i < nfull; i += CE_THREADS) {
      const uint4 u = STAGE ? ce_smem[i] : gv[i];
      mx = ce_max_bf16x2(mx, ce_max_bf16x2(ce_max_bf16x2(u.x, u.y), ce_max_bf16x2(u.z, u.w)));
    }
    const float2 m2 = unpack_bf16x2(mx);
    float m = fmaxf(m2.x, m2.y);
    if (ntail > 0 && threadIdx.x == 0)
      for (int j = 0; j < ntail; ++j) m = fmaxf(m, __bfloat162float(g[nfull * 8 + j]));
    gm = block_reduce_max(m, red);
  }
  // sum of exp(f - gm) = sum of exp2(f * log2e - gm * log2e)
  const float moff = gm * LOG2E;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int i = threadIdx.x; i < nfull; i += CE_THREADS) {
    const uint4 u = STAGE ? ce_smem[i] : gv[i];
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    float x0, x1, x2, x3, x4, x5, x6, x7;
    ce_fma2(x0, x1, a.x, a.y, LOG2E, LOG2E, -moff, -moff);
    ce_fma2(x2, x3, b.x, b.y, LOG2E, LOG2E, -moff, -moff);
    ce_fma2(x4, x5, c.x, c.y, LOG2E, LOG2E, -moff, -moff);
    ce_fma2(x6, x7, d.x, d.y, LOG2E, LOG2E, -moff, -moff);
    s0 += fast_exp2(x0) + fast_exp2(x1);
    s1 += fast_exp2(x2) + fast_exp2(x3);
    s2 += fast_exp2(x4) + fast_exp2(x5);
    s3 += fast_exp2(x6) + fast_exp2(x7);
  }
  float s = (s0 + s1) + (s2 + s3);
  if (ntail > 0 && threadIdx.x == 0)
    for (int j = 0; j < ntail; ++j) s += fast_exp2(__bfloat162float(g[nfull * 8 + j]) * LOG2E - moff);
  const float gs = block_reduce_sum(s, red);
  const float lse = gm + logf(gs);
  const bool active = tgt >= 0 && tgt < vocab;
  const float rs = (row_scale ? row_scale[row] : 1.f);
  const float vt = active ? __bfloat162float(g[tgt]) : 0.f;  // read before any gradient is written
  if (threadIdx.x == 0) {
    row_loss[row] = active ? (lse - vt + z_coef * lse * lse) * rs : 0.f;
    if (row_lse) row_lse[row] = lse;
  }
  if (!write_grad) return;
  __syncthreads();  // every thread holds vt; the staged row is complete

  // gradient in place: d = p * (1 + 2 z lse) * (1 - f^2 / cap^2) * coef, p = exp2(f log2e - lse log2e);
  // the "- [j == t]" term is added by one thread after the sweep
  const float coef = active ? grad_scale * rs : 0.f;
  const float A = (1.f + 2.f * z_coef * lse) * coef;
  const float loff = lse * LOG2E;
  const float nic2 = CAPPED ? -1.f / (cap * cap) : 0.f;
  uint4* gw = reinterpret_cast<uint4*>(g);
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    if (i < nfull) {
      const uint4 u = STAGE ? ce_smem[i] : gv[i];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
      uint32_t r[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        float x0, x1, d0, d1;
        ce_fma2(x0, x1, f.x, f.y, LOG2E, LOG2E, -loff, -loff);
        ce_mul2(d0, d1, fast_exp2(x0), fast_exp2(x1), A, A);
        if (CAPPED) {
          float q0, q1, t0, t1;
          ce_mul2(q0, q1, f.x, f.y, f.x, f.y);
          ce_fma2(t0, t1, q0, q1, nic2, nic2, 1.f, 1.f);
          ce_mul2(d0, d1, d0, d1, t0, t1);
        }
        r[j] = pack_bf16x2(d0, d1);
      }
      o = make_uint4(r[0], r[1], r[2], r[3]);
    } else if (i == nfull && ntail > 0) {
      float f[8];
      const uint4 u = STAGE ? ce_smem[i] : gv[i];
      {
        const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float d = 0.f;
        if (j < ntail) d = fast_exp2(f[j] * LOG2E - loff) * A * (1.f + f[j] * f[j] * nic2);
        f[j] = d;
      }
      o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
      o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
    }
    gw[i] = o;  // padding columns get zero gradient
  }
  if (active) {
    __syncthreads();  // the sweep's store of the target's vector has been issued by its owner
    if (threadIdx.x == ((tgt / 8) % CE_THREADS)) {  // the same thread that wrote that vector: program order suffices
      const float p = fast_exp2(vt * LOG2E - loff);
      const float d = (p * (1.f + 2.f * z_coef * lse) - 1.f) * (1.f + vt * vt * nic2) * coef;
      g[tgt] = __float2bfloat16(d);
    }
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
      cudaFuncSetAttribute(ce_fwd_bwd_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
      cudaFuncSetAttribute(ce_fwd_bwd_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
      attr[dev & 63] = true;
    }
  }
  const size_t dyn = stage ? smem : 0;
#define NFN_CE(S, C)                                                                                          \
  ce_fwd_bwd_kernel<S, C><<<rows, CE_THREADS, dyn, st>>>((__nv_bfloat16*)logits, targets, row_scale, row_loss, \
                                                         row_lse, rows, vocab, ld, cap, z_coef, grad_scale, write_grad)
  if (stage) {
    if (cap > 0.f) NFN_CE(true, true); else NFN_CE(true, false);
  } else {
    if (cap > 0.f) NFN_CE(false, true); else NFN_CE(false, false);
  }
#undef NFN_CE
  if (mean_loss) sum_rows_kernel<<<1, 1024, 0, st>>>(row_loss, mean_loss, rows, loss_scale, 0);
  return launch_check("cross_entropy", mean_loss ? 2 : 1);
}

extern "C" int nfn_sum_f32(const float* v, float* out, int n, float scale, int accumulate,
                           nfn_stream_t stream) {
  sum_rows_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(v, out, n, scale, accumulate);
  return launch_check("sum_f32");
}
