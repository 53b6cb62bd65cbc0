// K-quant (GGUF Q4_K / Q5_K / Q6_K) and NF4 weights: dequantisation to bf16 and a
// decode-time skinny product y[b, n] = sum_k W[n, k] x[b, k] that reads the weights in
// their quantised form (4.5 / 6.56 bits per weight instead of 16), which is what bounds a
// small-batch decode step.
//
// Super-block layouts (256 weights each, little endian, as published with ggml):
//   Q4_K 144 B: half d, half dmin, u8 scales[12] (8 x 6-bit scale + 8 x 6-bit min), u8 qs[128]
//   Q5_K 176 B: half d, half dmin, u8 scales[12], u8 qh[32], u8 qs[128]
//   Q6_K 210 B: u8 ql[128], u8 qh[64], i8 scales[16], half d
// NF4: 4-bit codes into the 16-entry normal-float table, two codes per byte (low nibble =
// even column, as in the reference's torch_backend.py:1060-1072), one fp32 absmax per group
// of 64 weights.
//
// Skinny product: a CTA of 8 warps owns 32 output rows whose quantised weights stream through
// a ring of bulk-copied shared-memory stages; the activations of up to 8 batch rows stay in
// shared memory; one warp multiplies one row, every lane decoding 8 weights per super-block.
// An optional second weight matrix gives the gated form silu(W1 x) * (W2 x) in the same pass.
//
// The reference's counterparts: glimmer_k_mmq.cu (fused K-quant products),
// kernels.cu:1324-2015 (dequantisation), torch_backend.py:990-1097 (NF4 LoRA linear).
#include <cuda_fp16.h>

#include <algorithm>

#include "common.h"
#include "nfn_kernels.h"
#include "sm100_ptx.cuh"

namespace nfn {

constexpr int Q4K_BYTES = 144, Q5K_BYTES = 176, Q6K_BYTES = 210;

__constant__ float c_nf4[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                                -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                                0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                                0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};

__device__ __forceinline__ float half_at(const uint8_t* p) {
  return __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(p)));
}

// 6-bit scale and min of sub-block j (0..7) from the 12 packed bytes
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t* q, float* sc, float* mn) {
  if (j < 4) {
    *sc = (float)(q[j] & 63);
    *mn = (float)(q[j + 4] & 63);
  } else {
    *sc = (float)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
    *mn = (float)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

// ---- lane decoders: 8 weights of one super-block per lane --------------------------------------
// They also report where those weights sit inside the block: two runs of 4 (Q4_K/Q5_K) or
// four runs of 2 (Q6_K), so the caller can fetch the matching activations.
struct Q4KLane {
  static constexpr int kBytes = Q4K_BYTES, kRuns = 2, kRunLen = 4;
  __device__ static void decode(const uint8_t* blk, int lane, float* w, int* run_start) {
    const int grp = lane >> 3, off = (lane & 7) * 4;
    const float d = half_at(blk), dmin = half_at(blk + 2);
    float s1, m1, s2, m2;
    scale_min_k4(2 * grp, blk + 4, &s1, &m1);
    scale_min_k4(2 * grp + 1, blk + 4, &s2, &m2);
    const uint32_t q = *reinterpret_cast<const uint32_t*>(blk + 16 + grp * 32 + off);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t byte = (q >> (8 * i)) & 0xffu;
      w[i] = d * s1 * (float)(byte & 0xF) - dmin * m1;
      w[4 + i] = d * s2 * (float)(byte >> 4) - dmin * m2;
    }
    run_start[0] = grp * 64 + off;
    run_start[1] = grp * 64 + 32 + off;
  }
};

struct Q5KLane {
  static constexpr int kBytes = Q5K_BYTES, kRuns = 2, kRunLen = 4;
  __device__ static void decode(const uint8_t* blk, int lane, float* w, int* run_start) {
    const int grp = lane >> 3, off = (lane & 7) * 4;
    const float d = half_at(blk), dmin = half_at(blk + 2);
    float s1, m1, s2, m2;
    scale_min_k4(2 * grp, blk + 4, &s1, &m1);
    scale_min_k4(2 * grp + 1, blk + 4, &s2, &m2);
    const uint32_t qh = *reinterpret_cast<const uint32_t*>(blk + 16 + off);
    const uint32_t q = *reinterpret_cast<const uint32_t*>(blk + 48 + grp * 32 + off);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t byte = (q >> (8 * i)) & 0xffu, hb = (qh >> (8 * i)) & 0xffu;
      w[i] = d * s1 * (float)((byte & 0xF) + (((hb >> (2 * grp)) & 1u) << 4)) - dmin * m1;
      w[4 + i] = d * s2 * (float)((byte >> 4) + (((hb >> (2 * grp + 1)) & 1u) << 4)) - dmin * m2;
    }
    run_start[0] = grp * 64 + off;
    run_start[1] = grp * 64 + 32 + off;
  }
};

struct Q6KLane {
  static constexpr int kBytes = Q6K_BYTES, kRuns = 4, kRunLen = 2;
  __device__ static void decode(const uint8_t* blk, int lane, float* w, int* run_start) {
    const int half = lane >> 4, l0 = (lane & 15) * 2, is = l0 >> 4;
    const uint8_t* ql = blk + half * 64;
    const uint8_t* qh = blk + 128 + half * 32;
    const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192) + half * 8 + is;
    const float d = half_at(blk + 208);
    const unsigned short a = *reinterpret_cast<const unsigned short*>(ql + l0);
    const unsigned short b = *reinterpret_cast<const unsigned short*>(ql + l0 + 32);
    const unsigned short h = *reinterpret_cast<const unsigned short*>(qh + l0);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int qa = (a >> (8 * i)) & 0xff, qb = (b >> (8 * i)) & 0xff, hh = (h >> (8 * i)) & 0xff;
      w[0 + i] = d * (float)sc[0] * (float)(((qa & 0xF) | (((hh >> 0) & 3) << 4)) - 32);
      w[2 + i] = d * (float)sc[2] * (float)(((qb & 0xF) | (((hh >> 2) & 3) << 4)) - 32);
      w[4 + i] = d * (float)sc[4] * (float)(((qa >> 4) | (((hh >> 4) & 3) << 4)) - 32);
      w[6 + i] = d * (float)sc[6] * (float)(((qb >> 4) | (((hh >> 6) & 3) << 4)) - 32);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) run_start[r] = half * 128 + l0 + 32 * r;
  }
};

// ---- dequantisation to bf16: one warp per super-block ------------------------------------------
template <class L>
__global__ void __launch_bounds__(256)
dequant_kquant_kernel(const uint8_t* __restrict__ blocks, long long n_blocks, __nv_bfloat16* __restrict__ out) {
  const long long blk = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (blk >= n_blocks) return;
  float w[8];
  int runs[L::kRuns];
  L::decode(blocks + blk * L::kBytes, threadIdx.x & 31, w, runs);
  __nv_bfloat16* o = out + blk * 256;
#pragma unroll
  for (int r = 0; r < L::kRuns; ++r)
#pragma unroll
    for (int i = 0; i < L::kRunLen; i += 2)
      *reinterpret_cast<uint32_t*>(o + runs[r] + i) = pack_bf16x2(w[r * L::kRunLen + i], w[r * L::kRunLen + i + 1]);
}

__global__ void __launch_bounds__(256)
dequant_nf4_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ absmax, long long n_pairs, int group,
                   __nv_bfloat16* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pairs) return;
  const uint8_t b = codes[i];
  const float s = absmax[(2 * i) / group];
  *reinterpret_cast<uint32_t*>(out + 2 * i) = pack_bf16x2(c_nf4[b & 0xF] * s, c_nf4[b >> 4] * s);
}

// ---- skinny product ---------------------------------------------------------------------------
// A CTA owns GEMV_ROWS_CTA consecutive output rows. Their quantised weights are one
// contiguous byte range (rows are stored back to back), which streams through a ring of
// shared-memory stages - GEMV_STAGE_ROWS rows per stage, one bulk async copy each - so tens of
// kilobytes are in flight per SM regardless of how few registers the math needs. The
// activations of all batch rows sit in shared memory for the whole kernel; warp w of a stage
// multiplies row w: every lane decodes 8 weights of each super-block from shared memory.
constexpr int GEMV_WARPS = 8, GEMV_STAGE_ROWS = GEMV_WARPS, GEMV_ROWS_CTA = 32;

__device__ __forceinline__ void gemv_bulk_g2s(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar)
               : "memory");
}

template <class L, int BT, bool GATED>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
kquant_gemv_kernel(const uint8_t* __restrict__ W1, const uint8_t* __restrict__ W2, const __nv_bfloat16* __restrict__ x, int ldx,
                   __nv_bfloat16* __restrict__ y, int ldy, const __nv_bfloat16* __restrict__ bias,
                   const __nv_bfloat16* __restrict__ resid, int ld_resid, int B, int N, int K, int n_stages, int* status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full[4];
  __shared__ int sh_abort;
  const int kblocks = K / 256;
  const uint32_t row_bytes = (uint32_t)kblocks * L::kBytes;
  const uint32_t stage_bytes = ((GEMV_STAGE_ROWS * row_bytes + 127u) / 128u) * 128u;
  constexpr int NM = GATED ? 2 : 1;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [BT][K]
  unsigned char* ring = smem_raw + (((size_t)BT * K * 2 + 127) / 128) * 128;  // [n_stages][NM][stage_bytes]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * GEMV_ROWS_CTA;
  const int rows_cta = min(GEMV_ROWS_CTA, N - row0);
  const int n_iters = (rows_cta + GEMV_STAGE_ROWS - 1) / GEMV_STAGE_ROWS;

  if (threadIdx.x == 0) {
    sh_abort = 0;
    for (int s = 0; s < n_stages; ++s) mbar_init(smem_u32(&full[s]), 1);
    fence_mbar_init();
  }
  __syncthreads();
  auto issue = [&](int it) {  // thread 0: one bulk copy per weight matrix (16-byte granules; a sub-16-byte tail is copied by hand)
    const int st = it % n_stages;
    const int r = row0 + it * GEMV_STAGE_ROWS, rows = min(GEMV_STAGE_ROWS, row0 + rows_cta - r);
    const uint32_t bytes = (uint32_t)rows * row_bytes, bulk = bytes & ~15u;
    const uint32_t bar = smem_u32(&full[st]);
    mbar_expect_tx(bar, NM * bulk);
    gemv_bulk_g2s(smem_u32(ring + ((size_t)st * NM) * stage_bytes), W1 + (size_t)r * row_bytes, bulk, bar);
    if (GATED) gemv_bulk_g2s(smem_u32(ring + ((size_t)st * NM + 1) * stage_bytes), W2 + (size_t)r * row_bytes, bulk, bar);
  };
  if (threadIdx.x == 0)
    for (int it = 0; it < min(n_stages, n_iters); ++it) issue(it);
  // activations: all batch rows, zero-filled beyond B
  for (int i = threadIdx.x * 8; i < BT * K; i += blockDim.x * 8) {
    const int b = i / K, kk = i % K;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (b < B) v = *reinterpret_cast<const uint4*>(x + (long long)b * ldx + kk);
    *reinterpret_cast<uint4*>(xs + (size_t)b * K + kk) = v;
  }
  __syncthreads();

  for (int it = 0; it < n_iters; ++it) {
    const int st = it % n_stages;
    const int r = row0 + it * GEMV_STAGE_ROWS, rows = min(GEMV_STAGE_ROWS, row0 + rows_cta - r);
    bool ok = mbar_wait_bounded(smem_u32(&full[st]), (it / n_stages) & 1, &sh_abort, status, NFN_ERR_WAIT_FULL);
    ok = __syncthreads_and(ok);
    if (!ok) {
      for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let copies in flight land before the CTA goes away
      return;
    }
    unsigned char* w1s = ring + ((size_t)st * NM) * stage_bytes;
    unsigned char* w2s = w1s + stage_bytes;
    {  // tail bytes the 16-byte bulk granularity left out (at most 15 per matrix)
      const uint32_t bytes = (uint32_t)rows * row_bytes, bulk = bytes & ~15u;
      if (threadIdx.x < bytes - bulk) {
        w1s[bulk + threadIdx.x] = W1[(size_t)r * row_bytes + bulk + threadIdx.x];
        if (GATED) w2s[bulk + threadIdx.x] = W2[(size_t)r * row_bytes + bulk + threadIdx.x];
      }
      if (bytes != bulk) __syncthreads();
    }
    if (warp < rows) {
      float acc[NM][BT];
#pragma unroll
      for (int m = 0; m < NM; ++m)
#pragma unroll
        for (int b = 0; b < BT; ++b) acc[m][b] = 0.f;
      const unsigned char* wr1 = w1s + (size_t)warp * row_bytes;
      const unsigned char* wr2 = w2s + (size_t)warp * row_bytes;
#pragma unroll 2
      for (int kb = 0; kb < kblocks; ++kb) {
        int runs[L::kRuns];
        float w[NM][8];
        L::decode(wr1 + (size_t)kb * L::kBytes, lane, w[0], runs);
        if (GATED) L::decode(wr2 + (size_t)kb * L::kBytes, lane, w[NM - 1], runs);
#pragma unroll
        for (int b = 0; b < BT; ++b) {
          float xv[8];
          const __nv_bfloat16* xr = xs + (size_t)b * K + kb * 256;
#pragma unroll
          for (int q = 0; q < L::kRuns; ++q) {
            if (L::kRunLen == 4) {
              const uint2 u = *reinterpret_cast<const uint2*>(xr + runs[q]);
              const float2 p0 = unpack_bf16x2(u.x), p1 = unpack_bf16x2(u.y);
              xv[q * 4] = p0.x; xv[q * 4 + 1] = p0.y; xv[q * 4 + 2] = p1.x; xv[q * 4 + 3] = p1.y;
            } else {
              const float2 p0 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(xr + runs[q]));
              xv[q * 2] = p0.x; xv[q * 2 + 1] = p0.y;
            }
          }
#pragma unroll
          for (int m = 0; m < NM; ++m) {
            float s = acc[m][b];
#pragma unroll
            for (int i = 0; i < 8; ++i) s = fmaf(w[m][i], xv[i], s);
            acc[m][b] = s;
          }
        }
      }
#pragma unroll
      for (int m = 0; m < NM; ++m)
#pragma unroll
        for (int b = 0; b < BT; ++b) {
          float s = acc[m][b];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
          acc[m][b] = s;
        }
      if (lane == 0) {
        const int row = r + warp;
#pragma unroll
        for (int b = 0; b < BT; ++b) {
          if (b >= B) continue;
          float v = acc[0][b];
          if (GATED) v = silu_f(v) * acc[NM - 1][b];
          if (bias) v += __bfloat162float(bias[row]);
          if (resid) v += __bfloat162float(resid[(long long)b * ld_resid + row]);
          y[(long long)b * ldy + row] = __float2bfloat16(v);
        }
      }
    }
    __syncthreads();  // everyone is done with this stage
    if (threadIdx.x == 0 && it + n_stages < n_iters) issue(it + n_stages);
  }
}

template <class L, int BT>
static int launch_gemv(const void* w1, const void* w2, const void* x, int ldx, void* y, int ldy, const void* bias, const void* resid,
                       int ld_resid, int B, int N, int K, cudaStream_t st) {
  const int nm = w2 ? 2 : 1;
  const size_t x_bytes = (((size_t)BT * K * 2 + 127) / 128) * 128;
  const size_t stage = ((((size_t)GEMV_STAGE_ROWS * (K / 256) * L::kBytes) + 127) / 128) * 128 * nm;
  const size_t budget = 200 * 1024;
  if (x_bytes + 2 * stage > budget) return fail(-1, "kquant_gemv: K too large for the shared-memory plan (split the batch or use the dequantised GEMM path)");
  const int n_stages = (int)std::min<size_t>(4, (budget - x_bytes) / stage);
  const size_t smem = x_bytes + (size_t)n_stages * stage;
  const dim3 grid((N + GEMV_ROWS_CTA - 1) / GEMV_ROWS_CTA);
  auto run = [&](auto kern) -> int {
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget) != cudaSuccess)
      return fail(-2, "kquant_gemv: cannot raise the dynamic shared memory limit");
    kern<<<grid, GEMV_WARPS * 32, smem, st>>>(static_cast<const uint8_t*>(w1), static_cast<const uint8_t*>(w2),
                                             static_cast<const __nv_bfloat16*>(x), ldx, static_cast<__nv_bfloat16*>(y), ldy,
                                             static_cast<const __nv_bfloat16*>(bias), static_cast<const __nv_bfloat16*>(resid),
                                             ld_resid, B, N, K, n_stages, status_ptr());
    return launch_check("kquant_gemv", 1);
  };
  return w2 ? run(kquant_gemv_kernel<L, BT, true>) : run(kquant_gemv_kernel<L, BT, false>);
}

template <class L>
static int dispatch_gemv(const void* w1, const void* w2, const void* x, int ldx, void* y, int ldy, const void* bias, const void* resid,
                         int ld_resid, int B, int N, int K, cudaStream_t st) {
  if (B <= 1) return launch_gemv<L, 1>(w1, w2, x, ldx, y, ldy, bias, resid, ld_resid, B, N, K, st);
  if (B <= 2) return launch_gemv<L, 2>(w1, w2, x, ldx, y, ldy, bias, resid, ld_resid, B, N, K, st);
  if (B <= 4) return launch_gemv<L, 4>(w1, w2, x, ldx, y, ldy, bias, resid, ld_resid, B, N, K, st);
  return launch_gemv<L, 8>(w1, w2, x, ldx, y, ldy, bias, resid, ld_resid, B, N, K, st);
}

}  // namespace nfn

using namespace nfn;

extern "C" int nfn_quant_block_bytes(int qtype) {
  switch (qtype) {
    case NFN_QTYPE_Q4_K: return Q4K_BYTES;
    case NFN_QTYPE_Q5_K: return Q5K_BYTES;
    case NFN_QTYPE_Q6_K: return Q6K_BYTES;
    default: return -1;
  }
}

extern "C" int nfn_dequant_kquant(int qtype, const void* blocks, long long n_blocks, void* out_bf16, nfn_stream_t stream) {
  if (n_blocks <= 0) return 0;
  if (!blocks || !out_bf16) return fail(-1, "dequant_kquant: null operand");
  const long long grid = (n_blocks + 7) / 8;
  if (grid > 0x7fffffffLL) return fail(-1, "dequant_kquant: too many blocks for one launch");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint8_t* b = static_cast<const uint8_t*>(blocks);
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out_bf16);
  if (qtype == NFN_QTYPE_Q4_K) {
    if (reinterpret_cast<uintptr_t>(blocks) % 4) return fail(-1, "dequant_kquant: Q4_K blocks must be 4-byte aligned");
    dequant_kquant_kernel<Q4KLane><<<(unsigned)grid, 256, 0, st>>>(b, n_blocks, o);
  } else if (qtype == NFN_QTYPE_Q5_K) {
    if (reinterpret_cast<uintptr_t>(blocks) % 4) return fail(-1, "dequant_kquant: Q5_K blocks must be 4-byte aligned");
    dequant_kquant_kernel<Q5KLane><<<(unsigned)grid, 256, 0, st>>>(b, n_blocks, o);
  } else if (qtype == NFN_QTYPE_Q6_K) {
    if (reinterpret_cast<uintptr_t>(blocks) % 2) return fail(-1, "dequant_kquant: Q6_K blocks must be 2-byte aligned");
    dequant_kquant_kernel<Q6KLane><<<(unsigned)grid, 256, 0, st>>>(b, n_blocks, o);
  } else {
    return fail(-1, "dequant_kquant: unknown quantisation type");
  }
  return launch_check("dequant_kquant", 1);
}

extern "C" int nfn_dequant_nf4(const void* codes, const float* absmax, long long n_weights, int group, void* out_bf16,
                               nfn_stream_t stream) {
  if (n_weights <= 0) return 0;
  if (!codes || !absmax || !out_bf16 || group <= 0 || group % 2 || n_weights % 2) return fail(-1, "dequant_nf4: bad arguments");
  const long long pairs = n_weights / 2, grid = (pairs + 255) / 256;
  if (grid > 0x7fffffffLL) return fail(-1, "dequant_nf4: too many weights for one launch");
  dequant_nf4_kernel<<<(unsigned)grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(codes), absmax, pairs, group, static_cast<__nv_bfloat16*>(out_bf16));
  return launch_check("dequant_nf4", 1);
}

// y[b, n] = act(W1[n, :] . x[b, :]) (* W2[n, :] . x[b, :] when w2 is given: silu-gated) + bias[n] + resid[b, n]
extern "C" int nfn_kquant_gemv(int qtype, const void* w1, const void* w2, const void* x, int ldx, void* y, int ldy,
                               const void* bias, const void* resid, int ld_resid, int B, int N, int K, nfn_stream_t stream) {
  if (B <= 0 || N <= 0) return 0;
  if (!w1 || !x || !y) return fail(-1, "kquant_gemv: null operand");
  if (B > 8) return fail(-1, "kquant_gemv: at most 8 batch rows per call (use the dequantised GEMM path beyond)");
  if (K <= 0 || K % 256) return fail(-1, "kquant_gemv: K must be a multiple of 256");
  if (ldx < K || ldx % 8 || reinterpret_cast<uintptr_t>(x) % 16) return fail(-1, "kquant_gemv: x rows must be 16-byte aligned");
  if (ldy < N || (resid && ld_resid < N)) return fail(-1, "kquant_gemv: output / residual stride smaller than N");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (qtype == NFN_QTYPE_Q4_K) {
    if (reinterpret_cast<uintptr_t>(w1) % 16 || reinterpret_cast<uintptr_t>(w2) % 16) return fail(-1, "kquant_gemv: weight matrices must be 16-byte aligned");
    return dispatch_gemv<Q4KLane>(w1, w2, x, ldx, y, ldy, bias, resid, ld_resid, B, N, K, st);
  }
  if (qtype == NFN_QTYPE_Q5_K) {
    if (reinterpret_cast<uintptr_t>(w1) % 16 || reinterpret_cast<uintptr_t>(w2) % 16) return fail(-1, "kquant_gemv: weight matrices must be 16-byte aligned");
    return dispatch_gemv<Q5KLane>(w1, w2, x, ldx, y, ldy, bias, resid, ld_resid, B, N, K, st);
  }
  if (qtype == NFN_QTYPE_Q6_K) {
    if (reinterpret_cast<uintptr_t>(w1) % 16 || reinterpret_cast<uintptr_t>(w2) % 16) return fail(-1, "kquant_gemv: weight matrices must be 16-byte aligned");
    return dispatch_gemv<Q6KLane>(w1, w2, x, ldx, y, ldy, bias, resid, ld_resid, B, N, K, st);
  }
  return fail(-1, "kquant_gemv: unknown quantisation type");
}
