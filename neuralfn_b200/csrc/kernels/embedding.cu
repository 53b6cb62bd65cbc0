// Token (+ absolute position) embedding forward and backward for bf16 tables.
//
// Forward gathers 16-byte vectors: out[n, :] = wte[token[n], :] (+ wpe[n % T, :]).
// Backward: dwpe is a deterministic sum over the batch. dwte has two forms, both adding on top of whatever the tied
// LM-head weight-gradient GEMM already wrote there: with the batch's tokens sorted (a stable sort, so equal tokens keep
// their row order) every vocabulary row that occurs is summed by one block, in row order, in fp32, and written once -
// the same bits on every run; without the sorted index it is a scatter-add with packed bf16x2 atomics, whose rounding
// depends on the order the atomics happen to land in.
//
// Reference counterparts: token_embedding* / absolute_position_embedding* kernels
// (neuralfn/csrc/tile_cuda/kernels.cu:13601-13861).
#include <cstdint>

#include "common.h"
#include "sm100_ptx.cuh"

namespace nfn {

__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const int* __restrict__ tokens, const __nv_bfloat16* __restrict__ wte,
                     const __nv_bfloat16* __restrict__ wpe, __nv_bfloat16* __restrict__ out, int n,
                     int T, int C, int vocab) {
  const int vec_per_row = C / 8;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * vec_per_row) return;
  const int row = (int)(idx / vec_per_row), v = (int)(idx % vec_per_row);
  int tok = tokens[row];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  uint4 a = reinterpret_cast<const uint4*>(wte + (size_t)tok * C)[v];
  if (wpe) {
    const uint4 b = reinterpret_cast<const uint4*>(wpe + (size_t)(row % T) * C)[v];
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 x = unpack_bf16x2(aw[j]), y = unpack_bf16x2(bw[j]);
      o[j] = pack_bf16x2(x.x + y.x, x.y + y.y);
    }
    a = make_uint4(o[0], o[1], o[2], o[3]);
  }
  reinterpret_cast<uint4*>(out + (size_t)row * C)[v] = a;
}

// dwpe[t, c] = sum_b dout[b*T + t, c]  (written, or accumulated when `accumulate`)
__global__ void __launch_bounds__(256)
wpe_bwd_kernel(const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ dwpe, int B,
               int T, int C, int accumulate) {
  const int pairs = C / 2;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * pairs) return;
  const int t = (int)(idx / pairs), c = (int)(idx % pairs) * 2;
  float a = 0.f, b = 0.f;
  for (int bi = 0; bi < B; ++bi) {
    float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dout + ((size_t)bi * T + t) * C + c));
    a += f.x; b += f.y;
  }
  uint32_t* dst = reinterpret_cast<uint32_t*>(dwpe + (size_t)t * C + c);
  if (accumulate) { float2 o = unpack_bf16x2(*dst); a += o.x; b += o.y; }
  *dst = pack_bf16x2(a, b);
}

__global__ void __launch_bounds__(256)
wte_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const int* __restrict__ tokens,
               __nv_bfloat16* __restrict__ dwte, int n, int C, int vocab) {
  const int pairs = C / 2;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * pairs) return;
  const int row = (int)(idx / pairs), c = (int)(idx % pairs) * 2;
  const int tok = tokens[row];
  if (tok < 0 || tok >= vocab) return;
  const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(dout + (size_t)row * C + c);
  atomicAdd(reinterpret_cast<__nv_bfloat162*>(dwte + (size_t)tok * C + c), g);
}

// One block per position of the sorted token list and per chunk of 256 columns; only the first position of every run of equal
// tokens works. A run of fewer than eight rows is summed by the block of chunk 0 alone, thread per 16-byte vector, row after
// row. For a longer run the eight warps of every chunk's block take the rows round-robin (row j of the run goes to warp j % 8, four rows in flight per
// warp), each lane keeps eight fp32 column sums, the warps' partial sums are added in a fixed order through shared memory, and
// warp 0 adds the total to the token's row of dwte: the order of every addition depends on the tokens alone.
constexpr int EMB_SORTED_WARPS = 8;

__global__ void __launch_bounds__(EMB_SORTED_WARPS * 32)
wte_bwd_sorted_kernel(const __nv_bfloat16* __restrict__ dout, const int* __restrict__ sorted_tokens, const long long* __restrict__ order,
                      __nv_bfloat16* __restrict__ dwte, int n, int C, int vocab) {
  __shared__ float part[EMB_SORTED_WARPS][32][8];
  const int p0 = blockIdx.x;
  const int tok = sorted_tokens[p0];
  if (tok < 0 || tok >= vocab || (p0 > 0 && sorted_tokens[p0 - 1] == tok)) return;      // block-uniform
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int p1 = p0 + 1;                                                                       // end of the run: 32 positions per look
  for (;;) {
    const int q = p1 + lane;
    const unsigned same = __ballot_sync(0xffffffffu, q < n && sorted_tokens[q] == tok);
    if (same == 0xffffffffu) { p1 += 32; continue; }
    p1 += __ffs(~same) - 1;
    break;
  }
  if (p1 - p0 < EMB_SORTED_WARPS) {
    // a short run (nearly all of them): the block of column chunk 0 does the whole row, one 16-byte vector per thread
    if (blockIdx.y) return;
    for (int cv = threadIdx.x * 8; cv < C; cv += EMB_SORTED_WARPS * 32 * 8) {
      float s8[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) s8[i] = 0.f;
      for (int q = p0; q < p1; ++q) {
        const uint4 v = *reinterpret_cast<const uint4*>(dout + (size_t)order[q] * C + cv);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 g = unpack_bf16x2(w[i]);
          s8[2 * i] += g.x;
          s8[2 * i + 1] += g.y;
        }
      }
      uint4* dst = reinterpret_cast<uint4*>(dwte + (size_t)tok * C + cv);
      const uint4 o = *dst;
      const uint32_t w[4] = {o.x, o.y, o.z, o.w};
      uint32_t r[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 g = unpack_bf16x2(w[i]);
        r[i] = pack_bf16x2(g.x + s8[2 * i], g.y + s8[2 * i + 1]);
      }
      *dst = make_uint4(r[0], r[1], r[2], r[3]);
    }
    return;
  }
  const int c = (blockIdx.y * 32 + lane) * 8;
  const bool live = c < C;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if (live) {
    constexpr int U = 4, STEP = EMB_SORTED_WARPS;
    for (int q = p0 + warp; q < p1; q += U * STEP) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int qq = q + u * STEP;
        v[u] = qq < p1 ? *reinterpret_cast<const uint4*>(dout + (size_t)order[qq] * C + c) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 g = unpack_bf16x2(w[i]);
          acc[2 * i] += g.x;
          acc[2 * i + 1] += g.y;
        }
      }
    }
  }
  {
#pragma unroll
    for (int i = 0; i < 8; ++i) part[warp][lane][i] = acc[i];
    __syncthreads();
    if (warp == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < EMB_SORTED_WARPS; ++w) t += part[w][lane][i];
        acc[i] = t;
      }
    }
  }
  if (warp == 0 && live) {
    uint4* dst = reinterpret_cast<uint4*>(dwte + (size_t)tok * C + c);
    const uint4 o = *dst;
    const uint32_t w[4] = {o.x, o.y, o.z, o.w};
    uint32_t r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 g = unpack_bf16x2(w[i]);
      r[i] = pack_bf16x2(g.x + acc[2 * i], g.y + acc[2 * i + 1]);
    }
    *dst = make_uint4(r[0], r[1], r[2], r[3]);
  }
}

// The same for widths that are not a multiple of 8: column pairs, one thread walks the run.
__global__ void __launch_bounds__(128)
wte_bwd_sorted_pairs_kernel(const __nv_bfloat16* __restrict__ dout, const int* __restrict__ sorted_tokens, const long long* __restrict__ order,
                            __nv_bfloat16* __restrict__ dwte, int n, int C, int vocab) {
  const int p0 = blockIdx.x;
  const int tok = sorted_tokens[p0];
  if (tok < 0 || tok >= vocab || (p0 > 0 && sorted_tokens[p0 - 1] == tok)) return;
  int p1 = p0 + 1;
  while (p1 < n && sorted_tokens[p1] == tok) ++p1;
  for (int c = threadIdx.x * 2; c < C; c += blockDim.x * 2) {
    float a = 0.f, b = 0.f;
    for (int q = p0; q < p1; ++q) {
      const float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dout + (size_t)order[q] * C + c));
      a += g.x;
      b += g.y;
    }
    uint32_t* dst = reinterpret_cast<uint32_t*>(dwte + (size_t)tok * C + c);
    const float2 old = unpack_bf16x2(*dst);
    *dst = pack_bf16x2(old.x + a, old.y + b);
  }
}

}  // namespace nfn

using namespace nfn;

// The deterministic form of the dwte part of nfn_embedding_backward: sorted_tokens / order = the batch's token ids in
// ascending order (stable) and the row each came from (int64, as a library sort returns it).
extern "C" int nfn_embedding_backward_sorted(const void* dout, const int* sorted_tokens, const long long* order, void* dwte, int n, int C, int vocab,
                                             nfn_stream_t stream) {
  if (n <= 0) return 0;
  if (!dout || !sorted_tokens || !order || !dwte || (C % 2)) return fail(-1, "embedding_backward_sorted: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (C % 8 == 0 && (reinterpret_cast<uintptr_t>(dout) % 16) == 0 && (reinterpret_cast<uintptr_t>(dwte) % 16) == 0) {
    const dim3 grid((unsigned)n, (unsigned)((C + 255) / 256));
    wte_bwd_sorted_kernel<<<grid, EMB_SORTED_WARPS * 32, 0, st>>>((const __nv_bfloat16*)dout, sorted_tokens, order, (__nv_bfloat16*)dwte, n, C, vocab);
  } else {
    wte_bwd_sorted_pairs_kernel<<<n, 128, 0, st>>>((const __nv_bfloat16*)dout, sorted_tokens, order, (__nv_bfloat16*)dwte, n, C, vocab);
  }
  return launch_check("embedding_bwd_sorted", 1);
}

extern "C" int nfn_embedding_forward(const int* tokens, const void* wte, const void* wpe, void* out,
                                     int n, int T, int C, int vocab, nfn_stream_t stream) {
  if (n <= 0) return 0;
  if (C % 8) return fail(-1, "embedding: C must be a multiple of 8");
  const long long total = (long long)n * (C / 8);
  embedding_fwd_kernel<<<(unsigned)((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      tokens, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, (__nv_bfloat16*)out, n, T, C,
      vocab);
  return launch_check("embedding_fwd");
}

extern "C" int nfn_embedding_backward(const void* dout, const int* tokens, void* dwte, void* dwpe,
                                      int B, int T, int C, int vocab, int accumulate_wpe,
                                      nfn_stream_t stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int n = B * T;
  if (n <= 0) return 0;
  if (C % 2) return fail(-1, "embedding: C must be even");
  if (dwpe) {
    const long long total = (long long)T * (C / 2);
    wpe_bwd_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        (const __nv_bfloat16*)dout, (__nv_bfloat16*)dwpe, B, T, C, accumulate_wpe);
  }
  if (dwte) {
    const long long total = (long long)n * (C / 2);
    wte_bwd_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        (const __nv_bfloat16*)dout, tokens, (__nv_bfloat16*)dwte, n, C, vocab);
  }
  return launch_check("embedding_bwd", (dwpe ? 1 : 0) + (dwte ? 1 : 0));
}
