// Token (+ absolute position) embedding forward and backward for bf16 tables.
//
// Forward gathers 16-byte vectors: out[n, :] = wte[token[n], :] (+ wpe[n % T, :]).
// Backward: dwpe is a deterministic sum over the batch; dwte is a scatter-add with
// packed bf16x2 reductions on top of whatever the tied LM-head weight-gradient GEMM
// already wrote there.
//
// Reference counterparts: token_embedding* / absolute_position_embedding* kernels
// (neuralfn/csrc/tile_cuda/kernels.cu:13601-13861).
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

}  // namespace nfn

using namespace nfn;

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
