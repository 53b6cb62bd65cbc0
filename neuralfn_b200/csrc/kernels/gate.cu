// Sigmoid output gate of gated attention, forward and backward, for training.
//
//   forward : out = att * sigmoid(gate)
//   backward: d(att) = d(out) * sigmoid(gate),  d(gate) = d(out) * att * sigmoid(gate) * (1 - sigmoid(gate))
//
// att / out / d(out) / d(att) are [rows, width] bf16 with their own row strides; gate and d(gate) are
// column blocks of the packed projection rows (q | k | v | gate), hence strided as well. One thread owns
// 8 consecutive elements. The inference path gates in place (nfn_sigmoid_gate_inplace); training keeps
// the ungated attention output because the attention backward pass needs it. Reference counterpart:
// the gated o_proj epilogues of neuralfn/csrc/native_gpt2/glimmer_k_mmq.cu:2521-2637 (inference only).
#include "common.h"
#include "nfn_kernels.h"
#include "sm100_ptx.cuh"

namespace nfn {

__device__ __forceinline__ void gate_unpack8(const uint4& u, float (&f)[8]) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 gate_pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

__global__ void __launch_bounds__(256)
gate_fwd_kernel(const __nv_bfloat16* __restrict__ att, int ld_att, const __nv_bfloat16* __restrict__ gate, int ld_gate,
                __nv_bfloat16* __restrict__ out, int ld_out, long long rows, int width) {
  const int vpr = width / 8;
  const long long total = rows * vpr;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const long long r = i / vpr;
    const int c = (int)(i - r * vpr) * 8;
    float a[8], g[8];
    gate_unpack8(*reinterpret_cast<const uint4*>(att + r * ld_att + c), a);
    gate_unpack8(*reinterpret_cast<const uint4*>(gate + r * ld_gate + c), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] *= 1.f / (1.f + __expf(-g[j]));
    *reinterpret_cast<uint4*>(out + r * ld_out + c) = gate_pack8(a);
  }
}

__global__ void __launch_bounds__(256)
gate_bwd_kernel(const __nv_bfloat16* __restrict__ dout, int ld_dout, const __nv_bfloat16* __restrict__ att, int ld_att,
                const __nv_bfloat16* __restrict__ gate, int ld_gate, __nv_bfloat16* __restrict__ datt, int ld_datt,
                __nv_bfloat16* __restrict__ dgate, int ld_dgate, long long rows, int width) {
  const int vpr = width / 8;
  const long long total = rows * vpr;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const long long r = i / vpr;
    const int c = (int)(i - r * vpr) * 8;
    float d[8], a[8], g[8], da[8], dg[8];
    gate_unpack8(*reinterpret_cast<const uint4*>(dout + r * ld_dout + c), d);
    gate_unpack8(*reinterpret_cast<const uint4*>(att + r * ld_att + c), a);
    gate_unpack8(*reinterpret_cast<const uint4*>(gate + r * ld_gate + c), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = 1.f / (1.f + __expf(-g[j]));
      da[j] = d[j] * s;
      dg[j] = d[j] * a[j] * s * (1.f - s);
    }
    *reinterpret_cast<uint4*>(datt + r * ld_datt + c) = gate_pack8(da);
    *reinterpret_cast<uint4*>(dgate + r * ld_dgate + c) = gate_pack8(dg);
  }
}

static int gate_grid(long long vecs) {
  long long b = (vecs + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}
static bool gate_ok(const void* p, int ld) { return p && !(reinterpret_cast<uintptr_t>(p) & 15) && !(ld & 7); }

}  // namespace nfn

using namespace nfn;

extern "C" int nfn_sigmoid_gate_forward(const void* att, int ld_att, const void* gate, int ld_gate, void* out, int ld_out,
                                        long long rows, int width, nfn_stream_t stream) {
  if (rows <= 0) return 0;
  if (width <= 0 || (width & 7) || !gate_ok(att, ld_att) || !gate_ok(gate, ld_gate) || !gate_ok(out, ld_out))
    return fail(-1, "sigmoid_gate_forward: operands must be 16-byte aligned, widths and strides multiples of 8");
  gate_fwd_kernel<<<gate_grid(rows * (width / 8)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(att), ld_att, static_cast<const __nv_bfloat16*>(gate), ld_gate, static_cast<__nv_bfloat16*>(out), ld_out,
      rows, width);
  return launch_check("sigmoid_gate_forward");
}

extern "C" int nfn_sigmoid_gate_backward(const void* dout, int ld_dout, const void* att, int ld_att, const void* gate, int ld_gate,
                                         void* datt, int ld_datt, void* dgate, int ld_dgate, long long rows, int width,
                                         nfn_stream_t stream) {
  if (rows <= 0) return 0;
  if (width <= 0 || (width & 7) || !gate_ok(dout, ld_dout) || !gate_ok(att, ld_att) || !gate_ok(gate, ld_gate) ||
      !gate_ok(datt, ld_datt) || !gate_ok(dgate, ld_dgate))
    return fail(-1, "sigmoid_gate_backward: operands must be 16-byte aligned, widths and strides multiples of 8");
  gate_bwd_kernel<<<gate_grid(rows * (width / 8)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dout), ld_dout, static_cast<const __nv_bfloat16*>(att), ld_att,
      static_cast<const __nv_bfloat16*>(gate), ld_gate, static_cast<__nv_bfloat16*>(datt), ld_datt, static_cast<__nv_bfloat16*>(dgate),
      ld_dgate, rows, width);
  return launch_check("sigmoid_gate_backward");
}
