// Gradient accumulation across micro-batches of one optimizer step. The engines write bf16
// gradients of one micro-batch into the flat gradient buffer; between micro-batches they
// are summed in an fp32 side buffer so that many small contributions do not round away:
//   mode 0 (first micro-batch):  acc  = g
//   mode 1 (middle):             acc += g
//   mode 2 (last):               g    = (acc + g) * scale        (scale = 1 / micro-batches)
// after which the optimizer consumes g exactly as in the no-accumulation case.
// Reference behaviour: zero_accumulated_gradients + gradient_accumulate
// (nfn_gpt2_native_train.cpp:28362-28400, kernels.cu:10659).
#include <algorithm>

#include "common.h"
#include "nfn_kernels.h"
#include "sm100_ptx.cuh"

namespace nfn {

__global__ void __launch_bounds__(256)
grad_accumulate_kernel(float* __restrict__ acc, __nv_bfloat16* __restrict__ g, long long n8, int mode, float scale) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    const uint4 u = *reinterpret_cast<const uint4*>(g + i * 8);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    float v[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
    float4* ap = reinterpret_cast<float4*>(acc + i * 8);
    if (mode != 0) {
      const float4 lo = ap[0], hi = ap[1];
      v[0] += lo.x; v[1] += lo.y; v[2] += lo.z; v[3] += lo.w;
      v[4] += hi.x; v[5] += hi.y; v[6] += hi.z; v[7] += hi.w;
    }
    if (mode == 2) {
      uint4 o;
      o.x = pack_bf16x2(v[0] * scale, v[1] * scale); o.y = pack_bf16x2(v[2] * scale, v[3] * scale);
      o.z = pack_bf16x2(v[4] * scale, v[5] * scale); o.w = pack_bf16x2(v[6] * scale, v[7] * scale);
      *reinterpret_cast<uint4*>(g + i * 8) = o;
    } else {
      ap[0] = make_float4(v[0], v[1], v[2], v[3]);
      ap[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
  }
}

}  // namespace nfn

extern "C" int nfn_grad_accumulate(float* acc, void* grads_bf16, long long n, int mode, float scale, nfn_stream_t stream) {
  using namespace nfn;
  if (n <= 0) return 0;
  if (!acc || !grads_bf16 || (n & 7) || mode < 0 || mode > 2) return fail(-1, "grad_accumulate: bad arguments (n must be a multiple of 8)");
  const long long n8 = n / 8;
  const int grid = (int)std::min<long long>((n8 + 255) / 256, (long long)sm_count() * 16);
  grad_accumulate_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(acc, static_cast<__nv_bfloat16*>(grads_bf16), n8, mode, scale);
  return launch_check("grad_accumulate", 1);
}
