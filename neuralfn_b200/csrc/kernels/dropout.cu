// Counter-based dropout for the adapter branch of LoRA training: out = keep(r, c) ? x / (1 - p) : 0.
//
// The mask is never stored. keep(r, c) is a pure function of (seed, stream, step, r, c): Philox4x32-10 keyed by the seed,
// counter = (index of the 8-element group, stream id, step), 16 random bits per element. The backward pass (and the
// recomputation of a checkpointed segment) calls the kernel again with the same stream id while the step counter - a device
// word the engine advances once per forward pass, so a replayed CUDA graph draws new masks - still holds the same value.
// With `accumulate` the masked, scaled input is added to `out` (d x += mask * d(dropped x) / (1 - p)).
//
// Reference counterpart: `nn.Dropout` in front of `lora_A` (neuralfn/torch_backend.py:977) and `--lora-dropout` of the native
// Glimmer trainer (neuralfn/csrc/native_train/muse_glimmer_native_train.cpp:141).
#include "common.h"
#include "nfn_kernels.h"
#include "sm100_ptx.cuh"

namespace nfn {

__device__ __forceinline__ uint4 drop_philox(uint4 ctr, uint2 key) {
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, ctr.x), lo0 = 0xD2511F53u * ctr.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, ctr.z), lo1 = 0xCD9E8D57u * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += 0x9E3779B9u;
    key.y += 0xBB67AE85u;
  }
  return ctr;
}

__global__ void __launch_bounds__(256)
dropout_kernel(const __nv_bfloat16* __restrict__ x, int ld_x, __nv_bfloat16* __restrict__ out, int ld_out, long long rows, int width,
               uint32_t threshold, float scale, uint2 key, uint32_t stream_id, const long long* __restrict__ step_dev, int accumulate) {
  const int vpr = width / 8;
  const long long total = rows * vpr;
  const unsigned long long step = step_dev ? (unsigned long long)*step_dev : 0ull;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const long long r = i / vpr;
    const int c = (int)(i - r * vpr) * 8;
    const uint4 rnd = drop_philox(make_uint4((uint32_t)i, (uint32_t)((unsigned long long)i >> 32) ^ (stream_id << 8), (uint32_t)step, (uint32_t)(step >> 32)), key);
    const uint32_t w[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
    const uint4 xv = *reinterpret_cast<const uint4*>(x + r * ld_x + c);
    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
    uint4 ov = make_uint4(0u, 0u, 0u, 0u);
    if (accumulate) ov = *reinterpret_cast<const uint4*>(out + r * ld_out + c);
    const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w};
    uint32_t res[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 v = unpack_bf16x2(xw[j]), o = unpack_bf16x2(ow[j]);
      const float a = ((w[j] & 0xFFFFu) >= threshold) ? v.x * scale : 0.f;
      const float b = ((w[j] >> 16) >= threshold) ? v.y * scale : 0.f;
      res[j] = pack_bf16x2(o.x + a, o.y + b);
    }
    *reinterpret_cast<uint4*>(out + r * ld_out + c) = make_uint4(res[0], res[1], res[2], res[3]);
  }
}

}  // namespace nfn

using namespace nfn;

// x, out: bf16 [rows, width] with row strides ld_x / ld_out (multiples of 8, 16-byte aligned); 0 <= p < 1; step_dev may be null.
extern "C" int nfn_dropout_apply(const void* x, int ld_x, void* out, int ld_out, long long rows, int width, float p, unsigned long long seed,
                                 int stream_id, const long long* step_dev, int accumulate, nfn_stream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  if (!x || !out || (width & 7) || (ld_x & 7) || (ld_out & 7) || ld_x < width || ld_out < width || !(p >= 0.f && p < 1.f))
    return fail(-1, "dropout: bad arguments");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) return fail(-1, "dropout: operands must be 16-byte aligned");
  const long long total = rows * (width / 8);
  const unsigned grid = (unsigned)std::min<long long>((total + 255) / 256, 148 * 16);
  const uint32_t threshold = (uint32_t)(p * 65536.f + 0.5f);
  dropout_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ld_x, static_cast<__nv_bfloat16*>(out), ld_out, rows, width, threshold, 1.f / (1.f - p),
      make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)), (uint32_t)stream_id, step_dev, accumulate);
  return launch_check("dropout", 1);
}
