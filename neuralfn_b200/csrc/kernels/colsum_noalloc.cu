// Column sum (bias gradient) for callers that cannot allocate device memory.
//
// nfn_colsum needs an fp32 scratch buffer of 64 * C floats from its caller. Some callers
// have no way to provide one: code running inside a CUDA-graph capture or replay-only
// serving loop where cudaMalloc is illegal or would stall, plug-ins handed only their
// input and output pointers by a host framework that owns all device memory, and
// real-time loops that must not take the allocator lock. For them this file offers one
// extra entry point whose scratch is a fixed array compiled into the library.
//
// Cost and limits of that choice:
//  * the array occupies NFN_COLSUM_NOALLOC_MAX_C * 64 floats (2 MiB) of every GPU that
//    loads the library, from load until the process exits;
//  * widths above NFN_COLSUM_NOALLOC_MAX_C are refused with an error (use nfn_colsum);
//  * the array is shared by all calls on a device and keeps whatever the previous call
//    left in it. Nothing needs to start at zero: every partial slot a call reads is
//    written by that same call first. Two calls that overlap on the GPU (different
//    streams, or graphs replayed concurrently) race on the array and give wrong sums;
//    order them on one stream.
//
// The first call on each device looks up the device address of the array
// (cudaGetSymbolAddress) and caches it. Make that first call before starting any stream
// capture on that device.
#include "colsum_noalloc.h"

#include <mutex>

#include "common.h"
#include "sm100_ptx.cuh"

namespace nfn {

constexpr int NA_ROW_SPLITS = 64;
static __device__ __align__(256) float g_colsum_scratch[NA_ROW_SPLITS * NFN_COLSUM_NOALLOC_MAX_C];

// block (cx, ry): 4 row-lanes x 64 column pairs; rows ry*4 + lane, stepping by 4 * gridDim.y
__global__ void __launch_bounds__(256)
na_colsum_partial_kernel(const __nv_bfloat16* __restrict__ dy, int ld, float* __restrict__ partial,
                         int rows, int C) {
  const int cp = threadIdx.x & 63, rlane = threadIdx.x >> 6;
  const int col = (blockIdx.x * 64 + cp) * 2;
  float a = 0.f, b = 0.f;
  if (col < C) {
    for (int r = blockIdx.y * 4 + rlane; r < rows; r += gridDim.y * 4) {
      const float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dy + (size_t)r * ld + col));
      a += f.x;
      b += f.y;
    }
  }
  __shared__ float sa[4][64], sb[4][64];
  sa[rlane][cp] = a;
  sb[rlane][cp] = b;
  __syncthreads();
  if (rlane == 0 && col < C) {
    partial[(size_t)blockIdx.y * C + col] = sa[0][cp] + sa[1][cp] + sa[2][cp] + sa[3][cp];
    partial[(size_t)blockIdx.y * C + col + 1] = sb[0][cp] + sb[1][cp] + sb[2][cp] + sb[3][cp];
  }
}

__global__ void na_colsum_final_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                                       int splits, int C, int accumulate) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= C) return;
  float a = 0.f;
  for (int r = 0; r < splits; ++r) a += partial[(size_t)r * C + col];
  out[col] = __float2bfloat16(a + (accumulate ? __bfloat162float(out[col]) : 0.f));
}

// Device address of the scratch array on the current device (looked up once per device).
static float* scratch_for_current_device(int* rc) {
  static float* cached[64] = {};
  static bool ready[64] = {};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    *rc = fail(-2, "colsum_noalloc: cannot identify the current device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(mu);
  if (!ready[dev]) {
    float* ptr = nullptr;
    // In host code the array's name is only a handle for the runtime; the kernels need
    // the address the runtime resolves for the device that is current right now.
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_colsum_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      *rc = fail(-2, "colsum_noalloc: cudaGetSymbolAddress failed for the scratch array");
      return nullptr;
    }
    cached[dev] = ptr;
    ready[dev] = true;
  }
  return cached[dev];
}

}  // namespace nfn

using namespace nfn;

extern "C" int nfn_colsum_noalloc(const void* dy, int ld, void* out, int rows, int C, int accumulate,
                                  nfn_stream_t stream) {
  if (rows <= 0) return 0;
  if (!dy || !out) return fail(-1, "colsum_noalloc: null operand");
  if (C <= 0 || (C % 2) || (ld % 2) || ld < C) return fail(-1, "colsum_noalloc: C and ld must be even, ld >= C");
  // the partial kernel reads dy two bf16 at a time: a view that starts at an odd element passes the
  // size checks above but would fault with a misaligned address on the device, so refuse it here
  if ((reinterpret_cast<uintptr_t>(dy) & 3) != 0)
    return fail(-1, "colsum_noalloc: dy must be 4-byte aligned (a view starting at an odd bf16 element is not)");
  if ((reinterpret_cast<uintptr_t>(out) & 1) != 0) return fail(-1, "colsum_noalloc: out must be 2-byte aligned");
  if (C > NFN_COLSUM_NOALLOC_MAX_C)
    return fail(-1, "colsum_noalloc: width exceeds NFN_COLSUM_NOALLOC_MAX_C (8192); use nfn_colsum with caller scratch");
  int rc = 0;
  float* scratch = scratch_for_current_device(&rc);
  if (!scratch) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(ceil_div(C, 128), NA_ROW_SPLITS);
  na_colsum_partial_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(dy), ld, scratch, rows, C);
  na_colsum_final_kernel<<<ceil_div(C, 256), 256, 0, st>>>(scratch, static_cast<__nv_bfloat16*>(out),
                                                           NA_ROW_SPLITS, C, accumulate);
  return launch_check("colsum_noalloc", 2);
}
