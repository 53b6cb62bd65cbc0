// Host-side helpers shared by every translation unit of the kernel library.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "nfn_kernels.h"

namespace nfn {

// Device pointer to the per-device status word kernels write error codes into.
int* status_ptr();
int sm_count();
int max_smem_optin();

void set_last_error(const char* msg);
int fail(int code, const char* msg);

// Cached TMA descriptors. `inner` is the contiguous dimension. Strides in elements.
bool make_tmap_2d(CUtensorMap* out, const void* ptr, int elem_size, uint64_t inner,
                  uint64_t outer, uint64_t ld_elems, uint32_t box_inner, uint32_t box_outer,
                  int swizzle_bytes);
bool make_tmap_3d(CUtensorMap* out, const void* ptr, int elem_size, uint64_t d0, uint64_t d1,
                  uint64_t d2, uint64_t stride1_elems, uint64_t stride2_elems, uint32_t b0,
                  uint32_t b1, uint32_t b2, int swizzle_bytes);

// Number of kernels this library has launched in this process (host-side count).
void count_launches(int n);
long long launches();

// Checks the launch(es) just issued; `n_kernels` of them are added to the launch count.
inline int launch_check(const char* what, int n_kernels = 1) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error(cudaGetErrorString(e));
    (void)what;
    return -100 - static_cast<int>(e);
  }
  count_launches(n_kernels);
  return 0;
}

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

}  // namespace nfn
