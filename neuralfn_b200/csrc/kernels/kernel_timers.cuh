// Optional per-role cycle counters for the warp-specialised kernels. Compiled in only with
// -DNFN_KERNEL_TIMERS (NFN_EXTRA_NVCC_FLAGS=-DNFN_KERNEL_TIMERS python -m neuralfn_b200.ops._build);
// otherwise every macro expands to nothing. One thread of a role accumulates clock64() laps into
// local counters and adds them to a per-translation-unit device array when it leaves the kernel;
// NFN_TIMER_EXPORT(name) defines `int name(unsigned long long* out32, int reset)` that copies the
// 32 counters to the host. Plays the role of the reference's device cycle counters
// (neuralfn/csrc/tile_cuda/kernels.cu:202-207).
#pragma once
#include <cuda_runtime.h>

#ifdef NFN_KERNEL_TIMERS
namespace nfn { static __device__ unsigned long long g_kernel_timers[32]; }
#define NFN_TIMER_DECL(n) long long nfn_t_[n] = {}; long long nfn_t_last_ = clock64();
#define NFN_TIMER_LAP(i) { const long long nfn_now_ = clock64(); nfn_t_[i] += nfn_now_ - nfn_t_last_; nfn_t_last_ = nfn_now_; }
#define NFN_TIMER_FLUSH(base, n) { for (int nfn_i_ = 0; nfn_i_ < (n); ++nfn_i_) atomicAdd(&nfn::g_kernel_timers[(base) + nfn_i_], (unsigned long long)nfn_t_[nfn_i_]); }
#define NFN_TIMER_EXPORT(name)                                                                          \
  extern "C" int name(unsigned long long* out32, int reset) {                                           \
    cudaDeviceSynchronize();                                                                            \
    int rc = (int)cudaMemcpyFromSymbol(out32, nfn::g_kernel_timers, sizeof(unsigned long long) * 32);   \
    if (reset) {                                                                                        \
      unsigned long long z[32] = {};                                                                    \
      rc |= (int)cudaMemcpyToSymbol(nfn::g_kernel_timers, z, sizeof(z));                                \
    }                                                                                                   \
    return rc;                                                                                          \
  }
#else
#define NFN_TIMER_DECL(n)
#define NFN_TIMER_LAP(i) {}
#define NFN_TIMER_FLUSH(base, n) {}
#define NFN_TIMER_EXPORT(name) extern "C" int name(unsigned long long*, int) { return -1; }
#endif
