// Allocation-free column sum. This entry point has no counterpart in the reference
// implementation; it exists for callers of this library that are not allowed to
// allocate device memory (stream capture / graph replay, host frameworks that own all
// device memory and pass only inputs and outputs, latency-critical loops).
#pragma once
#include "nfn_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

// Largest supported width. The library holds 64 * this many floats (2 MiB) of scratch in
// device memory on every GPU that loads it, until the process exits.
#define NFN_COLSUM_NOALLOC_MAX_C 8192

// out[c] = sum_r dy[r, c]  (+ out[c] when accumulate != 0)
//   dy : bf16 [rows, C], row stride ld elements (ld >= C, both even); the address must be
//        4-byte aligned (the kernel reads two elements at a time), so a view that starts at
//        an odd element is refused before anything is launched
//   out: bf16 [C]
// rows <= 0 returns 0 without touching out, also when accumulate == 0 (nfn_colsum does the same).
// The device address of the scratch array is looked up once per device and kept; after a
// cudaDeviceReset() in the same process it is stale, so do not reset a device this library has used.
// Same result as nfn_colsum, but the partial sums live in a fixed array inside the
// library instead of caller-provided scratch. Returns 0, or a negative code with a
// message in nfn_last_error() (null operands, odd sizes, C > NFN_COLSUM_NOALLOC_MAX_C).
// Calls no cudaMalloc/cudaFree and no allocating library routine.
// The first call on a device resolves the array's device address; issue it before any
// stream capture on that device. Calls that overlap on the GPU share the array and
// race: keep them ordered on one stream.
int nfn_colsum_noalloc(const void* dy, int ld, void* out, int rows, int C, int accumulate,
                       nfn_stream_t stream);

#ifdef __cplusplus
}
#endif
