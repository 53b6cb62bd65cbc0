// C ABI of the sm_100a kernel library (libnfn_b200_kernels.so).
//
// Every entry point takes raw device pointers plus the CUDA stream to launch on
// and returns 0 on success or a negative argument/launch error. Kernels never
// allocate; scratch is passed in by the caller. Waits inside kernels are bounded
// and report through a per-device status word (nfn_status_read_reset).
//
// Plays the role of the reference's dlopen kernel boundary
// (neuralfn/csrc/native_train/tile_ops.h), redesigned around tcgen05/TMA kernels.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* nfn_stream_t;

// ---- library / status -------------------------------------------------------
int nfn_abi_version(void);
// Returns the first non-zero error code recorded by any kernel on the current
// device since the last call (0 = none) and clears it. Synchronises the device.
int nfn_status_read_reset(void);
// Same, but does not synchronise (reads whatever has landed) and does not clear.
int nfn_status_peek(void);
const char* nfn_last_error(void);

// ---- GEMM family (tcgen05 + TMEM + TMA) -------------------------------------
// C[M,N] = epilogue( sum_k opA[m,k] * opB[n,k] )
//   a_mn = 0: A is stored [M,K] (K contiguous, leading dim lda)
//   a_mn = 1: A is stored [K,M] (M contiguous, leading dim lda)
//   b_mn = 0: B is stored [N,K] (K contiguous, leading dim ldb)
//   b_mn = 1: B is stored [K,N] (N contiguous, leading dim ldb)
// A, B are bf16. C is bf16 unless NFN_EPI_OUT_F32.
// Epilogue order: acc*alpha -> +bias[n] -> (save pre-activation to aux_out)
//   -> activation -> * act'(aux_in) (DACT) -> + aux_in (RESID) -> + C (ACCUM).
enum {
  NFN_EPI_BIAS = 1 << 0,      // add bf16 bias[N]
  NFN_EPI_SAVE_PRE = 1 << 1,  // write pre-activation to aux_out (bf16, ld = ld_aux_out)
  NFN_EPI_RESID = 1 << 2,     // add bf16 residual aux_in[M,N]
  NFN_EPI_DACT = 1 << 3,      // multiply by act'(aux_in[M,N]) (aux_in = saved pre-activation)
  NFN_EPI_ACCUM = 1 << 4,     // C += result
  NFN_EPI_OUT_F32 = 1 << 5,   // C is fp32
  NFN_EPI_ACT_SHIFT = 8,      // activation id in bits 8..11
};
enum { NFN_ACT_NONE = 0, NFN_ACT_GELU_TANH = 1, NFN_ACT_GELU_ERF = 2, NFN_ACT_SILU = 3,
       NFN_ACT_RELU2 = 4, NFN_ACT_TANH_CAP = 5 /* cap*tanh(x/cap), cap = act_param */ };

typedef struct {
  const void* a; const void* b; void* c;
  int m, n, k;
  int lda, ldb, ldc;
  int a_mn, b_mn;
  int flags;
  float alpha;
  float act_param;
  const void* bias;
  const void* aux_in; int ld_aux_in;
  void* aux_out; int ld_aux_out;
  // split-K (plain products only): 0 = choose automatically, 1 = never, n > 1 = force n.
  // Needs an fp32 workspace of split * M * N elements; without one no split happens.
  void* workspace; long long workspace_bytes; int split_k;
} nfn_gemm_args;

int nfn_gemm_bf16(const nfn_gemm_args* args, nfn_stream_t stream);

#ifdef __cplusplus
}
#endif
