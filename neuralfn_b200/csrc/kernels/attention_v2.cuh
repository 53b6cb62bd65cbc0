// Shared pieces of the pipelined flash-attention kernels (attention_fwd2.cu, attention_bwd2.cu).
//
// All three kernels (forward, dK/dV, dQ) have the same shape: four "math" warps own the 128 TMEM
// lanes (one thread per row of the 128-row accumulator tile), one warp issues tcgen05.mma and one
// issues the TMA loads. A math thread pulls its whole row of the score tile out of TMEM in one go
// and hands the TMEM columns back at once, so the tensor pipe computes the next score tile while
// the exponentials of this one run; two CTAs share an SM so that one CTA's exponentials also
// overlap the other's matrix products.
#pragma once
#include "common.h"
#include "sm100_ptx.cuh"

namespace nfn {

constexpr int AV2_MATH_WARPS = 4;
constexpr int AV2_MMA_WARP = 4;
constexpr int AV2_TMA_WARP = 5;
constexpr int AV2_THREADS = 6 * 32;

// Visibility of key position k for query position q under the mask options of a launch.
struct AttnMask {
  int T;
  int causal;   // 1: keys <= query
  int window;   // 0: unlimited; W: causal keys in (q-W, q]; bidirectional |q-k| < W
  const int* seq_ids;  // optional [B*T]: a key is visible only inside the query's own packed sequence
};

__device__ __forceinline__ bool attn_visible(const AttnMask& m, int q, int k) {
  if (k >= m.T) return false;
  if (m.causal) {
    if (k > q) return false;
    if (m.window > 0 && k <= q - m.window) return false;
  } else if (m.window > 0) {
    if (k <= q - m.window || k >= q + m.window) return false;
  }
  return true;
}

// Does a [q0, q0 + nq) x [k0, k0 + nk) block need per-element masking (any pair invisible)?
__device__ __forceinline__ bool attn_block_needs_mask(const AttnMask& m, int q0, int nq, int k0, int nk) {
  bool need = (k0 + nk > m.T) || (m.seq_ids != nullptr);
  if (m.causal) need |= (k0 + nk - 1 > q0);
  if (m.window > 0) {
    need |= (k0 <= q0 + nq - 1 - m.window);                    // lower window edge of the last query
    if (!m.causal) need |= (k0 + nk - 1 >= q0 + m.window);     // upper window edge of the first query
  }
  return need;
}

// Key range [k_lo, k_hi) that the queries [q0, q0 + nq) can see (sequence ids do not narrow it).
__device__ __forceinline__ void attn_key_range(const AttnMask& m, int q0, int nq, int& k_lo, int& k_hi) {
  k_lo = 0;
  k_hi = m.T;
  if (m.causal) {
    k_hi = min(m.T, q0 + nq);
    if (m.window > 0) k_lo = max(0, q0 - m.window + 1);
  } else if (m.window > 0) {
    k_lo = max(0, q0 - m.window + 1);
    k_hi = min(m.T, q0 + nq - 1 + m.window);
  }
}

// Query range [q_lo, q_hi) that can see any of the keys [k0, k0 + nk).
__device__ __forceinline__ void attn_query_range(const AttnMask& m, int k0, int nk, int& q_lo, int& q_hi) {
  q_lo = 0;
  q_hi = m.T;
  if (m.causal) {
    q_lo = k0;
    if (m.window > 0) q_hi = min(m.T, k0 + nk - 1 + m.window);
  } else if (m.window > 0) {
    q_lo = max(0, k0 - m.window + 1);
    q_hi = min(m.T, k0 + nk - 1 + m.window);
  }
}

// sm_100 packed / three-input fp32 arithmetic: one issue slot for two elements
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// (d0, d1) = (a0, a1) * b + c
__device__ __forceinline__ void fma2_bcast(float& d0, float& d1, float a0, float a1, float b, float c) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
// (d0, d1) += (a0, a1)
__device__ __forceinline__ void add2(float& d0, float& d1, float a0, float a1) {
  asm("{\n\t.reg .b64 ra, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rd, {%0, %1};\n\tadd.rn.f32x2 rd, rd, ra;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "+f"(d0), "+f"(d1)
      : "f"(a0), "f"(a1));
}
// (d0, d1) = (a0, a1) * (b0, b1)
__device__ __forceinline__ void mul2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmul.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}

// 32 consecutive fp32 TMEM columns of this thread's lane into a slice of a larger register array.
template <int N>
__device__ __forceinline__ void tmem_ld_row(uint32_t taddr, uint32_t (&dst)[N]) {
  static_assert(N % 32 == 0, "row length must be a multiple of 32 columns");
#pragma unroll
  for (int c = 0; c < N / 32; ++c)
    tmem_ld_32x32(taddr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&dst[c * 32]));
}

// 32 consecutive fp32 TMEM columns <- 32 registers
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16,"
      " %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
      "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// Row `r` of a K-major bf16 operand tile made of 64-element (128-byte, 128B-swizzled) panels of
// `rows` rows each: stores the 16 bytes holding elements [8 * chunk16, 8 * chunk16 + 8) of that row.
__device__ __forceinline__ void st_swizzled_row_chunk(uint8_t* tile, int rows, int r, int chunk16, const uint4& v) {
  const int panel = chunk16 >> 3, c = chunk16 & 7;
  *reinterpret_cast<uint4*>(tile + panel * (rows * 128) + r * 128 + ((c ^ (r & 7)) << 4)) = v;
}

}  // namespace nfn
