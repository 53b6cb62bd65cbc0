// Epilogue building blocks of the tcgen05 GEMM: activation math on 8-wide register
// groups (branches hoisted out of the element loops so only the selected activation
// is ever evaluated), TMA bulk stores out of a swizzled shared-memory staging tile,
// and the direct (bounds-checked) store path used for fp32 / accumulating outputs.
#pragma once
#include "common.h"
#include "sm100_ptx.cuh"

namespace nfn {

struct GemmParams {
  void* c;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* aux_in;
  __nv_bfloat16* aux_out;
  int m, n, k;
  int ldc, ld_aux_in, ld_aux_out;
  int flags;
  float alpha, act_param;
  int tiles_m, tiles_n;
  int split_k;        // >= 1; tile index space is tiles_m * tiles_n * split_k
  int kb_per_split;   // k-blocks handled by one split
  long long split_stride;  // elements between consecutive split slices of the fp32 workspace
  int* status;
  int raster_gw;      // tile order: bands of this many n-tiles, n fastest inside a band (1 = m fastest)
  // grouped contraction (weight gradients of MoE experts): split index g contracts rows [group_rows[g], group_rows[g + 1]) of
  // the K axis (multiples of BK; rows of a group's padding must be finite in both operands and zero in one) and writes slice
  // g of C (split_stride elements apart, bf16 or fp32). nullptr: the plain / split-K meaning of the fields above.
  const int* group_rows = nullptr;
};

// Tile index -> (m-tile, n-tile). CTAs that run at the same time hold consecutive indices, so a
// band of `raster_gw` n-tiles shares each A row panel while it is still in L2; with a band of 1
// the order is m-fastest and consecutive CTAs share the B tile instead.
__device__ __forceinline__ void tile_mn(const GemmParams& p, int t2, int& tm, int& tn) {
  if (p.raster_gw <= 1) {
    tm = t2 % p.tiles_m;
    tn = t2 / p.tiles_m;
    return;
  }
  const int band_tiles = p.raster_gw * p.tiles_m;
  const int band = t2 / band_tiles, r = t2 - band * band_tiles;
  const int n_first = band * p.raster_gw;
  const int w = min(p.raster_gw, p.tiles_n - n_first);
  tm = r / w;
  tn = n_first + r % w;
}

// Band width for a product with an [M, K] A operand and `tiles_n` column tiles: when A does not
// fit in L2 beside everything else, walk n first so that every A panel is fetched from HBM once.
inline int pick_raster_gw(long long m, long long k, int tiles_n) {
  const long long a_bytes = m * k * 2;
  if (tiles_n <= 1 || a_bytes <= (40ll << 20)) return 1;
  return tiles_n < 8 ? tiles_n : 8;
}

__device__ __forceinline__ void act8(float (&v)[8], int act, float prm) {
  if (act == NFN_ACT_GELU_TANH) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = gelu_tanh_f(v[j]);
  } else if (act == NFN_ACT_GELU_ERF) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = gelu_erf_f(v[j]);
  } else if (act == NFN_ACT_SILU) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = silu_f(v[j]);
  } else if (act == NFN_ACT_RELU2) {
#pragma unroll
    for (int j = 0; j < 8; ++j) { const float r = fmaxf(v[j], 0.f); v[j] = r * r; }
  } else if (act == NFN_ACT_RELU) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = fmaxf(v[j], 0.f);
  } else if (act == NFN_ACT_TANH_CAP) {
    const float inv = 1.f / prm;
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = prm * fast_tanh(v[j] * inv);
  }
}

// v[j] *= act'(pre[j])
__device__ __forceinline__ void dact8(float (&v)[8], const float (&pre)[8], int act, float prm) {
  if (act == NFN_ACT_GELU_TANH) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= dgelu_tanh_f(pre[j]);
  } else if (act == NFN_ACT_GELU_ERF) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= dgelu_erf_f(pre[j]);
  } else if (act == NFN_ACT_SILU) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= dsilu_f(pre[j]);
  } else if (act == NFN_ACT_RELU2) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= pre[j] > 0.f ? 2.f * pre[j] : 0.f;
  } else if (act == NFN_ACT_RELU) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = pre[j] > 0.f ? v[j] : 0.f;
  } else if (act == NFN_ACT_TANH_CAP) {
    const float inv = 1.f / prm;
#pragma unroll
    for (int j = 0; j < 8; ++j) { const float t = fast_tanh(pre[j] * inv); v[j] *= 1.f - t * t; }
  }
}

__device__ __forceinline__ void unpack8_bf16(const uint4& u, float (&f)[8]) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8_bf16(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// ---- TMA bulk store (shared -> global), bulk async-group completion ---------------
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t smem_src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(tmap), "r"(smem_src), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// one 32-byte store (a whole DRAM sector) of sixteen bf16 values; `addr` must be 32-byte aligned
__device__ __forceinline__ void st_global_v8(void* addr, const uint4& a, const uint4& b) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(addr), "r"(a.x), "r"(a.y), "r"(a.z),
               "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
               : "memory");
}
// internal epilogue flag (not part of the public ABI): bf16 outputs bypass the shared-memory
// staging tiles and TMA stores and go out as 32-byte stores straight from registers
constexpr int NFN_EPI_DIRECT_ST = 1 << 16;
// ---- specialised register epilogues ---------------------------------------------------------
// The generic epilogue tests every flag per 8-column group; with one row per thread and two
// warps per scheduler that is a long dependent instruction stream (about 16 instructions per
// element), long enough to outlast the main loop of a K = 768 tile. The combinations the
// trainers use are therefore compiled as straight-line code and selected once per launch.
enum : int {
  EPI_K_GENERIC = 0,
  EPI_K_PLAIN,           // C = acc
  EPI_K_BIAS,            // C = acc + bias
  EPI_K_BIAS_RESID,      // C = acc + bias + aux_in
  EPI_K_BIAS_GELU_SAVE,  // aux_out = acc + bias; C = gelu_tanh(aux_out)
  EPI_K_DGELU,           // C = acc * gelu_tanh'(aux_in)
  EPI_K_TANHCAP,         // C = cap * tanh(acc / cap)
  EPI_K_F32_PLAIN,       // fp32 C = acc (split-K partial slices)
};

__device__ __forceinline__ int epi_classify(const GemmParams& p) {
  if (p.alpha != 1.f) return EPI_K_GENERIC;
  const int act = (p.flags >> NFN_EPI_ACT_SHIFT) & 0xF;
  const int base = p.flags & 0x3F;
  if (act == NFN_ACT_NONE) {
    if (base == 0) return EPI_K_PLAIN;
    if (base == NFN_EPI_BIAS) return EPI_K_BIAS;
    if (base == (NFN_EPI_BIAS | NFN_EPI_RESID)) return EPI_K_BIAS_RESID;
    if (base == NFN_EPI_OUT_F32) return EPI_K_F32_PLAIN;
  } else if (act == NFN_ACT_GELU_TANH) {
    if (base == (NFN_EPI_BIAS | NFN_EPI_SAVE_PRE)) return EPI_K_BIAS_GELU_SAVE;
    if (base == NFN_EPI_DACT) return EPI_K_DGELU;
  } else if (act == NFN_ACT_TANH_CAP) {
    if (base == 0) return EPI_K_TANHCAP;
  }
  return EPI_K_GENERIC;
}

__device__ __forceinline__ void st_row32_bf16(__nv_bfloat16* cp, const uint4 (&o)[4], bool wide_st) {
  if (wide_st) {
    st_global_v8(cp, o[0], o[1]);
    st_global_v8(cp + 16, o[2], o[3]);
  } else {
#pragma unroll
    for (int g = 0; g < 4; ++g) *reinterpret_cast<uint4*>(cp + g * 8) = o[g];
  }
}

// One thread's 32 consecutive columns [nc, nc + 32) of row `row` (all inside the matrix).
// `taddr` addresses those columns of the thread's TMEM lane. The TMEM load is warp-collective,
// so every lane calls this; lanes with row_ok == false load and discard.
template <int KIND>
__device__ __forceinline__ void epi_chunk32(const GemmParams& p, uint32_t taddr, int row, bool row_ok, int nc, int sp,
                                            bool wide_st, bool wide_aux) {
  constexpr bool kBias = KIND == EPI_K_BIAS || KIND == EPI_K_BIAS_RESID || KIND == EPI_K_BIAS_GELU_SAVE;
  constexpr bool kAuxIn = KIND == EPI_K_BIAS_RESID || KIND == EPI_K_DGELU;
  uint4 aux[4], bias[4];
  if (kAuxIn && row_ok) {
    const uint4* ap = reinterpret_cast<const uint4*>(p.aux_in + (size_t)row * p.ld_aux_in + nc);
#pragma unroll
    for (int g = 0; g < 4; ++g) aux[g] = ap[g];
  }
  if (kBias) {
    const uint4* bp = reinterpret_cast<const uint4*>(p.bias + nc);
#pragma unroll
    for (int g = 0; g < 4; ++g) bias[g] = __ldg(bp + g);
  }
  uint32_t r[32];
  tmem_ld_32x32(taddr, r);
  tmem_ld_wait();
  if (!row_ok) return;
  if (KIND == EPI_K_F32_PLAIN) {
    float4* cp = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.c) + (size_t)sp * p.split_stride + (size_t)row * p.ldc + nc);
#pragma unroll
    for (int g = 0; g < 8; ++g)
      cp[g] = make_float4(__uint_as_float(r[4 * g]), __uint_as_float(r[4 * g + 1]), __uint_as_float(r[4 * g + 2]),
                          __uint_as_float(r[4 * g + 3]));
    return;
  }
  uint4 o[4], pre[4];
  const float cap = p.act_param, inv_cap = (KIND == EPI_K_TANHCAP) ? 1.f / p.act_param : 0.f;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[g * 8 + j]);
    if (kBias) {
      float b8[8];
      unpack8_bf16(bias[g], b8);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += b8[j];
    }
    if (KIND == EPI_K_BIAS_GELU_SAVE) {
      pre[g] = pack8_bf16(v);
#pragma unroll
      for (int j = 0; j < 8; j += 2) gelu_tanh_2(v[j], v[j + 1], v[j], v[j + 1]);
    }
    if (KIND == EPI_K_TANHCAP) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = cap * fast_tanh(v[j] * inv_cap);
    }
    if (kAuxIn) {
      float x8[8];
      unpack8_bf16(aux[g], x8);
      if (KIND == EPI_K_DGELU) {
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          float d0, d1;
          dgelu_tanh_2(d0, d1, x8[j], x8[j + 1]);
          mul2f(v[j], v[j + 1], v[j], v[j + 1], d0, d1);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] += x8[j];
      }
    }
    o[g] = pack8_bf16(v);
  }
  if (KIND == EPI_K_BIAS_GELU_SAVE) st_row32_bf16(p.aux_out + (size_t)row * p.ld_aux_out + nc, pre, wide_aux);
  st_row32_bf16(reinterpret_cast<__nv_bfloat16*>(p.c) + (size_t)row * p.ldc + nc, o, wide_st);
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Row r of a [128 x 64] bf16 staging tile with the 128-byte swizzle TMA expects:
// 16-byte chunk c of row r lives at chunk (c ^ (r & 7)).
__device__ __forceinline__ void stage_store8(uint8_t* tile, int r, int chunk, const uint4& v) {
  *reinterpret_cast<uint4*>(tile + r * 128 + ((chunk ^ (r & 7)) << 4)) = v;
}

}  // namespace nfn
