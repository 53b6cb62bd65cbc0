// TurboQuant KV cache: encode kernel and decode attention over compressed records.
//
// A record holds one head vector: its norm and, per coordinate of the ROTATED unit vector, the
// index of the nearest Lloyd-Max centroid (2, 3 or 4 bits, packed as consecutive little-endian
// bit fields); key records of the QJL profile also carry the norm of the quantisation residual
// and one sign bit per coordinate of a Gaussian projection of that residual. Layout
//     [ norm f32 | residual_norm f32 (qjl) | sign bits D/8 bytes (qjl) | packed indices | pad to 16 ].
//
// Attention never rebuilds a K or V matrix. Per (sequence, kv head) the CTA rotates the G query
// vectors once (and projects them once for QJL); every warp then walks its share of the cached
// tokens: a record is 16-20 words, one per lane, bit fields are cut out of two neighbouring
// words fetched by shuffle, the score is <R q, centroids> * norm (+ the sign correction), the
// value's centroids are accumulated IN ROTATED SPACE under an online softmax, and the result is
// rotated back once at the end. HBM traffic per token and kv head is two records (128 bytes at
// head_dim 128 instead of 512 for bf16).
//
// Behavioural counterparts in the reference: the codec (neuralfn/turboquant.py:298-475), the
// CPU session cache (csrc/native_gpt2/resident_turboquant.h:24-150) and the tile kernel
// turboquant_attention_forward_v1 (resident_tile_turboquant.*).
#include <cuda_bf16.h>

#include <algorithm>

#include "common.h"
#include "nfn_kernels.h"

namespace nfn {

constexpr int TQ_MAX_D = 128;
constexpr int TQ_MAX_G = 8;
constexpr int TQ_WARPS = 8;

struct TqTables {
  const float* rotation;    // [D, D], rotated = R x
  const float* projection;  // [D, D] (qjl)
  const float* centroids;   // [5][16]: row = bit width
  const int* key_fields;    // [D][2]: bit offset inside the index area, width
  const int* value_fields;
  int D, qjl, key_rec_bytes, value_rec_bytes;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Bit field [bit, bit + width) of a record whose word w sits in lane w of `word`.
__device__ __forceinline__ uint32_t record_field(uint32_t word, int bit, int width) {
  const uint32_t lo = __shfl_sync(0xffffffffu, word, bit >> 5);
  const uint32_t hi = __shfl_sync(0xffffffffu, word, ((bit >> 5) + 1) & 31);
  return __funnelshift_r(lo, hi, bit & 31) & ((1u << width) - 1u);
}

// ------------------------------------------------------------------------------------ encode
struct TqEncodeParams {
  TqTables t;
  const __nv_bfloat16* x;
  long long ld;
  const int* seq;   // [rows] destination sequence
  const int* slot;  // [rows] destination row inside the head's cache
  int rows, H, cap, is_key;
  uint8_t* out;     // [B][H][cap][rec_bytes]
};

__global__ void __launch_bounds__(128) tq_encode_kernel(const TqEncodeParams p) {
  __shared__ float s_vec[4][TQ_MAX_D];    // unit vector, later the residual
  __shared__ float s_q[4][TQ_MAX_D];      // quantised rotated coordinates
  __shared__ uint32_t s_rec[4][32];
  __shared__ float s_cent[5 * 16];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int D = p.t.D, KD = D / 32;
  for (int i = threadIdx.x; i < 80; i += blockDim.x) s_cent[i] = p.t.centroids[i];
  __syncthreads();
  const long long vec = (long long)blockIdx.x * 4 + warp;
  if (vec >= (long long)p.rows * p.H) return;
  const int row = (int)(vec / p.H), h = (int)(vec % p.H);
  if (p.slot[row] < 0 || p.slot[row] >= p.cap || p.seq[row] < 0) return;  // rows without a destination (idle sequences) are skipped
  const bool qjl = p.is_key && p.t.qjl;
  const int rec_bytes = p.is_key ? p.t.key_rec_bytes : p.t.value_rec_bytes;
  const int* fields = p.is_key ? p.t.key_fields : p.t.value_fields;
  const int index_bit0 = (qjl ? 8 + D / 8 : 4) * 8;

  float x[4], ss = 0.f;
  const __nv_bfloat16* src = p.x + (long long)row * p.ld + (long long)h * D;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    x[k] = k < KD ? __bfloat162float(src[lane + 32 * k]) : 0.f;
    ss += x[k] * x[k];
  }
  const float norm = sqrtf(warp_sum(ss));
  const float inv = norm > 0.f ? 1.f / norm : 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k)
    if (k < KD) s_vec[warp][lane + 32 * k] = x[k] * inv;
  s_rec[warp][lane] = 0u;
  __syncwarp();

  // rotate, pick the nearest centroid, pack
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (k >= KD) break;
    const int i = lane + 32 * k;
    const float* Ri = p.t.rotation + (size_t)i * D;
    float r = 0.f;
    for (int j = 0; j < D; ++j) r += Ri[j] * s_vec[warp][j];
    const int bit = fields[2 * i], width = fields[2 * i + 1];
    const float* cb = s_cent + width * 16;
    int best = 0;
    float bd = fabsf(r - cb[0]);
    for (int c = 1; c < (1 << width); ++c) {
      const float d = fabsf(r - cb[c]);
      if (d < bd) { bd = d; best = c; }
    }
    s_q[warp][i] = cb[best];
    const int abs_bit = index_bit0 + bit;
    atomicOr(&s_rec[warp][abs_bit >> 5], (uint32_t)best << (abs_bit & 31));
    if ((abs_bit & 31) + width > 32) atomicOr(&s_rec[warp][(abs_bit >> 5) + 1], (uint32_t)best >> (32 - (abs_bit & 31)));
  }
  __syncwarp();
  float rnorm = 0.f;
  if (qjl) {
    // residual = unit - R^T q ; signs of S residual
    float res[4], rs = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      res[k] = 0.f;
      if (k >= KD) continue;
      const int j = lane + 32 * k;
      float m = 0.f;
      for (int i = 0; i < D; ++i) m += p.t.rotation[(size_t)i * D + j] * s_q[warp][i];
      res[k] = s_vec[warp][j] - m;
      rs += res[k] * res[k];
    }
    rnorm = sqrtf(warp_sum(rs));
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (k < KD) s_vec[warp][lane + 32 * k] = res[k];
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (k >= KD) break;
      const int i = lane + 32 * k;
      const float* Si = p.t.projection + (size_t)i * D;
      float pr = 0.f;
      for (int j = 0; j < D; ++j) pr += Si[j] * s_vec[warp][j];
      const uint32_t bits = __ballot_sync(0xffffffffu, pr >= 0.f);
      if (lane == 0) s_rec[warp][2 + k] = bits;  // sign of coordinate 32 k + lane is bit `lane` of word 2 + k
    }
  }
  if (lane == 0) {
    s_rec[warp][0] = __float_as_uint(norm);
    if (qjl) s_rec[warp][1] = __float_as_uint(rnorm);
  }
  __syncwarp();
  uint32_t* dst = reinterpret_cast<uint32_t*>(p.out + (((size_t)p.seq[row] * p.H + h) * p.cap + p.slot[row]) * rec_bytes);
  if (lane < rec_bytes / 4) dst[lane] = s_rec[warp][lane];
}

// --------------------------------------------------------------------------------- attention
struct TqAttnParams {
  TqTables t;
  const __nv_bfloat16* q;
  int ld_q;
  const uint8_t* krec;
  const uint8_t* vrec;
  const int* lengths;
  __nv_bfloat16* out;
  int ld_o;
  int B, Hq, Hkv, cap;
  float scale;
};

template <int KD>  // head_dim / 32
__global__ void __launch_bounds__(TQ_WARPS * 32) tq_attention_kernel(const TqAttnParams p) {
  constexpr int D = KD * 32;
  extern __shared__ float tq_smem[];
  const int G = p.Hq / p.Hkv;
  float* s_q = tq_smem;                 // [G][D] query, later the merged rotated output
  float* s_qr = s_q + TQ_MAX_G * D;     // [G][D] rotated query
  float* s_qp = s_qr + TQ_MAX_G * D;    // [G][D] projected query (qjl)
  float* s_cent = s_qp + TQ_MAX_G * D;  // [80]
  int* s_kf = reinterpret_cast<int*>(s_cent + 80);  // [D][2]
  int* s_vf = s_kf + 2 * D;
  float* s_m = reinterpret_cast<float*>(s_vf + 2 * D);  // [WARPS][G]
  float* s_l = s_m + TQ_WARPS * TQ_MAX_G;
  float* s_acc = s_l + TQ_WARPS * TQ_MAX_G;             // [WARPS][G][D]

  const int hk = blockIdx.x, b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int len = min(p.lengths[b], p.cap);
  const bool qjl = p.t.qjl != 0;

  for (int i = threadIdx.x; i < 80; i += blockDim.x) s_cent[i] = p.t.centroids[i];
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) {
    s_kf[i] = p.t.key_fields[i];
    s_vf[i] = p.t.value_fields[i];
  }
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    s_q[i] = __bfloat162float(p.q[(size_t)b * p.ld_q + (size_t)(hk * G + g) * D + d]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, r = i % D;
    const float* Rr = p.t.rotation + (size_t)r * D;
    float a = 0.f, c = 0.f;
    for (int j = 0; j < D; ++j) a += Rr[j] * s_q[g * D + j];
    s_qr[i] = a;
    if (qjl) {
      const float* Sr = p.t.projection + (size_t)r * D;
      for (int j = 0; j < D; ++j) c += Sr[j] * s_q[g * D + j];
      s_qp[i] = c;
    }
  }
  __syncthreads();

  const int kwords = p.t.key_rec_bytes / 4, vwords = p.t.value_rec_bytes / 4;
  const int kbit0 = (qjl ? 8 + D / 8 : 4) * 8, vbit0 = 32;
  const float corr_k = 1.2533141373155001f / D;  // sqrt(pi / 2) / D
  float m_run[TQ_MAX_G], l_run[TQ_MAX_G], acc[TQ_MAX_G][KD];
#pragma unroll
  for (int g = 0; g < TQ_MAX_G; ++g) {
    m_run[g] = -INFINITY;
    l_run[g] = 0.f;
#pragma unroll
    for (int k = 0; k < KD; ++k) acc[g][k] = 0.f;
  }
  const uint8_t* kbase = p.krec + ((size_t)b * p.Hkv + hk) * p.cap * p.t.key_rec_bytes;
  const uint8_t* vbase = p.vrec + ((size_t)b * p.Hkv + hk) * p.cap * p.t.value_rec_bytes;

  for (int t = warp; t < len; t += TQ_WARPS) {
    const uint32_t kw = lane < kwords ? reinterpret_cast<const uint32_t*>(kbase + (size_t)t * p.t.key_rec_bytes)[lane] : 0u;
    const uint32_t vw = lane < vwords ? reinterpret_cast<const uint32_t*>(vbase + (size_t)t * p.t.value_rec_bytes)[lane] : 0u;
    const float knorm = __uint_as_float(__shfl_sync(0xffffffffu, kw, 0));
    const float rnorm = qjl ? __uint_as_float(__shfl_sync(0xffffffffu, kw, 1)) : 0.f;
    const float vnorm = __uint_as_float(__shfl_sync(0xffffffffu, vw, 0));
    float kc[KD], vc[KD], sg[KD];
#pragma unroll
    for (int k = 0; k < KD; ++k) {
      const int c = lane + 32 * k;
      const int kwid = s_kf[2 * c + 1], vwid = s_vf[2 * c + 1];
      kc[k] = s_cent[kwid * 16 + record_field(kw, kbit0 + s_kf[2 * c], kwid)];
      vc[k] = s_cent[vwid * 16 + record_field(vw, vbit0 + s_vf[2 * c], vwid)] * vnorm;
      sg[k] = 0.f;
      if (qjl) sg[k] = ((__shfl_sync(0xffffffffu, kw, 2 + k) >> lane) & 1u) ? 1.f : -1.f;
    }
#pragma unroll
    for (int g = 0; g < TQ_MAX_G; ++g) {
      if (g >= G) break;
      float base = 0.f, corr = 0.f;
#pragma unroll
      for (int k = 0; k < KD; ++k) {
        base += s_qr[g * D + lane + 32 * k] * kc[k];
        if (qjl) corr += s_qp[g * D + lane + 32 * k] * sg[k];
      }
      base = warp_sum(base);
      if (qjl) base += corr_k * rnorm * warp_sum(corr);
      const float s = knorm * base * p.scale;
      const float m_new = fmaxf(m_run[g], s);
      const float alpha = __expf(m_run[g] - m_new);  // first token: exp(-inf) = 0
      const float pw = __expf(s - m_new);
      l_run[g] = l_run[g] * alpha + pw;
      m_run[g] = m_new;
#pragma unroll
      for (int k = 0; k < KD; ++k) acc[g][k] = acc[g][k] * alpha + pw * vc[k];
    }
  }
  // merge the warps
#pragma unroll
  for (int g = 0; g < TQ_MAX_G; ++g) {
    if (g >= G) break;
    if (lane == 0) {
      s_m[warp * TQ_MAX_G + g] = m_run[g];
      s_l[warp * TQ_MAX_G + g] = l_run[g];
    }
#pragma unroll
    for (int k = 0; k < KD; ++k) s_acc[((size_t)warp * TQ_MAX_G + g) * D + lane + 32 * k] = acc[g][k];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    float M = -INFINITY;
    for (int w = 0; w < TQ_WARPS; ++w) M = fmaxf(M, s_m[w * TQ_MAX_G + g]);
    float L = 0.f, o = 0.f;
    if (M > -INFINITY) {
      for (int w = 0; w < TQ_WARPS; ++w) {
        const float e = __expf(s_m[w * TQ_MAX_G + g] - M);
        L += e * s_l[w * TQ_MAX_G + g];
        o += e * s_acc[((size_t)w * TQ_MAX_G + g) * D + d];
      }
    }
    s_q[i] = L > 0.f ? o / L : 0.f;  // rotated-space output
  }
  __syncthreads();
  // rotate back: out[d] = sum_i R[i][d] o_rot[i]
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    float a = 0.f;
    for (int r = 0; r < D; ++r) a += p.t.rotation[(size_t)r * D + d] * s_q[g * D + r];
    p.out[(size_t)b * p.ld_o + (size_t)(hk * G + g) * D + d] = __float2bfloat16(a);
  }
}

static bool tables_ok(const nfn_tq_tables* t) {
  return t && t->rotation && t->centroids && t->key_fields && t->value_fields && (t->D == 64 || t->D == 128) &&
         (!t->qjl || t->projection) && t->key_rec_bytes > 0 && t->key_rec_bytes <= 128 && t->key_rec_bytes % 16 == 0 &&
         t->value_rec_bytes > 0 && t->value_rec_bytes <= 128 && t->value_rec_bytes % 16 == 0;
}

static TqTables to_tables(const nfn_tq_tables* t) {
  return TqTables{t->rotation, t->projection, t->centroids, t->key_fields, t->value_fields, t->D, t->qjl, t->key_rec_bytes, t->value_rec_bytes};
}

}  // namespace nfn

using namespace nfn;

extern "C" int nfn_turboquant_encode(const nfn_tq_tables* tables, const void* x, long long ld, const int* seq, const int* slot, int rows,
                                     int n_heads, int cap, int is_key, void* records, nfn_stream_t stream) {
  if (rows <= 0) return 0;
  if (!tables_ok(tables) || !x || !seq || !slot || !records || n_heads <= 0 || cap <= 0) return fail(-1, "turboquant_encode: bad arguments");
  TqEncodeParams p{to_tables(tables), static_cast<const __nv_bfloat16*>(x), ld, seq, slot, rows, n_heads, cap, is_key, static_cast<uint8_t*>(records)};
  const long long vecs = (long long)rows * n_heads;
  tq_encode_kernel<<<(unsigned)((vecs + 3) / 4), 128, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return launch_check("turboquant_encode");
}

extern "C" int nfn_turboquant_attention(const nfn_tq_tables* tables, const void* q, int ld_q, const void* k_records, const void* v_records,
                                        const int* lengths, void* out, int ld_o, int B, int n_q_heads, int n_kv_heads, int cap, float scale,
                                        nfn_stream_t stream) {
  if (B <= 0) return 0;
  if (!tables_ok(tables) || !q || !k_records || !v_records || !lengths || !out) return fail(-1, "turboquant_attention: bad arguments");
  if (n_kv_heads <= 0 || n_q_heads % n_kv_heads || n_q_heads / n_kv_heads > TQ_MAX_G) return fail(-1, "turboquant_attention: at most 8 query heads per kv head");
  TqAttnParams p{to_tables(tables), static_cast<const __nv_bfloat16*>(q), ld_q, static_cast<const uint8_t*>(k_records),
                 static_cast<const uint8_t*>(v_records), lengths, static_cast<__nv_bfloat16*>(out), ld_o, B, n_q_heads, n_kv_heads, cap, scale};
  const int D = tables->D;
  const size_t smem = (size_t)(3 * TQ_MAX_G * D + 80 + 4 * D + 2 * TQ_WARPS * TQ_MAX_G + TQ_WARPS * TQ_MAX_G * D) * 4;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(n_kv_heads, B);
  if (D == 128) {
    static bool attr[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr[dev & 63]) {
      if (cudaFuncSetAttribute(tq_attention_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return launch_check("turboquant attr", 0);
      attr[dev & 63] = true;
    }
    tq_attention_kernel<4><<<grid, TQ_WARPS * 32, smem, st>>>(p);
  } else {
    static bool attr[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr[dev & 63]) {
      if (cudaFuncSetAttribute(tq_attention_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return launch_check("turboquant attr", 0);
      attr[dev & 63] = true;
    }
    tq_attention_kernel<2><<<grid, TQ_WARPS * 32, smem, st>>>(p);
  }
  return launch_check("turboquant_attention");
}
