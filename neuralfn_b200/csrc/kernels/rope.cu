// Rotary position embedding on the q and k head groups of packed QKV rows, in place.
//
// Pairing is the split-half one used by both of the reference's conventions
// (torch_backend.py:323-340): element i of the first half rotates with element i + half.
//   sign = -1  "legacy":  (x1 cos + x2 sin, -x1 sin + x2 cos)
//   sign = +1  "hf":      (x1 cos - x2 sin,  x2 cos + x1 sin)
// The backward of either is the same kernel with the opposite sign (rotations are
// orthogonal), so there is no separate backward entry point.
// cos/sin come from fp32 tables [max_pos, rot_dim/2] built on the host side, so every
// frequency-scaling rule (linear, NTK, YaRN, llama3) is a table, not a kernel variant.
//
// nfn_qk_norm_rope_forward fuses the per-head RMS norm (optional bf16 weights), the
// rotation and the query scale into one pass: one warp per (token, head).
#include "common.h"
#include "nfn_kernels.h"
#include "sm100_ptx.cuh"

namespace nfn {

// one thread: 2 low + 2 high elements of one head
__global__ void __launch_bounds__(256)
rope_inplace_kernel(__nv_bfloat16* __restrict__ qkv, int ld, long long n_items, int T, int heads, int hd, int rot_dim,
                    const float* __restrict__ cosT, const float* __restrict__ sinT, const int* __restrict__ positions,
                    int max_pos, float sign, float q_scale, int n_q_heads) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_items) return;
  const int half = rot_dim >> 1, per_head = half >> 1;
  const int j = (int)(idx % per_head);
  const long long th = idx / per_head;
  const int head = (int)(th % heads);
  const long long tok = th / heads;
  int pos = positions ? positions[tok] : (int)(tok % T);
  pos = min(max(pos, 0), max_pos - 1);
  __nv_bfloat16* base = qkv + tok * (long long)ld + (long long)head * hd;
  const float2 c = *reinterpret_cast<const float2*>(cosT + (long long)pos * half + 2 * j);
  const float2 s = *reinterpret_cast<const float2*>(sinT + (long long)pos * half + 2 * j);
  const float2 lo = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(base + 2 * j));
  const float2 hi = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(base + half + 2 * j));
  const float sc = head < n_q_heads ? q_scale : 1.f;
  float2 olo, ohi;
  olo.x = (lo.x * c.x - sign * hi.x * s.x) * sc;
  olo.y = (lo.y * c.y - sign * hi.y * s.y) * sc;
  ohi.x = (hi.x * c.x + sign * lo.x * s.x) * sc;
  ohi.y = (hi.y * c.y + sign * lo.y * s.y) * sc;
  *reinterpret_cast<uint32_t*>(base + 2 * j) = pack_bf16x2(olo.x, olo.y);
  *reinterpret_cast<uint32_t*>(base + half + 2 * j) = pack_bf16x2(ohi.x, ohi.y);
}

// one warp per (token, head); hd in {64, 128}; lane l owns low pair 2l and high pair half+2l
__global__ void __launch_bounds__(256)
qk_norm_rope_kernel(__nv_bfloat16* __restrict__ qkv, int ld, long long n_rows, int T, int heads, int hd,
                    const __nv_bfloat16* __restrict__ q_weight, const __nv_bfloat16* __restrict__ k_weight,
                    const float* __restrict__ cosT, const float* __restrict__ sinT, const int* __restrict__ positions,
                    int max_pos, float sign, float eps, float q_scale, int n_q_heads, float* __restrict__ rstd_out) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int lane = threadIdx.x & 31, half = hd >> 1, per_head = half >> 1;
  const int head = (int)(row % heads);
  const long long tok = row / heads;
  const bool live = lane < per_head;
  __nv_bfloat16* base = qkv + tok * (long long)ld + (long long)head * hd;
  float2 lo = make_float2(0.f, 0.f), hi = lo;
  if (live) {
    lo = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(base + 2 * lane));
    hi = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(base + half + 2 * lane));
  }
  float ss = lo.x * lo.x + lo.y * lo.y + hi.x * hi.x + hi.y * hi.y;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float rstd = rsqrtf(ss / (float)hd + eps);
  if (lane == 0 && rstd_out) rstd_out[row] = rstd;
  if (!live) return;
  const __nv_bfloat16* w = head < n_q_heads ? q_weight : k_weight;
  float2 wlo = make_float2(1.f, 1.f), whi = wlo;
  if (w) {
    wlo = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(w + 2 * lane));
    whi = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(w + half + 2 * lane));
  }
  lo.x *= rstd * wlo.x; lo.y *= rstd * wlo.y; hi.x *= rstd * whi.x; hi.y *= rstd * whi.y;
  int pos = positions ? positions[tok] : (int)(tok % T);
  pos = min(max(pos, 0), max_pos - 1);
  const float2 c = *reinterpret_cast<const float2*>(cosT + (long long)pos * half + 2 * lane);
  const float2 s = *reinterpret_cast<const float2*>(sinT + (long long)pos * half + 2 * lane);
  const float sc = head < n_q_heads ? q_scale : 1.f;
  *reinterpret_cast<uint32_t*>(base + 2 * lane) =
      pack_bf16x2((lo.x * c.x - sign * hi.x * s.x) * sc, (lo.y * c.y - sign * hi.y * s.y) * sc);
  *reinterpret_cast<uint32_t*>(base + half + 2 * lane) =
      pack_bf16x2((hi.x * c.x + sign * lo.x * s.x) * sc, (hi.y * c.y + sign * lo.y * s.y) * sc);
}

static int check_common(const void* qkv, int ld, long long tokens, int T, int hq, int hkv, int hd, int rot_dim, const void* c,
                        const void* s, int max_pos, float sign) {
  if (!qkv || !c || !s) return fail(-1, "rope: null operand");
  if (tokens <= 0 || T <= 0 || hq < 0 || hkv < 0 || hq + hkv <= 0 || max_pos <= 0) return fail(-1, "rope: bad sizes");
  if (hd % 4 || rot_dim % 4 || rot_dim <= 0 || rot_dim > hd) return fail(-1, "rope: head_dim and rot_dim must be multiples of 4, rot_dim <= head_dim");
  if (ld % 2 || ld < (hq + hkv) * hd) return fail(-1, "rope: row stride must be even and cover the q and k heads");
  if (sign != 1.f && sign != -1.f) return fail(-1, "rope: sign must be +1 (hf) or -1 (legacy)");
  return 0;
}

}  // namespace nfn

using namespace nfn;

extern "C" int nfn_rope_inplace(void* qkv, int ld, long long tokens, int T, int n_q_heads, int n_kv_heads, int head_dim,
                                int rot_dim, const float* cos_table, const float* sin_table, const int* positions,
                                int max_pos, float sign, float q_scale, nfn_stream_t stream) {
  if (int rc = check_common(qkv, ld, tokens, T, n_q_heads, n_kv_heads, head_dim, rot_dim, cos_table, sin_table, max_pos, sign)) return rc;
  if (q_scale != 1.f && rot_dim != head_dim) return fail(-1, "rope: q_scale needs rot_dim == head_dim");
  const int heads = n_q_heads + n_kv_heads;
  const long long items = tokens * heads * (rot_dim / 4);
  const long long blocks = (items + 255) / 256;
  if (blocks > 0x7fffffffLL) return fail(-1, "rope: too many elements for one launch");
  rope_inplace_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(qkv), ld, items, T, heads, head_dim, rot_dim, cos_table, sin_table, positions, max_pos, sign,
      q_scale, n_q_heads);
  return launch_check("rope_inplace", 1);
}

extern "C" int nfn_qk_norm_rope_forward(void* qkv, int ld, long long tokens, int T, int n_q_heads, int n_kv_heads, int head_dim,
                                        const void* q_weight, const void* k_weight, const float* cos_table,
                                        const float* sin_table, const int* positions, int max_pos, float sign, float eps,
                                        float q_scale, float* rstd_out, nfn_stream_t stream) {
  if (int rc = check_common(qkv, ld, tokens, T, n_q_heads, n_kv_heads, head_dim, head_dim, cos_table, sin_table, max_pos, sign)) return rc;
  if (head_dim != 64 && head_dim != 128) return fail(-1, "qk_norm_rope: head_dim must be 64 or 128");
  const long long rows = tokens * (n_q_heads + n_kv_heads);
  const long long blocks = (rows + 7) / 8;
  if (blocks > 0x7fffffffLL) return fail(-1, "qk_norm_rope: too many rows for one launch");
  qk_norm_rope_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(qkv), ld, rows, T, n_q_heads + n_kv_heads, head_dim,
      static_cast<const __nv_bfloat16*>(q_weight), static_cast<const __nv_bfloat16*>(k_weight), cos_table, sin_table, positions,
      max_pos, sign, eps, q_scale, n_q_heads, rstd_out);
  return launch_check("qk_norm_rope_forward", 1);
}
