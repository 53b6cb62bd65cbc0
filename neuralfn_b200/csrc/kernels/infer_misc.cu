// Small memory-bound pieces of the inference and Llama-style training paths:
//   * SwiGLU on a fused [rows, 2I] gate|up projection, forward and backward;
//   * token (+ learned position) embedding with an explicit position per row, for decode
//     batches where every sequence is at a different position;
//   * prefill -> KV-cache scatter: the k and v heads of packed QKV rows go to their cache
//     slots ((pos0 + t) % cap, so ring caches of local-attention layers work too).
#include "common.h"
#include "nfn_kernels.h"
#include "sm100_ptx.cuh"

namespace nfn {

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]); u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, int ld, __nv_bfloat16* __restrict__ out, int ld_out, long long rows, int I) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int vecs = I / 8;
  if (idx >= rows * vecs) return;
  const long long r = idx / vecs;
  const int c = (int)(idx % vecs) * 8;
  float g[8], u[8], o[8];
  unpack8(*reinterpret_cast<const uint4*>(gu + r * ld + c), g);
  unpack8(*reinterpret_cast<const uint4*>(gu + r * ld + I + c), u);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = silu_f(g[j]) * u[j];
  *reinterpret_cast<uint4*>(out + r * ld_out + c) = pack8(o);
}

// dgu = [dout * u * silu'(g) | dout * silu(g)]
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, int ld, const __nv_bfloat16* __restrict__ dout, int ld_dout,
                  __nv_bfloat16* __restrict__ dgu, int ld_dgu, long long rows, int I) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int vecs = I / 8;
  if (idx >= rows * vecs) return;
  const long long r = idx / vecs;
  const int c = (int)(idx % vecs) * 8;
  float g[8], u[8], d[8], dg[8], du[8];
  unpack8(*reinterpret_cast<const uint4*>(gu + r * ld + c), g);
  unpack8(*reinterpret_cast<const uint4*>(gu + r * ld + I + c), u);
  unpack8(*reinterpret_cast<const uint4*>(dout + r * ld_dout + c), d);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    dg[j] = d[j] * u[j] * dsilu_f(g[j]);
    du[j] = d[j] * silu_f(g[j]);
  }
  *reinterpret_cast<uint4*>(dgu + r * ld_dgu + c) = pack8(dg);
  *reinterpret_cast<uint4*>(dgu + r * ld_dgu + I + c) = pack8(du);
}

__global__ void __launch_bounds__(256)
embedding_pos_kernel(const int* __restrict__ tokens, const int* __restrict__ positions, const __nv_bfloat16* __restrict__ wte,
                     const __nv_bfloat16* __restrict__ wpe, __nv_bfloat16* __restrict__ out, int n, int C, int vocab, int max_pos,
                     float scale) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int vecs = C / 8;
  if (idx >= (long long)n * vecs) return;
  const int r = (int)(idx / vecs), c = (int)(idx % vecs) * 8;
  const int tok = min(max(tokens[r], 0), vocab - 1);
  float e[8];
  unpack8(*reinterpret_cast<const uint4*>(wte + (long long)tok * C + c), e);
  if (wpe) {
    const int pos = min(max(positions[r], 0), max_pos - 1);
    float p[8];
    unpack8(*reinterpret_cast<const uint4*>(wpe + (long long)pos * C + c), p);
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] += p[j];
  }
  if (scale != 1.f) {
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] *= scale;
  }
  *reinterpret_cast<uint4*>(out + (long long)r * C + c) = pack8(e);
}

// rows t in [t_first, n): k/v heads of row t -> cache slot (pos0 + t) % cap
__global__ void __launch_bounds__(256)
kv_cache_write_kernel(const __nv_bfloat16* __restrict__ qkv, int ld, __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc,
                      int n, int t_first, int Hq, int Hkv, int hd, int cap, int pos0) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int vecs = hd / 8;
  const long long total = (long long)(n - t_first) * Hkv * vecs;
  if (idx >= total) return;
  const int c = (int)(idx % vecs) * 8;
  const int h = (int)((idx / vecs) % Hkv);
  const int t = t_first + (int)(idx / ((long long)vecs * Hkv));
  const int slot = (pos0 + t) % cap;
  const __nv_bfloat16* row = qkv + (long long)t * ld;
  const long long dst = ((long long)h * cap + slot) * hd + c;
  *reinterpret_cast<uint4*>(kc + dst) = *reinterpret_cast<const uint4*>(row + (long long)(Hq + h) * hd + c);
  *reinterpret_cast<uint4*>(vc + dst) = *reinterpret_cast<const uint4*>(row + (long long)(Hq + Hkv + h) * hd + c);
}

}  // namespace nfn

using namespace nfn;

extern "C" int nfn_swiglu_forward(const void* gate_up, int ld, void* out, int ld_out, long long rows, int inter, nfn_stream_t stream) {
  if (rows <= 0) return 0;
  if (!gate_up || !out || inter <= 0 || (inter & 7) || (ld & 7) || (ld_out & 7) || ld < 2 * inter || ld_out < inter)
    return fail(-1, "swiglu_forward: bad arguments (sizes and strides must be multiples of 8)");
  const long long total = rows * (inter / 8), grid = (total + 255) / 256;
  if (grid > 0x7fffffffLL) return fail(-1, "swiglu_forward: too large for one launch");
  swiglu_fwd_kernel<<<(unsigned)grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate_up), ld, static_cast<__nv_bfloat16*>(out), ld_out, rows, inter);
  return launch_check("swiglu_forward", 1);
}

extern "C" int nfn_swiglu_backward(const void* gate_up, int ld, const void* dout, int ld_dout, void* dgate_up, int ld_dgu,
                                   long long rows, int inter, nfn_stream_t stream) {
  if (rows <= 0) return 0;
  if (!gate_up || !dout || !dgate_up || inter <= 0 || (inter & 7) || (ld & 7) || (ld_dout & 7) || (ld_dgu & 7) ||
      ld < 2 * inter || ld_dgu < 2 * inter || ld_dout < inter)
    return fail(-1, "swiglu_backward: bad arguments (sizes and strides must be multiples of 8)");
  const long long total = rows * (inter / 8), grid = (total + 255) / 256;
  if (grid > 0x7fffffffLL) return fail(-1, "swiglu_backward: too large for one launch");
  swiglu_bwd_kernel<<<(unsigned)grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate_up), ld, static_cast<const __nv_bfloat16*>(dout), ld_dout,
      static_cast<__nv_bfloat16*>(dgate_up), ld_dgu, rows, inter);
  return launch_check("swiglu_backward", 1);
}

extern "C" int nfn_embedding_positions(const int* tokens, const int* positions, const void* wte, const void* wpe, void* out, int n,
                                       int C, int vocab, int max_pos, float scale, nfn_stream_t stream) {
  if (n <= 0) return 0;
  if (!tokens || !wte || !out || (wpe && !positions) || C <= 0 || (C & 7) || vocab <= 0) return fail(-1, "embedding_positions: bad arguments");
  const long long total = (long long)n * (C / 8);
  embedding_pos_kernel<<<(unsigned)((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      tokens, positions, static_cast<const __nv_bfloat16*>(wte), static_cast<const __nv_bfloat16*>(wpe),
      static_cast<__nv_bfloat16*>(out), n, C, vocab, max_pos > 0 ? max_pos : 1, scale);
  return launch_check("embedding_positions", 1);
}

extern "C" int nfn_kv_cache_write(const void* qkv, int ld, void* k_cache, void* v_cache, int n, int n_q_heads, int n_kv_heads,
                                  int head_dim, int cap, int pos0, nfn_stream_t stream) {
  if (n <= 0) return 0;
  if (!qkv || !k_cache || !v_cache || cap <= 0 || pos0 < 0 || (head_dim & 7) || (ld & 7) || ld < (n_q_heads + 2 * n_kv_heads) * head_dim)
    return fail(-1, "kv_cache_write: bad arguments");
  const int t_first = n > cap ? n - cap : 0;  // earlier rows would be overwritten anyway (and would race)
  const long long total = (long long)(n - t_first) * n_kv_heads * (head_dim / 8);
  kv_cache_write_kernel<<<(unsigned)((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(qkv), ld, static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), n,
      t_first, n_q_heads, n_kv_heads, head_dim, cap, pos0);
  return launch_check("kv_cache_write", 1);
}

// ---- hidden-state taps: rows of the residual stream into per-slot position-indexed buffers ------
namespace nfn {

// one warp per row: row r belongs to sequence r / block_rows, block row j = r % block_rows, and lands at
// position lengths[sequence] + j + pos_offset of that sequence's [max_pos, C] region
__global__ void __launch_bounds__(256)
rows_to_slots_kernel(const __nv_bfloat16* __restrict__ x, int ldx, int rows, int C, __nv_bfloat16* __restrict__ dst, long long slot_stride,
                     int max_pos, const int* __restrict__ lengths, int block_rows, int pos_offset, const int* __restrict__ live_rows) {
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int b = r / block_rows, j = r % block_rows;
  if (live_rows && j >= live_rows[b]) return;
  const int pos = lengths[b] + j + pos_offset;
  if (pos < 0 || pos >= max_pos) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)r * ldx);
  uint4* out = reinterpret_cast<uint4*>(dst + b * slot_stride + (long long)pos * C);
  for (int i = threadIdx.x & 31; i < C / 8; i += 32) out[i] = src[i];
}

}  // namespace nfn

extern "C" int nfn_rows_to_slots(const void* x, int ldx, int rows, int C, void* dst, long long slot_stride, int max_pos, const int* lengths,
                                 int block_rows, int pos_offset, const int* live_rows, nfn_stream_t stream) {
  using namespace nfn;
  if (rows <= 0) return 0;
  if (!x || !dst || !lengths || (C & 7) || (ldx & 7) || block_rows <= 0 || max_pos <= 0 || slot_stride < (long long)max_pos * C)
    return fail(-1, "rows_to_slots: bad arguments");
  rows_to_slots_kernel<<<(rows + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, rows, C, static_cast<__nv_bfloat16*>(dst), slot_stride, max_pos, lengths, block_rows, pos_offset,
      live_rows);
  return launch_check("rows_to_slots", 1);
}

// ---- gated attention output and sandwich norms (Glimmer-style blocks) ---------------------------
namespace nfn {

// att[r, c] *= sigmoid(gate[r, c])
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(__nv_bfloat16* __restrict__ att, int ld_att, const __nv_bfloat16* __restrict__ gate, int ld_gate, long long rows, int width) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int vecs = width / 8;
  if (idx >= rows * vecs) return;
  const long long r = idx / vecs;
  const int c = (int)(idx % vecs) * 8;
  float a[8], g[8];
  unpack8(*reinterpret_cast<const uint4*>(att + r * ld_att + c), a);
  unpack8(*reinterpret_cast<const uint4*>(gate + r * ld_gate + c), g);
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] *= 1.f / (1.f + __expf(-g[j]));
  *reinterpret_cast<uint4*>(att + r * ld_att + c) = pack8(a);
}

// out[r, :] = resid[r, :] + RMS(x[r, :]) * (centered ? 1 + w : w); one 256-thread block per row
__global__ void __launch_bounds__(256)
rmsnorm_residual_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ resid,
                        __nv_bfloat16* __restrict__ out, int C, float eps, int centered) {
  __shared__ float red[8];
  const long long r = blockIdx.x;
  const int vecs = C / 8;
  float ss = 0.f;
  for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(x + r * C + v * 8), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float rstd = rsqrtf(tot / (float)C + eps);
  for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
    float f[8], wv[8], rv[8];
    unpack8(*reinterpret_cast<const uint4*>(x + r * C + v * 8), f);
    unpack8(*reinterpret_cast<const uint4*>(w + v * 8), wv);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * (centered ? 1.f + wv[j] : wv[j]);
    if (resid) {
      unpack8(*reinterpret_cast<const uint4*>(resid + r * C + v * 8), rv);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += rv[j];
    }
    *reinterpret_cast<uint4*>(out + r * C + v * 8) = pack8(f);
  }
}

}  // namespace nfn

extern "C" int nfn_sigmoid_gate_inplace(void* att, int ld_att, const void* gate, int ld_gate, long long rows, int width, nfn_stream_t stream) {
  using namespace nfn;
  if (rows <= 0) return 0;
  if (!att || !gate || width <= 0 || (width & 7) || (ld_att & 7) || (ld_gate & 7)) return fail(-1, "sigmoid_gate: bad arguments");
  const long long total = rows * (width / 8), grid = (total + 255) / 256;
  if (grid > 0x7fffffffLL) return fail(-1, "sigmoid_gate: too large for one launch");
  sigmoid_gate_kernel<<<(unsigned)grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<__nv_bfloat16*>(att), ld_att,
                                                                                    static_cast<const __nv_bfloat16*>(gate), ld_gate, rows, width);
  return launch_check("sigmoid_gate", 1);
}

// Contiguous rows of C elements. resid may be NULL; out may alias resid (each element is read
// before it is written by the same thread).
extern "C" int nfn_rmsnorm_residual(const void* x, const void* weight, const void* resid, void* out, long long rows, int C, float eps,
                                    int centered, nfn_stream_t stream) {
  using namespace nfn;
  if (rows <= 0) return 0;
  if (!x || !weight || !out || C <= 0 || (C & 7) || rows > 0x7fffffffLL) return fail(-1, "rmsnorm_residual: bad arguments");
  rmsnorm_residual_kernel<<<(unsigned)rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(weight), static_cast<const __nv_bfloat16*>(resid),
      static_cast<__nv_bfloat16*>(out), C, eps, centered);
  return launch_check("rmsnorm_residual", 1);
}
