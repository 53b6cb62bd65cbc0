// Resident inference engine (see nfn_engine.h for the contract).
//
// Memory plan, sized once at creation: weights (bf16, one allocation per tensor), per-layer
// K/V caches [max_batch, n_kv_head, cap_l, head_dim] with cap_l = window for local layers
// and max_seq for global ones, activation buffers for max(max_seq, max_batch) rows, fp32
// rotary tables, one pinned host block for the per-step inputs and outputs. Nothing is
// allocated after nfn_engine_finalize().
//
// A decode step always runs all max_batch rows (inactive rows carry length 0 and are
// skipped inside the attention kernel), so every launch has static shapes and pointers and
// the step can be replayed as one CUDA graph; per-step data (tokens, lengths, positions,
// sampling parameters, Philox offset) travels in a single host-to-device copy.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../kernels/nfn_kernels.h"
#include "nfn_engine.h"

extern "C" {
// kernel-library entry points that nfn_kernels.h does not declare
int nfn_norm_forward(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int rows, int C, float eps,
                     int mode, int centered, nfn_stream_t stream);
int nfn_attention_forward(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T, int Hq, int Hkv, int D,
                          int ld_q, int ld_k, int ld_v, int ld_o, int causal, int window, float scale, nfn_stream_t stream);
int nfn_qk_norm_forward(void* qkv, float* rstd, int tokens, int n_q_heads, int n_kv_heads, int head_dim, int ld, float eps,
                        float q_scale, nfn_stream_t stream);
int nfn_swiglu_forward(const void* gate_up, int ld, void* out, int ld_out, long long rows, int inter, nfn_stream_t stream);
int nfn_embedding_positions(const int* tokens, const int* positions, const void* wte, const void* wpe, void* out, int n, int C,
                            int vocab, int max_pos, float scale, nfn_stream_t stream);
int nfn_kv_cache_write(const void* qkv, int ld, void* k_cache, void* v_cache, int n, int n_q_heads, int n_kv_heads, int head_dim,
                       int cap, int pos0, nfn_stream_t stream);
int nfn_sigmoid_gate_inplace(void* att, int ld_att, const void* gate, int ld_gate, long long rows, int width, nfn_stream_t stream);
int nfn_rmsnorm_residual(const void* x, const void* weight, const void* resid, void* out, long long rows, int C, float eps, int centered,
                         nfn_stream_t stream);
long long nfn_launch_count(void);
}

namespace {

thread_local std::string t_err;
int efail(const std::string& m) {
  t_err = m;
  return -1;
}
#define CU(call)                                                                                       \
  do {                                                                                                 \
    cudaError_t e__ = (call);                                                                          \
    if (e__ != cudaSuccess) return efail(std::string(#call) + ": " + cudaGetErrorString(e__));         \
  } while (0)
#define K(call)                                                                        \
  do {                                                                                 \
    int rc__ = (call);                                                                 \
    if (rc__ != 0) return efail(std::string(#call) + " failed: " + nfn_last_error()); \
  } while (0)

struct DevTensor {
  void* ptr = nullptr;
  long long numel = 0;
  int qtype = 0;  // 0: bf16 values; NFN_QTYPE_Q4_K / Q5_K / Q6_K: packed super-blocks of 256 values, rows back to back
};

struct StepIO {  // layout of the pinned per-step block; device mirror has the same layout
  long long tokens, lengths, positions, row_params, offset, tq_seq, tq_slot_local, tq_slot_global, out_tokens, total;
};

}  // namespace

struct nfn_engine {
  nfn_engine_config c{};
  int device = 0;
  cudaStream_t stream = nullptr;
  std::map<std::string, DevTensor> w;
  std::vector<std::pair<std::string, long long>> expected;
  bool finalized = false;
  long long bytes = 0;
  // activations
  void *x = nullptr, *xn = nullptr, *qkv = nullptr, *att = nullptr, *ff = nullptr, *ffa = nullptr, *logits = nullptr;
  float *cosT = nullptr, *sinT = nullptr;
  std::vector<void*> kc, vc;
  std::vector<int> cap;
  void* dec_ws = nullptr;
  long long dec_ws_bytes = 0;
  void* gemm_ws = nullptr;      // fp32 partial slices of split-K products
  long long gemm_ws_bytes = 0;
  void* rstd = nullptr;         // scratch of the weightless prefill QK norm
  void* branch = nullptr;       // output of a block branch before its sandwich norm
  void* ones = nullptr;         // unit norm weights (weightless embedding norm)
  void* zero_pos = nullptr;     // int32 zeros: "position 0" for layers without rotary embedding
  std::vector<int> logit_row;   // row of e.logits holding each slot's latest logits
  int decode_calls = 0;
  int qkv_ld = 0, rows_max = 0;
  // per-step io
  unsigned char* h_io = nullptr;
  unsigned char* d_io = nullptr;
  StepIO io{};
  std::vector<int> len;  // tokens held per slot
  unsigned long long steps = 0;
  cudaGraphExec_t graph = nullptr;
  long long launches = 0, graph_launches = 0;
  // block verification (speculative decoding, appends at a position > 0); set up by nfn_engine_enable_verify
  int v_rows_max = 0, v_rows = 0;         // rows per slot: capacity / of the last verification
  std::vector<void*> stage_k, stage_v;    // per layer [max_batch * v_rows_max, n_kv_head * head_dim]
  void** d_tables = nullptr;              // device copies of stage_k | stage_v | kc | vc pointer arrays
  int* d_caps = nullptr;
  void* logits_v = nullptr;               // [max_batch * v_rows_max, padded_vocab] bf16
  void* blk_ws = nullptr;
  long long blk_ws_bytes = 0;
  int *d_vtok = nullptr, *d_vpos = nullptr, *d_vlen = nullptr, *d_vrows = nullptr, *d_vout = nullptr;
  void* argmax_ws = nullptr;
  std::vector<int> h_vrows;               // live rows per slot of the last verification
  std::vector<int> logit_src;             // 0: e.logits, 1: logits_v
  // hidden-state taps (inputs of a block-diffusion draft): residual stream after the listed layers, by slot and position
  // TurboQuant cache mode: K / V records instead of bf16 rows (kc / vc then hold records)
  bool tq = false;
  nfn_tq_tables tq_tables{};
  int* tq_idx = nullptr;                  // prompt scratch: sequence, local-ring slot and global slot of every prompt row
  std::vector<int> tap_layers;
  std::vector<void*> taps;                // per tap [max_batch][max_seq][d_model] bf16
  // K-quant resident projections: packed pointer -> type; products with more rows than the quantised GEMV takes decode the
  // tensor into wq_scratch (bf16, sized for the largest one) first
  std::map<const void*, int> qtype_of;
  long long wq_max_numel = 0;
  void* wq_scratch = nullptr;

  int alloc(void** p, long long nbytes) {
    CU(cudaMalloc(p, (size_t)nbytes));
    bytes += nbytes;
    return 0;
  }
  const void* W(const std::string& n) const { return w.at(n).ptr; }
  bool has(const std::string& n) const { return w.count(n) != 0; }
};

namespace {

std::string lname(int l, const char* s) {
  char buf[96];
  std::snprintf(buf, sizeof buf, "%d.%s", l, s);
  return buf;
}
std::string gname(int l, const char* s) { return "h." + lname(l, s); }        // GPT-2 family
std::string yname(int l, const char* s) { return "layers." + lname(l, s); }   // Llama family

bool layer_is_local(const nfn_engine_config& c, int l) {
  if (c.window <= 0) return false;
  if (c.global_every <= 0) return true;
  return ((l + 1) % c.global_every) != 0;
}

void build_expected(nfn_engine& e) {
  const nfn_engine_config& c = e.c;
  const long long C = c.d_model, F = c.d_ff, Vp = c.padded_vocab, HD = c.head_dim;
  const long long ATT = (long long)c.n_head * HD;
  const long long QKV = (long long)(c.n_head + 2 * c.n_kv_head) * HD + ((c.family == 1 && c.gated_attention) ? ATT : 0);
  auto add = [&](const std::string& n, long long numel) { e.expected.emplace_back(n, numel); };
  if (c.family == 0) {
    add("wte", Vp * C);
    add("wpe", (long long)c.max_seq * C);
    for (int l = 0; l < c.n_layer; ++l) {
      add(gname(l, "ln_1.weight"), C); add(gname(l, "ln_1.bias"), C);
      add(gname(l, "attn.c_attn.weight"), QKV * C); add(gname(l, "attn.c_attn.bias"), QKV);
      add(gname(l, "attn.c_proj.weight"), C * ATT); add(gname(l, "attn.c_proj.bias"), C);
      add(gname(l, "ln_2.weight"), C); add(gname(l, "ln_2.bias"), C);
      add(gname(l, "mlp.c_fc.weight"), F * C); add(gname(l, "mlp.c_fc.bias"), F);
      add(gname(l, "mlp.c_proj.weight"), C * F); add(gname(l, "mlp.c_proj.bias"), C);
    }
    add("ln_f.weight", C); add("ln_f.bias", C);
  } else {
    add("tok_embeddings", Vp * C);
    for (int l = 0; l < c.n_layer; ++l) {
      add(yname(l, "attn_norm"), C);
      add(yname(l, "wqkv"), QKV * C);
      if (c.qk_norm == 2) { add(yname(l, "q_norm"), HD); add(yname(l, "k_norm"), HD); }
      add(yname(l, "wo"), C * ATT);
      if (c.sandwich_norms) add(yname(l, "post_attn_norm"), C);
      add(yname(l, "ffn_norm"), C);
      add(yname(l, "w_gate_up"), 2 * F * C);
      add(yname(l, "w_down"), C * F);
      if (c.sandwich_norms) add(yname(l, "post_ffn_norm"), C);
    }
    add("norm", C);
    if (!c.tie_embeddings) add("lm_head", Vp * C);
  }
}

// C[M, N] = A[M, K] . B[N, K]^T with the epilogue selected by flags
int gemm(nfn_engine& e, const void* a, int lda, const void* b, void* cdst, int ldc, int m, int n, int k, int flags, const void* bias,
         const void* resid, int ld_resid, float act_param = 0.f, float alpha = 1.f) {
  if (!e.qtype_of.empty()) {
    const auto it = e.qtype_of.find(b);
    if (it != e.qtype_of.end()) {
      // a K-quant resident weight: up to eight rows with a bias / residual epilogue go to the quantised GEMV, which reads
      // the packed blocks once; everything else decodes the tensor into the scratch buffer and runs the bf16 product on it
      if (m <= 8 && flags == 0 && alpha == 1.f && (k % 256) == 0) {
        K(nfn_kquant_gemv(it->second, b, nullptr, a, lda, cdst, ldc, bias, resid, ld_resid, m, n, k, e.stream));
        return 0;
      }
      K(nfn_dequant_kquant(it->second, b, (long long)n * (k / 256), e.wq_scratch, e.stream));
      b = e.wq_scratch;
    }
  }
  nfn_gemm_args g{};
  g.a = a; g.b = b; g.c = cdst;
  g.m = m; g.n = n; g.k = k;
  g.lda = lda; g.ldb = k; g.ldc = ldc;
  // "+= into the residual stream" is an accumulating product; unlike a residual epilogue it may be
  // split along K, which is what lets a decode-sized product (a handful of rows) keep every SM
  // streaming weights instead of one CTA per 128 output columns
  const bool accumulate = m <= 128 && resid && resid == cdst && ld_resid == ldc && !bias && flags == 0;
  g.flags = flags | (bias ? NFN_EPI_BIAS : 0) | (accumulate ? NFN_EPI_ACCUM : (resid ? NFN_EPI_RESID : 0));
  g.alpha = alpha;
  g.act_param = act_param;
  g.bias = bias;
  g.aux_in = accumulate ? nullptr : resid;
  g.ld_aux_in = accumulate ? 0 : ld_resid;
  g.workspace = e.gemm_ws;
  g.workspace_bytes = e.gemm_ws_bytes;
  g.split_k = 0;  // automatic: only skinny, long-K products with a plain epilogue are split
  K(nfn_gemm_bf16(&g, e.stream));
  return 0;
}

// One transformer stack over `rows` rows of e.x. decode = true: one token per slot (row ==
// slot), attention over the caches; false: one sequence of `rows` tokens for `slot`. With
// block_rows > 0 (and decode = false) the rows are max_batch blocks of block_rows rows that
// continue each slot at d_lengths[slot]: attention reads the caches plus the block, the
// block's K/V go to the staging buffers, the caches stay untouched.
int forward_layers(nfn_engine& e, int rows, bool decode, int slot, const int* d_lengths, int block_rows = 0, const int* d_block_pos = nullptr,
                   const int* d_block_live = nullptr) {
  const nfn_engine_config& c = e.c;
  const int C = c.d_model, F = c.d_ff, HD = c.head_dim, Hq = c.n_head, Hkv = c.n_kv_head, ATT = Hq * HD;
  const float scale = 1.f / std::sqrt((float)HD);
  const float sign = c.rope_hf ? 1.f : -1.f;
  if (e.tq && block_rows > 0) return efail("engine: verification blocks are not available with the TurboQuant cache (decode only)");
  if (e.tq && !decode) {
    // a prompt: row r of `slot` is position r; its records go to ring row r % window on local layers, row r on global ones
    const int wcap = c.window > 0 ? std::min(c.window, c.max_seq) : c.max_seq;
    std::vector<int> idx(3 * (size_t)rows);
    for (int r = 0; r < rows; ++r) {
      idx[r] = slot;
      idx[rows + r] = r >= rows - wcap ? r % wcap : -1;       // earlier rows would be overwritten by later ones of this prompt
      idx[2 * rows + r] = r;
    }
    CU(cudaMemcpyAsync(e.tq_idx, idx.data(), idx.size() * 4, cudaMemcpyHostToDevice, e.stream));
    CU(cudaStreamSynchronize(e.stream));  // `idx` leaves scope
  }
  for (int l = 0; l < c.n_layer; ++l) {
    const bool local = layer_is_local(c, l);
    const int cap = e.cap[l];
    const long long cache_stride = (long long)Hkv * cap * HD;
    char* kc = static_cast<char*>(e.kc[l]);
    char* vc = static_cast<char*>(e.vc[l]);
    const void *qw = nullptr, *kw = nullptr;
    if (c.family == 0) {
      K(nfn_norm_forward(e.x, e.W(gname(l, "ln_1.weight")), e.W(gname(l, "ln_1.bias")), e.xn, nullptr, nullptr, rows, C, c.norm_eps, 0, 0, e.stream));
      if (gemm(e, e.xn, C, e.W(gname(l, "attn.c_attn.weight")), e.qkv, e.qkv_ld, rows, e.qkv_ld, C, 0, e.W(gname(l, "attn.c_attn.bias")), nullptr, 0)) return -1;
    } else {
      K(nfn_norm_forward(e.x, e.W(yname(l, "attn_norm")), nullptr, e.xn, nullptr, nullptr, rows, C, c.norm_eps, 1, c.centered_norms, e.stream));
      if (gemm(e, e.xn, C, e.W(yname(l, "wqkv")), e.qkv, e.qkv_ld, rows, e.qkv_ld, C, 0, nullptr, nullptr, 0)) return -1;
      if (c.qk_norm == 2) { qw = e.W(yname(l, "q_norm")); kw = e.W(yname(l, "k_norm")); }
    }
    const bool rope = c.family == 1 && (!c.rope_local_only || local);
    const float q_scale = (c.family == 1 && c.q_scale > 0.f) ? c.q_scale : 1.f;
    if (decode && e.tq) {
      // compressed cache: prepare q / k at their positions, encode the new token's K and V, attend over the records
      const int* d_pos = reinterpret_cast<const int*>(e.d_io + e.io.positions);
      if (rope && c.qk_norm) {
        K(nfn_qk_norm_rope_forward(e.qkv, e.qkv_ld, rows, rows, Hq, Hkv, HD, qw, kw, e.cosT, e.sinT, d_pos, c.max_seq, sign, c.qk_norm_eps, q_scale, nullptr, e.stream));
      } else if (rope) {
        K(nfn_rope_inplace(e.qkv, e.qkv_ld, rows, rows, Hq, Hkv, HD, HD, e.cosT, e.sinT, d_pos, c.max_seq, sign, q_scale, e.stream));
      } else if (c.qk_norm == 1) {
        K(nfn_qk_norm_forward(e.qkv, static_cast<float*>(e.rstd), rows, Hq, Hkv, HD, e.qkv_ld, c.qk_norm_eps, q_scale, e.stream));
      } else if (c.qk_norm == 2) {
        K(nfn_qk_norm_rope_forward(e.qkv, e.qkv_ld, rows, rows, Hq, Hkv, HD, qw, kw, e.cosT, e.sinT, static_cast<const int*>(e.zero_pos), c.max_seq, sign,
                                   c.qk_norm_eps, q_scale, nullptr, e.stream));
      } else if (q_scale != 1.f) {
        return efail("engine: a query scale without QK norm or rotary embedding is not supported with the TurboQuant cache");
      }
      const int* d_seq = reinterpret_cast<const int*>(e.d_io + e.io.tq_seq);
      const int* d_slot = reinterpret_cast<const int*>(e.d_io + (local ? e.io.tq_slot_local : e.io.tq_slot_global));
      const char* q = static_cast<const char*>(e.qkv);
      K(nfn_turboquant_encode(&e.tq_tables, q + (size_t)Hq * HD * 2, e.qkv_ld, d_seq, d_slot, rows, Hkv, cap, 1, kc, e.stream));
      K(nfn_turboquant_encode(&e.tq_tables, q + (size_t)(Hq + Hkv) * HD * 2, e.qkv_ld, d_seq, d_slot, rows, Hkv, cap, 0, vc, e.stream));
      K(nfn_turboquant_attention(&e.tq_tables, e.qkv, e.qkv_ld, kc, vc, d_lengths, e.att, ATT, rows, Hq, Hkv, cap, scale, e.stream));
    } else if (decode) {
      K(nfn_decode_attention(e.qkv, e.qkv_ld, kc, vc, cache_stride, d_lengths, e.att, rows, Hq, Hkv, HD, cap, qw, kw, c.qk_norm != 0,
                             c.qk_norm_eps, rope ? e.cosT : nullptr, rope ? e.sinT : nullptr, rope ? c.max_seq : 0, sign, scale * q_scale,
                             e.dec_ws, e.dec_ws_bytes, 0, e.stream));
    } else {
      if (rope && c.qk_norm) {
        K(nfn_qk_norm_rope_forward(e.qkv, e.qkv_ld, rows, rows, Hq, Hkv, HD, qw, kw, e.cosT, e.sinT, d_block_pos, c.max_seq, sign, c.qk_norm_eps, q_scale, nullptr, e.stream));
      } else if (rope) {
        K(nfn_rope_inplace(e.qkv, e.qkv_ld, rows, rows, Hq, Hkv, HD, HD, e.cosT, e.sinT, d_block_pos, c.max_seq, sign, q_scale, e.stream));
      } else if (c.qk_norm == 1) {
        K(nfn_qk_norm_forward(e.qkv, static_cast<float*>(e.rstd), rows, Hq, Hkv, HD, e.qkv_ld, c.qk_norm_eps, q_scale, e.stream));
      } else if (q_scale != 1.f && c.qk_norm != 2) {
        return efail("engine: a query scale without QK norm or rotary embedding is not supported in prefill");
      } else if (c.qk_norm == 2) {
        // no rotation on this layer: run the fused kernel at position 0 for every row (cos 1, sin 0)
        if (!e.cosT) return efail("engine: weighted QK norm / query scale need the rotary tables (family 1)");
        K(nfn_qk_norm_rope_forward(e.qkv, e.qkv_ld, rows, rows, Hq, Hkv, HD, qw, kw, e.cosT, e.sinT, static_cast<const int*>(e.zero_pos), c.max_seq, sign,
                                   c.qk_norm_eps, q_scale, nullptr, e.stream));
      }
      if (block_rows > 0) {
        K(nfn_block_attention(e.qkv, e.qkv_ld, kc, vc, d_lengths, d_block_live, e.att, ATT, e.stage_k[l], e.stage_v[l], c.max_batch, block_rows, Hq,
                              Hkv, HD, cap, local ? cap : 0, 1, scale, e.blk_ws, e.blk_ws_bytes, 0, e.stream));
      } else {
        const char* q = static_cast<const char*>(e.qkv);
        K(nfn_attention_forward(q, q + (size_t)Hq * HD * 2, q + (size_t)(Hq + Hkv) * HD * 2, e.att, nullptr, 1, rows, Hq, Hkv, HD, e.qkv_ld,
                                e.qkv_ld, e.qkv_ld, ATT, 1, local ? c.window : 0, scale, e.stream));
        if (e.tq) {
          const int* d_slot = e.tq_idx + (local ? rows : 2 * rows);
          K(nfn_turboquant_encode(&e.tq_tables, q + (size_t)Hq * HD * 2, e.qkv_ld, e.tq_idx, d_slot, rows, Hkv, cap, 1, kc, e.stream));
          K(nfn_turboquant_encode(&e.tq_tables, q + (size_t)(Hq + Hkv) * HD * 2, e.qkv_ld, e.tq_idx, d_slot, rows, Hkv, cap, 0, vc, e.stream));
        } else {
          K(nfn_kv_cache_write(e.qkv, e.qkv_ld, kc + (size_t)slot * cache_stride * 2, vc + (size_t)slot * cache_stride * 2, rows, Hq, Hkv, HD, cap, 0, e.stream));
        }
      }
    }
    if (c.family == 0) {
      if (gemm(e, e.att, ATT, e.W(gname(l, "attn.c_proj.weight")), e.x, C, rows, C, ATT, 0, e.W(gname(l, "attn.c_proj.bias")), e.x, C)) return -1;
      K(nfn_norm_forward(e.x, e.W(gname(l, "ln_2.weight")), e.W(gname(l, "ln_2.bias")), e.xn, nullptr, nullptr, rows, C, c.norm_eps, 0, 0, e.stream));
      if (gemm(e, e.xn, C, e.W(gname(l, "mlp.c_fc.weight")), e.ff, F, rows, F, C, (c.mlp_activation > 0 ? c.mlp_activation : NFN_ACT_GELU_TANH) << NFN_EPI_ACT_SHIFT, e.W(gname(l, "mlp.c_fc.bias")), nullptr, 0)) return -1;
      if (gemm(e, e.ff, F, e.W(gname(l, "mlp.c_proj.weight")), e.x, C, rows, C, F, 0, e.W(gname(l, "mlp.c_proj.bias")), e.x, C)) return -1;
    } else {
      const float post_eps = c.post_norm_eps > 0.f ? c.post_norm_eps : c.norm_eps;
      if (c.gated_attention) {
        const char* gate = static_cast<const char*>(e.qkv) + (size_t)(Hq + 2 * Hkv) * HD * 2;
        K(nfn_sigmoid_gate_inplace(e.att, ATT, gate, e.qkv_ld, rows, ATT, e.stream));
      }
      if (c.sandwich_norms) {
        if (gemm(e, e.att, ATT, e.W(yname(l, "wo")), e.branch, C, rows, C, ATT, 0, nullptr, nullptr, 0)) return -1;
        K(nfn_rmsnorm_residual(e.branch, e.W(yname(l, "post_attn_norm")), e.x, e.x, rows, C, post_eps, c.centered_norms, e.stream));
      } else if (gemm(e, e.att, ATT, e.W(yname(l, "wo")), e.x, C, rows, C, ATT, 0, nullptr, e.x, C)) {
        return -1;
      }
      K(nfn_norm_forward(e.x, e.W(yname(l, "ffn_norm")), nullptr, e.xn, nullptr, nullptr, rows, C, c.norm_eps, 1, c.centered_norms, e.stream));
      if (gemm(e, e.xn, C, e.W(yname(l, "w_gate_up")), e.ff, 2 * F, rows, 2 * F, C, 0, nullptr, nullptr, 0)) return -1;
      K(nfn_swiglu_forward(e.ff, 2 * F, e.ffa, F, rows, F, e.stream));
      if (c.sandwich_norms) {
        if (gemm(e, e.ffa, F, e.W(yname(l, "w_down")), e.branch, C, rows, C, F, 0, nullptr, nullptr, 0)) return -1;
        K(nfn_rmsnorm_residual(e.branch, e.W(yname(l, "post_ffn_norm")), e.x, e.x, rows, C, post_eps, c.centered_norms, e.stream));
      } else if (gemm(e, e.ffa, F, e.W(yname(l, "w_down")), e.x, C, rows, C, F, 0, nullptr, e.x, C)) {
        return -1;
      }
    }
    for (size_t t = 0; t < e.tap_layers.size(); ++t) {
      if (e.tap_layers[t] != l) continue;
      const long long stride = (long long)c.max_seq * C;
      if (!decode && block_rows == 0) {
        // a prompt: rows are positions 0 .. rows - 1 of `slot`
        CU(cudaMemcpyAsync(static_cast<char*>(e.taps[t]) + (size_t)slot * stride * 2, e.x, (size_t)rows * C * 2, cudaMemcpyDeviceToDevice, e.stream));
      } else if (decode) {
        // lengths count the new token: it sits at lengths[slot] - 1. Rows of idle slots have length 0 and are skipped.
        K(nfn_rows_to_slots(e.x, C, rows, C, e.taps[t], stride, c.max_seq, d_lengths, 1, -1, nullptr, e.stream));
      } else {
        // a verification block starts at lengths[slot]; rows past the committed length are overwritten before they are read
        K(nfn_rows_to_slots(e.x, C, rows, C, e.taps[t], stride, c.max_seq, d_lengths, block_rows, 0, d_block_live, e.stream));
      }
    }
  }
  return 0;
}

// final norm of rows [row0, row0 + n) -> logits[n, padded_vocab]
int head(nfn_engine& e, int row0, int n, void* logits_dst = nullptr) {
  const nfn_engine_config& c = e.c;
  const int C = c.d_model;
  const char* xin = static_cast<const char*>(e.x) + (size_t)row0 * C * 2;
  if (c.family == 0)
    K(nfn_norm_forward(xin, e.W("ln_f.weight"), e.W("ln_f.bias"), e.xn, nullptr, nullptr, n, C, c.norm_eps, 0, 0, e.stream));
  else
    K(nfn_norm_forward(xin, e.W("norm"), nullptr, e.xn, nullptr, nullptr, n, C, c.norm_eps, 1, 0, e.stream));
  const void* wh = c.family == 0 ? e.W("wte") : (c.tie_embeddings ? e.W("tok_embeddings") : e.W("lm_head"));
  const int flags = c.logit_softcap > 0.f ? (NFN_ACT_TANH_CAP << NFN_EPI_ACT_SHIFT) : 0;
  const float mult = (c.family == 1 && c.output_multiplier > 0.f) ? c.output_multiplier : 1.f;
  return gemm(e, e.xn, C, wh, logits_dst ? logits_dst : e.logits, c.padded_vocab, n, c.padded_vocab, C, flags, nullptr, nullptr, 0, c.logit_softcap, mult);
}

int sample(nfn_engine& e, int rows, const float* d_row_params, const unsigned long long* d_offset, int* d_out) {
  // every row carries its own (temperature, top_k, top_p); the Philox offset is a device word
  K(nfn_sample_rows(e.logits, 0, e.c.padded_vocab, rows, e.c.vocab, d_out, nullptr, 1.f, 0, 1.f, d_row_params, 0x5eedULL, 0ULL, d_offset, 0, e.stream));
  return 0;
}

int decode_body(nfn_engine& e) {
  const int B = e.c.max_batch;
  const int* d_tok = reinterpret_cast<const int*>(e.d_io + e.io.tokens);
  const int* d_len = reinterpret_cast<const int*>(e.d_io + e.io.lengths);
  const int* d_pos = reinterpret_cast<const int*>(e.d_io + e.io.positions);
  const float* d_rp = reinterpret_cast<const float*>(e.d_io + e.io.row_params);
  const unsigned long long* d_off = reinterpret_cast<const unsigned long long*>(e.d_io + e.io.offset);
  int* d_out = reinterpret_cast<int*>(e.d_io + e.io.out_tokens);
  const nfn_engine_config& c = e.c;
  if (c.family == 0)
    K(nfn_embedding_positions(d_tok, d_pos, e.W("wte"), e.W("wpe"), e.x, B, c.d_model, c.vocab, c.max_seq, c.embed_scale, e.stream));
  else
    K(nfn_embedding_positions(d_tok, nullptr, e.W("tok_embeddings"), nullptr, e.x, B, c.d_model, c.vocab, c.max_seq, c.embed_scale, e.stream));
  if (c.family == 1 && c.embed_norm) K(nfn_norm_forward(e.x, e.ones, nullptr, e.x, nullptr, nullptr, B, c.d_model, c.norm_eps, 1, 0, e.stream));
  if (forward_layers(e, B, true, 0, d_len)) return -1;
  if (head(e, 0, B)) return -1;
  return sample(e, B, d_rp, d_off, d_out);
}

void fill_params(const nfn_engine& e, float* rp, int row, const nfn_sampling& s) {
  rp[3 * row] = s.temperature;
  rp[3 * row + 1] = (float)s.top_k;
  rp[3 * row + 2] = s.top_p;
  (void)e;
}

}  // namespace

extern "C" {

int nfn_engine_abi_version(void) { return 1; }
const char* nfn_engine_last_error(void) { return t_err.c_str(); }

nfn_engine* nfn_engine_create(const nfn_engine_config* cfg, int device) {
  if (!cfg) {
    efail("engine_create: null config");
    return nullptr;
  }
  const nfn_engine_config& c = *cfg;
  if ((c.family != 0 && c.family != 1) || c.n_layer <= 0 || c.d_model <= 0 || c.n_head <= 0 || c.n_kv_head <= 0 || c.n_head % c.n_kv_head ||
      (c.head_dim != 64 && c.head_dim != 128) || c.d_ff <= 0 || c.vocab <= 0 || c.padded_vocab < c.vocab || (c.padded_vocab & 7) ||
      c.max_seq <= 0 || c.max_batch <= 0 || (c.d_model & 7) || (c.d_ff & 7)) {
    efail("engine_create: invalid geometry (head_dim must be 64 or 128; widths multiples of 8)");
    return nullptr;
  }
  if (c.family == 0 && (c.n_kv_head != c.n_head || c.n_head * c.head_dim != c.d_model)) {
    efail("engine_create: the GPT-2 family needs n_kv_head == n_head and n_head * head_dim == d_model");
    return nullptr;
  }
  auto e = std::make_unique<nfn_engine>();
  e->c = c;
  if (e->c.embed_scale == 0.f) e->c.embed_scale = 1.f;
  e->device = device;
  if (cudaSetDevice(device) != cudaSuccess || cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking) != cudaSuccess) {
    efail("engine_create: cannot select the device or create a stream");
    return nullptr;
  }
  build_expected(*e);
  e->len.assign(c.max_batch, 0);
  e->logit_row.assign(c.max_batch, 0);
  e->logit_src.assign(c.max_batch, 0);
  e->h_vrows.assign(c.max_batch, 0);
  return e.release();
}

void nfn_engine_destroy(nfn_engine* e) {
  if (!e) return;
  cudaSetDevice(e->device);
  if (e->stream) cudaStreamSynchronize(e->stream);
  if (e->graph) cudaGraphExecDestroy(e->graph);
  for (auto& kv : e->w) cudaFree(kv.second.ptr);
  for (void* p : {e->x, e->xn, e->qkv, e->att, e->ff, e->ffa, e->logits, (void*)e->cosT, (void*)e->sinT, e->dec_ws, (void*)e->d_io, e->rstd, e->branch, e->ones, e->zero_pos})
    if (p) cudaFree(p);
  for (void* p : e->kc) cudaFree(p);
  for (void* p : e->vc) cudaFree(p);
  if (e->wq_scratch) cudaFree(e->wq_scratch);
  if (e->h_io) cudaFreeHost(e->h_io);
  if (e->stream) cudaStreamDestroy(e->stream);
  delete e;
}

int nfn_engine_set_tensor(nfn_engine* e, const char* name, const void* host_bf16, long long numel) {
  if (!e || !name || !host_bf16 || numel <= 0) return efail("engine_set_tensor: bad arguments");
  CU(cudaSetDevice(e->device));
  long long want = -1;
  for (const auto& kv : e->expected)
    if (kv.first == name) want = kv.second;
  if (want < 0) return efail(std::string("engine_set_tensor: this configuration has no tensor named ") + name);
  if (want != numel) return efail(std::string("engine_set_tensor: ") + name + " has " + std::to_string(numel) + " elements, expected " + std::to_string(want));
  DevTensor& t = e->w[name];
  if (t.qtype) return efail(std::string("engine_set_tensor: ") + name + " holds K-quant blocks");
  if (!t.ptr) {
    if (e->alloc(&t.ptr, numel * 2)) return -1;
    t.numel = numel;
  }
  CU(cudaMemcpyAsync(t.ptr, host_bf16, (size_t)numel * 2, cudaMemcpyHostToDevice, e->stream));
  CU(cudaStreamSynchronize(e->stream));
  return 0;
}

// A projection weight kept in its K-quant blocks (Q4_K / Q5_K / Q6_K: `numel` values = rows of K / 256 super-blocks, rows back
// to back, the GGUF layout). Only 2-D projection weights qualify (the embedding is gathered, norms and biases are vectors);
// the row length must be a multiple of 256.
int nfn_engine_set_tensor_kquant(nfn_engine* e, const char* name, int qtype, const void* host_blocks, long long nbytes, long long numel) {
  if (!e || !name || !host_blocks || numel <= 0) return efail("engine_set_tensor_kquant: bad arguments");
  if (e->finalized) return efail("engine_set_tensor_kquant: call before nfn_engine_finalize");
  const int bb = nfn_quant_block_bytes(qtype);
  if (bb <= 0 || qtype == NFN_QTYPE_NF4) return efail("engine_set_tensor_kquant: qtype must be Q4_K, Q5_K or Q6_K");
  const std::string n = name;
  auto ends = [&](const char* suf) { const std::string s2 = suf; return n.size() >= s2.size() && n.compare(n.size() - s2.size(), s2.size(), s2) == 0; };
  const nfn_engine_config& c = e->c;
  long long row = 0;  // the contraction length of the product that reads this tensor
  if (c.family == 1) {
    if (ends(".wqkv") || ends(".w_gate_up") || n == "lm_head") row = c.d_model;
    else if (ends(".wo")) row = (long long)c.n_head * c.head_dim;
    else if (ends(".w_down")) row = c.d_ff;
  } else {
    if (ends("attn.c_attn.weight") || ends("mlp.c_fc.weight")) row = c.d_model;
    else if (ends("attn.c_proj.weight")) row = (long long)c.n_head * c.head_dim;
    else if (ends("mlp.c_proj.weight")) row = c.d_ff;
  }
  if (row <= 0) return efail("engine_set_tensor_kquant: " + n + " is not a projection weight (embeddings, norms and biases stay bf16)");
  if (row % 256) return efail("engine_set_tensor_kquant: " + n + " has rows of " + std::to_string(row) + " values, K-quant needs a multiple of 256");
  long long want = -1;
  for (const auto& kv : e->expected)
    if (kv.first == n) want = kv.second;
  if (want < 0) return efail("engine_set_tensor_kquant: this configuration has no tensor named " + n);
  if (want != numel || nbytes != numel / 256 * bb) return efail("engine_set_tensor_kquant: " + n + " has the wrong size");
  CU(cudaSetDevice(e->device));
  DevTensor& t = e->w[n];
  if (t.ptr) return efail("engine_set_tensor_kquant: " + n + " is already set");
  if (e->alloc(&t.ptr, nbytes)) return -1;
  t.numel = numel;
  t.qtype = qtype;
  CU(cudaMemcpyAsync(t.ptr, host_blocks, (size_t)nbytes, cudaMemcpyHostToDevice, e->stream));
  CU(cudaStreamSynchronize(e->stream));
  e->qtype_of[t.ptr] = qtype;
  e->wq_max_numel = std::max(e->wq_max_numel, numel);
  return 0;
}

int nfn_engine_expected_tensors(const nfn_engine* e, char* buf, int cap) {
  if (!e) return efail("engine_expected_tensors: null engine");
  std::string s;
  for (const auto& kv : e->expected) s += kv.first + " " + std::to_string(kv.second) + "\n";
  if (buf && cap > 0) {
    const size_t n = std::min<size_t>(s.size(), (size_t)cap - 1);
    std::memcpy(buf, s.data(), n);
    buf[n] = 0;
  }
  return (int)s.size();
}

int nfn_engine_load_dense_v5(nfn_engine* e, const char* path) {
  if (!e || !path) return efail("engine_load_dense_v5: bad arguments");
  if (e->c.family != 0) return efail("engine_load_dense_v5: dense GPT checkpoints load into family 0 engines");
  std::ifstream in(path, std::ios::binary);
  if (!in) return efail(std::string("engine_load_dense_v5: cannot open ") + path);
  int32_t h[256];
  in.read(reinterpret_cast<char*>(h), sizeof h);
  if (in.gcount() != (std::streamsize)sizeof h || h[0] != 20240326 || h[1] != 5) return efail("engine_load_dense_v5: not a version-5 dense GPT checkpoint");
  const nfn_engine_config& c = e->c;
  if (h[2] != c.max_seq || h[3] != c.vocab || h[4] != c.n_layer || h[5] != c.n_head || h[6] != c.d_model || h[7] != c.padded_vocab)
    return efail("engine_load_dense_v5: checkpoint geometry does not match the engine configuration");
  std::vector<char> stage;
  for (const auto& kv : e->expected) {  // the expected order of family 0 is the file order
    stage.resize((size_t)kv.second * 2);
    in.read(stage.data(), (std::streamsize)stage.size());
    if (in.gcount() != (std::streamsize)stage.size()) return efail("engine_load_dense_v5: payload is truncated at " + kv.first);
    if (nfn_engine_set_tensor(e, kv.first.c_str(), stage.data(), kv.second)) return -1;
  }
  if (in.peek() != std::ifstream::traits_type::eof()) return efail("engine_load_dense_v5: trailing bytes after the last tensor");
  return 0;
}

int nfn_engine_set_turboquant(nfn_engine* e, const void* tq_tables) {
  if (!e || !tq_tables) return efail("engine_set_turboquant: null argument");
  if (e->finalized) return efail("engine_set_turboquant: call it before nfn_engine_finalize (the caches are allocated there)");
  const nfn_tq_tables* t = static_cast<const nfn_tq_tables*>(tq_tables);
  const nfn_engine_config& c = e->c;
  if (c.kv_cache_mode != 1) return efail("engine_set_turboquant: the engine was created with kv_cache_mode 0");
  if (t->D != c.head_dim || (t->D != 64 && t->D != 128)) return efail("engine_set_turboquant: the codec dimension must equal head_dim (64 or 128)");
  if (!t->rotation || !t->centroids || !t->key_fields || !t->value_fields || t->key_rec_bytes <= 0 || t->value_rec_bytes <= 0 || (t->qjl && !t->projection))
    return efail("engine_set_turboquant: incomplete tables");
  if (c.n_head / c.n_kv_head > 8) return efail("engine_set_turboquant: the record attention kernel takes at most 8 query heads per kv head");
  e->tq_tables = *t;
  e->tq = true;
  return 0;
}

int nfn_engine_finalize(nfn_engine* e) {
  if (!e) return efail("engine_finalize: null engine");
  if (e->finalized) return 0;
  if (e->c.kv_cache_mode == 1 && !e->tq) return efail("engine_finalize: kv_cache_mode 1 needs nfn_engine_set_turboquant first");
  CU(cudaSetDevice(e->device));
  for (const auto& kv : e->expected)
    if (!e->has(kv.first)) return efail("engine_finalize: missing tensor " + kv.first);
  if (e->wq_max_numel > 0 && e->alloc(&e->wq_scratch, e->wq_max_numel * 2)) return -1;
  const nfn_engine_config& c = e->c;
  const int HD = c.head_dim;
  e->qkv_ld = (c.n_head + 2 * c.n_kv_head) * HD + ((c.family == 1 && c.gated_attention) ? c.n_head * HD : 0);
  e->rows_max = std::max(c.max_seq, c.max_batch);
  const long long R = e->rows_max;
  if (e->alloc(&e->x, R * c.d_model * 2) || e->alloc(&e->xn, R * c.d_model * 2) || e->alloc(&e->qkv, R * e->qkv_ld * 2) ||
      e->alloc(&e->att, R * c.n_head * HD * 2) || e->alloc(&e->ff, R * (c.family == 1 ? 2LL : 1LL) * c.d_ff * 2) ||
      e->alloc(&e->ffa, R * c.d_ff * 2) || e->alloc(&e->logits, (long long)c.max_batch * c.padded_vocab * 2) ||
      e->alloc(&e->rstd, R * (c.n_head + c.n_kv_head) * 4) || e->alloc(&e->branch, R * c.d_model * 2) ||
      e->alloc(&e->ones, (long long)c.d_model * 2) || e->alloc(&e->zero_pos, R * 4))
    return -1;
  {
    std::vector<uint16_t> one(c.d_model, 0x3F80);  // bf16 1.0
    CU(cudaMemcpy(e->ones, one.data(), one.size() * 2, cudaMemcpyHostToDevice));
    CU(cudaMemset(e->zero_pos, 0, (size_t)R * 4));
  }
  if (c.family == 1) {
    const int half = HD / 2;
    std::vector<float> cs((size_t)c.max_seq * half), sn((size_t)c.max_seq * half);
    for (int p = 0; p < c.max_seq; ++p)
      for (int i = 0; i < half; ++i) {
        const double ang = (double)p * std::pow((double)c.rope_theta, -2.0 * i / HD);
        cs[(size_t)p * half + i] = (float)std::cos(ang);
        sn[(size_t)p * half + i] = (float)std::sin(ang);
      }
    if (e->alloc((void**)&e->cosT, (long long)cs.size() * 4) || e->alloc((void**)&e->sinT, (long long)sn.size() * 4)) return -1;
    CU(cudaMemcpy(e->cosT, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice));
    CU(cudaMemcpy(e->sinT, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice));
  }
  e->kc.resize(c.n_layer);
  e->vc.resize(c.n_layer);
  e->cap.resize(c.n_layer);
  for (int l = 0; l < c.n_layer; ++l) {
    e->cap[l] = layer_is_local(c, l) ? std::min(c.window, c.max_seq) : c.max_seq;
    const long long rows_l = (long long)c.max_batch * c.n_kv_head * e->cap[l];
    const long long kbytes = rows_l * (e->tq ? e->tq_tables.key_rec_bytes : HD * 2), vbytes = rows_l * (e->tq ? e->tq_tables.value_rec_bytes : HD * 2);
    if (e->alloc(&e->kc[l], kbytes) || e->alloc(&e->vc[l], vbytes)) return -1;
    CU(cudaMemset(e->kc[l], 0, (size_t)kbytes));
    CU(cudaMemset(e->vc[l], 0, (size_t)vbytes));
  }
  if (e->tq && e->alloc((void**)&e->tq_idx, 3LL * c.max_seq * 4)) return -1;
  e->dec_ws_bytes = nfn_decode_attention_workspace_bytes(c.max_batch, c.n_head, c.n_kv_head, HD, 64);
  if (e->dec_ws_bytes <= 0) return efail("engine_finalize: bad decode attention geometry");
  if (e->alloc(&e->dec_ws, e->dec_ws_bytes)) return -1;
  e->gemm_ws_bytes = 64LL << 20;
  if (e->alloc(&e->gemm_ws, e->gemm_ws_bytes)) return -1;
  CU(cudaMemset(e->dec_ws, 0, (size_t)e->dec_ws_bytes));
  const long long B = c.max_batch;
  auto up = [](long long v) { return (v + 255) / 256 * 256; };
  e->io.tokens = 0;
  e->io.lengths = up(B * 4);
  e->io.positions = e->io.lengths + up(B * 4);
  e->io.row_params = e->io.positions + up(B * 4);
  e->io.offset = e->io.row_params + up(B * 12);
  e->io.tq_seq = e->io.offset + 256;
  e->io.tq_slot_local = e->io.tq_seq + up(B * 4);
  e->io.tq_slot_global = e->io.tq_slot_local + up(B * 4);
  e->io.out_tokens = e->io.tq_slot_global + up(B * 4);
  e->io.total = e->io.out_tokens + up(B * 4);
  CU(cudaMallocHost((void**)&e->h_io, (size_t)e->io.total));
  std::memset(e->h_io, 0, (size_t)e->io.total);
  if (e->alloc((void**)&e->d_io, e->io.total)) return -1;
  CU(cudaMemset(e->d_io, 0, (size_t)e->io.total));
  CU(cudaDeviceSynchronize());
  e->finalized = true;
  return 0;
}

long long nfn_engine_device_bytes(const nfn_engine* e) { return e ? e->bytes : -1; }
int nfn_engine_slot_length(const nfn_engine* e, int slot) { return (e && slot >= 0 && slot < e->c.max_batch) ? e->len[slot] : -1; }
long long nfn_engine_launches(const nfn_engine* e) { return e ? e->launches : -1; }

int nfn_engine_release(nfn_engine* e, int slot) {
  if (!e || slot < 0 || slot >= e->c.max_batch) return efail("engine_release: bad slot");
  e->len[slot] = 0;
  return 0;
}

}  // extern "C"

// layers, head on the last row, sampling and bookkeeping of a prompt whose layer-0 inputs sit in e->x
static int run_prompt_rows(nfn_engine* e, int slot, int n, const nfn_sampling* s, int32_t* next_token, long long before) {
  const nfn_engine_config& c = e->c;
  if (forward_layers(*e, n, false, slot, nullptr)) return -1;
  if (head(*e, n - 1, 1)) return -1;
  float* rp = reinterpret_cast<float*>(e->h_io + e->io.row_params);
  fill_params(*e, rp, 0, *s);
  unsigned long long* off = reinterpret_cast<unsigned long long*>(e->h_io + e->io.offset);
  *off = (s->seed << 20) ^ (++e->steps);
  CU(cudaMemcpyAsync(e->d_io + e->io.row_params, rp, 12, cudaMemcpyHostToDevice, e->stream));
  CU(cudaMemcpyAsync(e->d_io + e->io.offset, off, 8, cudaMemcpyHostToDevice, e->stream));
  if (sample(*e, 1, reinterpret_cast<const float*>(e->d_io + e->io.row_params),
             reinterpret_cast<const unsigned long long*>(e->d_io + e->io.offset), reinterpret_cast<int*>(e->d_io + e->io.out_tokens)))
    return -1;
  CU(cudaMemcpyAsync(e->h_io + e->io.out_tokens, e->d_io + e->io.out_tokens, 4, cudaMemcpyDeviceToHost, e->stream));
  CU(cudaStreamSynchronize(e->stream));
  *next_token = *reinterpret_cast<int*>(e->h_io + e->io.out_tokens);
  e->len[slot] = n;
  e->logit_row[slot] = 0;
  e->logit_src[slot] = 0;
  e->launches += nfn_launch_count() - before;
  if (nfn_status_peek() != 0) return efail("engine_prefill: a kernel reported error code " + std::to_string(nfn_status_read_reset()));
  return 0;
}


extern "C" {
int nfn_engine_prefill(nfn_engine* e, int slot, const int32_t* tokens, int n, const nfn_sampling* s, int32_t* next_token) {
  if (!e || !tokens || !s || !next_token) return efail("engine_prefill: null argument");
  if (!e->finalized) return efail("engine_prefill: call nfn_engine_finalize first");
  const nfn_engine_config& c = e->c;
  if (slot < 0 || slot >= c.max_batch) return efail("engine_prefill: bad slot");
  if (n <= 0 || n >= c.max_seq) return efail("engine_prefill: the prompt must hold between 1 and max_seq - 1 tokens");
  CU(cudaSetDevice(e->device));
  const long long before = nfn_launch_count();
  // prompt tokens ride in a temporary region of the qkv buffer until the embedding has run
  int* d_tok = static_cast<int*>(e->att);
  CU(cudaMemcpyAsync(d_tok, tokens, (size_t)n * 4, cudaMemcpyHostToDevice, e->stream));
  int* d_pos = d_tok + n;
  if (c.family == 0) {
    std::vector<int> pos(n);
    for (int i = 0; i < n; ++i) pos[i] = i;
    CU(cudaMemcpyAsync(d_pos, pos.data(), (size_t)n * 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaStreamSynchronize(e->stream));  // `pos` leaves scope
    K(nfn_embedding_positions(d_tok, d_pos, e->W("wte"), e->W("wpe"), e->x, n, c.d_model, c.vocab, c.max_seq, c.embed_scale, e->stream));
  } else {
    K(nfn_embedding_positions(d_tok, nullptr, e->W("tok_embeddings"), nullptr, e->x, n, c.d_model, c.vocab, c.max_seq, c.embed_scale, e->stream));
  }
  if (c.family == 1 && c.embed_norm) K(nfn_norm_forward(e->x, e->ones, nullptr, e->x, nullptr, nullptr, n, c.d_model, c.norm_eps, 1, 0, e->stream));
  return run_prompt_rows(e, slot, n, s, next_token, before);
}

int nfn_engine_prefill_rows(nfn_engine* e, int slot, const void* rows_bf16, int n, int rows_on_device, const nfn_sampling* s, int32_t* next_token) {
  if (!e || !rows_bf16 || !s || !next_token) return efail("engine_prefill_rows: null argument");
  if (!e->finalized) return efail("engine_prefill_rows: call nfn_engine_finalize first");
  const nfn_engine_config& c = e->c;
  if (slot < 0 || slot >= c.max_batch) return efail("engine_prefill_rows: bad slot");
  if (n <= 0 || n >= c.max_seq) return efail("engine_prefill_rows: the prompt must hold between 1 and max_seq - 1 rows");
  if (c.family == 0) return efail("engine_prefill_rows: the GPT-2 layout adds learned positions to its embeddings; pass token ids");
  CU(cudaSetDevice(e->device));
  const long long before = nfn_launch_count();
  CU(cudaMemcpyAsync(e->x, rows_bf16, (size_t)n * c.d_model * 2, rows_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, e->stream));
  return run_prompt_rows(e, slot, n, s, next_token, before);
}

int nfn_engine_decode(nfn_engine* e, const int32_t* tokens_in, const uint8_t* active, const nfn_sampling* s, const nfn_sampling* per_slot,
                      int32_t* next_tokens) {
  if (!e || !tokens_in || !active || !s || !next_tokens) return efail("engine_decode: null argument");
  if (!e->finalized) return efail("engine_decode: call nfn_engine_finalize first");
  const nfn_engine_config& c = e->c;
  const int B = c.max_batch;
  CU(cudaSetDevice(e->device));
  int* tok = reinterpret_cast<int*>(e->h_io + e->io.tokens);
  int* len = reinterpret_cast<int*>(e->h_io + e->io.lengths);
  int* pos = reinterpret_cast<int*>(e->h_io + e->io.positions);
  float* rp = reinterpret_cast<float*>(e->h_io + e->io.row_params);
  int n_active = 0;
  for (int b = 0; b < B; ++b) {
    const bool on = active[b] != 0;
    if (on && e->len[b] <= 0) return efail("engine_decode: slot " + std::to_string(b) + " is active but was never prefilled");
    if (on && e->len[b] + 1 > c.max_seq) return efail("engine_decode: slot " + std::to_string(b) + " reached max_seq");
    tok[b] = on ? tokens_in[b] : 0;
    len[b] = on ? e->len[b] + 1 : 0;
    pos[b] = on ? e->len[b] : 0;
    if (e->tq) {
      // where the new token's records go: ring row of the sliding-window layers, plain row of the global ones; -1 = idle
      const int wcap = c.window > 0 ? std::min(c.window, c.max_seq) : c.max_seq;
      reinterpret_cast<int*>(e->h_io + e->io.tq_seq)[b] = on ? b : -1;
      reinterpret_cast<int*>(e->h_io + e->io.tq_slot_local)[b] = on ? e->len[b] % wcap : -1;
      reinterpret_cast<int*>(e->h_io + e->io.tq_slot_global)[b] = on ? e->len[b] : -1;
    }
    fill_params(*e, rp, b, per_slot ? per_slot[b] : *s);
    n_active += on;
  }
  if (n_active == 0) return 0;
  *reinterpret_cast<unsigned long long*>(e->h_io + e->io.offset) = (s->seed << 20) ^ (++e->steps);
  CU(cudaMemcpyAsync(e->d_io, e->h_io, (size_t)e->io.out_tokens, cudaMemcpyHostToDevice, e->stream));
  if (c.use_cuda_graph && e->graph) {
    CU(cudaGraphLaunch(e->graph, e->stream));
    e->launches += e->graph_launches;
  } else if (c.use_cuda_graph && ++e->decode_calls > 1) {
    // second decode call: everything is warm (tensor maps cached, attributes set) - capture
    const long long before = nfn_launch_count();
    cudaGraph_t g = nullptr;
    CU(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
    const int rc = decode_body(*e);
    const cudaError_t ce = cudaStreamEndCapture(e->stream, &g);
    if (rc != 0 || ce != cudaSuccess || !g) {
      if (g) cudaGraphDestroy(g);
      return rc != 0 ? -1 : efail("engine_decode: stream capture failed");
    }
    CU(cudaGraphInstantiate(&e->graph, g, 0));
    cudaGraphDestroy(g);
    e->graph_launches = nfn_launch_count() - before;
    CU(cudaGraphLaunch(e->graph, e->stream));
    e->launches += e->graph_launches;
  } else {
    const long long before = nfn_launch_count();
    if (decode_body(*e)) return -1;
    e->launches += nfn_launch_count() - before;
  }
  CU(cudaMemcpyAsync(e->h_io + e->io.out_tokens, e->d_io + e->io.out_tokens, (size_t)B * 4, cudaMemcpyDeviceToHost, e->stream));
  CU(cudaStreamSynchronize(e->stream));
  const int* out = reinterpret_cast<const int*>(e->h_io + e->io.out_tokens);
  for (int b = 0; b < B; ++b)
    if (active[b]) {
      next_tokens[b] = out[b];
      e->len[b] += 1;
      e->logit_row[b] = b;
      e->logit_src[b] = 0;
    }
  if (nfn_status_peek() != 0) return efail("engine_decode: a kernel reported error code " + std::to_string(nfn_status_read_reset()));
  return 0;
}

int nfn_engine_last_logits(nfn_engine* e, int slot, float* out_vocab) {
  if (!e || !out_vocab || slot < 0 || slot >= e->c.max_batch || !e->finalized) return efail("engine_last_logits: bad arguments");
  CU(cudaSetDevice(e->device));
  std::vector<uint16_t> tmp(e->c.vocab);
  const char* src = static_cast<const char*>(e->logit_src[slot] ? e->logits_v : e->logits);
  CU(cudaMemcpy(tmp.data(), src + (size_t)e->logit_row[slot] * e->c.padded_vocab * 2, tmp.size() * 2, cudaMemcpyDeviceToHost));
  for (int i = 0; i < e->c.vocab; ++i) {
    const uint32_t bits = (uint32_t)tmp[i] << 16;
    std::memcpy(&out_vocab[i], &bits, 4);
  }
  return 0;
}

// ---- block verification, commit, truncate, fork -------------------------------------------------

int nfn_engine_enable_verify(nfn_engine* e, int max_rows) {
  if (!e || !e->finalized) return efail("engine_enable_verify: finalize the engine first");
  if (e->tq) return efail("engine_enable_verify: verification blocks are not available with the TurboQuant cache (decode only)");
  if (e->v_rows_max > 0) return max_rows <= e->v_rows_max ? 0 : efail("engine_enable_verify: already enabled with fewer rows");
  const nfn_engine_config& c = e->c;
  if (max_rows < 1 || max_rows > 128) return efail("engine_enable_verify: 1 <= max_rows <= 128");
  if ((long long)c.max_batch * max_rows > e->rows_max)
    return efail("engine_enable_verify: max_batch * max_rows exceeds the activation rows (max(max_seq, max_batch))");
  CU(cudaSetDevice(e->device));
  const long long B = c.max_batch, rows = B * max_rows, kvw = (long long)c.n_kv_head * c.head_dim;
  e->stage_k.assign(c.n_layer, nullptr);
  e->stage_v.assign(c.n_layer, nullptr);
  for (int l = 0; l < c.n_layer; ++l)
    if (e->alloc(&e->stage_k[l], rows * kvw * 2) || e->alloc(&e->stage_v[l], rows * kvw * 2)) return -1;
  std::vector<void*> tab;
  tab.insert(tab.end(), e->stage_k.begin(), e->stage_k.end());
  tab.insert(tab.end(), e->stage_v.begin(), e->stage_v.end());
  tab.insert(tab.end(), e->kc.begin(), e->kc.end());
  tab.insert(tab.end(), e->vc.begin(), e->vc.end());
  if (e->alloc((void**)&e->d_tables, (long long)tab.size() * sizeof(void*)) || e->alloc((void**)&e->d_caps, (long long)c.n_layer * 4)) return -1;
  CU(cudaMemcpy(e->d_tables, tab.data(), tab.size() * sizeof(void*), cudaMemcpyHostToDevice));
  CU(cudaMemcpy(e->d_caps, e->cap.data(), (size_t)c.n_layer * 4, cudaMemcpyHostToDevice));
  if (e->alloc(&e->logits_v, rows * c.padded_vocab * 2)) return -1;
  e->blk_ws_bytes = nfn_block_attention_workspace_bytes(c.max_batch, std::min(max_rows, 32), c.n_head, c.n_kv_head, c.head_dim, 8);
  if (e->blk_ws_bytes <= 0) return efail("engine_enable_verify: bad attention geometry");
  if (e->alloc(&e->blk_ws, e->blk_ws_bytes)) return -1;
  CU(cudaMemset(e->blk_ws, 0, (size_t)e->blk_ws_bytes));
  if (e->alloc((void**)&e->d_vtok, rows * 4) || e->alloc((void**)&e->d_vpos, rows * 4) || e->alloc((void**)&e->d_vout, rows * 4) ||
      e->alloc((void**)&e->d_vlen, B * 4) || e->alloc((void**)&e->d_vrows, B * 4) || e->alloc(&e->argmax_ws, rows * 512))
    return -1;
  e->v_rows_max = max_rows;
  return 0;
}

int nfn_engine_verify(nfn_engine* e, const int32_t* tokens, const int32_t* n_rows, int rows, int32_t* argmax_out) {
  if (!e || !tokens || !n_rows || !argmax_out) return efail("engine_verify: null argument");
  if (e->v_rows_max <= 0) return efail("engine_verify: call nfn_engine_enable_verify first");
  if (rows < 1 || rows > e->v_rows_max) return efail("engine_verify: rows outside [1, max_rows]");
  const nfn_engine_config& c = e->c;
  const int B = c.max_batch, total = B * rows;
  CU(cudaSetDevice(e->device));
  std::vector<int> tok(total, 0), pos(total, 0), len(B, 0), live(B, 0);
  int any = 0;
  for (int b = 0; b < B; ++b) {
    const int n = n_rows[b];
    if (n < 0 || n > rows) return efail("engine_verify: n_rows[slot] outside [0, rows]");
    if (n > 0 && e->len[b] + n > c.max_seq) return efail("engine_verify: slot " + std::to_string(b) + " would pass max_seq");
    live[b] = n;
    len[b] = e->len[b];
    any += n;
    for (int r = 0; r < rows; ++r) {
      tok[b * rows + r] = r < n ? tokens[b * rows + r] : 0;
      pos[b * rows + r] = std::min(e->len[b] + r, c.max_seq - 1);
    }
  }
  if (!any) return 0;
  const long long before = nfn_launch_count();
  CU(cudaMemcpyAsync(e->d_vtok, tok.data(), (size_t)total * 4, cudaMemcpyHostToDevice, e->stream));
  CU(cudaMemcpyAsync(e->d_vpos, pos.data(), (size_t)total * 4, cudaMemcpyHostToDevice, e->stream));
  CU(cudaMemcpyAsync(e->d_vlen, len.data(), (size_t)B * 4, cudaMemcpyHostToDevice, e->stream));
  CU(cudaMemcpyAsync(e->d_vrows, live.data(), (size_t)B * 4, cudaMemcpyHostToDevice, e->stream));
  CU(cudaStreamSynchronize(e->stream));  // the host vectors leave scope at return; also orders after earlier steps
  if (c.family == 0)
    K(nfn_embedding_positions(e->d_vtok, e->d_vpos, e->W("wte"), e->W("wpe"), e->x, total, c.d_model, c.vocab, c.max_seq, c.embed_scale, e->stream));
  else
    K(nfn_embedding_positions(e->d_vtok, nullptr, e->W("tok_embeddings"), nullptr, e->x, total, c.d_model, c.vocab, c.max_seq, c.embed_scale, e->stream));
  if (c.family == 1 && c.embed_norm) K(nfn_norm_forward(e->x, e->ones, nullptr, e->x, nullptr, nullptr, total, c.d_model, c.norm_eps, 1, 0, e->stream));
  if (forward_layers(*e, total, false, 0, e->d_vlen, rows, e->d_vpos, e->d_vrows)) return -1;
  if (head(*e, 0, total, e->logits_v)) return -1;
  K(nfn_argmax_rows(e->logits_v, 0, c.padded_vocab, total, c.vocab, e->d_vout, nullptr, e->argmax_ws, (long long)B * e->v_rows_max * 512, 0, e->stream));
  CU(cudaMemcpyAsync(argmax_out, e->d_vout, (size_t)total * 4, cudaMemcpyDeviceToHost, e->stream));
  CU(cudaStreamSynchronize(e->stream));
  e->v_rows = rows;
  e->h_vrows = live;
  e->launches += nfn_launch_count() - before;
  if (nfn_status_peek() != 0) return efail("engine_verify: a kernel reported error code " + std::to_string(nfn_status_read_reset()));
  return 0;
}

int nfn_engine_verify_logits(nfn_engine* e, int slot, int row, float* out_vocab) {
  if (!e || !out_vocab || e->v_rows <= 0 || slot < 0 || slot >= e->c.max_batch || row < 0 || row >= e->h_vrows[slot])
    return efail("engine_verify_logits: no such verification row");
  CU(cudaSetDevice(e->device));
  std::vector<uint16_t> tmp(e->c.vocab);
  CU(cudaMemcpy(tmp.data(), static_cast<const char*>(e->logits_v) + ((size_t)slot * e->v_rows + row) * e->c.padded_vocab * 2, tmp.size() * 2,
                cudaMemcpyDeviceToHost));
  for (int i = 0; i < e->c.vocab; ++i) {
    const uint32_t bits = (uint32_t)tmp[i] << 16;
    std::memcpy(&out_vocab[i], &bits, 4);
  }
  return 0;
}

int nfn_engine_commit(nfn_engine* e, const int32_t* accepted) {
  if (!e || !accepted) return efail("engine_commit: null argument");
  if (e->v_rows <= 0) return efail("engine_commit: no verification to commit");
  const nfn_engine_config& c = e->c;
  const int B = c.max_batch, L = c.n_layer;
  CU(cudaSetDevice(e->device));
  std::vector<int> acc(B, 0);
  int any = 0;
  for (int b = 0; b < B; ++b) {
    if (accepted[b] < 0 || accepted[b] > e->h_vrows[b]) return efail("engine_commit: accepted[slot] outside [0, verified rows]");
    acc[b] = accepted[b];
    any += acc[b];
  }
  if (any) {
    // d_vlen still holds the lengths the verification ran at; d_vrows is reused for the accepted counts
    CU(cudaMemcpyAsync(e->d_vrows, acc.data(), (size_t)B * 4, cudaMemcpyHostToDevice, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    const long long before = nfn_launch_count();
    K(nfn_kv_commit_layers(e->d_tables, e->d_tables + L, e->d_tables + 2 * L, e->d_tables + 3 * L, e->d_caps, e->d_vlen, e->d_vrows, L, B, e->v_rows,
                           c.n_kv_head, c.head_dim, e->stream));
    CU(cudaStreamSynchronize(e->stream));
    e->launches += nfn_launch_count() - before;
  }
  for (int b = 0; b < B; ++b)
    if (acc[b] > 0) {
      e->logit_row[b] = b * e->v_rows + acc[b] - 1;
      e->logit_src[b] = 1;
      e->len[b] += acc[b];
    }
  std::fill(e->h_vrows.begin(), e->h_vrows.end(), 0);  // a verification commits once
  return 0;
}

// A ring cache keeps only the newest `cap` positions: once it has wrapped, the rows an earlier
// length would need have been overwritten, so such a slot can only be truncated to its own length.
static bool ring_prefix_intact(const nfn_engine& e, int slot, int n) {
  if (n == e.len[slot]) return true;
  for (int l = 0; l < e.c.n_layer; ++l)
    if (layer_is_local(e.c, l) && e.len[slot] > e.cap[l]) return false;
  return true;
}

int nfn_engine_truncate(nfn_engine* e, int slot, int n) {
  if (!e || slot < 0 || slot >= e->c.max_batch) return efail("engine_truncate: bad slot");
  if (n < 0 || n > e->len[slot]) return efail("engine_truncate: length outside [0, current length]");
  if (n > 0 && !ring_prefix_intact(*e, slot, n)) return efail("engine_truncate: a sliding-window cache of this slot has wrapped; only a reset is possible");
  e->len[slot] = n;
  return 0;
}

int nfn_engine_fork(nfn_engine* e, int src_slot, int dst_slot, int n) {
  if (!e || !e->finalized) return efail("engine_fork: engine not ready");
  const nfn_engine_config& c = e->c;
  if (src_slot < 0 || src_slot >= c.max_batch || dst_slot < 0 || dst_slot >= c.max_batch || src_slot == dst_slot) return efail("engine_fork: bad slots");
  if (n < 0 || n > e->len[src_slot]) return efail("engine_fork: prefix longer than the source");
  if (n > 0 && !ring_prefix_intact(*e, src_slot, n)) return efail("engine_fork: a sliding-window cache of the source has wrapped past this prefix");
  CU(cudaSetDevice(e->device));
  for (int l = 0; l < c.n_layer && n > 0; ++l) {
    // rows [0, min(n, cap)) of every kv head; whole-slot copy when most of it is live
    char* caches[2] = {static_cast<char*>(e->kc[l]), static_cast<char*>(e->vc[l])};
    const size_t row_bytes[2] = {e->tq ? (size_t)e->tq_tables.key_rec_bytes : (size_t)c.head_dim * 2,
                                 e->tq ? (size_t)e->tq_tables.value_rec_bytes : (size_t)c.head_dim * 2};
    for (int which = 0; which < 2; ++which) {
      const size_t head_bytes = (size_t)e->cap[l] * row_bytes[which], slot_bytes = head_bytes * c.n_kv_head;
      const size_t live = (size_t)std::min(n, e->cap[l]) * row_bytes[which];
      CU(cudaMemcpy2DAsync(caches[which] + dst_slot * slot_bytes, head_bytes, caches[which] + src_slot * slot_bytes, head_bytes, live, c.n_kv_head,
                           cudaMemcpyDeviceToDevice, e->stream));
    }
  }
  for (size_t t = 0; t < e->taps.size() && n > 0; ++t) {
    const size_t stride = (size_t)c.max_seq * c.d_model * 2;
    CU(cudaMemcpyAsync(static_cast<char*>(e->taps[t]) + dst_slot * stride, static_cast<char*>(e->taps[t]) + src_slot * stride,
                       (size_t)n * c.d_model * 2, cudaMemcpyDeviceToDevice, e->stream));
  }
  CU(cudaStreamSynchronize(e->stream));
  e->len[dst_slot] = n;
  return 0;
}

int nfn_engine_enable_taps(nfn_engine* e, const int32_t* layers, int n) {
  if (!e || !e->finalized || !layers) return efail("engine_enable_taps: finalize the engine first");
  if (!e->taps.empty()) return efail("engine_enable_taps: taps are already enabled");
  if (e->graph || e->decode_calls > 0) return efail("engine_enable_taps: enable taps before the first decode step (the step is captured once)");
  const nfn_engine_config& c = e->c;
  if (n < 1 || n > 8) return efail("engine_enable_taps: between 1 and 8 tap layers");
  for (int i = 0; i < n; ++i)
    if (layers[i] < 0 || layers[i] >= c.n_layer) return efail("engine_enable_taps: tap layer outside the model");
  CU(cudaSetDevice(e->device));
  for (int i = 0; i < n; ++i) {
    void* p = nullptr;
    const long long bytes = (long long)c.max_batch * c.max_seq * c.d_model * 2;
    if (e->alloc(&p, bytes)) return -1;
    CU(cudaMemset(p, 0, (size_t)bytes));
    e->taps.push_back(p);
    e->tap_layers.push_back(layers[i]);
  }
  return 0;
}

int nfn_engine_read_taps(nfn_engine* e, int slot, int pos0, int n, void* dst, int dst_on_device) {
  if (!e || !dst || e->taps.empty()) return efail("engine_read_taps: taps are not enabled");
  const nfn_engine_config& c = e->c;
  if (slot < 0 || slot >= c.max_batch || pos0 < 0 || n < 0 || pos0 + n > e->len[slot]) return efail("engine_read_taps: positions outside the slot's cached tokens");
  if (n == 0) return 0;
  CU(cudaSetDevice(e->device));
  const size_t row = (size_t)c.d_model * 2, T = e->taps.size();
  for (size_t t = 0; t < T; ++t) {
    const char* src = static_cast<const char*>(e->taps[t]) + ((size_t)slot * c.max_seq + pos0) * row;
    CU(cudaMemcpy2DAsync(static_cast<char*>(dst) + t * row, T * row, src, row, row, (size_t)n,
                         dst_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, e->stream));
  }
  CU(cudaStreamSynchronize(e->stream));
  return 0;
}

}  // extern "C"
