// C ABI of the resident inference engine: weights, KV caches and activation buffers stay on
// the device for the life of the engine; the host sends token ids and receives token ids.
//
// One engine serves up to max_batch concurrent sequences ("slots"). `prefill` runs a whole
// prompt of one slot through the tcgen05 GEMM / flash-attention path and fills that slot's
// KV cache; `decode` advances every active slot by one token in a single batched step
// (split-KV decode attention with fused QK-norm + RoPE + cache append, on-device sampling)
// which is captured into a CUDA graph on first use and replayed afterwards.
//
// Families: 0 = GPT-2 style (LayerNorm, learned positions, GELU MLP, biases, MHA, tied head),
//           1 = Llama style (RMSNorm, RoPE, grouped-query attention, SwiGLU, optional per-head
//               QK norm with weights, optional sliding-window layers with ring caches).
// Behavioural counterpart in the reference: csrc/native_gpt2/resident_dense.{h,cpp},
// resident_llama.{h,cpp} and the `_native_inference` module (resident_binding.cpp).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct nfn_engine nfn_engine;

typedef struct {
  int family;
  int n_layer, d_model, n_head, n_kv_head, head_dim, d_ff;
  int vocab, padded_vocab, max_seq, max_batch;
  int qk_norm;          // 0 none, 1 weightless, 2 with bf16 weights [head_dim]
  int rope_hf;          // rotary convention: 1 = hf, 0 = legacy (family 1)
  float rope_theta;
  float norm_eps, qk_norm_eps;
  float logit_softcap;  // 0 = off
  int tie_embeddings;
  int window;           // sliding window of local layers (0 = every layer global)
  int global_every;     // with window > 0: layers l with (l + 1) % global_every == 0 are global
  float embed_scale;    // multiplies the token embedding (1 = off)
  int use_cuda_graph;
  // Glimmer-style blocks (family 1 only); all zero = plain Llama
  int gated_attention;  // wqkv carries n_head * head_dim extra gate rows; attention output *= sigmoid(gate)
  int sandwich_norms;   // h += RMS(branch; post_*_norm) instead of h += branch (needs post_attn_norm / post_ffn_norm tensors)
  int centered_norms;   // block norms apply (1 + w); the final norm never does
  int embed_norm;       // weightless RMS norm of the token embedding
  int rope_local_only;  // rotary embedding on sliding-window layers only (global layers have no position signal)
  float q_scale;        // multiplies the normalised, rotated query (0 = 1)
  float output_multiplier;  // multiplies the logits before the soft cap (0 = 1)
  float post_norm_eps;  // epsilon of the sandwich norms (0 = norm_eps)
} nfn_engine_config;

typedef struct {
  float temperature;    // <= 0: greedy
  int top_k;            // 0: off
  float top_p;          // 0 or 1: off
  uint64_t seed;
} nfn_sampling;

int nfn_engine_abi_version(void);
const char* nfn_engine_last_error(void);
nfn_engine* nfn_engine_create(const nfn_engine_config* cfg, int device);
void nfn_engine_destroy(nfn_engine* e);
// Copies one bf16 tensor to the device under `name` (replacing any earlier one).
int nfn_engine_set_tensor(nfn_engine* e, const char* name, const void* host_bf16, long long numel);
// Names the engine expects for its configuration, '\n'-separated "name numel" lines.
int nfn_engine_expected_tensors(const nfn_engine* e, char* buf, int cap);
// Loads a dense GPT checkpoint (model_%08d.bin, version 5) into a family-0 engine.
int nfn_engine_load_dense_v5(nfn_engine* e, const char* path);
// Verifies that every expected tensor is present with the right size.
int nfn_engine_finalize(nfn_engine* e);
long long nfn_engine_device_bytes(const nfn_engine* e);

// Runs the prompt of `slot` (resets the slot first). Writes the sampled next token.
int nfn_engine_prefill(nfn_engine* e, int slot, const int32_t* tokens, int n, const nfn_sampling* s, int32_t* next_token);
// One step for all slots: tokens_in[slot] is consumed for every slot with active[slot] != 0,
// next_tokens[slot] receives its successor. per_slot (optional, max_batch entries) overrides `s`.
int nfn_engine_decode(nfn_engine* e, const int32_t* tokens_in, const uint8_t* active, const nfn_sampling* s,
                      const nfn_sampling* per_slot, int32_t* next_tokens);
int nfn_engine_release(nfn_engine* e, int slot);
int nfn_engine_slot_length(const nfn_engine* e, int slot);
// Copies the bf16 logits of the last step for `slot` to the host as fp32 (vocab entries).
int nfn_engine_last_logits(nfn_engine* e, int slot, float* out_vocab);
// Kernel launches issued so far by this engine (graph replays count their captured launches).
long long nfn_engine_launches(const nfn_engine* e);

#ifdef __cplusplus
}
#endif
