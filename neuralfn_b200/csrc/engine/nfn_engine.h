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
  int mlp_activation;   // family 0: NFN_ACT_* id of the MLP activation (0 = GELU, tanh form); mixture-of-activations checkpoints name theirs
  int kv_cache_mode;    // 0: bf16 K / V rows; 1: TurboQuant records (nfn_engine_set_turboquant before finalize; decode only, no verification blocks)
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
// A projection weight kept resident in its K-quant blocks (qtype 12 / 13 / 14 = Q4_K / Q5_K / Q6_K, the GGUF row layout).
// Products with up to eight rows read the blocks directly (quantised GEMV); larger ones decode the tensor into one shared
// bf16 scratch buffer first. Before nfn_engine_finalize; embeddings, norms and biases stay bf16.
int nfn_engine_set_tensor_kquant(nfn_engine* e, const char* name, int qtype, const void* host_blocks, long long nbytes, long long numel);
int nfn_engine_expected_tensors(const nfn_engine* e, char* buf, int cap);
// Loads a dense GPT checkpoint (model_%08d.bin, version 5) into a family-0 engine.
int nfn_engine_load_dense_v5(nfn_engine* e, const char* path);
// kv_cache_mode 1: the codec tables (device pointers that stay valid for the engine's life, see nfn_tq_tables in
// nfn_kernels.h; D must equal head_dim). K and V of every layer are then kept as compressed records - keys after QK norm
// and rotary embedding - and decode attention runs on the records. Call before nfn_engine_finalize.
int nfn_engine_set_turboquant(nfn_engine* e, const void* tq_tables);
// Verifies that every expected tensor is present with the right size.
int nfn_engine_finalize(nfn_engine* e);
long long nfn_engine_device_bytes(const nfn_engine* e);

// Runs the prompt of `slot` (resets the slot first). Writes the sampled next token.
int nfn_engine_prefill(nfn_engine* e, int slot, const int32_t* tokens, int n, const nfn_sampling* s, int32_t* next_token);
// The same for a prompt given as its layer-0 input rows (bf16 [n][d_model], host or device memory): token embeddings after
// the embedding norm, with rows replaced by projected media features where the prompt holds media placeholders.
// Llama-family layouts only (the GPT-2 layout adds learned position embeddings inside the engine).
int nfn_engine_prefill_rows(nfn_engine* e, int slot, const void* rows_bf16, int n, int rows_on_device, const nfn_sampling* s,
                            int32_t* next_token);
// One step for all slots: tokens_in[slot] is consumed for every slot with active[slot] != 0,
// next_tokens[slot] receives its successor. per_slot (optional, max_batch entries) overrides `s`.
int nfn_engine_decode(nfn_engine* e, const int32_t* tokens_in, const uint8_t* active, const nfn_sampling* s,
                      const nfn_sampling* per_slot, int32_t* next_tokens);
int nfn_engine_release(nfn_engine* e, int slot);
int nfn_engine_slot_length(const nfn_engine* e, int slot);
// Copies the bf16 logits of the last step for `slot` to the host as fp32 (vocab entries).
int nfn_engine_last_logits(nfn_engine* e, int slot, float* out_vocab);

// ---- block verification (speculative decoding, appends at a position > 0) ---------------------
// Allocates the staging buffers once (max_rows <= 128 rows per slot and call;
// max_batch * max_rows must not exceed max(max_seq, max_batch)).
int nfn_engine_enable_verify(nfn_engine* e, int max_rows);
// Runs `rows` tokens per slot (tokens[slot * rows + r]; n_rows[slot] of them live, 0 = slot not
// in this call) through the model at positions length[slot] ..., WITHOUT touching the KV caches:
// attention reads the cache prefix plus the block, the block's K/V go to per-layer staging
// buffers. argmax_out[slot * rows + r] = most likely successor after row r.
int nfn_engine_verify(nfn_engine* e, const int32_t* tokens, const int32_t* n_rows, int rows, int32_t* argmax_out);
// fp32 logits of row `row` of `slot` in the last verification.
int nfn_engine_verify_logits(nfn_engine* e, int slot, int row, float* out_vocab);
// Appends the first accepted[slot] rows of the last verification to the caches (one launch for
// all layers) and advances the slot lengths; rows that were not accepted leave no trace.
int nfn_engine_commit(nfn_engine* e, const int32_t* accepted);
// Shortens a slot to its first n tokens. Fails when a sliding-window cache of the slot has
// already wrapped (its older rows are gone).
int nfn_engine_truncate(nfn_engine* e, int slot, int n);
// Copies the first n cached tokens of src_slot into dst_slot (device-to-device; the two slots
// are independent afterwards).
int nfn_engine_fork(nfn_engine* e, int src_slot, int dst_slot, int n);

// ---- hidden-state taps (context of a block-diffusion draft model) ------------------------------
// Keeps the residual stream after each listed layer (0-based) for every cached position of every slot:
// [max_batch][max_seq][d_model] bf16 per tap. Prefill, decode steps and verification blocks all write
// their rows; rows of a block that is not committed are overwritten before they can be read. Must be
// called after finalize and before the first decode step.
int nfn_engine_enable_taps(nfn_engine* e, const int32_t* layers, int n);
// Copies positions [pos0, pos0 + n) of `slot` to dst as bf16 [n][taps * d_model] (taps side by side in
// the order they were enabled). dst is device memory when dst_on_device != 0, else host memory.
int nfn_engine_read_taps(nfn_engine* e, int slot, int pos0, int n, void* dst, int dst_on_device);
// Kernel launches issued so far by this engine (graph replays count their captured launches).
long long nfn_engine_launches(const nfn_engine* e);

#ifdef __cplusplus
}
#endif
