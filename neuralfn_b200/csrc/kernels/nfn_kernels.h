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
// Host-side test hook: sets the status word of the current device.
int nfn_status_set(int code);
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
       NFN_ACT_RELU2 = 4, NFN_ACT_TANH_CAP = 5 /* cap*tanh(x/cap), cap = act_param */, NFN_ACT_RELU = 6 };

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
// Grouped contraction for expert weight gradients: C[g] = A[K rows of group g, M]^T . B[same rows, N] for every group in one
// launch. Both operands MN-major; group_rows = groups + 1 device ints (multiples of 64; padding rows zero); C slices
// group_stride elements apart. Only alpha, fp32 output and accumulate of the epilogue flags apply.
int nfn_gemm_grouped_k(const nfn_gemm_args* args, const int* group_rows, int groups, long long group_stride, nfn_stream_t stream);
// Routes eligible products (K-major A and B, bf16 output, no split-K, at least one 256 x 256
// tile per SM pair) to the CTA-pair kernel (tcgen05 cta_group::2, 256 x 256 tile per 2-CTA
// cluster). Returns the previous setting. On by default; NFN_GEMM_PAIR=0 turns it off.
int nfn_gemm_set_gemv_mode(int on);  // 1 (default): M <= 2 products use the weight-streaming GEMV kernel; returns the old setting
int nfn_gemm_set_pair_mode(int on);

// ---- GEMMs fused with their collective (gemm_tp.cu) ----------------------------------------
// K-major bf16 operands: A [M, K], B [N, K] (out x in), C = A . B^T. Buffers named "peer"
// are the same allocation on every rank (symmetric memory), indexed by rank.
//   NFN_TP_AG_A: `a` is the local gathered buffer [M, K] (lda == K); this rank's rows
//                [rank * rows_per_rank, +rows_per_rank) are already in it, the other rows are
//                pulled from peer_bufs[r] inside the kernel. C [M, N] = bias/activation epilogue.
//   NFN_TP_AG_B: the same with the gathered operand on the B side (`b` [N, K], ldb == K).
//   NFN_TP_RS:   C is not written; partial tiles go to peer_bufs[owner] (bf16 slots
//                [world, rows_per_rank, N]); the kernel then reduces this rank's slots into
//                `out` [rows_per_rank, N] (+ bias + resid).
// ctrl_*: per-rank control block of ctrl_ints int32 (zero-initialised once): [0, 8) flags
// written by peers, [16] ticket, [32, 32 + blocks) block flags. epoch must grow by one per
// call on every rank alike; the value used is epoch + *epoch_dev (epoch_dev may be NULL).
//   NFN_TP_GROUPED: single-rank grouped GEMM (mixture-of-experts): A rows sorted by group and
//                padded to 128-row tiles, B = [groups, N, K]; tile t uses B[tile_group[t]];
//                only the first *num_m_tiles_dev tiles are computed (device-side count).
enum { NFN_TP_AG_A = 0, NFN_TP_AG_B = 1, NFN_TP_RS = 2, NFN_TP_GROUPED = 3 };
typedef struct {
  int mode;
  const void* a; const void* b; void* c;
  int m, n, k;
  int lda, ldb, ldc;
  int flags; float act_param; const void* bias;   // NFN_EPI_BIAS and activation bits
  int rank, world, rows_per_rank;
  int epoch; const int* epoch_dev;
  const void* peer_bufs[8];
  int* ctrl_local; int* ctrl_peer[8]; int ctrl_ints;
  void* out; int ld_out; const void* resid; int ld_resid;   // NFN_TP_RS only
  int n_copy;                                               // gather CTAs (0 = default 16)
  const int* tile_group; const int* num_m_tiles_dev; int groups;   // NFN_TP_GROUPED only
} nfn_gemm_tp_args;
int nfn_gemm_tp(const nfn_gemm_tp_args* args, nfn_stream_t stream);

// ---- one-shot all-reduce + residual + RMS norm (allreduce_fused.cu) ---------------------------
// peer_bufs[r]: rank r's copy of the symmetric bf16 [rows, ld] partial-result buffer;
// multicast_buf: multicast address of that buffer (NVSwitch reduction) or NULL for peer loads.
// resid (optional) is updated in place with sum + bias + resid; out receives the RMS-normed
// row (norm_weight != NULL) or the reduced row itself. ctrl blocks: >= 32 int32, zeroed once.
int nfn_allreduce_resid_norm(const void* const* peer_bufs, const void* multicast_buf, int* ctrl_local, int* const* ctrl_peer,
                             int rank, int world, int epoch, const int* epoch_dev, int rows, int n, int ld,
                             const void* bias, void* resid, int ld_resid, const void* norm_weight, float eps,
                             int centered, void* out, int ld_out, nfn_stream_t stream);
// Stream-ordered wait until every peer finished reading this rank's buffer in call `epoch`.
int nfn_allreduce_wait_readers(const int* ctrl_local, int world, int epoch, const int* epoch_dev, nfn_stream_t stream);

// ---- flash attention for training and prefill (attention_fwd2.cu, attention_bwd2.cu) ----------------
// q: bf16 rows [B*T] x (Hq*D) with row stride ld_q; k, v: rows x (Hkv*D); o: rows x (Hq*D);
// lse: fp32 [B, Hq, T] (optional in the forward pass). head_dim D is 64 or 128.
//   causal = 1: keys <= query.  window = W > 0: causal keys in (q - W, q], or |q - k| < W when
//   not causal.  seq_ids (optional int32 [B*T]): a key is visible only when its id equals the
//   query's (packed sequences).  softcap = c > 0: scores become c * tanh(s * scale / c).
//   gate (optional bf16 [rows, Hq*D], forward only): o *= sigmoid(gate).
// The backward pass needs delta scratch (fp32 [B, Hq, T]); it runs two kernels, one that owns a
// key block (dK, dV) and one that owns a query tile (dQ), so no gradient is accumulated with atomics.
typedef struct {
  const void* q; const void* k; const void* v; void* o; float* lse;
  int B, T, Hq, Hkv, D;
  int ld_q, ld_k, ld_v, ld_o;
  int causal, window;
  float scale, softcap;
  const int* seq_ids;
  const void* gate; int ld_gate;
  // backward only
  const void* d_o; int ld_do;
  float* delta;
  void* dq; void* dk; void* dv; int ld_dq, ld_dk, ld_dv;
} nfn_attention_args;
int nfn_attention_forward_ex(const nfn_attention_args* args, nfn_stream_t stream);
int nfn_attention_backward_ex(const nfn_attention_args* args, nfn_stream_t stream);
int nfn_attention_forward(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T, int Hq,
                          int Hkv, int D, int ld_q, int ld_k, int ld_v, int ld_o, int causal, int window, float scale,
                          nfn_stream_t stream);
int nfn_attention_backward(const void* dout, const void* q, const void* k, const void* v, const void* o, const float* lse,
                           float* delta, float* dq_accum, void* dq, void* dk, void* dv, int B, int T, int Hq, int Hkv,
                           int D, int ld_do, int ld_q, int ld_k, int ld_v, int ld_o, int ld_dq, int ld_dk, int ld_dv,
                           int causal, int window, float scale, nfn_stream_t stream);
// 2 (default): pipelined kernels; 1: the first-generation kernels (plain masks only). Returns the old value.
int nfn_attention_set_impl(int impl);

// ---- rotary embedding (rope.cu) -----------------------------------------------------------------
// In place on the q and k heads of packed rows (q | k | v). sign = +1: "hf" convention,
// -1: "legacy"; the backward pass is the same call with the opposite sign. Tables are fp32
// [max_pos, rot_dim/2]; positions (optional int32 per row) default to row % T.
int nfn_rope_inplace(void* qkv, int ld, long long tokens, int T, int n_q_heads, int n_kv_heads, int head_dim,
                     int rot_dim, const float* cos_table, const float* sin_table, const int* positions,
                     int max_pos, float sign, float q_scale, nfn_stream_t stream);
// Per-head RMS norm (optional bf16 weights [head_dim]) + rotation + query scale in one pass.
int nfn_qk_norm_rope_forward(void* qkv, int ld, long long tokens, int T, int n_q_heads, int n_kv_heads, int head_dim,
                             const void* q_weight, const void* k_weight, const float* cos_table,
                             const float* sin_table, const int* positions, int max_pos, float sign, float eps,
                             float q_scale, float* rstd_out, nfn_stream_t stream);

// ---- token selection (sampling.cu) --------------------------------------------------------------
// logits: bf16 (is_fp32 = 0) or fp32 rows of V entries, row stride ld. Ties go to the lowest
// index. index_offset is added to every result (vocabulary shard offset under tensor
// parallelism). argmax workspace: rows * 8 bytes at least, rows * 512 for full parallelism.
int nfn_argmax_rows(const void* logits, int is_fp32, long long ld, int rows, int V, int* out_idx, float* out_val,
                    void* workspace, long long workspace_bytes, int index_offset, nfn_stream_t stream);
// Merges per-rank winners laid out [world, rows] (values and already-offset indices).
int nfn_argmax_merge(const float* vals, const int* idx, int world, int rows, int* out_idx, float* out_val,
                     nfn_stream_t stream);
// temperature <= 0 or top_k == 1: greedy. top_k = 0 and top_p in {0, 1}: no truncation.
// row_params (optional, fp32 [rows, 3] = temperature, top_k, top_p) overrides the scalars per
// row. Randomness: Philox4x32-10 keyed by seed, counter (element/4, row, offset + *offset_dev).
int nfn_sample_rows(const void* logits, int is_fp32, long long ld, int rows, int V, int* out_idx, float* out_logprob,
                    float temperature, int top_k, float top_p, const float* row_params, unsigned long long seed,
                    unsigned long long offset, const unsigned long long* offset_dev, int index_offset,
                    nfn_stream_t stream);

// ---- decode attention (decode_attention.cu) -----------------------------------------------------
// One new token per sequence. qkv: bf16 [B, ld] packed (q | k | v) rows of the new token;
// caches: bf16 [B, n_kv_heads, cap, head_dim] with cache_batch_stride elements between
// sequences; lengths[b] counts the new token; out: bf16 [B, n_q_heads * head_dim]. The call
// appends the (normed, rotated) k and v of the new token at slot (len - 1) % cap. The
// workspace must be zero-filled once before its first use and is left ready for the next call.
long long nfn_decode_attention_workspace_bytes(int B, int n_q_heads, int n_kv_heads, int head_dim, int max_splits);
// 1 (default): mma.sync kernel, 16 cache positions per warp step; 0: SIMT kernel. Returns the previous setting.
int nfn_decode_attention_set_impl(int impl);
int nfn_decode_attention(const void* qkv, int ld, void* k_cache, void* v_cache, long long cache_batch_stride,
                         const int* lengths, void* out, int B, int n_q_heads, int n_kv_heads, int head_dim, int cap,
                         const void* q_norm_weight, const void* k_norm_weight, int qk_norm, float eps,
                         const float* cos_table, const float* sin_table, int max_pos, float rope_sign, float scale,
                         void* workspace, long long workspace_bytes, int splits, nfn_stream_t stream);

// ---- block attention over a KV cache (block_attention.cu) ------------------------------------------
// `rows` (<= 128) new rows per sequence attend to the sequence's cached keys plus the block's own
// keys; the caches are only read. qkv: [B*rows, ld] packed q | k | v (norm / rotary already
// applied); caches [B][n_kv_heads][cap][head_dim]; lengths[b] = tokens already cached (the block
// starts at that position); n_rows (optional) = live rows per sequence, 0 skips the sequence.
// window = 0: every cached key is visible; otherwise keys inside (q - window, q] (window <= cap).
// causal = 0 lets every block row see the whole block (draft blocks). stage_k / stage_v
// (optional, [B*rows, n_kv_heads*head_dim]) receive the block's own K / V rows for a later
// nfn_kv_commit_layers. splits = 0 picks the KV split count.
long long nfn_block_attention_workspace_bytes(int B, int rows, int n_q_heads, int n_kv_heads, int head_dim, int max_splits);
int nfn_block_attention(const void* qkv, int ld, const void* k_cache, const void* v_cache, const int* lengths, const int* n_rows,
                        void* out, int ld_o, void* stage_k, void* stage_v, int B, int rows, int n_q_heads, int n_kv_heads,
                        int head_dim, int cap, int window, int causal, float scale, void* workspace, long long workspace_bytes,
                        int splits, nfn_stream_t stream);
// Appends the first accepted[b] staged rows of every layer to that layer's cache at positions
// lengths[b] ... (ring rows position % caps[layer]). All pointer arrays live in device memory.
int nfn_kv_commit_layers(const void* const* stage_k, const void* const* stage_v, void* const* k_caches, void* const* v_caches,
                         const int* caps, const int* lengths, const int* accepted, int n_layers, int B, int rows, int n_kv_heads,
                         int head_dim, nfn_stream_t stream);

// Products with a few rows over large K-major weights (decode batches, verification blocks): 1 (default) = 3 - 16 rows take the
// mma.sync weight-streaming kernel of gemm_skinny.cu, 2 = up to 64 rows do, 0 = none (tcgen05 split-K path). Returns the previous setting.
int nfn_gemm_skinny_set_impl(int mode);

// Hidden-state taps: row r of x (bf16 [rows, ldx], C columns used) belongs to sequence r / block_rows and is copied to
// position lengths[sequence] + r % block_rows + pos_offset of dst [sequences][max_pos][C] (slot_stride elements between
// sequences). live_rows (optional): rows at or past live_rows[sequence] are skipped. Positions outside [0, max_pos) are skipped.
int nfn_rows_to_slots(const void* x, int ldx, int rows, int C, void* dst, long long slot_stride, int max_pos, const int* lengths,
                      int block_rows, int pos_offset, const int* live_rows, nfn_stream_t stream);

// ---- GEMM over K-quant weights, dequantisation fused into the operand pipeline (gemm_kquant.cu) ----
// C[M, N] = A[M, K] . dequant(W)^T with args->b pointing at N rows of K / 256 super-blocks
// (qtype: NFN_QTYPE_Q4_K / Q5_K / Q6_K, declared below). K-major A, bf16 output, the bias /
// activation / residual epilogues of nfn_gemm_bf16; ldb, a_mn, b_mn and split_k are ignored or refused.
int nfn_gemm_kquant(int qtype, const nfn_gemm_args* args, nfn_stream_t stream);
// The same with NF4 base weights (qtype NFN_QTYPE_NF4: args->b = N rows of K / 2 code bytes, low
// nibble = even element; absmax fp32 [N, K / 64]) and / or a fused LoRA branch: lora_t = bf16
// [M, >= 64] holding scale * (x A^T) in its first r columns and zeros up to column 64, lora_b =
// bf16 [N, >= 64] holding the adapter's B matrix likewise. Pass NULL adapters for none.
int nfn_gemm_quant_lora(int qtype, const nfn_gemm_args* args, const float* absmax, const void* lora_t, int ld_t,
                        const void* lora_b, int ld_b, nfn_stream_t stream);

// ---- TurboQuant KV cache (turboquant.cu) ------------------------------------------------------------
// Device tables of one codec: rotation / projection [D, D] fp32 (rotated = R x), centroids [5][16]
// fp32 (row = bit width), fields [D][2] int32 (bit offset inside the index area, width).
// Record: [norm f32 | residual norm f32 + D/8 sign bytes (qjl keys) | packed indices | pad to 16].
typedef struct {
  const float* rotation; const float* projection; const float* centroids;
  const int* key_fields; const int* value_fields;
  int D, qjl, key_rec_bytes, value_rec_bytes;
} nfn_tq_tables;
// Encodes head vectors x[row, h * D ...] (bf16, row stride ld) into records[seq[row]][h][slot[row]].
int nfn_turboquant_encode(const nfn_tq_tables* tables, const void* x, long long ld, const int* seq, const int* slot, int rows,
                          int n_heads, int cap, int is_key, void* records, nfn_stream_t stream);
// One query row per sequence against records [B][n_kv_heads][cap]; the first min(lengths[b], cap)
// rows of every head are live. q: bf16 [B, ld_q]; out: bf16 [B, ld_o].
int nfn_turboquant_attention(const nfn_tq_tables* tables, const void* q, int ld_q, const void* k_records, const void* v_records,
                             const int* lengths, void* out, int ld_o, int B, int n_q_heads, int n_kv_heads, int cap, float scale,
                             nfn_stream_t stream);

// ---- quantised weights (quant.cu) ---------------------------------------------------------------
enum { NFN_QTYPE_Q4_K = 12, NFN_QTYPE_Q5_K = 13, NFN_QTYPE_Q6_K = 14, NFN_QTYPE_NF4 = 100 };  // GGUF type ids; NF4 is this library's own
int nfn_quant_block_bytes(int qtype);
int nfn_dequant_kquant(int qtype, const void* blocks, long long n_blocks, void* out_bf16, nfn_stream_t stream);
int nfn_dequant_nf4(const void* codes, const float* absmax, long long n_weights, int group, void* out_bf16,
                    nfn_stream_t stream);
// y[b, n] = W1[n, :] . x[b, :]  (silu(W1 x) * (W2 x) when w2 != NULL) + bias[n] + resid[b, n];
// W rows are K/256 consecutive super-blocks; B <= 8.
int nfn_kquant_gemv(int qtype, const void* w1, const void* w2, const void* x, int ldx, void* y, int ldy,
                    const void* bias, const void* resid, int ld_resid, int B, int N, int K, nfn_stream_t stream);

int nfn_allreduce_sandwich_norm(const void* const* peer_bufs, const void* multicast_buf, int* ctrl_local, int* const* ctrl_peer,
                                int rank, int world, int epoch, const int* epoch_dev, int rows, int n, int ld, const void* bias,
                                const void* post_weight, float post_eps, void* resid, int ld_resid, const void* norm_weight,
                                float eps, int centered, void* out, int ld_out, nfn_stream_t stream);

// ---- gated attention, training (gate.cu) ----
int nfn_sigmoid_gate_forward(const void* att, int ld_att, const void* gate, int ld_gate, void* out, int ld_out, long long rows, int width,
                             nfn_stream_t stream);
int nfn_sigmoid_gate_backward(const void* dout, int ld_dout, const void* att, int ld_att, const void* gate, int ld_gate, void* datt,
                              int ld_datt, void* dgate, int ld_dgate, long long rows, int width, nfn_stream_t stream);

// ---- counter-based dropout for the LoRA adapter branch (dropout.cu) ----
// out (+)= keep ? x / (1 - p) : 0 with keep = f(seed, stream_id, *step_dev, row, column): calling it again with the same ids
// reproduces the mask (backward pass, recomputation). bf16 [rows, width], width a multiple of 8.
int nfn_dropout_apply(const void* x, int ld_x, void* out, int ld_out, long long rows, int width, float p, unsigned long long seed,
                      int stream_id, const long long* step_dev, int accumulate, nfn_stream_t stream);

// ---- differential attention glue (diff_attention.cu) ----
int nfn_diff_partials(void);
int nfn_diff_q_expand(const void* q, int ldq, void* q2, long long tokens, int H, int D, nfn_stream_t stream);
int nfn_diff_q_collapse(const void* dq2, void* dq, int lddq, long long tokens, int H, int D, nfn_stream_t stream);
int nfn_diff_combine(const void* a, const void* lambda, float out_scale, float eps, void* out, float* rstd,
                     long long tokens, int H, int D, nfn_stream_t stream);
int nfn_diff_combine_backward(const void* dout, const void* a, const void* lambda, float out_scale, const float* rstd,
                              void* da, float* partial, void* dlambda, long long tokens, int H, int D, nfn_stream_t stream);

#ifdef __cplusplus
}
#endif
