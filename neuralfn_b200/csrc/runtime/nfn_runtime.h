// C ABI of the host-side native runtime (libnfn_b200_runtime.so): training-data readers,
// checkpoint containers, GGUF import. Every function returns >= 0 on success and a
// negative value on failure, with the message available from nfn_rt_last_error() on the
// calling thread. Handles are opaque pointers owned by the library.
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* nfn_rt_last_error(void);
int nfn_rt_sha256_file(const char* path, char* out65);
int nfn_rt_sha256(const void* data, uint64_t bytes, char* out65);
// shipped preset catalogue compiled into the runtime (shipped_presets.h)
int nfn_rt_preset_count(void);
const char* nfn_rt_preset_name(int index);
const char* nfn_rt_preset_family(const char* name);

// ---- token / byte shard datasets -------------------------------------------------------
// On-disk formats (compatible with the reference's token_shards.cpp:48-59,151-200):
//   legacy  : optional 512-byte header starting with bytes 88 d8 34 01, then uint16 tokens
//   v2      : 512-byte header "NFNTSH2\0", u32 version=2, u32 header=512, u32 dtype=2 (uint32),
//             u32 endian=0x01020304, u64 token_count, u32 vocab, u32 flags=0, then fixed
//             strings tokenizer_sha256@40(65) revision@105(96) split@201(32) objective@233(32)
//             name@265(128), zero padding; payload uint32 tokens
//   byte    : raw uint8 stream, no header
// kind: 0 = token shards (fineweb_{train,val}_*.bin, TinyStories_{train,val}.bin, direct file),
//       1 = byte shards ({byte,hnet}_{train,val}_*.bin, bytes_{train,val}.bin).
typedef struct nfn_dataset nfn_dataset;
typedef struct nfn_sampler nfn_sampler;
typedef struct nfn_prefetcher nfn_prefetcher;

nfn_dataset* nfn_dataset_open(const char* alias_or_path, int kind, int allow_train_as_val, int require_validation);
void nfn_dataset_close(nfn_dataset* ds);
// JSON description: path, shard tables, token totals and - when seq_len > 0 - the batch plan
// (micro-batch tokens, grad-accum steps, sequences, micro-batches, optimizer steps / epoch).
int nfn_dataset_json(const nfn_dataset* ds, int64_t seq_len, int64_t batch_size, int64_t train_batch_tokens,
                     char* buf, int cap);
int64_t nfn_dataset_tokens(const nfn_dataset* ds, int split);  // split: 0 train, 1 validation
int64_t nfn_dataset_max_token(const nfn_dataset* ds, int split);

// Sequential sampler over contiguous windows: window i of a shard is tokens[i*T, i*T+T) with
// targets tokens[i*T+1, i*T+T+1); a shard yields (tokens-1)/T windows; a global batch is
// world*batch consecutive windows (across shard boundaries) of which rank r takes rows
// [r*batch, (r+1)*batch). With world == 1 this is the reference's sequential order.
nfn_sampler* nfn_sampler_open(const nfn_dataset* ds, int split, int64_t seq_len, int64_t batch_size, int rank, int world);
void nfn_sampler_close(nfn_sampler* s);
int64_t nfn_sampler_total_batches(const nfn_sampler* s);
int64_t nfn_sampler_position(const nfn_sampler* s);  // index of the next batch
// Positions the cursor at batch_index modulo total_batches (resume). Returns 0/-1.
int nfn_sampler_seek(nfn_sampler* s, int64_t batch_index);
void nfn_sampler_reset(nfn_sampler* s);
// Writes batch*seq int32 tokens and targets. Returns 1 when a batch was produced, 0 at the
// end of the epoch (cursor stays at the end; call reset/seek), negative on error.
int nfn_sampler_next_i32(nfn_sampler* s, int32_t* tokens, int32_t* targets, int64_t capacity);
// Same, wrapping around at the end of the data (never returns 0 when total_batches > 0).
int nfn_sampler_next_wrap_i32(nfn_sampler* s, int32_t* tokens, int32_t* targets, int64_t capacity);

// Background reader: one thread keeps `slots` caller-owned (pinned) buffer pairs filled in
// sampler order, wrapping at the end of the epoch. acquire() blocks until the next batch is
// ready and returns its slot; release() hands the slot back for refilling.
nfn_prefetcher* nfn_prefetcher_open(nfn_sampler* s, int slots, int32_t* const* token_bufs, int32_t* const* target_bufs,
                                    int64_t capacity);
int nfn_prefetcher_acquire(nfn_prefetcher* p, int64_t* batch_index);
int nfn_prefetcher_release(nfn_prefetcher* p, int slot);
void nfn_prefetcher_close(nfn_prefetcher* p);

// Writers (used by the dataset tools and the tests).
int nfn_write_legacy_shard(const char* path, const uint16_t* tokens, uint64_t count, int with_header);
int nfn_write_v2_shard(const char* path, const uint32_t* tokens, uint64_t count, uint32_t vocab_size,
                       const char* tokenizer_sha256, const char* tokenizer_revision, const char* split,
                       const char* objective, const char* tokenizer_name);

// ---- structured post-training records ---------------------------------------------------
// Fixed-width records behind a 512-byte header (magic NFNSFT1 / NFNPRF1 / NFNPPO1, u32
// version=1, u32 header=512, u32 endian, u32 flags=0, u64 records@24, u32 seq@32, u32 vocab@36,
// u32 pad@40, strings tokenizer_sha256@48(65) chat_template_sha256@113(65) revision@178(96)
// split@274(32) objective@306(32)):
//   kind 0 SFT        : uint32 input_ids[T], int32 targets[T] (-100 ignored), float32 loss_mask[T],
//                       int32 sequence_ids[T]
//   kind 1 preference : chosen SFT record followed by rejected SFT record
//   kind 2 PPO prompt : uint32 input_ids[T], float32 attention_mask[T] (contiguous prefix)
typedef struct nfn_records nfn_records;
nfn_records* nfn_records_open(const char* alias_or_path, int kind, int split, int allow_train_as_val, int64_t batch_size,
                              int rank, int world);
void nfn_records_close(nfn_records* r);
int nfn_records_json(const nfn_records* r, char* buf, int cap);
int64_t nfn_records_total_batches(const nfn_records* r);
int64_t nfn_records_seq_len(const nfn_records* r);
int nfn_records_seek(nfn_records* r, int64_t batch_index);
void nfn_records_reset(nfn_records* r);
// SFT: fills the four arrays (batch*T each). Preference: arrays hold 2*batch*T, chosen rows
// first. PPO prompt: input_ids and loss_mask (= attention mask); targets/sequence_ids ignored.
int nfn_records_next(nfn_records* r, int32_t* input_ids, int32_t* targets, float* loss_mask, int32_t* sequence_ids,
                     int64_t capacity);
int nfn_write_records(const char* path, int kind, uint64_t records, uint32_t seq_len, uint32_t vocab_size,
                      uint32_t pad_token_id, const char* tokenizer_sha256, const char* chat_template_sha256,
                      const char* tokenizer_revision, const char* split, const void* payload, uint64_t payload_bytes);

// ---- checkpoint containers --------------------------------------------------------------
// header + N caller-described segments. Writing is exclusive (never overwrites, follows no
// symlink, staged + fsync + link); reading demands the exact size. out_sha65 (optional)
// receives the SHA-256 of the whole file as lower-case hex + NUL.
int nfn_ckpt_write(const char* path, const void* header, uint64_t header_bytes, const void* const* segments,
                   const uint64_t* segment_bytes, int n_segments, char* out_sha65);
int nfn_ckpt_read(const char* path, void* header, uint64_t header_bytes, void* const* segments,
                  const uint64_t* segment_bytes, int n_segments, char* out_sha65);
int nfn_ckpt_peek(const char* path, void* header, uint64_t header_bytes, uint64_t* file_bytes);
int nfn_ckpt_publish_dir(const char* staging_dir, const char* final_dir);

#ifdef __cplusplus
}
#endif
