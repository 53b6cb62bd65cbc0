// Token / byte shard datasets, the sequential window sampler and the background prefetcher.
//
// Layout choices: every shard is memory-mapped once per sampler and windows are addressed
// through a prefix table of window counts, so `seek` is a binary search and a batch is a
// handful of widening copies straight from the page cache into the caller's (pinned)
// int32 staging buffer - the dtype the device-side embedding kernel consumes.
#include <algorithm>
#include <condition_variable>
#include <cstdlib>
#include <filesystem>
#include <fstream>
#include <memory>
#include <mutex>
#include <thread>

#include "nfn_runtime.h"
#include "runtime_common.h"

namespace fs = std::filesystem;
using namespace nfnrt;

namespace {

constexpr std::uint32_t kV2Header = 512, kEndian = 0x01020304u;
const unsigned char kV2Magic[8] = {'N', 'F', 'N', 'T', 'S', 'H', '2', 0};
const unsigned char kLegacyMagic[4] = {0x88, 0xd8, 0x34, 0x01};

struct Shard {
  std::string path;
  std::uint64_t bytes = 0, header_bytes = 0, tokens = 0;
  int elem_bytes = 2;  // 1 byte stream, 2 legacy uint16, 4 v2 uint32
  std::uint32_t vocab = 0, max_token = 0;
  std::string tokenizer_sha256, tokenizer_revision, split, objective, tokenizer_name;
};

std::uint32_t scan_max(const unsigned char* p, std::uint64_t n, int elem) {
  std::uint32_t mx = 0;
  if (elem == 1) {
    for (std::uint64_t i = 0; i < n; ++i) mx = std::max<std::uint32_t>(mx, p[i]);
  } else if (elem == 2) {
    for (std::uint64_t i = 0; i < n; ++i) mx = std::max<std::uint32_t>(mx, (std::uint32_t)p[2 * i] | ((std::uint32_t)p[2 * i + 1] << 8));
  } else {
    for (std::uint64_t i = 0; i < n; ++i) mx = std::max(mx, le32(p + 4 * i));
  }
  return mx;
}

Shard probe_shard(const std::string& path, int kind) {
  Shard s;
  s.path = path;
  s.bytes = fs::file_size(path);
  if (kind == 1) {
    s.elem_bytes = 1;
    s.tokens = s.bytes;
    if (s.tokens < 2) throw std::runtime_error("byte shard is too small: " + path);
    MappedFile m(path);
    s.max_token = scan_max(m.data(), s.tokens, 1);
    s.vocab = 256;
    return s;
  }
  MappedFile m(path);
  if (m.size() >= 8 && std::memcmp(m.data(), kV2Magic, 8) == 0) {
    if (m.size() < kV2Header) throw std::runtime_error("token shard v2 is smaller than its header: " + path);
    const unsigned char* h = m.data();
    const std::uint32_t version = le32(h + 8), header = le32(h + 12), dtype = le32(h + 16), endian = le32(h + 20);
    const std::uint64_t count = le64(h + 24);
    const std::uint32_t vocab = le32(h + 32), flags = le32(h + 36);
    if (version != 2 || header != kV2Header) throw std::runtime_error("unsupported token shard v2 version/header size: " + path);
    if (dtype != 2) throw std::runtime_error("unsupported token shard v2 dtype code " + std::to_string(dtype) + ": " + path);
    if (endian != kEndian) throw std::runtime_error("token shard v2 endian marker mismatch: " + path);
    if (count == 0 || vocab == 0 || flags != 0) throw std::runtime_error("invalid token shard v2 token count, vocab, or flags: " + path);
    if (count > (UINT64_MAX - header) / 4 || s.bytes != header + count * 4)
      throw std::runtime_error("token shard v2 byte size does not match token_count: " + path);
    s.tokenizer_sha256 = fixed_field(h, 40, 65, "tokenizer_sha256");
    s.tokenizer_revision = fixed_field(h, 105, 96, "tokenizer_revision");
    s.split = fixed_field(h, 201, 32, "split");
    s.objective = fixed_field(h, 233, 32, "objective");
    s.tokenizer_name = fixed_field(h, 265, 128, "tokenizer_name");
    if (!is_lower_hex_sha256(s.tokenizer_sha256) || s.tokenizer_revision.empty() || s.tokenizer_name.empty() ||
        (s.split != "train" && s.split != "validation" && s.split != "test") ||
        (s.objective != "ar" && s.objective != "pretrain"))
      throw std::runtime_error("invalid token shard v2 tokenizer/split/objective metadata: " + path);
    for (std::size_t i = 393; i < kV2Header; ++i)
      if (h[i] != 0) throw std::runtime_error("token shard v2 reserved header bytes must be zero: " + path);
    s.header_bytes = header;
    s.elem_bytes = 4;
    s.tokens = count;
    s.vocab = vocab;
    s.max_token = scan_max(h + header, count, 4);
    if (s.max_token >= vocab) throw std::runtime_error("token shard v2 holds a token id >= its vocab size: " + path);
    return s;
  }
  s.header_bytes = (m.size() >= 4 && std::memcmp(m.data(), kLegacyMagic, 4) == 0) ? 512 : 0;
  if (s.bytes < s.header_bytes + 4 || ((s.bytes - s.header_bytes) % 2) != 0)
    throw std::runtime_error("legacy uint16 token shard has an odd or empty payload: " + path);
  s.elem_bytes = 2;
  s.tokens = (s.bytes - s.header_bytes) / 2;
  s.max_token = scan_max(m.data() + s.header_bytes, s.tokens, 2);
  s.vocab = 65536;
  return s;
}

std::string datasets_dir() {
  if (const char* v = std::getenv("NFN_DATASETS_DIR"); v != nullptr && *v) return v;
  const char* home = std::getenv("HOME");
  return (fs::path(home ? home : ".") / ".cache" / "nfn" / "datasets").string();
}

std::vector<std::string> files_with_prefix(const fs::path& dir, const std::vector<std::string>& prefixes, const std::string& ext) {
  std::vector<std::string> out;
  if (!fs::is_directory(dir)) return out;
  for (const auto& entry : fs::directory_iterator(dir)) {
    if (!entry.is_regular_file() || entry.path().extension() != ext) continue;
    const std::string name = entry.path().filename().string();
    for (const auto& p : prefixes)
      if (name.rfind(p, 0) == 0) {
        out.push_back(entry.path().string());
        break;
      }
  }
  std::sort(out.begin(), out.end());
  return out;
}

std::vector<std::string> files_with_stem(const fs::path& dir, const std::vector<std::string>& stems, const std::string& ext) {
  std::vector<std::string> out;
  for (const auto& stem : stems) {
    const fs::path p = dir / (stem + ext);
    if (fs::is_regular_file(p)) out.push_back(p.string());
  }
  return out;
}

// a direct "..._train..." file implies its "..._val..." sibling
std::string sibling_validation(const fs::path& train) {
  const std::string name = train.filename().string();
  for (const char* from : {"_train", "train"}) {
    const auto pos = name.find(from);
    if (pos == std::string::npos) continue;
    for (const char* to : {"val", "valid", "validation"}) {
      std::string cand = name;
      const std::string rep = (from[0] == '_') ? std::string("_") + to : std::string(to);
      cand.replace(pos, std::strlen(from), rep);
      const fs::path p = train.parent_path() / cand;
      if (fs::is_regular_file(p)) return p.string();
    }
  }
  return {};
}

}  // namespace

struct nfn_dataset {
  std::string path;
  int kind = 0;
  std::vector<Shard> train, val;
  std::uint64_t train_tokens = 0, val_tokens = 0;
};

namespace {

fs::path resolve_path(const std::string& alias_or_path) {
  fs::path p(alias_or_path);
  if (p.is_absolute() || fs::exists(p)) return p;
  return fs::path(datasets_dir()) / alias_or_path;
}

std::unique_ptr<nfn_dataset> open_dataset(const std::string& alias_or_path, int kind, bool train_as_val, bool need_val) {
  auto ds = std::make_unique<nfn_dataset>();
  ds->kind = kind;
  const fs::path root = resolve_path(alias_or_path);
  ds->path = root.string();
  std::vector<std::string> train, val;
  if (fs::is_regular_file(root)) {
    train = {root.string()};
    if (need_val) {
      const std::string v = sibling_validation(root);
      if (!v.empty()) val = {v};
    }
  } else if (fs::is_directory(root)) {
    if (kind == 0) {
      train = files_with_prefix(root, {"fineweb_train_"}, ".bin");
      if (train.empty()) train = files_with_stem(root, {"TinyStories_train", "TinyStoriesV2-GPT4_train", "train"}, ".bin");
      if (need_val) {
        val = files_with_prefix(root, {"fineweb_val_"}, ".bin");
        if (val.empty())
          val = files_with_stem(root, {"TinyStories_val", "TinyStories_valid", "TinyStoriesV2-GPT4_val", "TinyStoriesV2-GPT4_valid", "val", "valid"}, ".bin");
      }
    } else {
      train = files_with_prefix(root, {"byte_train_", "hnet_train_"}, ".bin");
      if (train.empty()) train = files_with_stem(root, {"bytes_train", "hnet_train"}, ".bin");
      if (need_val) {
        val = files_with_prefix(root, {"byte_val_", "hnet_val_"}, ".bin");
        if (val.empty()) val = files_with_stem(root, {"bytes_val", "bytes_valid", "hnet_val", "hnet_valid"}, ".bin");
      }
    }
  } else {
    throw std::runtime_error("dataset directory not found: " + root.string());
  }
  if (train.empty())
    throw std::runtime_error("no native train shard found under " + root.string() +
                             (kind == 0 ? " (expected fineweb_train_*.bin, TinyStories_train.bin or train.bin)"
                                        : " (expected byte_train_*.bin or bytes_train.bin)"));
  for (const auto& p : train) ds->train.push_back(probe_shard(p, kind));
  for (const auto& p : val) ds->val.push_back(probe_shard(p, kind));
  if (need_val && ds->val.empty()) {
    if (!train_as_val) throw std::runtime_error("no native validation shard found under " + root.string());
    ds->val = ds->train;
  }
  for (const auto& s : ds->train) ds->train_tokens += s.tokens;
  for (const auto& s : ds->val) ds->val_tokens += s.tokens;
  return ds;
}

std::string shard_json(const Shard& s) {
  JsonObject o;
  o.add("path", s.path).add("bytes", s.bytes).add("header_bytes", s.header_bytes).add("tokens", s.tokens);
  o.add("element_bytes", s.elem_bytes);
  o.add("dtype", s.elem_bytes == 4 ? "uint32_le" : (s.elem_bytes == 2 ? "legacy_uint16_le" : "uint8"));
  o.add("tokenizer_vocab_size", (std::int64_t)s.vocab).add("max_token_id", (std::int64_t)s.max_token);
  if (s.elem_bytes == 4) {
    o.add("tokenizer_sha256", s.tokenizer_sha256).add("tokenizer_revision", s.tokenizer_revision);
    o.add("split", s.split).add("objective", s.objective).add("tokenizer_name", s.tokenizer_name);
  }
  return o.str();
}

std::int64_t windows_of(const std::vector<Shard>& v, std::int64_t T) {
  std::int64_t n = 0;
  for (const auto& s : v) n += s.tokens > 0 ? (std::int64_t)((s.tokens - 1) / (std::uint64_t)T) : 0;
  return n;
}
std::int64_t cdiv(std::int64_t a, std::int64_t b) { return (a + b - 1) / b; }

}  // namespace

struct nfn_sampler {
  std::vector<Shard> shards;
  std::vector<MappedFile> maps;
  std::vector<std::int64_t> first_window;  // prefix sums, size shards+1
  std::int64_t T = 0, B = 0, total_batches = 0, cursor = 0;
  int rank = 0, world = 1;

  void copy_window(std::int64_t w, std::int32_t* tok, std::int32_t* tgt) const {
    const std::size_t si = std::upper_bound(first_window.begin(), first_window.end(), w) - first_window.begin() - 1;
    const Shard& s = shards[si];
    const std::uint64_t start = (std::uint64_t)(w - first_window[si]) * (std::uint64_t)T;
    const unsigned char* base = maps[si].data() + s.header_bytes + start * (std::uint64_t)s.elem_bytes;
    if (s.elem_bytes == 4) {
      // little-endian host: the payload is already int32-compatible
      std::memcpy(tok, base, (std::size_t)T * 4);
      std::memcpy(tgt, base + 4, (std::size_t)T * 4);
    } else if (s.elem_bytes == 2) {
      const std::uint16_t* p = reinterpret_cast<const std::uint16_t*>(base);
      std::int32_t prev = p[0];
      for (std::int64_t i = 0; i < T; ++i) {
        const std::int32_t nxt = p[i + 1];
        tok[i] = prev;
        tgt[i] = nxt;
        prev = nxt;
      }
    } else {
      for (std::int64_t i = 0; i < T; ++i) {
        tok[i] = base[i];
        tgt[i] = base[i + 1];
      }
    }
  }

  bool fill(std::int64_t batch, std::int32_t* tok, std::int32_t* tgt) const {
    if (batch < 0 || batch >= total_batches) return false;
    const std::int64_t w0 = (batch * world + rank) * B;
    for (std::int64_t r = 0; r < B; ++r) copy_window(w0 + r, tok + r * T, tgt + r * T);
    return true;
  }
};

struct nfn_prefetcher {
  nfn_sampler* sampler = nullptr;
  std::vector<std::int32_t*> tok, tgt;
  std::vector<int> state;            // 0 free, 1 ready, 2 held by the consumer
  std::vector<std::int64_t> index;   // batch index held by each slot
  std::int64_t next_fill = 0;        // batch the worker reads next
  int fill_slot = 0, take_slot = 0;
  bool stop = false, failed = false;
  std::string failure;
  std::mutex mu;
  std::condition_variable cv;
  std::thread worker;

  void run() {
    for (;;) {
      int slot;
      std::int64_t batch;
      {
        std::unique_lock<std::mutex> lk(mu);
        cv.wait(lk, [&] { return stop || state[fill_slot] == 0; });
        if (stop) return;
        slot = fill_slot;
        batch = next_fill;
      }
      bool ok = false;
      try {
        ok = sampler->fill(batch % sampler->total_batches, tok[slot], tgt[slot]);
        if (!ok) failure = "prefetcher: sampler produced no batch";
      } catch (const std::exception& e) {
        failure = e.what();
      }
      {
        std::lock_guard<std::mutex> lk(mu);
        if (!ok) {
          failed = true;
          cv.notify_all();
          return;
        }
        state[slot] = 1;
        index[slot] = batch;
        fill_slot = (fill_slot + 1) % (int)state.size();
        ++next_fill;
      }
      cv.notify_all();
    }
  }
};

extern "C" {

nfn_dataset* nfn_dataset_open(const char* alias_or_path, int kind, int allow_train_as_val, int require_validation) {
  nfn_dataset* out = nullptr;
  guarded([&] {
    if (alias_or_path == nullptr || (kind != 0 && kind != 1)) throw std::runtime_error("dataset_open: bad arguments");
    out = open_dataset(alias_or_path, kind, allow_train_as_val != 0, require_validation != 0).release();
    return 0;
  });
  return out;
}

void nfn_dataset_close(nfn_dataset* ds) { delete ds; }

int64_t nfn_dataset_tokens(const nfn_dataset* ds, int split) { return ds ? (int64_t)(split ? ds->val_tokens : ds->train_tokens) : -1; }

int64_t nfn_dataset_max_token(const nfn_dataset* ds, int split) {
  if (!ds) return -1;
  std::uint32_t mx = 0;
  for (const auto& s : (split ? ds->val : ds->train)) mx = std::max(mx, s.max_token);
  return mx;
}

int nfn_dataset_json(const nfn_dataset* ds, int64_t seq_len, int64_t batch_size, int64_t train_batch_tokens, char* buf, int cap) {
  return guarded([&] {
    if (!ds) throw std::runtime_error("dataset_json: null dataset");
    JsonObject o;
    o.add("dataset_path", ds->path).add("kind", ds->kind == 0 ? "token" : "byte");
    std::vector<std::string> tr, va;
    for (const auto& s : ds->train) tr.push_back(shard_json(s));
    for (const auto& s : ds->val) va.push_back(shard_json(s));
    o.add_raw("train_shards", json_array(tr)).add_raw("val_shards", json_array(va));
    o.add("train_tokens", ds->train_tokens).add("val_tokens", ds->val_tokens);
    if (seq_len > 0 && batch_size > 0) {
      if (train_batch_tokens <= 0) train_batch_tokens = seq_len * batch_size;
      JsonObject p;
      const std::int64_t micro = seq_len * batch_size, accum = cdiv(train_batch_tokens, micro);
      const std::int64_t tseq = windows_of(ds->train, seq_len), vseq = windows_of(ds->val, seq_len);
      p.add("microbatch_tokens", micro).add("grad_accum_steps", accum).add("effective_train_batch_tokens", accum * micro);
      p.add("train_sequences", tseq).add("train_microbatches", cdiv(tseq, batch_size));
      p.add("train_optimizer_steps_per_epoch", cdiv(cdiv(tseq, batch_size), accum));
      p.add("val_sequences", vseq).add("val_microbatches", cdiv(vseq, batch_size));
      o.add_raw("batch_plan", p.str());
    }
    return copy_out(o.str(), buf, cap);
  });
}

nfn_sampler* nfn_sampler_open(const nfn_dataset* ds, int split, int64_t seq_len, int64_t batch_size, int rank, int world) {
  nfn_sampler* out = nullptr;
  guarded([&] {
    if (!ds || seq_len <= 0 || batch_size <= 0 || world <= 0 || rank < 0 || rank >= world)
      throw std::runtime_error("sampler_open: bad arguments");
    auto s = std::make_unique<nfn_sampler>();
    s->shards = split ? ds->val : ds->train;
    s->T = seq_len;
    s->B = batch_size;
    s->rank = rank;
    s->world = world;
    s->first_window.push_back(0);
    for (const auto& sh : s->shards) {
      s->maps.emplace_back(sh.path);
      if (s->maps.back().size() != sh.bytes) throw std::runtime_error("shard changed size since it was validated: " + sh.path);
      s->first_window.push_back(s->first_window.back() + (sh.tokens > 0 ? (std::int64_t)((sh.tokens - 1) / (std::uint64_t)seq_len) : 0));
    }
    s->total_batches = s->first_window.back() / (batch_size * world);
    out = s.release();
    return 0;
  });
  return out;
}

void nfn_sampler_close(nfn_sampler* s) { delete s; }
int64_t nfn_sampler_total_batches(const nfn_sampler* s) { return s ? s->total_batches : -1; }
int64_t nfn_sampler_position(const nfn_sampler* s) { return s ? s->cursor : -1; }
void nfn_sampler_reset(nfn_sampler* s) {
  if (s) s->cursor = 0;
}

int nfn_sampler_seek(nfn_sampler* s, int64_t batch_index) {
  if (!s || batch_index < 0 || s->total_batches <= 0) {
    set_error("sampler_seek: negative index or empty sampler");
    return -1;
  }
  s->cursor = batch_index % s->total_batches;
  return 0;
}

int nfn_sampler_next_i32(nfn_sampler* s, int32_t* tokens, int32_t* targets, int64_t capacity) {
  return guarded([&] {
    if (!s || !tokens || !targets) throw std::runtime_error("sampler_next: null argument");
    if (capacity < s->B * s->T) throw std::runtime_error("sampler_next: destination smaller than batch_size * seq_len");
    if (!s->fill(s->cursor, tokens, targets)) return 0;
    ++s->cursor;
    return 1;
  });
}

int nfn_sampler_next_wrap_i32(nfn_sampler* s, int32_t* tokens, int32_t* targets, int64_t capacity) {
  if (s && s->total_batches > 0 && s->cursor >= s->total_batches) s->cursor = 0;
  return nfn_sampler_next_i32(s, tokens, targets, capacity);
}

nfn_prefetcher* nfn_prefetcher_open(nfn_sampler* s, int slots, int32_t* const* token_bufs, int32_t* const* target_bufs, int64_t capacity) {
  nfn_prefetcher* out = nullptr;
  guarded([&] {
    if (!s || slots < 2 || !token_bufs || !target_bufs) throw std::runtime_error("prefetcher_open: need a sampler and >= 2 slots");
    if (capacity < s->B * s->T) throw std::runtime_error("prefetcher_open: slot smaller than batch_size * seq_len");
    if (s->total_batches <= 0) throw std::runtime_error("prefetcher_open: the sampler has no full batch");
    auto p = std::make_unique<nfn_prefetcher>();
    p->sampler = s;
    p->tok.assign(token_bufs, token_bufs + slots);
    p->tgt.assign(target_bufs, target_bufs + slots);
    p->state.assign(slots, 0);
    p->index.assign(slots, -1);
    p->next_fill = s->cursor;
    p->worker = std::thread([raw = p.get()] { raw->run(); });
    out = p.release();
    return 0;
  });
  return out;
}

int nfn_prefetcher_acquire(nfn_prefetcher* p, int64_t* batch_index) {
  if (!p) return -1;
  std::unique_lock<std::mutex> lk(p->mu);
  p->cv.wait(lk, [&] { return p->failed || p->state[p->take_slot] == 1; });
  if (p->failed) {
    set_error(p->failure);
    return -1;
  }
  const int slot = p->take_slot;
  p->state[slot] = 2;
  p->take_slot = (slot + 1) % (int)p->state.size();
  if (batch_index) *batch_index = p->index[slot];
  p->sampler->cursor = (p->index[slot] + 1) % p->sampler->total_batches;
  return slot;
}

int nfn_prefetcher_release(nfn_prefetcher* p, int slot) {
  if (!p || slot < 0 || slot >= (int)p->state.size()) return -1;
  {
    std::lock_guard<std::mutex> lk(p->mu);
    if (p->state[slot] != 2) {
      set_error("prefetcher_release: slot is not held");
      return -1;
    }
    p->state[slot] = 0;
  }
  p->cv.notify_all();
  return 0;
}

void nfn_prefetcher_close(nfn_prefetcher* p) {
  if (!p) return;
  {
    std::lock_guard<std::mutex> lk(p->mu);
    p->stop = true;
  }
  p->cv.notify_all();
  if (p->worker.joinable()) p->worker.join();
  delete p;
}

int nfn_write_legacy_shard(const char* path, const uint16_t* tokens, uint64_t count, int with_header) {
  return guarded([&] {
    std::ofstream out(path, std::ios::binary | std::ios::trunc);
    if (!out) throw std::runtime_error(std::string("cannot create ") + path);
    if (with_header) {
      unsigned char header[512] = {0};
      std::memcpy(header, kLegacyMagic, 4);
      header[4] = 1;  // version word
      const std::uint32_t n32 = (std::uint32_t)count;
      std::memcpy(header + 8, &n32, 4);
      out.write(reinterpret_cast<const char*>(header), sizeof header);
    }
    out.write(reinterpret_cast<const char*>(tokens), (std::streamsize)(count * 2));
    if (!out) throw std::runtime_error(std::string("short write to ") + path);
    return 0;
  });
}

int nfn_write_v2_shard(const char* path, const uint32_t* tokens, uint64_t count, uint32_t vocab_size, const char* tokenizer_sha256,
                       const char* tokenizer_revision, const char* split, const char* objective, const char* tokenizer_name) {
  return guarded([&] {
    if (count == 0 || vocab_size == 0) throw std::runtime_error("write_v2_shard: empty shard or zero vocab");
    unsigned char h[kV2Header] = {0};
    std::memcpy(h, kV2Magic, 8);
    auto put32 = [&](std::size_t off, std::uint32_t v) { std::memcpy(h + off, &v, 4); };
    put32(8, 2);
    put32(12, kV2Header);
    put32(16, 2);
    put32(20, kEndian);
    std::memcpy(h + 24, &count, 8);
    put32(32, vocab_size);
    put32(36, 0);
    auto puts = [&](std::size_t off, std::size_t width, const char* s, const char* what) {
      const std::size_t n = s ? std::strlen(s) : 0;
      if (n + 1 > width) throw std::runtime_error(std::string("write_v2_shard: field too long: ") + what);
      if (n) std::memcpy(h + off, s, n);
    };
    puts(40, 65, tokenizer_sha256, "tokenizer_sha256");
    puts(105, 96, tokenizer_revision, "tokenizer_revision");
    puts(201, 32, split, "split");
    puts(233, 32, objective, "objective");
    puts(265, 128, tokenizer_name, "tokenizer_name");
    for (std::uint64_t i = 0; i < count; ++i)
      if (tokens[i] >= vocab_size) throw std::runtime_error("write_v2_shard: token id >= vocab size");
    std::ofstream out(path, std::ios::binary | std::ios::trunc);
    if (!out) throw std::runtime_error(std::string("cannot create ") + path);
    out.write(reinterpret_cast<const char*>(h), sizeof h);
    out.write(reinterpret_cast<const char*>(tokens), (std::streamsize)(count * 4));
    if (!out) throw std::runtime_error(std::string("short write to ") + path);
    return 0;
  });
}

}  // extern "C"
