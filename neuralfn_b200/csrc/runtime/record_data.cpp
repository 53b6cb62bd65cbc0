// Structured post-training records (SFT, preference pairs, PPO prompts): validation on
// open, memory-mapped sequential batch reader with rank striding and seek-for-resume.
// File layouts follow the reference's token_shards.h:76-233 so datasets interchange.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <filesystem>
#include <fstream>
#include <memory>

#include "nfn_runtime.h"
#include "runtime_common.h"

namespace fs = std::filesystem;
using namespace nfnrt;

namespace {

constexpr std::uint32_t kHeader = 512, kEndian = 0x01020304u;

struct KindInfo {
  const char* magic;      // 7 chars + NUL
  const char* objective;
  const char* train_prefix;
  std::vector<std::string> val_prefixes;
  const char* ext;
  std::uint32_t bytes_per_token;  // per record
};

const KindInfo& kind_info(int kind) {
  static const KindInfo table[3] = {
      {"NFNSFT1", "sft", "sft_train_", {"sft_val_", "sft_validation_"}, ".sft", 16},
      {"NFNPRF1", "preference", "preference_train_", {"preference_val_", "preference_validation_"}, ".preference", 32},
      {"NFNPPO1", "ppo_prompt", "ppo_prompt_train_", {"ppo_prompt_val_", "ppo_prompt_validation_"}, ".ppo_prompt", 8},
  };
  if (kind < 0 || kind > 2) throw std::runtime_error("record kind must be 0 (sft), 1 (preference) or 2 (ppo prompt)");
  return table[kind];
}

struct RecordFile {
  std::string path;
  std::uint64_t bytes = 0, records = 0;
  std::uint32_t seq = 0, vocab = 0, pad = 0;
  std::string tokenizer_sha256, chat_template_sha256, tokenizer_revision, split;
};

// one SFT-shaped branch: ids, targets, mask, sequence ids
void check_sft_branch(const unsigned char* base, std::uint32_t T, std::uint32_t vocab, const std::string& path) {
  const unsigned char *tg = base + 4ull * T, *mk = tg + 4ull * T, *sg = mk + 4ull * T;
  double mask_sum = 0.0;
  std::int32_t prev_seg = 0;
  for (std::uint32_t t = 0; t < T; ++t) {
    const std::uint32_t id = le32(base + 4ull * t);
    const std::int32_t target = le_i32(tg + 4ull * t), seg = le_i32(sg + 4ull * t);
    const float m = le_f32(mk + 4ull * t);
    if (id >= vocab || (target != -100 && (target < 0 || (std::uint32_t)target >= vocab)) || !std::isfinite(m) || m < 0.0f ||
        seg < 0 || (t == 0 && seg != 0) || (t > 0 && seg != prev_seg && seg != prev_seg + 1))
      throw std::runtime_error("structured record holds an out-of-range id, target, mask or sequence id: " + path);
    if (m > 0.0f && target == -100) throw std::runtime_error("structured record has loss mask on an ignored target: " + path);
    mask_sum += m;
    prev_seg = seg;
  }
  if (!(mask_sum > 0.0)) throw std::runtime_error("structured record has an all-zero loss mask: " + path);
}

void check_ppo_record(const unsigned char* base, std::uint32_t T, std::uint32_t vocab, std::uint32_t pad, const std::string& path) {
  const unsigned char* mk = base + 4ull * T;
  bool ended = false;
  std::uint32_t live = 0;
  for (std::uint32_t t = 0; t < T; ++t) {
    const float m = le_f32(mk + 4ull * t);
    if (le32(base + 4ull * t) >= vocab || (m != 0.0f && m != 1.0f) || (m == 0.0f && le32(base + 4ull * t) != pad))
      throw std::runtime_error("PPO prompt record holds an out-of-range id or a non-binary mask: " + path);
    if (m == 0.0f) ended = true;
    else if (ended) throw std::runtime_error("PPO prompt attention mask is not a contiguous prefix: " + path);
    else ++live;
  }
  if (live == 0 || live >= T) throw std::runtime_error("PPO prompt must be non-empty and leave room for a response: " + path);
}

RecordFile probe(const std::string& path, int kind) {
  const KindInfo& k = kind_info(kind);
  RecordFile f;
  f.path = path;
  MappedFile m(path);
  f.bytes = m.size();
  if (f.bytes < kHeader) throw std::runtime_error("structured record file is smaller than its header: " + path);
  const unsigned char* h = m.data();
  if (std::memcmp(h, k.magic, 8) != 0 || le32(h + 8) != 1 || le32(h + 12) != kHeader || le32(h + 16) != kEndian || le32(h + 20) != 0)
    throw std::runtime_error("invalid structured record magic/version/endian/flags: " + path);
  f.records = le64(h + 24);
  f.seq = le32(h + 32);
  f.vocab = le32(h + 36);
  f.pad = le32(h + 40);
  if (f.records == 0 || f.seq == 0 || (kind == 2 && f.seq <= 1) || f.vocab == 0 || f.pad >= f.vocab)
    throw std::runtime_error("invalid structured record geometry: " + path);
  const std::uint64_t rec_bytes = (std::uint64_t)f.seq * k.bytes_per_token;
  if (f.records > (UINT64_MAX - kHeader) / rec_bytes || f.bytes != kHeader + f.records * rec_bytes)
    throw std::runtime_error("structured record byte size does not match its record table: " + path);
  f.tokenizer_sha256 = fixed_field(h, 48, 65, "tokenizer_sha256");
  f.chat_template_sha256 = fixed_field(h, 113, 65, "chat_template_sha256");
  f.tokenizer_revision = fixed_field(h, 178, 96, "tokenizer_revision");
  f.split = fixed_field(h, 274, 32, "split");
  const std::string objective = fixed_field(h, 306, 32, "objective");
  if (!is_lower_hex_sha256(f.tokenizer_sha256) || !is_lower_hex_sha256(f.chat_template_sha256) || f.tokenizer_revision.empty() ||
      (f.split != "train" && f.split != "validation" && f.split != "test") || objective != k.objective)
    throw std::runtime_error("invalid structured record lineage/split/objective metadata: " + path);
  for (std::size_t i = 338; i < kHeader; ++i)
    if (h[i] != 0) throw std::runtime_error("structured record reserved header bytes must be zero: " + path);
  for (std::uint64_t r = 0; r < f.records; ++r) {
    const unsigned char* base = h + kHeader + r * rec_bytes;
    if (kind == 0) check_sft_branch(base, f.seq, f.vocab, path);
    else if (kind == 1) {
      check_sft_branch(base, f.seq, f.vocab, path);
      check_sft_branch(base + 16ull * f.seq, f.seq, f.vocab, path);
    } else check_ppo_record(base, f.seq, f.vocab, f.pad, path);
  }
  return f;
}

std::vector<std::string> matching(const fs::path& dir, const std::vector<std::string>& prefixes, const std::string& ext) {
  std::vector<std::string> out;
  if (!fs::is_directory(dir)) return out;
  for (const auto& e : fs::directory_iterator(dir)) {
    if (!e.is_regular_file() || e.path().extension() != ext) continue;
    const std::string name = e.path().filename().string();
    for (const auto& p : prefixes)
      if (name.rfind(p, 0) == 0) {
        out.push_back(e.path().string());
        break;
      }
  }
  std::sort(out.begin(), out.end());
  return out;
}

}  // namespace

struct nfn_records {
  int kind = 0, rank = 0, world = 1;
  std::string path;
  std::vector<RecordFile> files;
  std::vector<MappedFile> maps;
  std::vector<std::int64_t> first_record;
  std::int64_t B = 0, T = 0, total_batches = 0, cursor = 0;
};

extern "C" {

nfn_records* nfn_records_open(const char* alias_or_path, int kind, int split, int allow_train_as_val, int64_t batch_size, int rank,
                              int world) {
  nfn_records* out = nullptr;
  guarded([&] {
    const KindInfo& k = kind_info(kind);
    if (!alias_or_path || batch_size <= 0 || world <= 0 || rank < 0 || rank >= world) throw std::runtime_error("records_open: bad arguments");
    fs::path root(alias_or_path);
    if (!root.is_absolute() && !fs::exists(root)) {
      const char* env = std::getenv("NFN_DATASETS_DIR");
      const char* home = std::getenv("HOME");
      root = (env && *env ? fs::path(env) : fs::path(home ? home : ".") / ".cache" / "nfn" / "datasets") / alias_or_path;
    }
    auto r = std::make_unique<nfn_records>();
    r->kind = kind;
    r->rank = rank;
    r->world = world;
    r->path = root.string();
    r->B = batch_size;
    std::vector<std::string> paths;
    if (fs::is_regular_file(root)) {
      paths = {root.string()};
    } else if (fs::is_directory(root)) {
      if (split == 0) {
        paths = matching(root, {k.train_prefix}, k.ext);
      } else {
        paths = matching(root, k.val_prefixes, k.ext);
        if (paths.empty() && allow_train_as_val) paths = matching(root, {k.train_prefix}, k.ext);
      }
    } else {
      throw std::runtime_error("dataset directory not found: " + root.string());
    }
    if (paths.empty())
      throw std::runtime_error(std::string("no native structured ") + k.objective + " records found under " + root.string() +
                               " (expected " + (split == 0 ? k.train_prefix : k.val_prefixes[0].c_str()) + "*" + k.ext + ")");
    r->first_record.push_back(0);
    for (const auto& p : paths) {
      RecordFile f = probe(p, kind);
      if (!r->files.empty()) {
        const RecordFile& a = r->files.front();
        if (f.seq != a.seq || f.vocab != a.vocab || f.pad != a.pad || f.tokenizer_sha256 != a.tokenizer_sha256 ||
            f.chat_template_sha256 != a.chat_template_sha256)
          throw std::runtime_error("structured record files disagree on geometry or tokenizer lineage: " + p);
      }
      if (fs::is_directory(root) && split == 0 && f.split != "train")
        throw std::runtime_error("structured train filename has non-train split metadata: " + p);
      r->maps.emplace_back(p);
      r->first_record.push_back(r->first_record.back() + (std::int64_t)f.records);
      r->files.push_back(std::move(f));
    }
    r->T = r->files.front().seq;
    r->total_batches = r->first_record.back() / (batch_size * world);
    out = r.release();
    return 0;
  });
  return out;
}

void nfn_records_close(nfn_records* r) { delete r; }
int64_t nfn_records_total_batches(const nfn_records* r) { return r ? r->total_batches : -1; }
int64_t nfn_records_seq_len(const nfn_records* r) { return r ? r->T : -1; }
void nfn_records_reset(nfn_records* r) {
  if (r) r->cursor = 0;
}

int nfn_records_seek(nfn_records* r, int64_t batch_index) {
  if (!r || batch_index < 0 || r->total_batches <= 0) {
    set_error("records_seek: negative index or empty reader");
    return -1;
  }
  r->cursor = batch_index % r->total_batches;
  return 0;
}

int nfn_records_json(const nfn_records* r, char* buf, int cap) {
  return guarded([&] {
    if (!r) throw std::runtime_error("records_json: null reader");
    const KindInfo& k = kind_info(r->kind);
    JsonObject o;
    o.add("dataset_path", r->path).add("objective", k.objective).add("sequence_length", r->T).add("batch_size", r->B);
    o.add("records", r->first_record.back()).add("total_batches", r->total_batches);
    std::vector<std::string> files;
    for (const auto& f : r->files) {
      JsonObject fo;
      fo.add("path", f.path).add("bytes", f.bytes).add("records", f.records).add("sequence_length", (std::int64_t)f.seq);
      fo.add("tokenizer_vocab_size", (std::int64_t)f.vocab).add("pad_token_id", (std::int64_t)f.pad);
      fo.add("tokenizer_sha256", f.tokenizer_sha256).add("chat_template_sha256", f.chat_template_sha256);
      fo.add("tokenizer_revision", f.tokenizer_revision).add("split", f.split);
      files.push_back(fo.str());
    }
    o.add_raw("files", json_array(files));
    return copy_out(o.str(), buf, cap);
  });
}

int nfn_records_next(nfn_records* r, int32_t* input_ids, int32_t* targets, float* loss_mask, int32_t* sequence_ids, int64_t capacity) {
  return guarded([&] {
    if (!r || !input_ids || !loss_mask) throw std::runtime_error("records_next: null argument");
    if (r->kind != 2 && (!targets || !sequence_ids)) throw std::runtime_error("records_next: targets and sequence_ids are required");
    const std::int64_t rows = r->kind == 1 ? 2 * r->B : r->B, T = r->T;
    if (capacity < rows * T) throw std::runtime_error("records_next: destination smaller than the batch");
    if (r->cursor >= r->total_batches) return 0;
    const std::int64_t first = (r->cursor * r->world + r->rank) * r->B;
    const std::uint64_t rec_bytes = (std::uint64_t)T * kind_info(r->kind).bytes_per_token;
    for (std::int64_t b = 0; b < r->B; ++b) {
      const std::int64_t g = first + b;
      const std::size_t fi = std::upper_bound(r->first_record.begin(), r->first_record.end(), g) - r->first_record.begin() - 1;
      const unsigned char* base = r->maps[fi].data() + kHeader + (std::uint64_t)(g - r->first_record[fi]) * rec_bytes;
      const std::size_t row = (std::size_t)T * 4;
      if (r->kind == 2) {
        std::memcpy(input_ids + b * T, base, row);
        std::memcpy(loss_mask + b * T, base + row, row);
        continue;
      }
      const int branches = r->kind == 1 ? 2 : 1;
      for (int br = 0; br < branches; ++br) {
        const unsigned char* p = base + (std::uint64_t)br * 16ull * T;
        const std::int64_t dst = (br * r->B + b) * T;  // chosen rows first, then rejected
        std::memcpy(input_ids + dst, p, row);
        std::memcpy(targets + dst, p + row, row);
        std::memcpy(loss_mask + dst, p + 2 * row, row);
        std::memcpy(sequence_ids + dst, p + 3 * row, row);
      }
    }
    ++r->cursor;
    return 1;
  });
}

int nfn_write_records(const char* path, int kind, uint64_t records, uint32_t seq_len, uint32_t vocab_size, uint32_t pad_token_id,
                      const char* tokenizer_sha256, const char* chat_template_sha256, const char* tokenizer_revision, const char* split,
                      const void* payload, uint64_t payload_bytes) {
  return guarded([&] {
    const KindInfo& k = kind_info(kind);
    if (!path || !payload || records == 0 || seq_len == 0) throw std::runtime_error("write_records: bad arguments");
    if (payload_bytes != records * (std::uint64_t)seq_len * k.bytes_per_token)
      throw std::runtime_error("write_records: payload size does not match records * seq_len * bytes-per-token");
    unsigned char h[kHeader] = {0};
    std::memcpy(h, k.magic, 8);
    auto put32 = [&](std::size_t off, std::uint32_t v) { std::memcpy(h + off, &v, 4); };
    put32(8, 1);
    put32(12, kHeader);
    put32(16, kEndian);
    put32(20, 0);
    std::memcpy(h + 24, &records, 8);
    put32(32, seq_len);
    put32(36, vocab_size);
    put32(40, pad_token_id);
    auto puts = [&](std::size_t off, std::size_t width, const char* s, const char* what) {
      const std::size_t n = s ? std::strlen(s) : 0;
      if (n + 1 > width) throw std::runtime_error(std::string("write_records: field too long: ") + what);
      if (n) std::memcpy(h + off, s, n);
    };
    puts(48, 65, tokenizer_sha256, "tokenizer_sha256");
    puts(113, 65, chat_template_sha256, "chat_template_sha256");
    puts(178, 96, tokenizer_revision, "tokenizer_revision");
    puts(274, 32, split, "split");
    puts(306, 32, k.objective, "objective");
    const std::string tmp = std::string(path) + ".staging";
    {
      std::ofstream out(tmp, std::ios::binary | std::ios::trunc);
      if (!out) throw std::runtime_error("cannot create " + tmp);
      out.write(reinterpret_cast<const char*>(h), sizeof h);
      out.write(static_cast<const char*>(payload), (std::streamsize)payload_bytes);
      if (!out) throw std::runtime_error("short write to " + tmp);
    }
    try {
      probe(tmp, kind);  // refuse to publish a file the reader would reject
    } catch (...) {
      fs::remove(tmp);
      throw;
    }
    fs::rename(tmp, path);
    return 0;
  });
}

}  // extern "C"
