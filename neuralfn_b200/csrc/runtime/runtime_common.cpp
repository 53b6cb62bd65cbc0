#include "runtime_common.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdio>
#include <fstream>

namespace nfnrt {

static thread_local std::string t_error;

void set_error(const std::string& msg) { t_error = msg; }
const char* last_error() { return t_error.c_str(); }

std::string fixed_field(const unsigned char* header, std::size_t offset, std::size_t width, const char* what) {
  std::size_t len = 0;
  while (len < width && header[offset + len] != 0) ++len;
  if (len == width) throw std::runtime_error(std::string("header field is not NUL-terminated: ") + what);
  for (std::size_t i = len; i < width; ++i)
    if (header[offset + i] != 0) throw std::runtime_error(std::string("header field has bytes after its terminator: ") + what);
  return std::string(reinterpret_cast<const char*>(header + offset), len);
}

bool is_lower_hex_sha256(const std::string& s) {
  if (s.size() != 64) return false;
  for (char c : s)
    if (!((c >= '0' && c <= '9') || (c >= 'a' && c <= 'f'))) return false;
  return true;
}

MappedFile::MappedFile(const std::string& path) {
  const int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
  if (fd < 0) throw std::runtime_error("cannot open " + path);
  struct stat st {};
  if (::fstat(fd, &st) != 0) {
    ::close(fd);
    throw std::runtime_error("cannot stat " + path);
  }
  size_ = static_cast<std::size_t>(st.st_size);
  if (size_ > 0) {
    void* p = ::mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd, 0);
    if (p == MAP_FAILED) {
      ::close(fd);
      throw std::runtime_error("cannot map " + path);
    }
    ::madvise(p, size_, MADV_SEQUENTIAL);
    data_ = static_cast<const unsigned char*>(p);
  }
  ::close(fd);
}

MappedFile::MappedFile(MappedFile&& o) noexcept : data_(o.data_), size_(o.size_) {
  o.data_ = nullptr;
  o.size_ = 0;
}

MappedFile& MappedFile::operator=(MappedFile&& o) noexcept {
  if (this != &o) {
    release();
    data_ = o.data_;
    size_ = o.size_;
    o.data_ = nullptr;
    o.size_ = 0;
  }
  return *this;
}

MappedFile::~MappedFile() { release(); }

void MappedFile::release() {
  if (data_ != nullptr) ::munmap(const_cast<unsigned char*>(data_), size_);
  data_ = nullptr;
  size_ = 0;
}

std::string json_quote(const std::string& s) {
  std::string out = "\"";
  for (unsigned char c : s) {
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\r': out += "\\r"; break;
      case '\t': out += "\\t"; break;
      default:
        if (c < 0x20) {
          char buf[8];
          std::snprintf(buf, sizeof buf, "\\u%04x", c);
          out += buf;
        } else {
          out += static_cast<char>(c);
        }
    }
  }
  return out + "\"";
}

void JsonObject::sep() {
  if (!body_.empty()) body_ += ", ";
}
JsonObject& JsonObject::add(const std::string& key, const std::string& value) {
  sep();
  body_ += json_quote(key) + ": " + json_quote(value);
  return *this;
}
JsonObject& JsonObject::add(const std::string& key, std::int64_t value) {
  sep();
  body_ += json_quote(key) + ": " + std::to_string(value);
  return *this;
}
JsonObject& JsonObject::add(const std::string& key, double value) {
  sep();
  char buf[40];
  if (std::isfinite(value)) std::snprintf(buf, sizeof buf, "%.9g", value);
  else std::snprintf(buf, sizeof buf, "null");
  body_ += json_quote(key) + ": " + buf;
  return *this;
}
JsonObject& JsonObject::add(const std::string& key, bool value) {
  sep();
  body_ += json_quote(key) + ": " + (value ? "true" : "false");
  return *this;
}
JsonObject& JsonObject::add_raw(const std::string& key, const std::string& json) {
  sep();
  body_ += json_quote(key) + ": " + json;
  return *this;
}

std::string json_array(const std::vector<std::string>& raw_items) {
  std::string out = "[";
  for (std::size_t i = 0; i < raw_items.size(); ++i) {
    if (i) out += ", ";
    out += raw_items[i];
  }
  return out + "]";
}

int copy_out(const std::string& s, char* buf, int cap) {
  if (buf != nullptr && cap > 0) {
    const std::size_t n = std::min<std::size_t>(s.size(), static_cast<std::size_t>(cap - 1));
    std::memcpy(buf, s.data(), n);
    buf[n] = 0;
  }
  return static_cast<int>(s.size());
}

// ---- SHA-256 (FIPS 180-4) ----------------------------------------------------------
namespace {
struct Sha256 {
  std::uint32_t h[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au, 0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};
  unsigned char block[64];
  std::size_t fill = 0;
  std::uint64_t total = 0;

  static std::uint32_t rotr(std::uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

  void compress(const unsigned char* p) {
    static const std::uint32_t K[64] = {
        0x428a2f98u, 0x71374491u, 0xb5c0fbcfu, 0xe9b5dba5u, 0x3956c25bu, 0x59f111f1u, 0x923f82a4u, 0xab1c5ed5u,
        0xd807aa98u, 0x12835b01u, 0x243185beu, 0x550c7dc3u, 0x72be5d74u, 0x80deb1feu, 0x9bdc06a7u, 0xc19bf174u,
        0xe49b69c1u, 0xefbe4786u, 0x0fc19dc6u, 0x240ca1ccu, 0x2de92c6fu, 0x4a7484aau, 0x5cb0a9dcu, 0x76f988dau,
        0x983e5152u, 0xa831c66du, 0xb00327c8u, 0xbf597fc7u, 0xc6e00bf3u, 0xd5a79147u, 0x06ca6351u, 0x14292967u,
        0x27b70a85u, 0x2e1b2138u, 0x4d2c6dfcu, 0x53380d13u, 0x650a7354u, 0x766a0abbu, 0x81c2c92eu, 0x92722c85u,
        0xa2bfe8a1u, 0xa81a664bu, 0xc24b8b70u, 0xc76c51a3u, 0xd192e819u, 0xd6990624u, 0xf40e3585u, 0x106aa070u,
        0x19a4c116u, 0x1e376c08u, 0x2748774cu, 0x34b0bcb5u, 0x391c0cb3u, 0x4ed8aa4au, 0x5b9cca4fu, 0x682e6ff3u,
        0x748f82eeu, 0x78a5636fu, 0x84c87814u, 0x8cc70208u, 0x90befffau, 0xa4506cebu, 0xbef9a3f7u, 0xc67178f2u};
    std::uint32_t w[64];
    for (int i = 0; i < 16; ++i)
      w[i] = ((std::uint32_t)p[4 * i] << 24) | ((std::uint32_t)p[4 * i + 1] << 16) | ((std::uint32_t)p[4 * i + 2] << 8) | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const std::uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const std::uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    std::uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int i = 0; i < 64; ++i) {
      const std::uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25);
      const std::uint32_t ch = (e & f) ^ (~e & g);
      const std::uint32_t t1 = hh + S1 + ch + K[i] + w[i];
      const std::uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22);
      const std::uint32_t mj = (a & b) ^ (a & c) ^ (b & c);
      const std::uint32_t t2 = S0 + mj;
      hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
  }

  void update(const unsigned char* p, std::size_t n) {
    total += n;
    while (n > 0) {
      if (fill == 0 && n >= 64) {
        compress(p);
        p += 64;
        n -= 64;
        continue;
      }
      const std::size_t take = std::min<std::size_t>(64 - fill, n);
      std::memcpy(block + fill, p, take);
      fill += take;
      p += take;
      n -= take;
      if (fill == 64) {
        compress(block);
        fill = 0;
      }
    }
  }

  std::string finish() {
    const std::uint64_t bits = total * 8;
    unsigned char pad[72] = {0x80};
    const std::size_t padlen = (fill < 56) ? (56 - fill) : (120 - fill);
    unsigned char len[8];
    for (int i = 0; i < 8; ++i) len[i] = static_cast<unsigned char>(bits >> (56 - 8 * i));
    update(pad, padlen);
    update(len, 8);
    static const char* hex = "0123456789abcdef";
    std::string out(64, '0');
    for (int i = 0; i < 8; ++i)
      for (int j = 0; j < 4; ++j) {
        const unsigned char byte = static_cast<unsigned char>(h[i] >> (24 - 8 * j));
        out[8 * i + 2 * j] = hex[byte >> 4];
        out[8 * i + 2 * j + 1] = hex[byte & 15];
      }
    return out;
  }
};
}  // namespace

std::string sha256_hex(const void* data, std::size_t bytes) {
  Sha256 s;
  s.update(static_cast<const unsigned char*>(data), bytes);
  return s.finish();
}

std::string sha256_file_hex(const std::string& path) {
  std::ifstream in(path, std::ios::binary);
  if (!in) throw std::runtime_error("cannot open " + path);
  Sha256 s;
  std::vector<unsigned char> buf(1 << 20);
  while (in) {
    in.read(reinterpret_cast<char*>(buf.data()), static_cast<std::streamsize>(buf.size()));
    const std::streamsize got = in.gcount();
    if (got > 0) s.update(buf.data(), static_cast<std::size_t>(got));
  }
  return s.finish();
}

}  // namespace nfnrt

extern "C" const char* nfn_rt_last_error() { return nfnrt::last_error(); }

extern "C" int nfn_rt_sha256_file(const char* path, char* out65) {
  return nfnrt::guarded([&] {
    const std::string h = nfnrt::sha256_file_hex(path);
    std::memcpy(out65, h.c_str(), 65);
    return 0;
  });
}

extern "C" int nfn_rt_sha256(const void* data, std::uint64_t bytes, char* out65) {
  return nfnrt::guarded([&] {
    const std::string h = nfnrt::sha256_hex(data, static_cast<std::size_t>(bytes));
    std::memcpy(out65, h.c_str(), 65);
    return 0;
  });
}

// ---- shipped preset catalogue (generated header) --------------------------------------------------
#include "shipped_presets.h"

extern "C" int nfn_rt_preset_count(void) { return nfn_rt::kShippedPresetCount; }

// Name of preset `index` (nullptr when out of range).
extern "C" const char* nfn_rt_preset_name(int index) {
  return index >= 0 && index < nfn_rt::kShippedPresetCount ? nfn_rt::kShippedPresets[index].name : nullptr;
}

// Family a shipped preset trains under, or nullptr for an unknown name.
extern "C" const char* nfn_rt_preset_family(const char* name) {
  if (!name) return nullptr;
  for (const auto& p : nfn_rt::kShippedPresets)
    if (std::strcmp(p.name, name) == 0) return p.family;
  return nullptr;
}
