// Shared helpers of the host-side native runtime: error reporting over the C ABI,
// little-endian field access, read-only memory maps, a small JSON string builder.
#pragma once

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace nfnrt {

// Last error message of the calling thread; C entry points return a negative code and
// leave the text here (nfn_rt_last_error()).
void set_error(const std::string& msg);
const char* last_error();

// Runs `fn`, converting C++ exceptions into (-1, message).
template <class F>
int guarded(F&& fn) {
  try {
    return fn();
  } catch (const std::exception& e) {
    set_error(e.what());
    return -1;
  } catch (...) {
    set_error("unknown native error");
    return -1;
  }
}

inline std::uint32_t le32(const unsigned char* p) {
  return (std::uint32_t)p[0] | ((std::uint32_t)p[1] << 8) | ((std::uint32_t)p[2] << 16) | ((std::uint32_t)p[3] << 24);
}
inline std::uint64_t le64(const unsigned char* p) { return (std::uint64_t)le32(p) | ((std::uint64_t)le32(p + 4) << 32); }
inline std::int32_t le_i32(const unsigned char* p) {
  const std::uint32_t u = le32(p);
  std::int32_t v;
  std::memcpy(&v, &u, 4);
  return v;
}
inline float le_f32(const unsigned char* p) {
  const std::uint32_t u = le32(p);
  float v;
  std::memcpy(&v, &u, 4);
  return v;
}

// NUL-terminated string stored in a fixed-width header field. Throws when the field has
// no terminator or carries bytes after it.
std::string fixed_field(const unsigned char* header, std::size_t offset, std::size_t width, const char* what);
bool is_lower_hex_sha256(const std::string& s);

// Read-only mapping of a whole file (MAP_PRIVATE | PROT_READ, sequential advice).
class MappedFile {
 public:
  MappedFile() = default;
  explicit MappedFile(const std::string& path);
  MappedFile(MappedFile&& o) noexcept;
  MappedFile& operator=(MappedFile&& o) noexcept;
  MappedFile(const MappedFile&) = delete;
  MappedFile& operator=(const MappedFile&) = delete;
  ~MappedFile();
  const unsigned char* data() const { return data_; }
  std::size_t size() const { return size_; }

 private:
  void release();
  const unsigned char* data_ = nullptr;
  std::size_t size_ = 0;
};

// Minimal JSON object writer (keys in insertion order).
class JsonObject {
 public:
  JsonObject& add(const std::string& key, const std::string& value);
  JsonObject& add(const std::string& key, const char* value) { return add(key, std::string(value)); }
  JsonObject& add(const std::string& key, std::int64_t value);
  JsonObject& add(const std::string& key, std::uint64_t value) { return add(key, (std::int64_t)value); }
  JsonObject& add(const std::string& key, int value) { return add(key, (std::int64_t)value); }
  JsonObject& add(const std::string& key, double value);
  JsonObject& add(const std::string& key, bool value);
  JsonObject& add_raw(const std::string& key, const std::string& json);
  std::string str() const { return "{" + body_ + "}"; }

 private:
  void sep();
  std::string body_;
};
std::string json_quote(const std::string& s);
std::string json_array(const std::vector<std::string>& raw_items);

// Copies `s` into a caller buffer; returns the length needed (excluding the NUL).
int copy_out(const std::string& s, char* buf, int cap);

// SHA-256 of a byte range / file, lower-case hex.
std::string sha256_hex(const void* data, std::size_t bytes);
std::string sha256_file_hex(const std::string& path);

}  // namespace nfnrt
