// Checkpoint container I/O: a file is one fixed header followed by N byte segments that
// the caller describes as (pointer, length) pairs, so flat parameter buffers can be
// written in any tensor order without staging copies.
//
// Safety rules shared by every checkpoint format of the framework (they mirror what the
// reference enforces for its dense files, nfn_gpt2_native_train.cpp:319-452): the final
// path is created exclusively (never overwritten), symlinks are not followed, data is
// written to "<path>.staging", fsync'ed and then linked into place, the reader demands
// the exact expected size (no truncation, no trailing bytes), and both directions return
// the SHA-256 of the whole file.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstdio>

#include "nfn_runtime.h"
#include "runtime_common.h"

using namespace nfnrt;

namespace {

struct Fd {
  int fd = -1;
  ~Fd() {
    if (fd >= 0) ::close(fd);
  }
};

void write_all(int fd, const unsigned char* p, std::uint64_t n, const std::string& path) {
  while (n > 0) {
    const ssize_t w = ::write(fd, p, (std::size_t)std::min<std::uint64_t>(n, 1u << 30));
    if (w < 0) {
      if (errno == EINTR) continue;
      throw std::runtime_error("write failed: " + path);
    }
    p += w;
    n -= (std::uint64_t)w;
  }
}

void read_all(int fd, unsigned char* p, std::uint64_t n, const std::string& path) {
  while (n > 0) {
    const ssize_t r = ::read(fd, p, (std::size_t)std::min<std::uint64_t>(n, 1u << 30));
    if (r < 0) {
      if (errno == EINTR) continue;
      throw std::runtime_error("read failed: " + path);
    }
    if (r == 0) throw std::runtime_error("checkpoint payload is truncated: " + path);
    p += r;
    n -= (std::uint64_t)r;
  }
}

}  // namespace

// A tiny incremental hasher built on the one-shot helpers would re-read the data, so the
// container hashes by streaming each segment through sha256 once after writing; files are
// in the page cache at that point.
extern "C" {

int nfn_ckpt_write(const char* path, const void* header, uint64_t header_bytes, const void* const* segments,
                   const uint64_t* segment_bytes, int n_segments, char* out_sha65) {
  return guarded([&] {
    if (!path || (!header && header_bytes) || n_segments < 0) throw std::runtime_error("ckpt_write: bad arguments");
    const std::string final_path(path), staging = final_path + ".staging";
    struct stat st {};
    if (::lstat(final_path.c_str(), &st) == 0) throw std::runtime_error("refusing to overwrite an existing checkpoint: " + final_path);
    {
      Fd f;
      f.fd = ::open(staging.c_str(), O_WRONLY | O_CREAT | O_EXCL | O_NOFOLLOW | O_CLOEXEC, 0644);
      if (f.fd < 0) throw std::runtime_error("cannot create (exclusive, no symlink) " + staging);
      try {
        write_all(f.fd, static_cast<const unsigned char*>(header), header_bytes, staging);
        for (int i = 0; i < n_segments; ++i)
          write_all(f.fd, static_cast<const unsigned char*>(segments[i]), segment_bytes[i], staging);
        if (::fsync(f.fd) != 0) throw std::runtime_error("fsync failed: " + staging);
      } catch (...) {
        ::unlink(staging.c_str());
        throw;
      }
    }
    // link() fails if the target appeared meanwhile: exclusive publication without a race
    if (::link(staging.c_str(), final_path.c_str()) != 0) {
      ::unlink(staging.c_str());
      throw std::runtime_error("refusing to overwrite an existing checkpoint: " + final_path);
    }
    ::unlink(staging.c_str());
    if (out_sha65) {
      const std::string h = sha256_file_hex(final_path);
      std::memcpy(out_sha65, h.c_str(), 65);
    }
    return 0;
  });
}

int nfn_ckpt_read(const char* path, void* header, uint64_t header_bytes, void* const* segments, const uint64_t* segment_bytes,
                  int n_segments, char* out_sha65) {
  return guarded([&] {
    if (!path || n_segments < 0) throw std::runtime_error("ckpt_read: bad arguments");
    const std::string p(path);
    Fd f;
    f.fd = ::open(p.c_str(), O_RDONLY | O_NOFOLLOW | O_CLOEXEC);
    if (f.fd < 0) throw std::runtime_error("cannot open checkpoint (missing, or a symlink): " + p);
    struct stat st {};
    if (::fstat(f.fd, &st) != 0 || !S_ISREG(st.st_mode)) throw std::runtime_error("checkpoint is not a regular file: " + p);
    std::uint64_t expect = header_bytes;
    for (int i = 0; i < n_segments; ++i) expect += segment_bytes[i];
    if ((std::uint64_t)st.st_size != expect)
      throw std::runtime_error("checkpoint file size " + std::to_string(st.st_size) + " does not match the expected " +
                               std::to_string(expect) + " bytes: " + p);
    if (header_bytes) read_all(f.fd, static_cast<unsigned char*>(header), header_bytes, p);
    for (int i = 0; i < n_segments; ++i) read_all(f.fd, static_cast<unsigned char*>(segments[i]), segment_bytes[i], p);
    if (out_sha65) {
      const std::string h = sha256_file_hex(p);
      std::memcpy(out_sha65, h.c_str(), 65);
    }
    return 0;
  });
}

// Reads only the first header_bytes of a file (to learn the geometry before allocating).
int nfn_ckpt_peek(const char* path, void* header, uint64_t header_bytes, uint64_t* file_bytes) {
  return guarded([&] {
    const std::string p(path ? path : "");
    Fd f;
    f.fd = ::open(p.c_str(), O_RDONLY | O_NOFOLLOW | O_CLOEXEC);
    if (f.fd < 0) throw std::runtime_error("cannot open checkpoint (missing, or a symlink): " + p);
    struct stat st {};
    if (::fstat(f.fd, &st) != 0 || !S_ISREG(st.st_mode)) throw std::runtime_error("checkpoint is not a regular file: " + p);
    if ((std::uint64_t)st.st_size < header_bytes) throw std::runtime_error("checkpoint header is truncated: " + p);
    read_all(f.fd, static_cast<unsigned char*>(header), header_bytes, p);
    if (file_bytes) *file_bytes = (std::uint64_t)st.st_size;
    return 0;
  });
}

// Publishes a directory written under "<dir>.staging" by renaming it; refuses when the
// target exists.
int nfn_ckpt_publish_dir(const char* staging_dir, const char* final_dir) {
  return guarded([&] {
    struct stat st {};
    if (::lstat(final_dir, &st) == 0) throw std::runtime_error(std::string("refusing to overwrite an existing checkpoint directory: ") + final_dir);
    if (::rename(staging_dir, final_dir) != 0) throw std::runtime_error(std::string("cannot publish checkpoint directory: ") + final_dir);
    return 0;
  });
}

}  // extern "C"
