// Checkpoint chunk I/O: many array chunks written / read concurrently with positional I/O, each
// through a temporary name that is renamed into place, plus CRC-32C of the payload so that a reader can
// tell a torn chunk from a complete one.  Replaces the role of the C++ array-store runtime behind the
// reference's checkpoint manager.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>

#include "host/thread_pool.h"

extern "C" uint32_t recml_crc32c(const uint8_t* p, long long n);

namespace {

bool write_all(int fd, const uint8_t* p, long long n) {
  while (n > 0) {
    const ssize_t w = ::write(fd, p, static_cast<size_t>(n > (1 << 30) ? (1 << 30) : n));
    if (w <= 0) return false;
    p += w;
    n -= w;
  }
  return true;
}

}  // namespace

extern "C" {

// Writes count files: paths[i] receives bufs[i][0:sizes[i]].  crcs (optional) receives each CRC-32C.
// Returns 0, or -(1+i) for the first file that failed.
int recml_write_chunks(int count, const char* const* paths, const uint8_t* const* bufs, const long long* sizes,
                       uint32_t* crcs, int fsync_files) {
  std::atomic<int> failed{0};
  recml::ThreadPool::global().parallel_for(count, [&](long long i0, long long i1, int) {
    for (long long i = i0; i < i1; ++i) {
      const std::string tmp = std::string(paths[i]) + ".partial";
      const int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
      bool ok = fd >= 0 && write_all(fd, bufs[i], sizes[i]);
      if (fd >= 0) {
        if (ok && fsync_files) ok = ::fsync(fd) == 0;
        ::close(fd);
      }
      if (ok) ok = ::rename(tmp.c_str(), paths[i]) == 0;
      if (ok && crcs != nullptr) crcs[i] = recml_crc32c(bufs[i], sizes[i]);
      if (!ok) {
        int expected = 0;
        failed.compare_exchange_strong(expected, static_cast<int>(-(1 + i)));
      }
    }
  });
  return failed.load();
}

// CRC-32C of count buffers, computed by all host threads (the per-segment checksums stored beside raw chunks).
void recml_crc32c_many(int count, const uint8_t* const* bufs, const long long* sizes, uint32_t* out) {
  recml::ThreadPool::global().parallel_for(count, [&](long long i0, long long i1, int) {
    for (long long i = i0; i < i1; ++i) out[i] = recml_crc32c(bufs[i], sizes[i]);
  }, 1);
}

// Reads count files fully into caller buffers of the given sizes; short files fail.
int recml_read_chunks(int count, const char* const* paths, uint8_t* const* bufs, const long long* sizes) {
  std::atomic<int> failed{0};
  recml::ThreadPool::global().parallel_for(count, [&](long long i0, long long i1, int) {
    for (long long i = i0; i < i1; ++i) {
      const int fd = ::open(paths[i], O_RDONLY);
      bool ok = fd >= 0;
      long long got = 0;
      while (ok && got < sizes[i]) {
        const ssize_t r = ::pread(fd, bufs[i] + got, static_cast<size_t>(sizes[i] - got), got);
        if (r <= 0) ok = false; else got += r;
      }
      if (fd >= 0) ::close(fd);
      if (!ok) {
        int expected = 0;
        failed.compare_exchange_strong(expected, static_cast<int>(-(1 + i)));
      }
    }
  });
  return failed.load();
}

// Writes bufs[i][0:sizes[i]] at file_offsets[i] of the EXISTING file paths[i] (the caller creates the
// temporary files, splits large chunks into segments so that many threads write one file, and renames the
// files once every segment is in).  Returns 0, or -(1+i) for the first item that failed.
int recml_write_ranges(int count, const char* const* paths, const long long* file_offsets, const uint8_t* const* bufs,
                       const long long* sizes) {
  std::atomic<int> failed{0};
  recml::ThreadPool::global().parallel_for(count, [&](long long i0, long long i1, int) {
    for (long long i = i0; i < i1; ++i) {
      const int fd = ::open(paths[i], O_WRONLY);
      bool ok = fd >= 0;
      long long put = 0;
      while (ok && put < sizes[i]) {
        const ssize_t r = ::pwrite(fd, bufs[i] + put, static_cast<size_t>(sizes[i] - put), file_offsets[i] + put);
        if (r <= 0) ok = false; else put += r;
      }
      if (fd >= 0) ::close(fd);
      if (!ok) {
        int expected = 0;
        failed.compare_exchange_strong(expected, static_cast<int>(-(1 + i)));
      }
    }
  }, 1);
  return failed.load();
}

// Reads sizes[i] bytes at file_offsets[i] of paths[i] into bufs[i]; a large chunk is read by several
// items (one per segment) so that one file is read by many threads.  A short file fails, except that
// allow_short lets an item end at the end of its file (the rest of the buffer is left as it is).
int recml_read_ranges(int count, const char* const* paths, const long long* file_offsets, uint8_t* const* bufs,
                      const long long* sizes, int allow_short) {
  std::atomic<int> failed{0};
  recml::ThreadPool::global().parallel_for(count, [&](long long i0, long long i1, int) {
    for (long long i = i0; i < i1; ++i) {
      const int fd = ::open(paths[i], O_RDONLY);
      bool ok = fd >= 0;
      long long got = 0;
      while (ok && got < sizes[i]) {
        const ssize_t r = ::pread(fd, bufs[i] + got, static_cast<size_t>(sizes[i] - got), file_offsets[i] + got);
        if (r < 0) ok = false;
        else if (r == 0) { ok = allow_short != 0; break; }
        else got += r;
      }
      if (fd >= 0) ::close(fd);
      if (!ok) {
        int expected = 0;
        failed.compare_exchange_strong(expected, static_cast<int>(-(1 + i)));
      }
    }
  }, 1);
  return failed.load();
}

}  // extern "C"
