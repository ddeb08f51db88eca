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

}  // extern "C"
