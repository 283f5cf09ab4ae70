// File IO for the filesystem KV-cache tier: whole-buffer reads and writes that run outside the
// Python interpreter lock (ctypes releases it for the duration of the call) and split large
// transfers over a few threads of positional IO.  Writes go to a temporary name and are renamed
// into place, so a reader never sees a partial file.
//
// Role parity: the reference's csrc/fs_io.cpp (GIL-releasing file IO for the FS offload tier).
#include <errno.h>
#include <fcntl.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <string>
#include <thread>
#include <vector>

#define SONAR_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

constexpr size_t kChunk = 8u << 20;   // bytes per positional IO call

template <bool WRITE>
int io_range(int fd, uint8_t* buf, size_t off, size_t len) {
  while (len > 0) {
    size_t n = std::min(len, kChunk);
    ssize_t r = WRITE ? pwrite(fd, buf, n, (off_t)off) : pread(fd, buf, n, (off_t)off);
    if (r < 0) { if (errno == EINTR) continue; return errno ? errno : EIO; }
    if (r == 0) return EIO;   // short file
    buf += r; off += (size_t)r; len -= (size_t)r;
  }
  return 0;
}

template <bool WRITE>
int io_parallel(int fd, void* ptr, size_t nbytes, int threads) {
  uint8_t* buf = static_cast<uint8_t*>(ptr);
  if (threads <= 1 || nbytes < 4 * kChunk) return io_range<WRITE>(fd, buf, 0, nbytes);
  threads = std::min<int>(threads, (int)((nbytes + kChunk - 1) / kChunk));
  const size_t per = ((nbytes + threads - 1) / threads + 4095) & ~size_t(4095);
  std::atomic<int> err{0};
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t) {
    size_t off = per * t;
    if (off >= nbytes) break;
    size_t len = std::min(per, nbytes - off);
    pool.emplace_back([=, &err] {
      int e = io_range<WRITE>(fd, buf + off, off, len);
      if (e) err.store(e);
    });
  }
  for (auto& th : pool) th.join();
  return err.load();
}

}  // namespace

// 0 on success, else errno.
SONAR_EXPORT int sonar_fs_write(const char* path, const void* ptr, size_t nbytes, int threads, int do_fsync) {
  std::string tmp = std::string(path) + ".tmp." + std::to_string((long)getpid());
  int fd = open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
  if (fd < 0) return errno;
  int e = io_parallel<true>(fd, const_cast<void*>(ptr), nbytes, threads);
  if (!e && do_fsync && fsync(fd) != 0) e = errno;
  close(fd);
  if (!e && rename(tmp.c_str(), path) != 0) e = errno;
  if (e) unlink(tmp.c_str());
  return e;
}

// 0 on success, else errno (EIO when the file is shorter than nbytes).
SONAR_EXPORT int sonar_fs_read(const char* path, void* ptr, size_t nbytes, int threads) {
  int fd = open(path, O_RDONLY);
  if (fd < 0) return errno;
  int e = io_parallel<false>(fd, ptr, nbytes, threads);
  close(fd);
  return e;
}

// file size in bytes, or -1
SONAR_EXPORT long long sonar_fs_size(const char* path) {
  struct stat st;
  if (stat(path, &st) != 0) return -1;
  return (long long)st.st_size;
}
