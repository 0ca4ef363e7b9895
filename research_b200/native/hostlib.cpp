// Host-side native runtime pieces (no CUDA): threaded file write/read for checkpoint chunks, and a threaded
// gather of token windows from memory-mapped uint32 shards into a caller-provided (pinned) batch buffer.
// The reference delegates these jobs to tensorstore (inside Orbax) and to Grain's C++ data loader; this is
// the stand-alone counterpart used by research_b200/services/checkpoints.py and research_b200/data.
#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <thread>
#include <vector>

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

namespace {

constexpr size_t kChunk = size_t(8) << 20;

int clamp_threads(int requested, size_t nbytes) {
  int hw = static_cast<int>(std::thread::hardware_concurrency());
  if (hw <= 0) hw = 4;
  int n = requested > 0 ? requested : std::min(hw, 8);
  const size_t by_size = std::max<size_t>(1, nbytes / kChunk);
  return static_cast<int>(std::min<size_t>(static_cast<size_t>(n), by_size));
}

}  // namespace

extern "C" {

// Writes nbytes from data to path (created / truncated) with positional writes from several threads.
// Returns 0 on success, errno-style code otherwise.
int b200h_write_file(const char* path, const void* data, unsigned long long nbytes, int threads) {
  const int fd = ::open(path, O_WRONLY | O_CREAT | O_TRUNC, 0644);
  if (fd < 0) return errno ? errno : -1;
  if (nbytes > 0 && ::ftruncate(fd, static_cast<off_t>(nbytes)) != 0) {
    const int e = errno;
    ::close(fd);
    return e ? e : -1;
  }
  const int n = clamp_threads(threads, nbytes);
  std::atomic<int> err{0};
  std::atomic<unsigned long long> next{0};
  auto worker = [&]() {
    while (true) {
      const unsigned long long off = next.fetch_add(kChunk);
      if (off >= nbytes || err.load()) return;
      size_t left = static_cast<size_t>(std::min<unsigned long long>(kChunk, nbytes - off));
      const char* src = static_cast<const char*>(data) + off;
      off_t pos = static_cast<off_t>(off);
      while (left > 0) {
        const ssize_t w = ::pwrite(fd, src, left, pos);
        if (w < 0) {
          if (errno == EINTR) continue;
          err.store(errno ? errno : -1);
          return;
        }
        src += w;
        pos += w;
        left -= static_cast<size_t>(w);
      }
    }
  };
  std::vector<std::thread> pool;
  for (int i = 1; i < n; ++i) pool.emplace_back(worker);
  worker();
  for (auto& t : pool) t.join();
  if (::fsync(fd) != 0 && !err.load()) err.store(errno ? errno : -1);
  ::close(fd);
  return err.load();
}

// Reads exactly nbytes from path into data.  Returns 0 on success.
int b200h_read_file(const char* path, void* data, unsigned long long nbytes, int threads) {
  const int fd = ::open(path, O_RDONLY);
  if (fd < 0) return errno ? errno : -1;
  struct stat st;
  if (::fstat(fd, &st) != 0 || static_cast<unsigned long long>(st.st_size) < nbytes) {
    ::close(fd);
    return EIO;
  }
  const int n = clamp_threads(threads, nbytes);
  std::atomic<int> err{0};
  std::atomic<unsigned long long> next{0};
  auto worker = [&]() {
    while (true) {
      const unsigned long long off = next.fetch_add(kChunk);
      if (off >= nbytes || err.load()) return;
      size_t left = static_cast<size_t>(std::min<unsigned long long>(kChunk, nbytes - off));
      char* dst = static_cast<char*>(data) + off;
      off_t pos = static_cast<off_t>(off);
      while (left > 0) {
        const ssize_t r = ::pread(fd, dst, left, pos);
        if (r < 0) {
          if (errno == EINTR) continue;
          err.store(errno ? errno : -1);
          return;
        }
        if (r == 0) {
          err.store(EIO);
          return;
        }
        dst += r;
        pos += r;
        left -= static_cast<size_t>(r);
      }
    }
  };
  std::vector<std::thread> pool;
  for (int i = 1; i < n; ++i) pool.emplace_back(worker);
  worker();
  for (auto& t : pool) t.join();
  ::close(fd);
  return err.load();
}

// Gathers `rows` windows of `window` uint32 tokens each from a set of memory-mapped shards into
// inputs[rows][window-1] and targets[rows][window-1] (int32): inputs = window[:-1], targets = window[1:].
// shard_ptrs[i] points at the first token of shard i, which covers absolute tokens [shard_starts[i],
// shard_starts[i+1]).  starts[r] is the absolute first token of row r.  Returns 0, or -1 if a window leaves
// the shards.
int b200h_gather_windows(const uint32_t* const* shard_ptrs, const long long* shard_starts, int num_shards,
                         const long long* starts, int rows, int window, int32_t* inputs, int32_t* targets,
                         int threads) {
  if (rows <= 0 || window < 2 || num_shards <= 0) return -1;
  std::atomic<int> err{0};
  std::atomic<int> next{0};
  const int n = std::max(1, std::min(threads > 0 ? threads : 4, rows));
  auto worker = [&]() {
    std::vector<uint32_t> tmp(static_cast<size_t>(window));
    while (true) {
      const int r = next.fetch_add(1);
      if (r >= rows || err.load()) return;
      long long pos = starts[r];
      int filled = 0;
      while (filled < window) {
        // locate the shard of `pos`
        int s = static_cast<int>(std::upper_bound(shard_starts, shard_starts + num_shards + 1, pos) - shard_starts) - 1;
        if (s < 0 || s >= num_shards) {
          err.store(-1);
          return;
        }
        const long long avail = shard_starts[s + 1] - pos;
        const int take = static_cast<int>(std::min<long long>(avail, window - filled));
        if (take <= 0) {
          err.store(-1);
          return;
        }
        std::memcpy(tmp.data() + filled, shard_ptrs[s] + (pos - shard_starts[s]), sizeof(uint32_t) * take);
        filled += take;
        pos += take;
      }
      int32_t* in = inputs + static_cast<size_t>(r) * (window - 1);
      int32_t* tg = targets + static_cast<size_t>(r) * (window - 1);
      for (int i = 0; i < window - 1; ++i) {
        in[i] = static_cast<int32_t>(tmp[i]);
        tg[i] = static_cast<int32_t>(tmp[i + 1]);
      }
    }
  };
  std::vector<std::thread> pool;
  for (int i = 1; i < n; ++i) pool.emplace_back(worker);
  worker();
  for (auto& t : pool) t.join();
  return err.load();
}

}  // extern "C"
