// Parallel positional reads of one file region into caller memory: checkpoint loading is a
// copy from the page cache (or the disk) into one large buffer, which one thread does at about
// 1 GB/s and several threads do at memory speed.  The reference streams its state dicts with a
// buffered reader (ferrotorch-serialize/src/state_dict.rs:167-260); the tensors there are copies,
// here they are views into the one buffer this call fills.
//
//   ftio_read(path, offset, nbytes, dst, threads) -> 0, or -errno / -1 (short file)
#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cstdint>
#include <fcntl.h>
#include <thread>
#include <unistd.h>
#include <vector>

#define FTIO_API extern "C" __attribute__((visibility("default")))

FTIO_API int ftio_read(const char* path, long long offset, long long nbytes, void* dst, int threads) {
  if (!path || !dst || offset < 0 || nbytes < 0) return -EINVAL;
  if (nbytes == 0) return 0;
  const int fd = open(path, O_RDONLY | O_CLOEXEC);
  if (fd < 0) return -errno;
  const long long chunk = 8ll << 20;                                   // work unit: 8 MiB
  const long long n_chunks = (nbytes + chunk - 1) / chunk;
  const int n_threads = static_cast<int>(std::max(1ll, std::min<long long>(threads > 0 ? threads : 4, n_chunks)));
  std::atomic<long long> next{0};
  std::atomic<int> error{0};
  auto work = [&]() {
    for (;;) {
      const long long c = next.fetch_add(1);
      if (c >= n_chunks || error.load() != 0) return;
      long long done = c * chunk;
      const long long end = std::min(nbytes, done + chunk);
      while (done < end) {
        const ssize_t r = pread(fd, static_cast<char*>(dst) + done, static_cast<size_t>(end - done), offset + done);
        if (r < 0) {
          if (errno == EINTR) continue;
          error.store(errno);
          return;
        }
        if (r == 0) {                                                  // the file ends before the region does
          error.store(-1);
          return;
        }
        done += r;
      }
    }
  };
  std::vector<std::thread> pool;
  for (int t = 1; t < n_threads; ++t) pool.emplace_back(work);
  work();
  for (auto& t : pool) t.join();
  close(fd);
  const int e = error.load();
  return e == 0 ? 0 : (e > 0 ? -e : -1);
}
