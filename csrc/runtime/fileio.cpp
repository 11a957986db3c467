// Parallel positional reads: fill many destination buffers from byte ranges of one file with a few threads.
//
// Loading a checkpoint is a list of (file offset, size, destination) triples once the header has been validated.
// One thread issuing read() after read() leaves most of an NVMe array (or a parallel file system) idle; here the
// ranges are cut into pieces of at most 64 MiB, and `threads` workers take pieces from a shared counter and pread()
// them straight into their destinations (typically pinned host tensors), so the result does not depend on the order in
// which pieces finish.  Used by the safetensors loader of the Python package for multi-GB shards.
#include <atomic>
#include <cerrno>
#include <cstdint>
#include <fcntl.h>
#include <thread>
#include <unistd.h>
#include <vector>

#define API extern "C" __attribute__((visibility("default")))

namespace {
struct Piece {
  int64_t off, size;
  uint8_t* dst;
};
constexpr int64_t kPiece = 64ll << 20;
}  // namespace

// 0 = ok, 1 = cannot open, 2 = read error or short file, 3 = bad arguments.
API int incin_file_read_ranges(const char* path, int64_t n, const int64_t* offsets, const int64_t* sizes, void* const* dst,
                               int threads) {
  if (!path || n < 0 || (n > 0 && (!offsets || !sizes || !dst))) return 3;
  std::vector<Piece> pieces;
  for (int64_t i = 0; i < n; ++i) {
    if (offsets[i] < 0 || sizes[i] < 0 || (sizes[i] > 0 && !dst[i])) return 3;
    for (int64_t done = 0; done < sizes[i]; done += kPiece) {
      const int64_t len = sizes[i] - done < kPiece ? sizes[i] - done : kPiece;
      pieces.push_back({offsets[i] + done, len, static_cast<uint8_t*>(dst[i]) + done});
    }
  }
  if (pieces.empty()) return 0;
  const int fd = ::open(path, O_RDONLY | O_CLOEXEC);
  if (fd < 0) return 1;
  std::atomic<size_t> next{0};
  std::atomic<int> failed{0};
  auto work = [&] {
    for (;;) {
      const size_t k = next.fetch_add(1);
      if (k >= pieces.size() || failed.load()) return;
      const Piece& p = pieces[k];
      int64_t got = 0;
      while (got < p.size) {
        const ssize_t r = ::pread(fd, p.dst + got, static_cast<size_t>(p.size - got), static_cast<off_t>(p.off + got));
        if (r < 0 && errno == EINTR) continue;
        if (r <= 0) {  // error, or the file ends before the range does
          failed.store(1);
          return;
        }
        got += r;
      }
    }
  };
  int nt = threads < 1 ? 1 : (threads > 64 ? 64 : threads);
  if (static_cast<size_t>(nt) > pieces.size()) nt = static_cast<int>(pieces.size());
  std::vector<std::thread> pool;
  for (int t = 1; t < nt; ++t) pool.emplace_back(work);
  work();
  for (auto& t : pool) t.join();
  ::close(fd);
  return failed.load() ? 2 : 0;
}
