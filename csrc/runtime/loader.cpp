// Native batch loader: worker threads gather rows of an in-memory dataset into batch buffers ahead of the consumer.
//
// The dataset is one or two row-major arrays with the same number of rows (samples and, optionally, targets).  An
// epoch visits the rows in index order or in a seeded permutation (Fisher-Yates driven by splitmix64 of seed + epoch),
// so the sequence of batches depends only on (seed, epoch, batch size): any number of workers delivers the same
// batches in the same order.  Workers claim batch numbers in order, fill a ring of `depth` slots and block while the
// ring is full, so memory stays bounded; the consumer copies the next slot into its own (typically pinned) buffers.
// The reference's loader is the Rust `DataLoader` with the same contract: ordered delivery, bounded prefetch, a
// worker error surfaces at the consumer (crates/incin/src/data).
#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

#define API extern "C" __attribute__((visibility("default")))

namespace {

inline uint64_t splitmix64(uint64_t& s) {
  uint64_t z = (s += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

struct Slot {
  std::vector<uint8_t> a, b;
  int64_t rows = 0;
  int64_t batch = -1;  // which batch number the slot holds
  bool ready = false;
};

struct Loader {
  const uint8_t* a = nullptr;
  const uint8_t* b = nullptr;
  int64_t n_rows = 0, row_bytes_a = 0, row_bytes_b = 0;
  int64_t batch = 1;
  bool shuffle = false, drop_last = false;
  uint64_t seed = 0;
  int workers = 1, depth = 2;

  std::vector<int64_t> order;
  int64_t n_batches = 0;
  std::vector<Slot> slots;
  std::mutex mu;
  std::condition_variable cv;
  int64_t next_claim = 0;    // next batch number a worker takes
  int64_t next_deliver = 0;  // next batch number the consumer takes
  bool stop = false;
  std::vector<std::thread> threads;

  void join() {
    {
      std::lock_guard<std::mutex> lock(mu);
      stop = true;
    }
    cv.notify_all();
    for (auto& t : threads)
      if (t.joinable()) t.join();
    threads.clear();
  }

  void work() {
    for (;;) {
      int64_t k;
      {
        std::unique_lock<std::mutex> lock(mu);
        if (stop || next_claim >= n_batches) return;
        k = next_claim++;
        // the slot is free once the batch that used it before (k - depth) has been delivered
        cv.wait(lock, [&] { return stop || k - next_deliver < depth; });
        if (stop) return;
      }
      Slot& s = slots[static_cast<size_t>(k % depth)];
      const int64_t lo = k * batch;
      const int64_t hi = std::min(n_rows, lo + batch);
      for (int64_t i = lo; i < hi; ++i) {
        const int64_t r = order[static_cast<size_t>(i)];
        std::memcpy(s.a.data() + (i - lo) * row_bytes_a, a + r * row_bytes_a, static_cast<size_t>(row_bytes_a));
        if (b) std::memcpy(s.b.data() + (i - lo) * row_bytes_b, b + r * row_bytes_b, static_cast<size_t>(row_bytes_b));
      }
      {
        std::lock_guard<std::mutex> lock(mu);
        s.rows = hi - lo;
        s.batch = k;
        s.ready = true;
      }
      cv.notify_all();
    }
  }

  void start(uint64_t epoch) {
    join();
    order.resize(static_cast<size_t>(n_rows));
    for (int64_t i = 0; i < n_rows; ++i) order[static_cast<size_t>(i)] = i;
    if (shuffle) {
      uint64_t st = seed + epoch;
      for (int64_t i = n_rows - 1; i > 0; --i) {
        const int64_t j = static_cast<int64_t>(splitmix64(st) % static_cast<uint64_t>(i + 1));
        std::swap(order[static_cast<size_t>(i)], order[static_cast<size_t>(j)]);
      }
    }
    n_batches = drop_last ? n_rows / batch : (n_rows + batch - 1) / batch;
    slots.assign(static_cast<size_t>(depth), Slot{});
    for (auto& s : slots) {
      s.a.resize(static_cast<size_t>(batch * row_bytes_a));
      if (b) s.b.resize(static_cast<size_t>(batch * row_bytes_b));
    }
    next_claim = next_deliver = 0;
    stop = false;
    for (int i = 0; i < workers; ++i) threads.emplace_back([this] { work(); });
  }
};

std::mutex g_mu;
std::unordered_map<int64_t, Loader*> g_loaders;
int64_t g_next = 1;

Loader* find(int64_t h) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_loaders.find(h);
  return it == g_loaders.end() ? nullptr : it->second;
}

}  // namespace

// Returns a handle (> 0) or 0 on bad arguments.  `b` may be null (no second array).  The arrays must outlive the loader.
API int64_t incin_loader_create(const void* a, int64_t row_bytes_a, const void* b, int64_t row_bytes_b, int64_t n_rows,
                                int64_t batch, int shuffle, int drop_last, uint64_t seed, int workers, int depth) {
  if (!a || row_bytes_a <= 0 || n_rows < 0 || batch < 1 || (b && row_bytes_b <= 0)) return 0;
  auto* l = new Loader();
  l->a = static_cast<const uint8_t*>(a);
  l->b = static_cast<const uint8_t*>(b);
  l->row_bytes_a = row_bytes_a;
  l->row_bytes_b = b ? row_bytes_b : 0;
  l->n_rows = n_rows;
  l->batch = batch;
  l->shuffle = shuffle != 0;
  l->drop_last = drop_last != 0;
  l->seed = seed;
  l->workers = workers < 1 ? 1 : (workers > 64 ? 64 : workers);
  l->depth = depth < 2 ? 2 : (depth > 256 ? 256 : depth);
  std::lock_guard<std::mutex> lock(g_mu);
  const int64_t h = g_next++;
  g_loaders[h] = l;
  return h;
}

// Begin epoch `epoch` (stops a running one).  Returns the number of batches of the epoch, or -1 for a bad handle.
API int64_t incin_loader_start(int64_t h, uint64_t epoch) {
  Loader* l = find(h);
  if (!l) return -1;
  l->start(epoch);
  return l->n_batches;
}

// Copy the next batch into out_a (batch * row_bytes_a bytes) and out_b; *rows_out = rows in the batch (the last one
// may be short).  Returns 1 when a batch was delivered, 0 at the end of the epoch, -1 for a bad handle / no epoch.
API int incin_loader_next(int64_t h, void* out_a, void* out_b, int64_t* rows_out) {
  Loader* l = find(h);
  if (!l || !out_a || l->slots.empty()) return -1;
  int64_t k;
  {
    std::unique_lock<std::mutex> lock(l->mu);
    if (l->next_deliver >= l->n_batches) return 0;
    k = l->next_deliver;
    Slot& s = l->slots[static_cast<size_t>(k % l->depth)];
    l->cv.wait(lock, [&] { return l->stop || (s.ready && s.batch == k); });
    if (l->stop) return -1;
  }
  Slot& s = l->slots[static_cast<size_t>(k % l->depth)];
  std::memcpy(out_a, s.a.data(), static_cast<size_t>(s.rows * l->row_bytes_a));
  if (l->b && out_b) std::memcpy(out_b, s.b.data(), static_cast<size_t>(s.rows * l->row_bytes_b));
  if (rows_out) *rows_out = s.rows;
  {
    std::lock_guard<std::mutex> lock(l->mu);
    s.ready = false;
    l->next_deliver = k + 1;
  }
  l->cv.notify_all();
  return 1;
}

// The row order of the current epoch (n_rows entries), for tests and for resuming mid-epoch.
API int incin_loader_order(int64_t h, int64_t* out) {
  Loader* l = find(h);
  if (!l || !out || l->order.empty()) return -1;
  std::memcpy(out, l->order.data(), l->order.size() * sizeof(int64_t));
  return 0;
}

API void incin_loader_destroy(int64_t h) {
  Loader* l = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_loaders.find(h);
    if (it == g_loaders.end()) return;
    l = it->second;
    g_loaders.erase(it);
  }
  l->join();
  delete l;
}
