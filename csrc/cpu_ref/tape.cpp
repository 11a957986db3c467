// Tape autograd for the CPU backend, and the native MLP training loop built on it.
//
// Same model as the reference's autograd core (crates/incin-core/src/exec/tape.rs:49-306):
// every tensor has a process-unique id; each differentiable op pushes a node
// {output id, input ids, backward closure} onto a thread-local tape while
// gradient mode is on; backward() seeds ones at the loss, walks the nodes in
// reverse, calls each closure once and ACCUMULATES contributions per input id
// (fan-out sums), draining the tape.  A non-finite gradient is reported
// according to the NaN policy instead of being silently propagated.
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <mutex>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <algorithm>
#include <memory>
#include <thread>
#include <unordered_map>
#include <vector>

#define API extern "C" __attribute__((visibility("default")))

extern "C" void incin_cpu_philox_uniform_f32(float* out, int64_t n, uint64_t seed, uint64_t offset);
extern "C" void incin_cpu_philox_normal_f32(float* out, int64_t n, uint64_t seed, uint64_t offset, float mean,
                                            float std_);

namespace {

struct T {
  std::vector<float> v;
  int64_t rows = 0, cols = 0;  // everything the tape needs is rank <= 2
  uint64_t id = 0;
  bool requires_grad = false;
};
using TP = std::shared_ptr<T>;

std::atomic<uint64_t> g_next_id{1};

struct Node {
  uint64_t out;
  std::vector<uint64_t> ins;
  std::function<std::vector<std::vector<float>>(const std::vector<float>&)> backward;
};

struct Tape {
  std::vector<Node> nodes;
  bool grad_mode = true;
  int nan_policy = 0;  // 0 = ignore, 1 = report
  bool saw_non_finite = false;
  std::unordered_map<uint64_t, std::vector<float>> grads;
  std::unordered_map<int64_t, TP> handles;
  int64_t next_handle = 1;
};
thread_local Tape g_tape;

TP make(int64_t r, int64_t c, bool rg) {
  auto t = std::make_shared<T>();
  t->rows = r;
  t->cols = c;
  t->v.assign((size_t)(r * c), 0.f);
  t->id = g_next_id.fetch_add(1);
  t->requires_grad = rg;
  return t;
}
int64_t put(const TP& t) {
  const int64_t h = g_tape.next_handle++;
  g_tape.handles[h] = t;
  return h;
}
TP get(int64_t h) {
  auto it = g_tape.handles.find(h);
  return it == g_tape.handles.end() ? nullptr : it->second;
}
void push(Node n) {
  if (g_tape.grad_mode) g_tape.nodes.push_back(std::move(n));
}

// C[M,N] += A[M,K] * B[K,N].  A is addressed through (a_rs, a_cs) so a transposed left operand needs no copy; B
// and C are row-major.  Every output element accumulates its K products one at a time in ascending k, with
// separate multiply and add (the file is compiled without contraction), so the result does not depend on the
// tile sizes, on the instruction set the loader picked, or on how rows were split over threads.
// Vector types reach the templates through a traits struct: as template arguments themselves they would lose
// `aligned(4)` (loads from any float address) and `may_alias`.
struct Vec8 {
  typedef float type __attribute__((vector_size(32), aligned(4), may_alias));
};
struct Vec16 {
  typedef float type __attribute__((vector_size(64), aligned(4), may_alias));
};

// MR rows by NV vectors of columns held in registers over the whole K loop
template <class VT, int MR, int NV>
__attribute__((always_inline)) inline void gemm_tile_v(const float* A, int64_t a_rs, int64_t a_cs, const float* B,
                                                       int64_t ldb, float* C, int64_t ldc, int64_t K) {
  typedef typename VT::type V;
  constexpr int W = sizeof(V) / sizeof(float);
  V acc[MR][NV];
  for (int r = 0; r < MR; ++r)
    for (int c = 0; c < NV; ++c) acc[r][c] = *(const V*)(C + r * ldc + W * c);
  for (int64_t k = 0; k < K; ++k) {
    V b[NV];
    for (int c = 0; c < NV; ++c) b[c] = *(const V*)(B + k * ldb + W * c);
    for (int r = 0; r < MR; ++r) {
      const V av = A[r * a_rs + k * a_cs] - V{};  // scalar op vector broadcasts; x - (+0) is x for every x
      for (int c = 0; c < NV; ++c) acc[r][c] += av * b[c];
    }
  }
  for (int r = 0; r < MR; ++r)
    for (int c = 0; c < NV; ++c) *(V*)(C + r * ldc + W * c) = acc[r][c];
}

__attribute__((always_inline)) inline void gemm_col(const float* A, int64_t a_rs, int64_t a_cs, const float* B,
                                                    int64_t ldb, float* C, int64_t ldc, int64_t i0, int64_t i1,
                                                    int64_t K) {
  for (int64_t i = i0; i < i1; ++i) {
    float acc = C[i * ldc];
    for (int64_t k = 0; k < K; ++k) acc += A[i * a_rs + k * a_cs] * B[k * ldb];
    C[i * ldc] = acc;
  }
}

// NV vectors of columns at a time: that K-deep panel of B stays in cache while every row block of [i0, i1) passes
template <class VT, int NV>
__attribute__((always_inline)) inline void gemm_panel(const float* A, int64_t a_rs, int64_t a_cs, const float* B,
                                                      float* C, int64_t i0, int64_t i1, int64_t N, int64_t K) {
  constexpr int MR = 4;
  int64_t i = i0;
  for (; i + MR <= i1; i += MR) gemm_tile_v<VT, MR, NV>(A + i * a_rs, a_rs, a_cs, B, N, C + i * N, N, K);
  for (; i < i1; ++i) gemm_tile_v<VT, 1, NV>(A + i * a_rs, a_rs, a_cs, B, N, C + i * N, N, K);
}

template <class VT>
__attribute__((always_inline)) inline void gemm_rows_impl(const float* A, int64_t a_rs, int64_t a_cs, const float* B,
                                                          float* C, int64_t i0, int64_t i1, int64_t N, int64_t K) {
  constexpr int W = sizeof(typename VT::type) / sizeof(float);
  int64_t j = 0;
  for (; j + 2 * W <= N; j += 2 * W) gemm_panel<VT, 2>(A, a_rs, a_cs, B + j, C + j, i0, i1, N, K);
  for (; j + W <= N; j += W) gemm_panel<VT, 1>(A, a_rs, a_cs, B + j, C + j, i0, i1, N, K);
  for (; j + 8 <= N; j += 8) gemm_panel<Vec8, 1>(A, a_rs, a_cs, B + j, C + j, i0, i1, N, K);
  for (; j < N; ++j) gemm_col(A, a_rs, a_cs, B + j, N, C + j, N, i0, i1, K);
}

// 256-bit tiles for AVX2 / AVX / baseline (the loader picks the clone), 512-bit tiles where the CPU has AVX-512
__attribute__((target_clones("avx2", "avx", "default"))) void gemm_rows_256(const float* A, int64_t a_rs,
                                                                            int64_t a_cs, const float* B, float* C,
                                                                            int64_t i0, int64_t i1, int64_t N,
                                                                            int64_t K) {
  gemm_rows_impl<Vec8>(A, a_rs, a_cs, B, C, i0, i1, N, K);
}
__attribute__((target("avx512f"))) void gemm_rows_512(const float* A, int64_t a_rs, int64_t a_cs, const float* B,
                                                      float* C, int64_t i0, int64_t i1, int64_t N, int64_t K) {
  gemm_rows_impl<Vec16>(A, a_rs, a_cs, B, C, i0, i1, N, K);
}
void gemm_rows(const float* A, int64_t a_rs, int64_t a_cs, const float* B, float* C, int64_t i0, int64_t i1,
               int64_t N, int64_t K) {
  static const bool wide = __builtin_cpu_supports("avx512f");
  (wide ? gemm_rows_512 : gemm_rows_256)(A, a_rs, a_cs, B, C, i0, i1, N, K);
}

// A small pool of sleeping workers splits the rows of one product.  Starting threads per product costs about as
// much as the products of a small MLP; waking sleeping ones costs a few microseconds.  A forked child has no
// workers (threads do not survive fork) and computes on the calling thread.
class RowPool {
 public:
  static RowPool& get() {
    static RowPool p;
    return p;
  }
  // runs fn(lo, hi) over [0, M) in `parts` row ranges whose sizes are multiples of `align`
  void run(int64_t M, int64_t parts, int64_t align, const std::function<void(int64_t, int64_t)>& fn) {
    parts = std::min<int64_t>(parts, (int64_t)workers_->size() + 1);
    if (parts <= 1 || owner_ != getpid() || busy_.exchange(true)) {  // nested or concurrent callers run inline
      fn(0, M);
      return;
    }
    const int64_t per = ((M + parts - 1) / parts + align - 1) / align * align;
    const int64_t n_parts = (M + per - 1) / per;
    {
      std::lock_guard<std::mutex> l(m_);
      fn_ = &fn;
      M_ = M;
      per_ = per;
      n_parts_ = n_parts;
      next_part_ = 1;   // part 0 is the caller's
      pending_.store(n_parts - 1);
    }
    cv_.notify_all();
    fn(0, std::min(M, per));
    // the caller takes parts too, then waits for the ones the workers hold.  A part is claimed under the mutex
    // together with the job it belongs to, and this function returns only after every claimed part has finished
    // with no part left to claim, so a worker that wakes late never sees a job of an earlier call.
    for (;;) {
      int64_t part;
      {
        std::lock_guard<std::mutex> l(m_);
        if (next_part_ >= n_parts_) break;
        part = next_part_++;
      }
      fn(part * per, std::min(M, (part + 1) * per));
      pending_.fetch_sub(1, std::memory_order_release);
    }
    for (int spins = 0; pending_.load(std::memory_order_acquire) > 0; ++spins)
      if (spins > 2000) std::this_thread::yield();
    busy_.store(false);
  }

 private:
  RowPool() : workers_(new std::vector<std::thread>), owner_(getpid()) {
    const unsigned hc = std::max(1u, std::thread::hardware_concurrency());
    for (unsigned i = 1; i < std::min(hc, 8u); ++i) workers_->emplace_back([this] { work(); });
  }
  ~RowPool() {
    if (owner_ != getpid()) return;   // a forked child has no such threads: their handles are left alone
    {
      std::lock_guard<std::mutex> l(m_);
      stop_ = true;
    }
    cv_.notify_all();
    for (auto& t : *workers_) t.join();
    delete workers_;
  }
  void work() {
    std::unique_lock<std::mutex> l(m_);
    for (;;) {
      cv_.wait(l, [&] { return stop_ || next_part_ < n_parts_; });
      if (stop_) return;
      const int64_t part = next_part_++, M = M_, per = per_;
      const std::function<void(int64_t, int64_t)>* fn = fn_;
      l.unlock();
      (*fn)(part * per, std::min(M, (part + 1) * per));
      pending_.fetch_sub(1, std::memory_order_release);
      l.lock();
    }
  }
  std::vector<std::thread>* workers_;
  std::mutex m_;
  std::condition_variable cv_;
  const std::function<void(int64_t, int64_t)>* fn_ = nullptr;
  int64_t M_ = 0, per_ = 0, n_parts_ = 0, next_part_ = 0;   // guarded by m_
  std::atomic<int64_t> pending_{0};
  std::atomic<bool> busy_{false};
  bool stop_ = false;
  pid_t owner_;
};

void gemm_acc(const float* A, int64_t a_rs, int64_t a_cs, const float* B, float* C, int64_t M, int64_t N,
              int64_t K) {
  const int64_t flops = 2 * M * N * K;
  const int64_t parts = std::min<int64_t>({8, M / 8, flops >> 20});
  if (parts <= 1) {
    gemm_rows(A, a_rs, a_cs, B, C, 0, M, N, K);
    return;
  }
  RowPool::get().run(M, parts, 4,
                     [&](int64_t lo, int64_t hi) { gemm_rows(A, a_rs, a_cs, B, C, lo, hi, N, K); });
}

// out[C,R] = in[R,C]^T in 16x16 blocks (both sides stay within a few cache lines per block)
void transpose(const float* in, float* out, int64_t R, int64_t Cn) {
  constexpr int64_t TB = 16;
  for (int64_t r0 = 0; r0 < R; r0 += TB)
    for (int64_t c0 = 0; c0 < Cn; c0 += TB)
      for (int64_t r = r0; r < std::min(R, r0 + TB); ++r)
        for (int64_t c = c0; c < std::min(Cn, c0 + TB); ++c) out[c * R + r] = in[r * Cn + c];
}

// y[M,N] = x[M,K] * w[N,K]^T + b[N]
TP linear(const TP& x, const TP& w, const TP& b) {
  const int64_t M = x->rows, K = x->cols, N = w->rows;
  TP y = make(M, N, true);
  // The vector loop runs over the columns of a row-major right operand, so one side has to be transposed:
  // either w (N*K elements) for y = x * w^T, or x and the result (M*(K+N)) for y^T = w * x^T.  Both forms add
  // the K products of an output in the same order; the cheaper transposition wins.
  if (M * (K + N) < N * K) {
    std::vector<float> xt((size_t)(K * M)), yt((size_t)(N * M));
    transpose(x->v.data(), xt.data(), M, K);
    for (int64_t j = 0; j < N; ++j)
      for (int64_t i = 0; i < M; ++i) yt[(size_t)(j * M + i)] = b ? b->v[(size_t)j] : 0.f;
    gemm_acc(w->v.data(), K, 1, xt.data(), yt.data(), N, M, K);
    transpose(yt.data(), y->v.data(), N, M);
  } else {
    std::vector<float> wt((size_t)(K * N));
    transpose(w->v.data(), wt.data(), N, K);
    for (int64_t i = 0; i < M; ++i)
      for (int64_t j = 0; j < N; ++j) y->v[(size_t)(i * N + j)] = b ? b->v[(size_t)j] : 0.f;
    gemm_acc(x->v.data(), K, 1, wt.data(), y->v.data(), M, N, K);
  }
  std::vector<uint64_t> ins = {x->id, w->id};
  if (b) ins.push_back(b->id);
  push({y->id, ins, [x, w, b, M, N, K](const std::vector<float>& g) {
          std::vector<std::vector<float>> out;
          // dx[M,K] = g[M,N] * w[N,K] (skipped for an input that takes no gradient); dw[N,K] = g^T[N,M] * x[M,K]
          std::vector<float> dx, dw((size_t)(N * K), 0.f);
          if (x->requires_grad) {
            dx.assign((size_t)(M * K), 0.f);
            gemm_acc(g.data(), N, 1, w->v.data(), dx.data(), M, K, N);
          }
          gemm_acc(g.data(), 1, N, x->v.data(), dw.data(), N, K, M);
          out.push_back(std::move(dx));
          out.push_back(std::move(dw));
          if (b) {
            std::vector<float> db((size_t)N, 0.f);
            for (int64_t i = 0; i < M; ++i)
              for (int64_t j = 0; j < N; ++j) db[(size_t)j] += g[(size_t)(i * N + j)];
            out.push_back(std::move(db));
          }
          return out;
        }});
  return y;
}

TP relu(const TP& x) {
  TP y = make(x->rows, x->cols, true);
  for (size_t i = 0; i < x->v.size(); ++i) y->v[i] = x->v[i] > 0 ? x->v[i] : 0.f;
  push({y->id, {x->id}, [x](const std::vector<float>& g) {
          std::vector<float> dx(g.size());
          for (size_t i = 0; i < g.size(); ++i) dx[i] = x->v[i] > 0 ? g[i] : 0.f;
          return std::vector<std::vector<float>>{std::move(dx)};
        }});
  return y;
}

// mean over rows of -log_softmax(logits)[target]
TP cross_entropy(const TP& logits, const std::vector<int64_t>& tgt) {
  const int64_t R = logits->rows, V = logits->cols;
  TP loss = make(1, 1, true);
  auto prob = std::make_shared<std::vector<float>>((size_t)(R * V));
  double total = 0;
  for (int64_t r = 0; r < R; ++r) {
    const float* lr = &logits->v[(size_t)(r * V)];
    float m = lr[0];
    for (int64_t c = 1; c < V; ++c) m = std::max(m, lr[c]);
    double s = 0;
    for (int64_t c = 0; c < V; ++c) s += std::exp((double)lr[c] - m);
    const double lse = m + std::log(s);
    total += lse - lr[tgt[(size_t)r]];
    for (int64_t c = 0; c < V; ++c) (*prob)[(size_t)(r * V + c)] = (float)std::exp((double)lr[c] - lse);
  }
  loss->v[0] = (float)(total / R);
  push({loss->id, {logits->id}, [prob, tgt, R, V](const std::vector<float>& g) {
          std::vector<float> d((size_t)(R * V));
          for (int64_t r = 0; r < R; ++r)
            for (int64_t c = 0; c < V; ++c)
              d[(size_t)(r * V + c)] =
                  g[0] * ((*prob)[(size_t)(r * V + c)] - (c == tgt[(size_t)r] ? 1.f : 0.f)) / (float)R;
          return std::vector<std::vector<float>>{std::move(d)};
        }});
  return loss;
}

void backward(const TP& root) {
  auto& grads = g_tape.grads;
  grads.clear();
  grads[root->id] = std::vector<float>(root->v.size(), 1.0f);  // ones_like seed
  for (auto it = g_tape.nodes.rbegin(); it != g_tape.nodes.rend(); ++it) {
    auto g = grads.find(it->out);
    if (g == grads.end()) continue;  // not on a path to the root
    auto contrib = it->backward(g->second);
    for (size_t i = 0; i < it->ins.size() && i < contrib.size(); ++i) {
      auto& c = contrib[i];
      if (c.empty()) continue;  // this input takes no gradient
      if (g_tape.nan_policy)
        for (float f : c)
          if (!std::isfinite(f)) {
            g_tape.saw_non_finite = true;
            break;
          }
      auto slot = grads.find(it->ins[i]);
      if (slot == grads.end()) {
        grads.emplace(it->ins[i], std::move(c));
      } else {
        for (size_t k = 0; k < c.size(); ++k) slot->second[k] += c[k];  // fan-out accumulates
      }
    }
  }
  g_tape.nodes.clear();  // the tape is drained once
}

}  // namespace

// ---- handle API ---------------------------------------------------------------------------------
API int64_t incin_tape_tensor(const float* data, int64_t rows, int64_t cols, int requires_grad) {
  TP t = make(rows, cols, requires_grad != 0);
  if (data) std::memcpy(t->v.data(), data, sizeof(float) * (size_t)(rows * cols));
  return put(t);
}
API int64_t incin_tape_linear(int64_t x, int64_t w, int64_t b) {
  TP tx = get(x), tw = get(w), tb = b ? get(b) : nullptr;
  if (!tx || !tw || tx->cols != tw->cols || (tb && (int64_t)tb->v.size() != tw->rows)) return 0;
  return put(linear(tx, tw, tb));
}
API int64_t incin_tape_relu(int64_t x) {
  TP tx = get(x);
  return tx ? put(relu(tx)) : 0;
}
API int64_t incin_tape_cross_entropy(int64_t logits, const int64_t* targets) {
  TP tl = get(logits);
  if (!tl) return 0;
  std::vector<int64_t> t(targets, targets + tl->rows);
  for (int64_t v : t)
    if (v < 0 || v >= tl->cols) return 0;
  return put(cross_entropy(tl, t));
}
API int incin_tape_backward(int64_t root) {
  TP t = get(root);
  if (!t) return 1;
  backward(t);
  return g_tape.saw_non_finite ? 2 : 0;
}
API int incin_tape_read(int64_t h, float* out) {
  TP t = get(h);
  if (!t) return 1;
  std::memcpy(out, t->v.data(), sizeof(float) * t->v.size());
  return 0;
}
API int incin_tape_grad(int64_t h, float* out) {
  TP t = get(h);
  if (!t) return 1;
  auto g = g_tape.grads.find(t->id);
  if (g == g_tape.grads.end()) return 2;
  std::memcpy(out, g->second.data(), sizeof(float) * g->second.size());
  return 0;
}
API int64_t incin_tape_depth(void) { return (int64_t)g_tape.nodes.size(); }
API void incin_tape_set_grad_mode(int on) { g_tape.grad_mode = on != 0; }
API void incin_tape_set_nan_policy(int p) {
  g_tape.nan_policy = p;
  g_tape.saw_non_finite = false;
}
API void incin_tape_reset(void) {
  g_tape.nodes.clear();
  g_tape.grads.clear();
  g_tape.handles.clear();
  g_tape.saw_non_finite = false;
}
API uint64_t incin_tape_tensor_id(int64_t h) {
  TP t = get(h);
  return t ? t->id : 0;
}

// ---- the CPU-backend MLP benchmark, end to end in native code ---------------------------------------
// Linear(in -> hidden) -> ReLU -> Linear(hidden -> out), softmax cross-entropy, plain SGD.
// Seed-0 generator: Philox4x32-10 keyed by `seed`.  Stream offsets: 0/1 = layer-1 weight/bias,
// 2/3 = layer-2 weight/bias (Kaiming-uniform with a = sqrt(5): U(-1/sqrt(fan_in), 1/sqrt(fan_in)),
// the bias uses the same bound), 16 = inputs ~ N(0,1), 17 = labels = floor(u * out).
API int incin_cpu_mlp_train(int steps, int batch, int n_in, int n_hidden, int n_out, float lr, uint64_t seed,
                            float* losses_out, float* final_params_out) {
  incin_tape_reset();
  auto kaiming = [&](int64_t rows, int64_t cols, int64_t fan_in, uint64_t off) {
    TP t = make(rows, cols, true);
    incin_cpu_philox_uniform_f32(t->v.data(), rows * cols, seed, off);
    const float bound = 1.0f / std::sqrt((float)fan_in);
    for (auto& f : t->v) f = (2.f * f - 1.f) * bound;
    return t;
  };
  TP w1 = kaiming(n_hidden, n_in, n_in, 0), b1 = kaiming(1, n_hidden, n_in, 1);
  TP w2 = kaiming(n_out, n_hidden, n_hidden, 2), b2 = kaiming(1, n_out, n_hidden, 3);
  TP x = make(batch, n_in, false);
  incin_cpu_philox_normal_f32(x->v.data(), (int64_t)batch * n_in, seed, 16, 0.f, 1.f);
  std::vector<float> u((size_t)batch);
  incin_cpu_philox_uniform_f32(u.data(), batch, seed, 17);
  std::vector<int64_t> y((size_t)batch);
  for (int i = 0; i < batch; ++i) y[(size_t)i] = std::min<int64_t>(n_out - 1, (int64_t)(u[(size_t)i] * n_out));
  for (int s = 0; s < steps; ++s) {
    TP h = relu(linear(x, w1, b1));
    TP loss = cross_entropy(linear(h, w2, b2), y);
    if (losses_out) losses_out[s] = loss->v[0];
    backward(loss);
    for (const TP& p : {w1, b1, w2, b2}) {
      const auto& g = g_tape.grads[p->id];
      for (size_t i = 0; i < p->v.size(); ++i) p->v[i] -= lr * g[i];
    }
  }
  if (final_params_out) {
    float* o = final_params_out;
    for (const TP& p : {w1, b1, w2, b2}) {
      std::memcpy(o, p->v.data(), sizeof(float) * p->v.size());
      o += p->v.size();
    }
  }
  return 0;
}
