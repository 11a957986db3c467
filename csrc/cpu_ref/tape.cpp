// Tape autograd for the CPU backend, and the native MLP training loop built on it.
//
// Same model as the reference's autograd core (crates/incin-core/src/exec/tape.rs:49-306):
// every tensor has a process-unique id; each differentiable op pushes a node
// {output id, input ids, backward closure} onto a thread-local tape while
// gradient mode is on; backward() seeds ones at the loss, walks the nodes in
// reverse, calls each closure once and ACCUMULATES contributions per input id
// (fan-out sums), draining the tape.  A non-finite gradient is reported
// according to the NaN policy instead of being silently propagated.
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <memory>
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

// y[M,N] = x[M,K] * w[N,K]^T + b[N]
TP linear(const TP& x, const TP& w, const TP& b) {
  const int64_t M = x->rows, K = x->cols, N = w->rows;
  TP y = make(M, N, true);
  // y[i, :] = b + sum_k x[i, k] * wt[k, :]: the inner loop runs over independent outputs, so it vectorises
  // without reassociating the reduction (bit-stable across compilers, unlike a dot-product inner loop)
  std::vector<float> wt((size_t)(K * N));
  for (int64_t j = 0; j < N; ++j)
    for (int64_t k = 0; k < K; ++k) wt[(size_t)(k * N + j)] = w->v[(size_t)(j * K + k)];
  for (int64_t i = 0; i < M; ++i) {
    float* yr = &y->v[(size_t)(i * N)];
    for (int64_t j = 0; j < N; ++j) yr[j] = b ? b->v[(size_t)j] : 0.f;
    const float* xr = &x->v[(size_t)(i * K)];
    for (int64_t k = 0; k < K; ++k) {
      const float xv = xr[k];
      const float* wr = &wt[(size_t)(k * N)];
      for (int64_t j = 0; j < N; ++j) yr[j] += xv * wr[j];
    }
  }
  std::vector<uint64_t> ins = {x->id, w->id};
  if (b) ins.push_back(b->id);
  push({y->id, ins, [x, w, b, M, N, K](const std::vector<float>& g) {
          std::vector<std::vector<float>> out;
          std::vector<float> dx((size_t)(M * K), 0.f), dw((size_t)(N * K), 0.f);
          for (int64_t i = 0; i < M; ++i)
            for (int64_t j = 0; j < N; ++j) {
              const float gy = g[(size_t)(i * N + j)];
              if (gy == 0.f) continue;
              const float *xr = &x->v[(size_t)(i * K)], *wr = &w->v[(size_t)(j * K)];
              float *dxr = &dx[(size_t)(i * K)], *dwr = &dw[(size_t)(j * K)];
              for (int64_t k = 0; k < K; ++k) {
                dxr[k] += gy * wr[k];
                dwr[k] += gy * xr[k];
              }
            }
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
