// N-rank TCP rendezvous and control channel (rank 0 is the root of a star).
//
// Mirrors the behaviour of the reference's two-rank rendezvous
// (crates/incin-core/src/dist/context.rs:967-1254), generalised to any world
// size: fixed-size framed messages with a magic, bounded accept/connect/read
// deadlines everywhere, validation of world size / rank / run id before a peer
// is admitted, and a control channel that stays open for Abort / Shutdown so a
// failing rank can fail-stop the others from the host, without touching a GPU.
//
// Startup frame, 160 bytes:  magic "INCINRV1"[0..8] kind[8] rank[9] world[10]
//   code[12..14] BE  local_cuda_device[16..24] BE  run_id_len[24..26] BE  run_id[32..160]
// Control frame, 16 bytes:   magic[0..8] kind[8] rank[9] code[10..12] BE
// Kinds: Hello=1 Accepted=2 Reject=3 Shutdown=4 Abort=5 Data=6 (payload length in a second frame).
#include <arpa/inet.h>
#include <cerrno>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <fcntl.h>
#include <mutex>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <string>
#include <sys/socket.h>
#include <unistd.h>
#include <unordered_map>
#include <vector>

#define API extern "C" __attribute__((visibility("default")))

namespace {

constexpr char MAGIC[8] = {'I', 'N', 'C', 'I', 'N', 'R', 'V', '1'};
enum Kind : uint8_t { Hello = 1, Accepted = 2, Reject = 3, Shutdown = 4, Abort = 5, Data = 6 };
enum State : int { Active = 0, ShuttingDown = 1, ShutdownDone = 2, Failed = 3 };
enum Err : int {
  OK = 0, E_TIMEOUT = 1, E_IO = 2, E_MAGIC = 3, E_WORLD = 4, E_RANK = 5, E_RUN_ID = 6, E_REJECTED = 7, E_STATE = 8,
  E_ABORTED = 9, E_ARG = 10, E_DUP_RANK = 11
};

using Clock = std::chrono::steady_clock;
int64_t ms_left(Clock::time_point deadline) {
  return std::chrono::duration_cast<std::chrono::milliseconds>(deadline - Clock::now()).count();
}

struct Ctx {
  int rank = 0, world = 1;
  int state = Active;
  int failure_code = 0;
  int listen_fd = -1;
  std::vector<int> fds;  // root: fd per rank (own slot -1); others: fds[0] = root
  std::vector<int64_t> peer_devices;
  std::mutex mu;
};

std::mutex g_mu;
std::unordered_map<int64_t, Ctx*> g_ctx;
int64_t g_next = 1;

Ctx* find(int64_t h) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_ctx.find(h);
  return it == g_ctx.end() ? nullptr : it->second;
}

int wait_fd(int fd, short ev, Clock::time_point deadline) {
  for (;;) {
    const int64_t left = ms_left(deadline);
    if (left <= 0) return E_TIMEOUT;
    pollfd p{fd, ev, 0};
    const int r = ::poll(&p, 1, (int)std::min<int64_t>(left, 200));
    if (r > 0) return (p.revents & (POLLERR | POLLNVAL)) ? E_IO : OK;
    if (r < 0 && errno != EINTR) return E_IO;
  }
}
int write_all(int fd, const void* buf, size_t n, Clock::time_point deadline) {
  const char* p = (const char*)buf;
  while (n) {
    int w = wait_fd(fd, POLLOUT, deadline);
    if (w) return w;
    const ssize_t k = ::send(fd, p, n, MSG_NOSIGNAL);
    if (k < 0) {
      if (errno == EAGAIN || errno == EINTR) continue;
      return E_IO;
    }
    p += k;
    n -= (size_t)k;
  }
  return OK;
}
int read_all(int fd, void* buf, size_t n, Clock::time_point deadline) {
  char* p = (char*)buf;
  while (n) {
    int w = wait_fd(fd, POLLIN, deadline);
    if (w) return w;
    const ssize_t k = ::recv(fd, p, n, 0);
    if (k == 0) return E_IO;  // peer closed
    if (k < 0) {
      if (errno == EAGAIN || errno == EINTR) continue;
      return E_IO;
    }
    p += k;
    n -= (size_t)k;
  }
  return OK;
}
void put16(uint8_t* p, uint16_t v) { p[0] = v >> 8; p[1] = v & 0xff; }
uint16_t get16(const uint8_t* p) { return (uint16_t)((p[0] << 8) | p[1]); }
void put64(uint8_t* p, uint64_t v) { for (int i = 0; i < 8; ++i) p[i] = (uint8_t)(v >> (56 - 8 * i)); }
uint64_t get64(const uint8_t* p) { uint64_t v = 0; for (int i = 0; i < 8; ++i) v = (v << 8) | p[i]; return v; }

void startup_frame(uint8_t* f, Kind k, int rank, int world, int code, int64_t dev, const std::string& run) {
  std::memset(f, 0, 160);
  std::memcpy(f, MAGIC, 8);
  f[8] = k; f[9] = (uint8_t)rank; f[10] = (uint8_t)world;
  put16(f + 12, (uint16_t)code);
  put64(f + 16, (uint64_t)dev);
  const size_t n = std::min<size_t>(run.size(), 128);
  put16(f + 24, (uint16_t)n);
  std::memcpy(f + 32, run.data(), n);
}
void control_frame(uint8_t* f, Kind k, int rank, int code) {
  std::memset(f, 0, 16);
  std::memcpy(f, MAGIC, 8);
  f[8] = k; f[9] = (uint8_t)rank;
  put16(f + 10, (uint16_t)code);
}
void set_nonblock(int fd) {
  const int fl = fcntl(fd, F_GETFL, 0);
  fcntl(fd, F_SETFL, fl | O_NONBLOCK);
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
}
bool split_addr(const char* addr, std::string& host, int& port) {
  const std::string a(addr ? addr : "");
  const size_t c = a.rfind(':');
  if (c == std::string::npos) return false;
  host = a.substr(0, c);
  port = std::atoi(a.c_str() + c + 1);
  return port > 0 && port < 65536 && !host.empty();
}
void fail(Ctx* c, int code) {
  c->state = Failed;
  c->failure_code = code;
}
void close_all(Ctx* c) {
  for (int& fd : c->fds)
    if (fd >= 0) { ::close(fd); fd = -1; }
  if (c->listen_fd >= 0) { ::close(c->listen_fd); c->listen_fd = -1; }
}

}  // namespace

// Returns 0 and a handle, or an error code (no handle).  Every wait is bounded by timeout_ms.
API int incin_rdv_connect(int rank, int world, const char* addr, const char* run_id, int64_t local_device,
                          int timeout_ms, int64_t* handle_out) {
  if (world < 1 || world > 255 || rank < 0 || rank >= world || !handle_out) return E_ARG;
  std::string host;
  int port = 0;
  if (world > 1 && !split_addr(addr, host, port)) return E_ARG;
  const std::string run(run_id ? run_id : "");
  const auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  Ctx* c = new Ctx();
  c->rank = rank;
  c->world = world;
  c->peer_devices.assign((size_t)world, -1);
  c->peer_devices[(size_t)rank] = local_device;
  int err = OK;
  if (world == 1) {
    // nothing to connect
  } else if (rank == 0) {
    c->fds.assign((size_t)world, -1);
    c->listen_fd = ::socket(AF_INET, SOCK_STREAM, 0);
    int one = 1;
    setsockopt(c->listen_fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in sa{};
    sa.sin_family = AF_INET;
    sa.sin_port = htons((uint16_t)port);
    if (inet_pton(AF_INET, host.c_str(), &sa.sin_addr) != 1) sa.sin_addr.s_addr = htonl(INADDR_ANY);
    if (::bind(c->listen_fd, (sockaddr*)&sa, sizeof(sa)) != 0 || ::listen(c->listen_fd, world) != 0) err = E_IO;
    set_nonblock(c->listen_fd);
    int admitted = 0;
    while (!err && admitted < world - 1) {
      err = wait_fd(c->listen_fd, POLLIN, deadline);
      if (err) break;
      const int fd = ::accept(c->listen_fd, nullptr, nullptr);
      if (fd < 0) continue;
      set_nonblock(fd);
      uint8_t f[160], reply[160];
      int verdict = OK;
      if (read_all(fd, f, 160, deadline) != OK) { ::close(fd); continue; }
      if (std::memcmp(f, MAGIC, 8) != 0 || f[8] != Hello) verdict = E_MAGIC;
      else if (f[10] != world) verdict = E_WORLD;
      else if (f[9] == 0 || f[9] >= world) verdict = E_RANK;
      else if (c->fds[f[9]] >= 0) verdict = E_DUP_RANK;
      else if (std::string((const char*)f + 32, std::min<size_t>(get16(f + 24), 128)) != run) verdict = E_RUN_ID;
      if (verdict != OK) {
        startup_frame(reply, Reject, 0, world, verdict, local_device, run);
        write_all(fd, reply, 160, deadline);
        ::close(fd);
        continue;  // a bad peer does not take the slot of a good one; the deadline still bounds us
      }
      c->fds[f[9]] = fd;
      c->peer_devices[f[9]] = (int64_t)get64(f + 16);
      ++admitted;
    }
    if (!err) {
      uint8_t reply[160];
      startup_frame(reply, Accepted, 0, world, 0, local_device, run);
      // the Accepted frame is followed by the device table (8 bytes per rank), so every rank knows where each peer's
      // memory lives without a further exchange
      std::vector<uint8_t> table((size_t)world * 8);
      for (int r = 0; r < world; ++r) put64(table.data() + 8 * r, (uint64_t)c->peer_devices[(size_t)r]);
      for (int r = 1; r < world && !err; ++r) {
        err = write_all(c->fds[(size_t)r], reply, 160, deadline);
        if (!err) err = write_all(c->fds[(size_t)r], table.data(), table.size(), deadline);
      }
    }
  } else {
    c->fds.assign(1, -1);
    sockaddr_in sa{};
    sa.sin_family = AF_INET;
    sa.sin_port = htons((uint16_t)port);
    if (inet_pton(AF_INET, host.c_str(), &sa.sin_addr) != 1) err = E_ARG;
    int fd = -1;
    while (!err) {  // the root may not be listening yet: retry until the deadline
      fd = ::socket(AF_INET, SOCK_STREAM, 0);
      if (::connect(fd, (sockaddr*)&sa, sizeof(sa)) == 0) break;
      ::close(fd);
      fd = -1;
      if (ms_left(deadline) <= 0) { err = E_TIMEOUT; break; }
      ::usleep(20000);
    }
    if (!err) {
      set_nonblock(fd);
      c->fds[0] = fd;
      uint8_t f[160];
      startup_frame(f, Hello, rank, world, 0, local_device, run);
      err = write_all(fd, f, 160, deadline);
      if (!err) err = read_all(fd, f, 160, deadline);
      if (!err) {
        if (std::memcmp(f, MAGIC, 8) != 0) err = E_MAGIC;
        else if (f[8] == Reject) err = get16(f + 12) ? (int)get16(f + 12) : E_REJECTED;
        else if (f[8] != Accepted) err = E_MAGIC;
        else {
          std::vector<uint8_t> table((size_t)world * 8);
          err = read_all(fd, table.data(), table.size(), deadline);
          for (int r = 0; r < world && !err; ++r) c->peer_devices[(size_t)r] = (int64_t)get64(table.data() + 8 * r);
        }
      }
    }
  }
  if (err) {
    close_all(c);
    delete c;
    return err;
  }
  std::lock_guard<std::mutex> l(g_mu);
  const int64_t h = g_next++;
  g_ctx[h] = c;
  *handle_out = h;
  return OK;
}

API int incin_rdv_state(int64_t h) {
  Ctx* c = find(h);
  return c ? c->state : Failed;
}
API int incin_rdv_failure_code(int64_t h) {
  Ctx* c = find(h);
  return c ? c->failure_code : E_ARG;
}
API void incin_rdv_invalidate(int64_t h, int code) {
  if (Ctx* c = find(h)) {
    std::lock_guard<std::mutex> l(c->mu);
    if (c->state == Active) fail(c, code);
  }
}
API int incin_rdv_ensure_active(int64_t h) {
  Ctx* c = find(h);
  return (c && c->state == Active) ? OK : E_STATE;
}

static int send_control(Ctx* c, Kind k, int code, int timeout_ms) {
  uint8_t f[16];
  control_frame(f, k, c->rank, code);
  const auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  int err = OK;
  for (int fd : c->fds)
    if (fd >= 0) {
      const int e = write_all(fd, f, 16, deadline);
      if (e && !err) err = e;
    }
  return err;
}

// Tell every reachable peer that this rank failed; the local context becomes Failed.
API int incin_rdv_abort(int64_t h, int code, int timeout_ms) {
  Ctx* c = find(h);
  if (!c) return E_ARG;
  std::lock_guard<std::mutex> l(c->mu);
  const int e = send_control(c, Abort, code, timeout_ms);
  fail(c, code);
  return e;
}

// Wait (bounded) for the next control frame from any peer.  Returns OK with kind/code/from, E_TIMEOUT when
// nothing arrived, E_IO when a peer closed its socket (treated as a failure of that peer).
API int incin_rdv_wait_for_peer(int64_t h, int timeout_ms, int* kind, int* code, int* from) {
  Ctx* c = find(h);
  if (!c) return E_ARG;
  std::lock_guard<std::mutex> l(c->mu);
  const auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  std::vector<pollfd> ps;
  for (int fd : c->fds)
    if (fd >= 0) ps.push_back({fd, POLLIN, 0});
  if (ps.empty()) return E_TIMEOUT;
  for (;;) {
    const int64_t left = ms_left(deadline);
    if (left <= 0) return E_TIMEOUT;
    const int r = ::poll(ps.data(), ps.size(), (int)std::min<int64_t>(left, 100));
    if (r <= 0) continue;
    for (auto& p : ps) {
      if (!(p.revents & (POLLIN | POLLHUP | POLLERR))) continue;
      uint8_t f[16];
      const int e = read_all(p.fd, f, 16, deadline);
      if (e == E_IO) {
        fail(c, E_IO);
        return E_IO;
      }
      if (e) return e;
      if (std::memcmp(f, MAGIC, 8) != 0) {
        fail(c, E_MAGIC);
        return E_MAGIC;
      }
      if (kind) *kind = f[8];
      if (code) *code = get16(f + 10);
      if (from) *from = f[9];
      if (f[8] == Abort) {
        // the root relays an abort to everyone else so the whole job stops
        if (c->rank == 0) {
          uint8_t g[16];
          control_frame(g, Abort, f[9], get16(f + 10));
          for (int fd : c->fds)
            if (fd >= 0 && fd != p.fd) write_all(fd, g, 16, deadline);
        }
        fail(c, E_ABORTED);
      } else if (f[8] == Shutdown && c->state == Active) {
        c->state = ShuttingDown;
      }
      return OK;
    }
  }
}

// Orderly shutdown: non-root ranks send Shutdown and wait for the root's echo; the root waits for all, then echoes.
API int incin_rdv_shutdown(int64_t h, int timeout_ms) {
  Ctx* c = find(h);
  if (!c) return E_ARG;
  std::lock_guard<std::mutex> l(c->mu);
  if (c->state == Failed) return E_STATE;
  c->state = ShuttingDown;
  const auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  int err = OK;
  uint8_t f[16];
  if (c->world > 1) {
    if (c->rank != 0) {
      err = send_control(c, Shutdown, 0, timeout_ms);
      if (!err) err = read_all(c->fds[0], f, 16, deadline);
      if (!err && (std::memcmp(f, MAGIC, 8) != 0 || f[8] != Shutdown)) err = f[8] == Abort ? E_ABORTED : E_MAGIC;
    } else {
      for (int r = 1; r < c->world && !err; ++r) {
        err = read_all(c->fds[(size_t)r], f, 16, deadline);
        if (!err && (std::memcmp(f, MAGIC, 8) != 0 || f[8] != Shutdown)) err = f[8] == Abort ? E_ABORTED : E_MAGIC;
      }
      if (!err) err = send_control(c, Shutdown, 0, timeout_ms);
    }
  }
  if (err) fail(c, err);
  else c->state = ShutdownDone;
  close_all(c);
  return err;
}

// All-gather of one fixed-size blob per rank through the root (bootstrap data: plan hashes, IPC handles).
API int incin_rdv_allgather(int64_t h, const void* mine, int bytes, void* all, int timeout_ms) {
  Ctx* c = find(h);
  if (!c || bytes <= 0) return E_ARG;
  std::lock_guard<std::mutex> l(c->mu);
  if (c->state != Active) return E_STATE;
  const auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  uint8_t* out = (uint8_t*)all;
  std::memcpy(out + (size_t)c->rank * bytes, mine, (size_t)bytes);
  int err = OK;
  if (c->world > 1) {
    if (c->rank == 0) {
      for (int r = 1; r < c->world && !err; ++r) err = read_all(c->fds[(size_t)r], out + (size_t)r * bytes, bytes, deadline);
      for (int r = 1; r < c->world && !err; ++r) err = write_all(c->fds[(size_t)r], out, (size_t)bytes * c->world, deadline);
    } else {
      err = write_all(c->fds[0], mine, (size_t)bytes, deadline);
      if (!err) err = read_all(c->fds[0], out, (size_t)bytes * c->world, deadline);
    }
  }
  if (err) fail(c, err);
  return err;
}

API int64_t incin_rdv_peer_device(int64_t h, int rank) {
  Ctx* c = find(h);
  return (c && rank >= 0 && rank < c->world) ? c->peer_devices[(size_t)rank] : -1;
}

API void incin_rdv_destroy(int64_t h) {
  Ctx* c = nullptr;
  {
    std::lock_guard<std::mutex> l(g_mu);
    auto it = g_ctx.find(h);
    if (it == g_ctx.end()) return;
    c = it->second;
    g_ctx.erase(it);
  }
  close_all(c);
  delete c;
}
