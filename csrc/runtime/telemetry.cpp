// Telemetry sink: schema-versioned JSON-lines events written by a background thread.
//
// Emitting an event from the training loop must never block on the file system, so events go into a bounded queue
// (when it is full the NEWEST event is dropped and counted: memory stays bounded and the loss of events is visible in
// the file as a "dropped" record) and one writer thread appends them to the file.  The line format is the one the
// Python emitter writes and the terminal viewer reads: {"v":1,"kind":"scalar","name":...,"value":...,"step":...,
// "ts":unix seconds}.  Counterpart of the reference's telemetry hook (crates/incin-backends/src/telemetry.rs:25-71:
// emit_scalar / emit_memory through a process-wide emitter).
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <deque>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>

#define API extern "C" __attribute__((visibility("default")))

namespace {

struct Sink {
  FILE* f = nullptr;
  size_t capacity = 4096;
  std::deque<std::string> q;
  std::mutex mu;
  std::condition_variable cv;
  bool stop = false;
  uint64_t dropped = 0, written = 0;
  size_t pending = 0;  // queued or being written: flush() waits for 0
  std::thread writer;

  void run() {
    for (;;) {
      std::deque<std::string> batch;
      {
        std::unique_lock<std::mutex> lock(mu);
        cv.wait(lock, [&] { return stop || !q.empty(); });
        batch.swap(q);
        if (batch.empty() && stop) break;
      }
      for (auto& line : batch) {
        std::fputs(line.c_str(), f);
        std::fputc('\n', f);
      }
      std::fflush(f);
      {
        std::lock_guard<std::mutex> lock(mu);
        written += batch.size();
        pending -= batch.size();
      }
      cv.notify_all();  // wakes a flush() that waits for pending == 0
    }
  }

  static double now() {   // wall clock, seconds since the Unix epoch (the viewer aligns runs by it)
    return std::chrono::duration<double>(std::chrono::system_clock::now().time_since_epoch()).count();
  }

  bool push(std::string line) {
    {
      std::lock_guard<std::mutex> lock(mu);
      if (q.size() >= capacity) {
        ++dropped;
        return false;
      }
      q.push_back(std::move(line));
      ++pending;
    }
    cv.notify_all();
    return true;
  }
};

std::mutex g_mu;
std::unordered_map<int64_t, Sink*> g_sinks;
int64_t g_next = 1;

Sink* find(int64_t h) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_sinks.find(h);
  return it == g_sinks.end() ? nullptr : it->second;
}

// JSON string escaping for names (quotes, backslashes and control characters).
std::string quoted(const char* s) {
  std::string out = "\"";
  for (const char* p = s ? s : ""; *p; ++p) {
    const unsigned char c = static_cast<unsigned char>(*p);
    if (c == '"' || c == '\\') {
      out += '\\';
      out += static_cast<char>(c);
    } else if (c < 0x20) {
      char buf[8];
      std::snprintf(buf, sizeof(buf), "\\u%04x", c);
      out += buf;
    } else {
      out += static_cast<char>(c);
    }
  }
  out += '"';
  return out;
}

std::string number(double v) {
  if (!std::isfinite(v)) return "null";  // JSON has no NaN / Infinity
  char buf[40];
  std::snprintf(buf, sizeof(buf), "%.17g", v);
  return buf;
}

}  // namespace

// Open (append) a JSON-lines sink with room for `capacity` queued events.  Returns a handle > 0, or 0 on failure.
API int64_t incin_telemetry_open(const char* path, int64_t capacity) {
  if (!path) return 0;
  FILE* f = std::fopen(path, "a");
  if (!f) return 0;
  auto* s = new Sink();
  s->f = f;
  if (capacity > 0) s->capacity = static_cast<size_t>(capacity);
  s->writer = std::thread([s] { s->run(); });
  std::lock_guard<std::mutex> lock(g_mu);
  const int64_t h = g_next++;
  g_sinks[h] = s;
  return h;
}

// 1 = queued, 0 = dropped (queue full), -1 = bad handle.
API int incin_telemetry_scalar(int64_t h, const char* name, double value, int64_t step) {
  Sink* s = find(h);
  if (!s) return -1;
  std::string line = "{\"v\":1,\"kind\":\"scalar\",\"name\":" + quoted(name) + ",\"value\":" + number(value) +
                     ",\"step\":" + std::to_string(step) + ",\"ts\":" + number(s->now()) + "}";
  return s->push(std::move(line)) ? 1 : 0;
}

// Bytes in use / reserved on a device at a step.
API int incin_telemetry_memory(int64_t h, int device, int64_t allocated, int64_t reserved, int64_t step) {
  Sink* s = find(h);
  if (!s) return -1;
  std::string line = "{\"v\":1,\"kind\":\"memory\",\"device\":" + std::to_string(device) + ",\"allocated\":" +
                     std::to_string(allocated) + ",\"reserved\":" + std::to_string(reserved) + ",\"step\":" +
                     std::to_string(step) + ",\"ts\":" + number(s->now()) + "}";
  return s->push(std::move(line)) ? 1 : 0;
}

// A pre-formatted JSON object (the caller guarantees that it is one line of valid JSON).
API int incin_telemetry_raw(int64_t h, const char* json_line) {
  Sink* s = find(h);
  if (!s || !json_line) return -1;
  return s->push(std::string(json_line)) ? 1 : 0;
}

// Wait until everything queued so far is on disk.  Returns the number of events dropped since the sink was opened.
API int64_t incin_telemetry_flush(int64_t h) {
  Sink* s = find(h);
  if (!s) return -1;
  std::unique_lock<std::mutex> lock(s->mu);
  s->cv.wait(lock, [&] { return s->pending == 0; });
  return static_cast<int64_t>(s->dropped);
}

// Flush, write a final {"kind":"dropped","count":N} record if events were lost, close the file.
API int64_t incin_telemetry_close(int64_t h) {
  Sink* s = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_sinks.find(h);
    if (it == g_sinks.end()) return -1;
    s = it->second;
    g_sinks.erase(it);
  }
  {
    std::lock_guard<std::mutex> lock(s->mu);
    s->stop = true;
  }
  s->cv.notify_all();
  if (s->writer.joinable()) s->writer.join();
  const uint64_t dropped = s->dropped;
  if (dropped) std::fprintf(s->f, "{\"v\":1,\"kind\":\"dropped\",\"count\":%llu}\n", static_cast<unsigned long long>(dropped));
  std::fclose(s->f);
  delete s;
  return static_cast<int64_t>(dropped);
}
