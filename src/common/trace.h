// Tracing: an event ring that costs one relaxed atomic load when it is off, plus NVTX ranges for
// tools that inject an NVTX backend. The reference has neither (its substitutes are verbose logs
// with hierarchical ids, tensorpipe/core/pipe_impl.cc:240,1117-1199, and the state-machine dump
// tool); this keeps those and adds a timeline.
//
//   TPB_TRACE=/path/trace.%p.json   record from start-up and write a chrome://tracing file at exit
//                                   (%p = process id)
//   tpb::trace::enable(path) / tpb::trace::dump()   the same from code (Python: trace_enable / trace_dump)
//
// Events are fixed-size slots claimed with one fetch_add; the ring keeps the most recent
// kCapacity events. Writers never block and never allocate.
#pragma once

#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>

#include <nvtx3/nvToolsExt.h>
#include <sys/syscall.h>
#include <unistd.h>

namespace tpb {
namespace trace {

struct Event {
  uint64_t ns;
  uint64_t id;
  uint32_t tid;
  char phase;  // 'B' begin, 'E' end, 'i' instant
  char name[43];
};
static_assert(sizeof(Event) == 64, "one cache line per event");

class Tracer {
 public:
  static constexpr size_t kCapacity = 1u << 16;

  static Tracer& get() {
    static Tracer* t = new Tracer();  // leaked on purpose: threads may trace during static destruction
    return *t;
  }

  bool enabled() const { return enabled_.load(std::memory_order_relaxed); }

  void enable(const std::string& path) {
    std::unique_lock<std::mutex> lock(m_);
    if (!ring_) ring_.reset(new Event[kCapacity]());
    path_ = path;
    // "%p" in the path becomes the process id, so that ranks sharing an environment do not
    // overwrite one another's file.
    const size_t at = path_.find("%p");
    if (at != std::string::npos) path_.replace(at, 2, std::to_string(::getpid()));
    enabled_.store(true, std::memory_order_release);
  }
  void disable() { enabled_.store(false, std::memory_order_release); }

  void record(char phase, const char* name, uint64_t id) {
    if (!enabled()) return;
    const uint64_t slot = next_.fetch_add(1, std::memory_order_relaxed);
    Event& e = ring_[slot % kCapacity];
    e.ns = static_cast<uint64_t>(std::chrono::duration_cast<std::chrono::nanoseconds>(
                                     std::chrono::steady_clock::now().time_since_epoch())
                                     .count());
    e.id = id;
    e.tid = threadId();
    e.phase = phase;
    std::strncpy(e.name, name, sizeof(e.name) - 1);
    e.name[sizeof(e.name) - 1] = 0;
  }

  // Number of events recorded since enable() (may exceed the capacity; older ones are gone).
  uint64_t count() const { return next_.load(std::memory_order_relaxed); }

  // Writes the ring as a chrome://tracing JSON array. Returns false if tracing never started or
  // the file cannot be written. Safe to call while other threads keep recording (events being
  // written at that instant may come out torn; they are skipped if their phase byte is not set).
  bool dump(const std::string& pathOverride = "") {
    std::unique_lock<std::mutex> lock(m_);
    if (!ring_) return false;
    const std::string path = pathOverride.empty() ? path_ : pathOverride;
    if (path.empty()) return false;
    FILE* f = std::fopen(path.c_str(), "w");
    if (!f) return false;
    const uint64_t end = next_.load(std::memory_order_acquire);
    const uint64_t begin = end > kCapacity ? end - kCapacity : 0;
    std::fputs("[\n", f);
    bool first = true;
    const int pid = static_cast<int>(::getpid());
    for (uint64_t i = begin; i < end; ++i) {
      const Event& e = ring_[i % kCapacity];
      if (e.phase != 'B' && e.phase != 'E' && e.phase != 'i') continue;
      std::fprintf(f, "%s{\"name\":\"", first ? "" : ",\n");
      for (const char* c = e.name; *c; ++c) {
        if (*c == '"' || *c == '\\') std::fputc('\\', f);
        std::fputc(*c, f);
      }
      std::fprintf(f, "\",\"ph\":\"%c\",\"ts\":%.3f,\"pid\":%d,\"tid\":%u,\"args\":{\"id\":%llu}%s}", e.phase,
                   static_cast<double>(e.ns) / 1000.0, pid, e.tid, static_cast<unsigned long long>(e.id),
                   e.phase == 'i' ? ",\"s\":\"t\"" : "");
      first = false;
    }
    std::fputs("\n]\n", f);
    std::fclose(f);
    return true;
  }

 private:
  Tracer() {
    const char* p = std::getenv("TPB_TRACE");
    if (p && *p) {
      enable(p);
      std::atexit([] { Tracer::get().dump(); });
    }
  }
  static uint32_t threadId() {
    static thread_local uint32_t tid = static_cast<uint32_t>(::syscall(SYS_gettid));
    return tid;
  }

  std::atomic<bool> enabled_{false};
  std::atomic<uint64_t> next_{0};
  std::unique_ptr<Event[]> ring_;
  std::mutex m_;
  std::string path_;
};

inline void instant(const char* name, uint64_t id = 0) { Tracer::get().record('i', name, id); }

// A begin/end pair on this thread, mirrored as an NVTX range (a no-op unless a tool injected an
// NVTX backend into the process).
class Scope {
 public:
  explicit Scope(const char* name, uint64_t id = 0) : name_(name), id_(id) {
    nvtxRangePushA(name);
    Tracer::get().record('B', name, id);
  }
  ~Scope() {
    Tracer::get().record('E', name_, id_);
    nvtxRangePop();
  }
  Scope(const Scope&) = delete;
  Scope& operator=(const Scope&) = delete;

 private:
  const char* name_;
  uint64_t id_;
};

}  // namespace trace
}  // namespace tpb
