// One process-wide timer thread ("TP_timer"), started on first use: schedule(delay, fn) runs fn
// on that thread once the delay has passed. Callers hand it closures that only hop to their own
// loop, so the timer thread never runs user code for long. The reference has no timers at all
// (no operation ever times out there); this backs the optional per-pipe deadlines.
#pragma once

#include <pthread.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <functional>
#include <map>
#include <mutex>
#include <thread>

#include "common/loop.h"

namespace tpb {

class TimerThread {
 public:
  using Clock = std::chrono::steady_clock;

  static TimerThread& get() {
    // Never destroyed: lives as long as the process. A forked child starts over with a fresh one
    // (the parent's thread does not exist there, and its mutex may have been held at the fork).
    static std::once_flag once;
    std::call_once(once, []() { ::pthread_atfork(nullptr, nullptr, []() { instance().store(nullptr); }); });
    TimerThread* t = instance().load(std::memory_order_acquire);
    if (t == nullptr) {
      auto* fresh = new TimerThread();
      if (instance().compare_exchange_strong(t, fresh)) return *fresh;
      delete fresh;
    }
    return *t;
  }

  void schedule(std::chrono::milliseconds delay, std::function<void()> fn) {
    std::unique_lock<std::mutex> lock(m_);
    queue_.emplace(Clock::now() + delay, std::move(fn));
    if (!started_) {
      started_ = true;
      std::thread([this]() { run(); }).detach();
    }
    cv_.notify_one();
  }

 private:
  static std::atomic<TimerThread*>& instance() {
    static std::atomic<TimerThread*> p{nullptr};
    return p;
  }

  void run() {
    setThreadName("TP_timer");
    std::unique_lock<std::mutex> lock(m_);
    for (;;) {
      if (queue_.empty()) {
        cv_.wait(lock);
        continue;
      }
      auto first = queue_.begin();
      if (first->first > Clock::now()) {
        cv_.wait_until(lock, first->first);
        continue;
      }
      auto fn = std::move(first->second);
      queue_.erase(first);
      lock.unlock();
      fn();
      lock.lock();
    }
  }

  std::mutex m_;
  std::condition_variable cv_;
  std::multimap<Clock::time_point, std::function<void()>> queue_;
  bool started_ = false;
};

}  // namespace tpb
