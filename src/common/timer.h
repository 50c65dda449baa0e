// One process-wide timer thread ("TP_timer"), started on first use: schedule(delay, fn) runs fn
// on that thread once the delay has passed. Callers hand it closures that only hop to their own
// loop, so the timer thread never runs user code for long. The reference has no timers at all
// (no operation ever times out there); this backs the optional per-pipe deadlines.
#pragma once

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
    static TimerThread* t = new TimerThread();  // never destroyed: lives as long as the process
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
