// Completion poller: a thread that watches conditions produced by the GPU (a host-visible flag a
// kernel writes, a CUDA event) and fires a one-shot callback when one turns true, so that
// channel loops never block on the device and never need a host callback enqueued on a stream.
// It sleeps when there is nothing to watch. Plays the role of the reference's CudaLoop
// (tensorpipe/common/cuda_loop.cc:34-124), which bounces cudaStreamAddCallback through a thread.
#pragma once

#include <condition_variable>
#include <functional>
#include <list>
#include <mutex>
#include <thread>
#include <vector>

#include "common/loop.h"

namespace tpb {

class Poller {
 public:
  Poller() = default;
  ~Poller() { stop(); }

  // `ready` is polled from the poller thread until it returns true (an exception counts as
  // true); `fire` then runs once on the poller thread — it should only defer work elsewhere.
  void watch(std::function<bool()> ready, std::function<void()> fire) {
    {
      std::unique_lock<std::mutex> l(mu_);
      if (stop_) {
        l.unlock();
        fire();
        return;
      }
      items_.push_back({std::move(ready), std::move(fire)});
      if (!started_) {
        started_ = true;
        thread_ = std::thread([this]() {
          setThreadName("TP_CUDA_poller");
          run();
        });
      }
    }
    cv_.notify_one();
  }

  void stop() {
    {
      std::unique_lock<std::mutex> l(mu_);
      if (stop_) return;
      stop_ = true;
    }
    cv_.notify_all();
    if (thread_.joinable()) thread_.join();
    // Whatever was still being watched fires now so that nobody waits forever.
    std::list<Item> rest;
    {
      std::unique_lock<std::mutex> l(mu_);
      rest.swap(items_);
    }
    for (auto& it : rest) it.fire();
  }

 private:
  struct Item {
    std::function<bool()> ready;
    std::function<void()> fire;
  };
  void run() {
    std::unique_lock<std::mutex> l(mu_);
    for (;;) {
      cv_.wait(l, [&] { return stop_ || !items_.empty(); });
      if (stop_) return;
      std::vector<std::function<void()>> fired;
      for (auto it = items_.begin(); it != items_.end();) {
        bool ok;
        try {
          ok = it->ready();
        } catch (...) {
          ok = true;  // a failing query must not wedge the list; the callback re-checks state
        }
        if (ok) {
          fired.push_back(std::move(it->fire));
          it = items_.erase(it);
        } else {
          ++it;
        }
      }
      l.unlock();
      for (auto& f : fired) f();
      if (fired.empty()) std::this_thread::yield();
      l.lock();
    }
  }

  std::mutex mu_;
  std::condition_variable cv_;
  std::list<Item> items_;
  bool stop_ = false;
  bool started_ = false;
  std::thread thread_;
};

}  // namespace tpb
