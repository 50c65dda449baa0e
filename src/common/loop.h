// The threading model. Every object's state is only touched "from its loop"; callers defer
// closures to it. Counterpart of tensorpipe/common/deferred_executor.h:38-278 and
// busy_polling_loop.h:21-53.
//
//  * OnDemandLoop owns no thread: the first thread that defers work while the loop is idle
//    becomes the loop until the queue drains. This is what gives one context "one callback
//    thread" — no two closures of the same loop ever run concurrently.
//  * ThreadLoop owns a thread running a subclass-provided event loop; once that thread has
//    exited, late deferrals are run by an on-demand loop so nothing leaks or hangs.
#pragma once

#include <pthread.h>

#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <future>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "common/defs.h"

namespace tpb {

inline void setThreadName(const std::string& name) {
  pthread_setname_np(pthread_self(), name.substr(0, 15).c_str());
}

class DeferredExecutor {
 public:
  using TTask = std::function<void()>;
  virtual void deferToLoop(TTask fn) = 0;
  virtual bool inLoop() const = 0;

  // Run synchronously: inline when already in the loop, else defer and wait.
  template <typename F>
  void runInLoop(F&& fn) {
    if (inLoop()) {
      fn();
      return;
    }
    std::promise<void> done;
    std::exception_ptr ex;
    deferToLoop([&]() {
      try {
        fn();
      } catch (...) {
        ex = std::current_exception();
      }
      done.set_value();
    });
    done.get_future().wait();
    if (ex) std::rethrow_exception(ex);
  }
  virtual ~DeferredExecutor() = default;
};

class OnDemandLoop final : public DeferredExecutor {
 public:
  void deferToLoop(TTask fn) override {
    {
      std::unique_lock<std::mutex> lock(mutex_);
      pending_.push_back(std::move(fn));
      if (owner_.load(std::memory_order_relaxed) != std::thread::id()) return;  // someone drains
      owner_.store(std::this_thread::get_id(), std::memory_order_relaxed);
    }
    for (;;) {
      TTask task;
      {
        std::unique_lock<std::mutex> lock(mutex_);
        if (pending_.empty()) {
          owner_.store(std::thread::id(), std::memory_order_relaxed);
          return;
        }
        task = std::move(pending_.front());
        pending_.pop_front();
      }
      task();
    }
  }
  bool inLoop() const override {
    return owner_.load(std::memory_order_relaxed) == std::this_thread::get_id();
  }

 private:
  std::mutex mutex_;
  std::deque<TTask> pending_;
  std::atomic<std::thread::id> owner_{std::thread::id()};
};

// Base for loops that own a thread. Subclasses implement eventLoop() (which must call
// runDeferredFunctions() regularly and return once `closed_ && ready to stop`) and
// wakeupEventLoop().
class ThreadLoop : public DeferredExecutor {
 public:
  void deferToLoop(TTask fn) override {
    {
      std::unique_lock<std::mutex> lock(mutex_);
      if (likelyRunning_) {
        fns_.push_back(std::move(fn));
        lock.unlock();
        wakeupEventLoop();
        return;
      }
    }
    fallback_.deferToLoop(std::move(fn));
  }
  bool inLoop() const override {
    {
      std::unique_lock<std::mutex> lock(mutex_);
      if (likelyRunning_) return std::this_thread::get_id() == thread_.get_id();
    }
    return fallback_.inLoop();
  }

 protected:
  void startThread(std::string name) {
    thread_ = std::thread([this, name = std::move(name)]() {
      setThreadName(name);
      eventLoop();
      // Hand over: whatever is still queued, and whatever arrives later, runs on demand.
      std::vector<TTask> rest;
      {
        std::unique_lock<std::mutex> lock(mutex_);
        likelyRunning_ = false;
        rest.swap(fns_);
      }
      for (auto& f : rest) fallback_.deferToLoop(std::move(f));
    });
  }
  void joinThread() {
    if (thread_.joinable()) thread_.join();
  }
  // Returns the number of functions run.
  size_t runDeferredFunctions() {
    std::vector<TTask> fns;
    {
      std::unique_lock<std::mutex> lock(mutex_);
      fns.swap(fns_);
    }
    for (auto& f : fns) f();
    return fns.size();
  }
  bool hasDeferred() const {
    std::unique_lock<std::mutex> lock(mutex_);
    return !fns_.empty();
  }
  virtual void eventLoop() = 0;
  virtual void wakeupEventLoop() = 0;

 private:
  mutable std::mutex mutex_;
  std::thread thread_;
  std::vector<TTask> fns_;
  bool likelyRunning_ = true;
  OnDemandLoop fallback_;
};

}  // namespace tpb
