// An event loop thread built on epoll: file-descriptor handlers and deferred closures all run
// on the one loop thread, so objects living on it need no locks. Handlers are registered under
// a fresh *record id* carried in the epoll user data, which makes an event that was already
// harvested for a closed (and possibly reused) fd harmless: its record no longer exists.
// Counterpart of tensorpipe/common/epoll_loop.h:26-138 (there the epoll thread forwards to a
// separate reactor thread; here they are the same thread).
#pragma once

#include <sys/epoll.h>
#include <sys/eventfd.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdlib>
#include <cstdint>
#include <memory>
#include <unordered_map>

#include "common/loop.h"

namespace tpb {

class EpollEventHandler {
 public:
  virtual void handleEventsFromLoop(int events) = 0;
  virtual ~EpollEventHandler() = default;
};

class EpollLoop : public ThreadLoop {
 public:
  explicit EpollLoop(const std::string& threadName) {
    epollFd_ = ::epoll_create1(EPOLL_CLOEXEC);
    TPB_THROW_SYSTEM_IF(epollFd_ < 0, errno, "epoll_create1");
    eventFd_ = ::eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
    TPB_THROW_SYSTEM_IF(eventFd_ < 0, errno, "eventfd");
    epoll_event ev{};
    ev.events = EPOLLIN;
    ev.data.u64 = 0;  // record 0 = wakeup
    TPB_THROW_SYSTEM_IF(::epoll_ctl(epollFd_, EPOLL_CTL_ADD, eventFd_, &ev) < 0, errno, "epoll_ctl");
    startThread(threadName);
  }

  ~EpollLoop() override {
    join();
    ::close(eventFd_);
    ::close(epollFd_);
  }

  // All three must be called from the loop thread.
  void registerDescriptor(int fd, int events, std::shared_ptr<EpollEventHandler> h) {
    TPB_DCHECK(inLoop());
    uint64_t rec;
    auto it = fdToRecord_.find(fd);
    epoll_event ev{};
    ev.events = events;
    if (it == fdToRecord_.end()) {
      rec = nextRecord_++;
      fdToRecord_[fd] = rec;
      ev.data.u64 = rec;
      TPB_THROW_SYSTEM_IF(::epoll_ctl(epollFd_, EPOLL_CTL_ADD, fd, &ev) < 0, errno, "epoll_ctl add");
    } else {
      rec = it->second;
      ev.data.u64 = rec;
      TPB_THROW_SYSTEM_IF(::epoll_ctl(epollFd_, EPOLL_CTL_MOD, fd, &ev) < 0, errno, "epoll_ctl mod");
    }
    handlers_[rec] = std::move(h);
  }
  void unregisterDescriptor(int fd) {
    TPB_DCHECK(inLoop());
    auto it = fdToRecord_.find(fd);
    if (it == fdToRecord_.end()) return;
    ::epoll_ctl(epollFd_, EPOLL_CTL_DEL, fd, nullptr);
    handlers_.erase(it->second);
    fdToRecord_.erase(it);
  }
  bool isRegistered(int fd) const { return fdToRecord_.count(fd) != 0; }

  void close() {
    if (!closed_.exchange(true)) wakeupEventLoop();
  }
  void join() {
    close();
    joinThread();
  }

 protected:
  void eventLoop() override {
    constexpr int kBatch = 64;
    epoll_event events[kBatch];
    bool sawEvents = false;
    auto activeUntil = std::chrono::steady_clock::now();
    for (;;) {
      // Functions often defer further functions (a callback that writes): run a few rounds of
      // them before looking at the descriptors, but not for ever, so that a chain of functions
      // cannot keep the descriptors waiting.
      bool more = false;
      for (int round = 0; round < 8; ++round) {
        more = runDeferredFunctions() > 0;
        if (!more) break;
      }
      const bool closing = closed_.load();
      // Leave once closed and nobody holds a registration any more.
      if (closing && handlers_.empty() && !hasDeferred()) break;
      // For a short while after the last sign of life the loop polls instead of blocking: a stream
      // of frames that is paced by the socket buffers would otherwise pay a thread wake-up for
      // every time the socket drains or fills.
      const auto now = std::chrono::steady_clock::now();
      if (more || sawEvents) activeUntil = now + spinWindow_;
      int timeout = (more || now < activeUntil) ? 0 : (closing ? 10 : -1);
      if (timeout != 0) {
        // About to block: from here on, whoever defers a function or closes the loop must write
        // the eventfd. Either this thread sees their change in the check below, or they see
        // `asleep_` set (both sides store first and load second, sequentially consistent).
        asleep_.store(true, std::memory_order_seq_cst);
        if (hasDeferred() || closed_.load() != closing) {
          asleep_.store(false, std::memory_order_seq_cst);
          continue;
        }
      }
      int n = ::epoll_wait(epollFd_, events, kBatch, timeout);
      if (timeout != 0) asleep_.store(false, std::memory_order_seq_cst);
      sawEvents = n > 0;
      if (n < 0) {
        if (errno == EINTR) continue;
        TPB_LOG_ERROR << "epoll_wait: " << std::strerror(errno);
        break;
      }
      for (int i = 0; i < n; ++i) {
        uint64_t rec = events[i].data.u64;
        if (rec == 0) {
          uint64_t v;
          ssize_t r = ::read(eventFd_, &v, sizeof(v));  // one read empties the counter
          (void)r;
          continue;
        }
        auto it = handlers_.find(rec);
        if (it == handlers_.end()) continue;  // stale event for a record that is gone
        std::shared_ptr<EpollEventHandler> h = it->second;
        h->handleEventsFromLoop(static_cast<int>(events[i].events));
      }
    }
  }
  // Called after a function was queued or the loop was closed. The loop only needs the eventfd
  // when it is blocked (or about to block) in epoll_wait; while it is running, what was queued is
  // found on its next pass, and a system call per deferred function is saved: most of them are
  // deferred by the loop thread itself.
  void wakeupEventLoop() override {
    if (!asleep_.load(std::memory_order_seq_cst)) return;
    uint64_t one = 1;
    ssize_t r = ::write(eventFd_, &one, sizeof(one));
    (void)r;
  }

 private:
  int epollFd_ = -1;
  int eventFd_ = -1;
  std::atomic<bool> closed_{false};
  std::atomic<bool> asleep_{false};
  // TPB_EPOLL_SPIN_US: how long the loop keeps polling after activity before it blocks.
  const std::chrono::nanoseconds spinWindow_ = [] {
    const char* s = std::getenv("TPB_EPOLL_SPIN_US");
    return std::chrono::microseconds(s ? std::strtol(s, nullptr, 10) : 50);
  }();
  uint64_t nextRecord_ = 1;
  std::unordered_map<int, uint64_t> fdToRecord_;
  std::unordered_map<uint64_t, std::shared_ptr<EpollEventHandler>> handlers_;
};

}  // namespace tpb
