// An event loop whose thread polls instead of blocking: it runs deferred functions, calls
// pollOnce() to look for work that arrives through memory (a token queue in a shared segment, a
// completion queue), and spins while either finds something. What happens when nothing does is
// the subclass's choice through onIdle(): the default yields the core, the shm reactor goes to
// sleep on an eventfd after a while. Role of tensorpipe/common/busy_polling_loop.h:21-53.
#pragma once

#include <atomic>
#include <cstdint>
#include <thread>

#include "common/loop.h"

namespace tpb {

class BusyPollingLoop : public ThreadLoop {
 public:
  // Ask the loop to end; it does so once readyToClose() says nothing needs the thread any more.
  void close() {
    if (!closed_.exchange(true)) wakeupEventLoop();
  }
  void join() {
    close();
    joinThread();
  }

 protected:
  // Look for work once; true if something was found (and handled).
  virtual bool pollOnce() = 0;
  // True when the loop may end after close(): no registered handler still needs the thread.
  virtual bool readyToClose() = 0;
  // Called after every pass that found nothing; `idlePasses` counts such passes in a row.
  virtual void onIdle(uint64_t idlePasses) {
    if ((idlePasses & 0x3f) == 0) std::this_thread::yield();
    else pause();
  }
  // A spinning loop needs no wake-up; a subclass that sleeps in onIdle overrides this.
  void wakeupEventLoop() override {}
  bool closing() const { return closed_.load(std::memory_order_acquire); }

  static void pause() {
#if defined(__x86_64__)
    __builtin_ia32_pause();
#endif
  }

  void eventLoop() override {
    uint64_t idle = 0;
    for (;;) {
      bool worked = runDeferredFunctions() > 0;
      if (pollOnce()) worked = true;
      if (worked) {
        idle = 0;
        onWork();
        continue;
      }
      if (closing() && readyToClose() && !hasDeferred()) break;
      onIdle(++idle);
    }
  }
  // Called after every pass that found something (for subclasses that time their idleness).
  virtual void onWork() {}

 private:
  std::atomic<bool> closed_{false};
};

}  // namespace tpb
