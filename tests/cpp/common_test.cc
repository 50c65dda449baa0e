// Unit tests of the common runtime: byte ring (wrap-around, partial reads and writes, a forked
// producer), the backend registry, the on-demand loop, the completion
// poller, system probes. (Reference counterparts: tensorpipe/test/common/ringbuffer_test.cc,
// shm_ringbuffer_test.cc, epoll_loop_test.cc.)
#include <atomic>
#include <random>

#include "common/epoll_loop.h"
#include "common/loop.h"
#include "common/url.h"
#include "core/backends.h"
#include "common/poller.h"
#include "common/ringbuffer.h"
#include "common/shm_segment.h"
#include "common/system.h"
#include <thread>
#include "test_util.h"

using namespace tpb;
using namespace tpbtest;

TPB_TEST(Common, RingWriteReadAndWrap) {
  std::vector<uint8_t> mem(Ring::bytesNeeded(64));
  Ring ring(mem.data(), 64, true);
  EXPECT_TRUE(ring.valid(mem.size()));
  EXPECT_EQ(ring.freeBytes(), uint64_t(64));
  uint8_t in[48], out[48];
  for (int i = 0; i < 48; ++i) in[i] = static_cast<uint8_t>(i);
  EXPECT_EQ(ring.write(in, 48), uint64_t(48));
  EXPECT_EQ(ring.usedBytes(), uint64_t(48));
  EXPECT_EQ(ring.read(out, 40), uint64_t(40));
  EXPECT_TRUE(std::memcmp(in, out, 40) == 0);
  // 8 left; writing 48 more wraps around the end of the data area.
  EXPECT_EQ(ring.write(in, 48), uint64_t(48));
  EXPECT_EQ(ring.freeBytes(), uint64_t(8));
  // A write larger than the free space is partial.
  EXPECT_EQ(ring.write(in, 20), uint64_t(8));
  EXPECT_EQ(ring.write(in, 1), uint64_t(0));
  EXPECT_EQ(ring.read(out, 8), uint64_t(8));
  EXPECT_TRUE(std::memcmp(in + 40, out, 8) == 0);
  EXPECT_EQ(ring.read(out, 48), uint64_t(48));
  EXPECT_TRUE(std::memcmp(in, out, 48) == 0);
  EXPECT_EQ(ring.read(out, 48), uint64_t(8));
  EXPECT_EQ(ring.read(out, 1), uint64_t(0));
}

TPB_TEST(Common, RingBetweenProcessesThroughSharedMemory) {
  auto [e, seg] = ShmSegment::create(Ring::bytesNeeded(4096));
  EXPECT_FALSE(bool(e));
  Ring ring(seg.ptr(), 4096, true);
  constexpr size_t kTotal = 1 << 20;
  pid_t pid = ::fork();
  if (pid == 0) {
    // producer: a deterministic byte stream, written in odd-sized pieces
    std::mt19937 rng(1);
    size_t sent = 0;
    std::vector<uint8_t> buf(997);
    while (sent < kTotal) {
      size_t n = std::min(buf.size(), kTotal - sent);
      for (size_t i = 0; i < n; ++i) buf[i] = static_cast<uint8_t>((sent + i) * 31);
      size_t off = 0;
      while (off < n) off += ring.write(buf.data() + off, n - off);
      sent += n;
    }
    ::_exit(0);
  }
  size_t got = 0;
  std::vector<uint8_t> buf(1500);
  auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(30);
  while (got < kTotal) {
    uint64_t n = ring.read(buf.data(), buf.size());
    for (uint64_t i = 0; i < n; ++i) EXPECT_EQ(int(buf[i]), int(static_cast<uint8_t>((got + i) * 31)));
    got += n;
    EXPECT_TRUE(std::chrono::steady_clock::now() < deadline);
  }
  int st = 0;
  ::waitpid(pid, &st, 0);
  EXPECT_TRUE(WIFEXITED(st) && WEXITSTATUS(st) == 0);
}

TPB_TEST(Common, ShmSegmentIsSharedThroughItsFd) {
  auto [e, seg] = ShmSegment::create(1 << 16);
  EXPECT_FALSE(bool(e));
  std::memset(seg.ptr(), 0x5a, seg.size());
  auto [e2, again] = ShmSegment::load(::dup(seg.fd()));
  EXPECT_FALSE(bool(e2));
  EXPECT_EQ(again.size(), seg.size());
  EXPECT_EQ(int(static_cast<uint8_t*>(again.ptr())[12345]), 0x5a);
  static_cast<uint8_t*>(again.ptr())[7] = 9;
  EXPECT_EQ(int(static_cast<uint8_t*>(seg.ptr())[7]), 9);
}

namespace {
struct FakeBackend {
  explicit FakeBackend(bool viable) : viable(viable) {}
  bool isViable() const { return viable; }
  bool viable;
};
}  // namespace

TPB_TEST(Common, BackendsAreKeptBestFirstAndRefuseDuplicates) {
  core::Backends<FakeBackend> reg("backend");
  EXPECT_TRUE(reg.add(10, "mid", std::make_shared<FakeBackend>(true)));
  EXPECT_TRUE(reg.add(-5, "low", std::make_shared<FakeBackend>(true)));
  EXPECT_TRUE(reg.add(400, "top", std::make_shared<FakeBackend>(true)));
  // not viable: skipped without an error, and its name and priority stay free
  EXPECT_FALSE(reg.add(50, "broken", std::make_shared<FakeBackend>(false)));
  EXPECT_TRUE(reg.find("broken") == nullptr);
  EXPECT_TRUE(reg.add(50, "fine", std::make_shared<FakeBackend>(true)));
  std::vector<std::string> order;
  for (const auto& slot : reg.bestFirst()) order.push_back(slot.name);
  EXPECT_EQ(order.size(), size_t(4));
  EXPECT_EQ(order[0], std::string("top"));
  EXPECT_EQ(order[1], std::string("fine"));
  EXPECT_EQ(order[2], std::string("mid"));
  EXPECT_EQ(order[3], std::string("low"));
  EXPECT_THROWS(reg.add(7, "mid", std::make_shared<FakeBackend>(true)));    // name taken
  EXPECT_THROWS(reg.add(10, "other", std::make_shared<FakeBackend>(true))); // priority taken
  EXPECT_THROWS(reg.add(1, "", std::make_shared<FakeBackend>(true)));
  EXPECT_THROWS(reg.require("nobody"));
  EXPECT_TRUE(reg.require("low") != nullptr);
}

TPB_TEST(Common, UrlSplitsAtTheScheme) {
  auto [scheme, rest] = splitSchemeOfURL("shm://some/name");
  EXPECT_EQ(scheme, std::string("shm"));
  EXPECT_EQ(rest, std::string("some/name"));
  auto [s2, r2] = splitSchemeOfURL("uv://[::1]:80");
  EXPECT_EQ(s2, std::string("uv"));
  EXPECT_EQ(r2, std::string("[::1]:80"));
  EXPECT_THROWS(splitSchemeOfURL("no-scheme-here"));
}

TPB_TEST(Common, OnDemandLoopRunsOneTaskAtATimeAndNeverNests) {
  OnDemandLoop loop;
  std::atomic<int> inside{0}, maxInside{0}, count{0};
  std::vector<std::thread> threads;
  for (int t = 0; t < 8; ++t) {
    threads.emplace_back([&] {
      for (int i = 0; i < 200; ++i) {
        loop.deferToLoop([&] {
          int now = ++inside;
          int prev = maxInside.load();
          while (now > prev && !maxInside.compare_exchange_weak(prev, now)) {}
          // deferring from inside the loop queues instead of nesting
          if (count.load() % 50 == 0) loop.deferToLoop([&] { ++count; });
          ++count;
          --inside;
        });
      }
    });
  }
  for (auto& t : threads) t.join();
  loop.runInLoop([] {});
  EXPECT_EQ(maxInside.load(), 1);
  EXPECT_TRUE(count.load() >= 1600);
  bool in = false;
  loop.runInLoop([&] { in = loop.inLoop(); });
  EXPECT_TRUE(in);
  EXPECT_FALSE(loop.inLoop());
}

TPB_TEST(Common, EpollLoopDefersAndDeliversFdEvents) {
  struct Handler : EpollEventHandler {
    std::promise<int> got;
    int fd = -1;
    void handleEventsFromLoop(int events) override {
      char c;
      if (::read(fd, &c, 1) == 1) got.set_value(events);  // level-triggered: consume the byte
    }
  };
  EpollLoop loop("TP_test_loop");
  int fds[2];
  EXPECT_EQ(::pipe(fds), 0);
  auto h = std::make_shared<Handler>();
  h->fd = fds[0];
  loop.runInLoop([&] { loop.registerDescriptor(fds[0], EPOLLIN, h); });
  EXPECT_EQ(::write(fds[1], "x", 1), ssize_t(1));
  auto f = h->got.get_future();
  EXPECT_TRUE((waitFor(f) & EPOLLIN) != 0);
  loop.runInLoop([&] { loop.unregisterDescriptor(fds[0]); });
  std::promise<std::thread::id> where;
  loop.deferToLoop([&] { where.set_value(std::this_thread::get_id()); });
  auto fw = where.get_future();
  EXPECT_TRUE(waitFor(fw) != std::this_thread::get_id());
  loop.join();
  // After the thread is gone, deferrals still run (on the caller).
  bool ran = false;
  loop.deferToLoop([&] { ran = true; });
  EXPECT_TRUE(ran);
  ::close(fds[0]);
  ::close(fds[1]);
}

// The loop is only poked through its eventfd while it is blocked: closures deferred from other
// threads at every possible moment (while it runs, while it polls after activity, while it is
// about to block, while it sleeps) must all run, promptly, and closures that defer closures too.
TPB_TEST(Common, EpollLoopNeverLosesADeferredClosure) {
  for (const char* spin : {"0", "50"}) {
    ::setenv("TPB_EPOLL_SPIN_US", spin, 1);
    EpollLoop loop("TP_test_loop");
    ::unsetenv("TPB_EPOLL_SPIN_US");
    constexpr int kThreads = 4, kPerThread = 3000;
    std::atomic<int> ran{0};
    std::atomic<long> worstUs{0};
    std::vector<std::thread> threads;
    for (int t = 0; t < kThreads; ++t)
      threads.emplace_back([&, t] {
        std::mt19937 rng(77 + t);
        for (int i = 0; i < kPerThread; ++i) {
          // Pauses from nothing to longer than the polling window, so that the loop is caught in
          // every state.
          const int pause = static_cast<int>(rng() % 4);
          if (pause == 1) std::this_thread::yield();
          if (pause == 2) std::this_thread::sleep_for(std::chrono::microseconds(rng() % 30));
          if (pause == 3 && i % 16 == 0) std::this_thread::sleep_for(std::chrono::microseconds(100 + rng() % 200));
          const auto t0 = std::chrono::steady_clock::now();
          std::promise<void> done;
          loop.deferToLoop([&] {
            ++ran;
            loop.deferToLoop([&] {  // from the loop thread itself: no poke, must still run
              ++ran;
              done.set_value();
            });
          });
          auto f = done.get_future();
          if (f.wait_for(std::chrono::seconds(10)) != std::future_status::ready)
            throw TestFailure(std::string("a deferred closure never ran (spin window ") + spin + " us)");
          const long us = std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
          long prev = worstUs.load();
          while (us > prev && !worstUs.compare_exchange_weak(prev, us)) {
          }
        }
      });
    for (auto& th : threads) th.join();
    EXPECT_EQ(ran.load(), 2 * kThreads * kPerThread);
    // Generous: a lost poke would only be rescued by the next unrelated event, i.e. never here.
    EXPECT_TRUE(worstUs.load() < 2'000'000);
    loop.join();
  }
}

TPB_TEST(Common, PollerFiresOnceWhenTheConditionTurnsTrue) {
  Poller poller;
  std::atomic<bool> flag{false};
  std::atomic<int> fired{0};
  std::promise<void> done;
  poller.watch([&] { return flag.load(); }, [&] {
    ++fired;
    done.set_value();
  });
  std::this_thread::sleep_for(std::chrono::milliseconds(20));
  EXPECT_EQ(fired.load(), 0);
  flag = true;
  auto f = done.get_future();
  waitFor(f);
  std::this_thread::sleep_for(std::chrono::milliseconds(5));
  EXPECT_EQ(fired.load(), 1);
  // Stopping fires what is still pending, so nobody waits forever.
  std::atomic<int> late{0};
  poller.watch([] { return false; }, [&] { ++late; });
  poller.stop();
  EXPECT_EQ(late.load(), 1);
}

TPB_TEST(Common, SystemProbes) {
  auto boot = getBootID();
  EXPECT_TRUE(boot.has_value() && boot->size() >= 8);
  auto net = getLinuxNamespaceId(LinuxNamespace::kNet);
  auto pid = getLinuxNamespaceId(LinuxNamespace::kPid);
  EXPECT_TRUE(net.has_value() && pid.has_value());
  EXPECT_TRUE(net->find('_') != std::string::npos);
  EXPECT_TRUE(isPow2(64) && !isPow2(65) && !isPow2(0));
  EXPECT_EQ(nextPow2(65), uint64_t(128));
  EXPECT_EQ(nextPow2(64), uint64_t(64));
}

#include "common/allocator.h"
#include "common/queue.h"

TPB_TEST(Common, AllocatorServesInOrderAndRecyclesChunks) {
  std::vector<uint8_t> mem(4 * 100);
  Allocator alloc(mem.data(), 4, 100);
  std::vector<Allocator::TChunk> held;
  std::vector<int> order;
  int failedWaiters = 0;
  for (int i = 0; i < 6; ++i) {
    alloc.alloc(50, [&, i](const Error& e, Allocator::TChunk c) {
      if (e) {
        EXPECT_TRUE(e.isOfType<AllocatorClosedError>());
        ++failedWaiters;
        return;
      }
      order.push_back(i);
      held.push_back(std::move(c));
    });
  }
  // four chunks exist: requests 0-3 are served, 4 and 5 wait
  EXPECT_EQ(order.size(), size_t(4));
  EXPECT_EQ(alloc.numPending(), size_t(2));
  // chunks are distinct and inside the pool
  for (size_t i = 0; i < 4; ++i)
    for (size_t j = i + 1; j < 4; ++j) EXPECT_TRUE(held[i].get() != held[j].get());
  uint8_t* freed = held[1].get();
  held[1].reset();  // returning one chunk serves request 4 with that very chunk
  EXPECT_EQ(order.size(), size_t(5));
  EXPECT_EQ(order.back(), 4);
  EXPECT_TRUE(held.back().get() == freed);
  // too large a request is an error, not a wait
  bool failed = false;
  alloc.alloc(101, [&](const Error& e, Allocator::TChunk) { failed = bool(e); });
  EXPECT_TRUE(failed);
  // closing fails the remaining waiter and every later request
  Error closedError;
  alloc.close();
  EXPECT_EQ(alloc.numPending(), size_t(0));
  EXPECT_EQ(failedWaiters, 1);  // request 5 never got a chunk
  alloc.alloc(10, [&](const Error& e, Allocator::TChunk) { closedError = e; });
  EXPECT_TRUE(closedError.isOfType<AllocatorClosedError>());
  held.clear();  // chunks may outlive close()
}

TPB_TEST(Common, QueueBlocksProducersAtCapacity) {
  Queue<int> q(2);
  std::atomic<int> produced{0};
  std::thread producer([&] {
    for (int i = 0; i < 10; ++i) {
      q.push(i);
      ++produced;
    }
  });
  std::this_thread::sleep_for(std::chrono::milliseconds(20));
  EXPECT_TRUE(produced.load() <= 3);  // two queued (+ one in flight at most)
  for (int i = 0; i < 10; ++i) EXPECT_EQ(q.pop(), i);
  producer.join();
  EXPECT_EQ(produced.load(), 10);
}
