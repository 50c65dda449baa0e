// A very small test framework (no gtest offline) plus the "cluster on one machine" helpers the
// suites share. Modelled on how the reference tests are organised (tensorpipe/test/peer_group.h:
// two peers and a string mailbox, as threads or as forked processes) but written for this repo.
#pragma once

#include <sys/wait.h>
#include <unistd.h>

#include <chrono>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <functional>
#include <future>
#include <iostream>
#include <mutex>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

namespace tpb {
namespace kernels {
bool debugKernels();
uint64_t boundsViolations();
}  // namespace kernels
}  // namespace tpb

namespace tpbtest {

struct TestCase {
  std::string name;
  bool needsGpu;
  int minGpus;
  std::function<void()> fn;
};
std::vector<TestCase>& registry();
struct Registrar {
  Registrar(std::string name, bool gpu, int minGpus, std::function<void()> fn) {
    registry().push_back({std::move(name), gpu, minGpus, std::move(fn)});
  }
};

struct TestFailure : std::runtime_error {
  using std::runtime_error::runtime_error;
};
struct TestSkipped : std::runtime_error {
  using std::runtime_error::runtime_error;
};

#define TPB_TEST(suite, name)                                                        \
  static void tpbtest_##suite##_##name();                                           \
  static ::tpbtest::Registrar tpbtest_reg_##suite##_##name(#suite "." #name, false, 0, \
                                                          tpbtest_##suite##_##name);  \
  static void tpbtest_##suite##_##name()
#define TPB_GPU_TEST(suite, name, mingpus)                                           \
  static void tpbtest_##suite##_##name();                                           \
  static ::tpbtest::Registrar tpbtest_reg_##suite##_##name(#suite "." #name, true, mingpus, \
                                                          tpbtest_##suite##_##name);  \
  static void tpbtest_##suite##_##name()

#define EXPECT_TRUE(c)                                                                  \
  do {                                                                                  \
    if (!(c)) {                                                                         \
      std::ostringstream tpb_ss_;                                                       \
      tpb_ss_ << __FILE__ << ":" << __LINE__ << ": expected " #c;                       \
      throw ::tpbtest::TestFailure(tpb_ss_.str());                                      \
    }                                                                                   \
  } while (0)
#define EXPECT_FALSE(c) EXPECT_TRUE(!(c))
#define EXPECT_EQ(a, b)                                                                 \
  do {                                                                                  \
    auto&& tpb_a_ = (a);                                                                \
    auto&& tpb_b_ = (b);                                                                \
    if (!(tpb_a_ == tpb_b_)) {                                                          \
      std::ostringstream tpb_ss_;                                                       \
      tpb_ss_ << __FILE__ << ":" << __LINE__ << ": expected " #a " == " #b " (" << tpb_a_ \
              << " vs " << tpb_b_ << ")";                                               \
      throw ::tpbtest::TestFailure(tpb_ss_.str());                                      \
    }                                                                                   \
  } while (0)
#define EXPECT_THROWS(stmt)                                                             \
  do {                                                                                  \
    bool tpb_threw_ = false;                                                            \
    try {                                                                               \
      stmt;                                                                             \
    } catch (const ::tpbtest::TestFailure&) {                                           \
      throw;                                                                            \
    } catch (const std::exception&) {                                                   \
      tpb_threw_ = true;                                                                \
    }                                                                                   \
    if (!tpb_threw_) {                                                                  \
      std::ostringstream tpb_ss_;                                                       \
      tpb_ss_ << __FILE__ << ":" << __LINE__ << ": expected an exception from " #stmt;  \
      throw ::tpbtest::TestFailure(tpb_ss_.str());                                      \
    }                                                                                   \
  } while (0)
#define SKIP_TEST(msg) throw ::tpbtest::TestSkipped(msg)

// Wait on a future with a deadline so a broken test fails instead of hanging the suite.
template <typename T>
T waitFor(std::future<T>& f, int seconds = 30) {
  if (f.wait_for(std::chrono::seconds(seconds)) != std::future_status::ready)
    throw TestFailure("timed out waiting for a callback");
  return f.get();
}
inline void waitFor(std::future<void>& f, int seconds = 30) {
  if (f.wait_for(std::chrono::seconds(seconds)) != std::future_status::ready)
    throw TestFailure("timed out waiting for a callback");
  f.get();
}

// Blocking string mailbox.
class Mailbox {
 public:
  void send(std::string s) {
    std::unique_lock<std::mutex> l(m_);
    q_.push_back(std::move(s));
    cv_.notify_all();
  }
  std::string recv(int seconds = 30) {
    std::unique_lock<std::mutex> l(m_);
    if (!cv_.wait_for(l, std::chrono::seconds(seconds), [&] { return !q_.empty(); }))
      throw TestFailure("timed out waiting for the peer's message");
    std::string s = std::move(q_.front());
    q_.pop_front();
    return s;
  }

 private:
  std::mutex m_;
  std::condition_variable cv_;
  std::deque<std::string> q_;
};

// Two peers as threads of this process. Each side gets send/recv to talk to the other, and the
// group joins both; a failure in either side fails the test.
class ThreadPeers {
 public:
  using Fn = std::function<void(ThreadPeers&)>;
  void sendToClient(std::string s) { toClient_.send(std::move(s)); }
  void sendToServer(std::string s) { toServer_.send(std::move(s)); }
  std::string recvFromServer() { return toClient_.recv(); }
  std::string recvFromClient() { return toServer_.recv(); }

  void run(Fn server, Fn client) {
    std::exception_ptr es, ec;
    std::thread ts([&] { try { server(*this); } catch (...) { es = std::current_exception(); } });
    std::thread tc([&] { try { client(*this); } catch (...) { ec = std::current_exception(); } });
    ts.join();
    tc.join();
    if (es) std::rethrow_exception(es);
    if (ec) std::rethrow_exception(ec);
  }

 private:
  Mailbox toClient_, toServer_;
};

// Two peers as forked processes with pipe(2) mailboxes (length-prefixed strings). Needed when
// the code under test requires distinct PIDs (cross-process shared memory, CUDA IPC, cma).
class ProcessPeers {
 public:
  struct Side {
    int rfd = -1, wfd = -1;
    void send(const std::string& s) const {
      uint64_t n = s.size();
      if (::write(wfd, &n, sizeof(n)) != sizeof(n)) throw TestFailure("mailbox write");
      if (n && ::write(wfd, s.data(), n) != static_cast<ssize_t>(n)) throw TestFailure("mailbox write");
    }
    std::string recv() const {
      uint64_t n = 0;
      if (readFull(&n, sizeof(n)) != sizeof(n)) throw TestFailure("mailbox closed (peer died?)");
      std::string s(n, '\0');
      if (n && readFull(s.data(), n) != static_cast<ssize_t>(n)) throw TestFailure("mailbox closed");
      return s;
    }
    ssize_t readFull(void* p, size_t n) const {
      size_t got = 0;
      while (got < n) {
        ssize_t r = ::read(rfd, static_cast<char*>(p) + got, n - got);
        if (r < 0 && errno == EINTR) continue;
        if (r <= 0) break;
        got += static_cast<size_t>(r);
      }
      return static_cast<ssize_t>(got);
    }
  };
  using Fn = std::function<void(const Side&)>;

  // Returns the two exit codes; 0/0 means both sides passed.
  // `clientMayBeKilled`: the client is expected to end by a signal (tests that kill a peer).
  static void run(Fn server, Fn client, bool clientMayBeKilled = false) {
    int s2c[2], c2s[2];
    if (::pipe(s2c) != 0 || ::pipe(c2s) != 0) throw TestFailure("pipe");
    pid_t ps = spawn([&] { ::close(s2c[0]); ::close(c2s[1]); Side me{c2s[0], s2c[1]}; server(me); });
    pid_t pc = spawn([&] { ::close(s2c[1]); ::close(c2s[0]); Side me{s2c[0], c2s[1]}; client(me); });
    ::close(s2c[0]); ::close(s2c[1]); ::close(c2s[0]); ::close(c2s[1]);
    int ss = 0, sc = 0;
    ::waitpid(ps, &ss, 0);
    ::waitpid(pc, &sc, 0);
    bool okS = WIFEXITED(ss) && WEXITSTATUS(ss) == 0;
    bool okC = (WIFEXITED(sc) && WEXITSTATUS(sc) == 0) || (clientMayBeKilled && WIFSIGNALED(sc));
    if (!okS || !okC) {
      std::ostringstream m;
      m << "peer processes failed: server status " << ss << ", client status " << sc;
      throw TestFailure(m.str());
    }
  }

 private:
  static pid_t spawn(std::function<void()> body) {
    std::cout.flush();
    std::cerr.flush();
    pid_t pid = ::fork();
    if (pid < 0) throw TestFailure("fork");
    if (pid == 0) {
      int rc = 0;
      try {
        body();
        if (tpb::kernels::debugKernels() && tpb::kernels::boundsViolations() != 0)
          throw TestFailure("out-of-range addresses computed by the kernels in a peer process");
      } catch (const std::exception& e) {
        std::cerr << "  [child " << ::getpid() << "] " << e.what() << std::endl;
        rc = 1;
      }
      std::cout.flush();
      std::cerr.flush();
      ::_exit(rc);
    }
    return pid;
  }
};

int numGpus();  // counted in a forked child so the parent never initialises CUDA

}  // namespace tpbtest
