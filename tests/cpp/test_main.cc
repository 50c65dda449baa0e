// Test runner: `tpb_test [--list] [--gpu] [--filter=substr[,substr...]]`. CPU tests run by
// default; --gpu runs the GPU tests instead (skipping those that need more GPUs than present).
#include <signal.h>

#include <cuda_runtime.h>

#include "kernels/push.h"
#include "test_util.h"

namespace tpbtest {
std::vector<TestCase>& registry() {
  static std::vector<TestCase> r;
  return r;
}
int numGpus() {
  static int cached = [] {
    int fds[2];
    if (::pipe(fds) != 0) return 0;
    pid_t pid = ::fork();
    if (pid == 0) {
      int n = 0;
      if (cudaGetDeviceCount(&n) != cudaSuccess) n = 0;
      ssize_t r = ::write(fds[1], &n, sizeof(n));
      (void)r;
      ::_exit(0);
    }
    ::close(fds[1]);
    int n = 0;
    if (::read(fds[0], &n, sizeof(n)) != sizeof(n)) n = 0;
    ::close(fds[0]);
    int st;
    ::waitpid(pid, &st, 0);
    return n;
  }();
  return cached;
}
}  // namespace tpbtest

int main(int argc, char** argv) {
  ::signal(SIGPIPE, SIG_IGN);
  bool list = false, gpu = false;
  std::vector<std::string> filters;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    if (a == "--list") list = true;
    else if (a == "--gpu") gpu = true;
    else if (a.rfind("--filter=", 0) == 0) {
      std::stringstream ss(a.substr(9));
      std::string item;
      while (std::getline(ss, item, ',')) filters.push_back(item);
    }
  }
  int failed = 0, passed = 0, skipped = 0, matched = 0;
  for (auto& t : tpbtest::registry()) {
    if (t.needsGpu != gpu) continue;
    if (!filters.empty()) {
      bool match = false;
      for (auto& f : filters) match = match || t.name.find(f) != std::string::npos;
      if (!match) continue;
    }
    ++matched;
    if (list) {
      std::cout << t.name << "\n";
      continue;
    }
    if (t.needsGpu && tpbtest::numGpus() < t.minGpus) {
      std::cout << "[ SKIP ] " << t.name << " (needs " << t.minGpus << " GPUs)" << std::endl;
      ++skipped;
      continue;
    }
    std::cout << "[ RUN  ] " << t.name << std::endl;
    auto t0 = std::chrono::steady_clock::now();
    try {
      if (gpu) {
        // Each GPU test runs in a child so that this process never initialises CUDA (tests that
        // fork peer processes need a CUDA-free parent) and one test's device state cannot leak
        // into the next.
        std::cout.flush();
        pid_t pid = ::fork();
        if (pid == 0) {
          int rc = 0;
          try {
            t.fn();
            // In a build with self-checking kernels, an address outside its entry fails the test.
            if (tpb::kernels::debugKernels()) {
              const uint64_t bad = tpb::kernels::boundsViolations();
              if (bad) throw tpbtest::TestFailure(std::to_string(bad) + " out-of-range addresses computed by the kernels");
            }
          } catch (const tpbtest::TestSkipped& e) {
            std::cout << "  skipped: " << e.what() << std::endl;
            rc = 77;
          } catch (const std::exception& e) {
            std::cout << "  " << e.what() << std::endl;
            rc = 1;
          }
          std::cout.flush();
          ::_exit(rc);
        }
        int st = 0;
        ::waitpid(pid, &st, 0);
        if (WIFEXITED(st) && WEXITSTATUS(st) == 77) throw tpbtest::TestSkipped("see above");
        if (!WIFEXITED(st) || WEXITSTATUS(st) != 0)
          throw tpbtest::TestFailure("child exited with status " + std::to_string(st));
      } else {
        t.fn();
      }
      auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
      std::cout << "[  OK  ] " << t.name << " (" << ms << " ms)" << std::endl;
      ++passed;
    } catch (const tpbtest::TestSkipped& e) {
      std::cout << "[ SKIP ] " << t.name << ": " << e.what() << std::endl;
      ++skipped;
    } catch (const std::exception& e) {
      std::cout << "[ FAIL ] " << t.name << ": " << e.what() << std::endl;
      ++failed;
    }
  }
  if (!list) std::cout << passed << " passed, " << failed << " failed, " << skipped << " skipped" << std::endl;
  if (!filters.empty() && matched == 0) {
    // A filter that selects nothing is a typo in whoever runs the suites, not a pass.
    std::cout << "no " << (gpu ? "GPU" : "CPU") << " test matches the filter" << std::endl;
    return 2;
  }
  return failed ? 1 : 0;
}
