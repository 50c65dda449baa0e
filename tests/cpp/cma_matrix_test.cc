// The rules that decide whether the cma channel may be used, checked two ways: against a table of
// environments (the container and security set-ups of tensorpipe/test/channel/cma/
// docker_tests.sh:1-458, written down as facts instead of started as containers), and against
// the kernel, for the pairs of processes a test can make on its own (children that change user,
// drop capabilities, enter new namespaces, make themselves non-dumpable): wherever the rules say
// yes the system call must work, and where a child cannot read its parent the rules must say no.
#include <linux/capability.h>
#include <sched.h>
#include <sys/prctl.h>
#include <sys/syscall.h>
#include <sys/uio.h>
#include <sys/wait.h>
#include <unistd.h>

#include "channel/cma/environment.h"
#include "test_util.h"

using namespace tpb;
using namespace tpbtest;
using channel::cma::Environment;
using channel::cma::describe;
using channel::cma::predictedToWork;

namespace {
Environment host() {
  Environment e;
  e.bootId = "3b2c7a9e-boot";
  e.pidNamespace = "4_f0000001";
  e.userNamespace = "4_f0000002";
  e.effectiveUid = 1000;
  e.effectiveGid = 1000;
  e.securityModules = std::vector<std::string>{"lockdown", "capability", "yama", "apparmor"};
  e.permittedCapabilities = "0000000000000000";
  e.yamaScope = 1;
  return e;
}
}  // namespace

TPB_TEST(CmaMatrix, PredictionOverATableOfEnvironments) {
  const Environment a = host();
  struct Case {
    const char* name;
    Environment other;
    bool expected;
  };
  std::vector<Case> cases;
  auto add = [&](const char* name, bool expected, std::function<void(Environment&)> change) {
    Environment e = host();
    change(e);
    cases.push_back({name, e, expected});
  };
  add("two processes of one user on the host", true, [](Environment&) {});
  add("containers sharing the host's PID namespace (--pid=host)", true, [](Environment&) {});
  add("a container with its own PID namespace", false, [](Environment& e) { e.pidNamespace = "4_f0000099"; });
  add("a container with its own user namespace (userns-remap)", false, [](Environment& e) { e.userNamespace = "4_f0000077"; });
  add("another user", false, [](Environment& e) { e.effectiveUid = 1001; });
  add("another group", false, [](Environment& e) { e.effectiveGid = 1001; });
  add("another machine (boot id)", false, [](Environment& e) { e.bootId = "another-boot"; });
  add("the peer holds more capabilities (--cap-add SYS_PTRACE on one side only)", false,
      [](Environment& e) { e.permittedCapabilities = "0000000000080000"; });
  add("the peer made itself non-dumpable", false, [](Environment& e) { e.dumpable = false; });
  add("the peer's seccomp profile filters process_vm_readv (docker's default profile)", false,
      [](Environment& e) { e.selfProbeWorks = false; });
  add("the peer cannot declare tracers under YAMA scope 1", false, [](Environment& e) { e.canDeclareAnyTracer = false; });
  add("the peer cannot read its namespaces (no /proc)", false, [](Environment& e) { e.pidNamespace.reset(); });
  for (auto& c : cases) {
    if (predictedToWork(a, c.other) != c.expected) throw TestFailure(std::string("wrong prediction for: ") + c.name);
    if (predictedToWork(c.other, a) != c.expected) throw TestFailure(std::string("prediction is not symmetric for: ") + c.name);
  }
  // Properties of the machine both ends share.
  auto both = [&](std::function<void(Environment&)> change) {
    Environment x = host(), y = host();
    change(x);
    change(y);
    return predictedToWork(x, y);
  };
  EXPECT_TRUE(both([](Environment& e) { e.yamaScope = 0; }));
  EXPECT_TRUE(both([](Environment& e) { e.yamaScope = 1; }));
  EXPECT_FALSE(both([](Environment& e) { e.yamaScope = 2; }));  // admin-only attach
  EXPECT_FALSE(both([](Environment& e) { e.yamaScope = 3; }));  // no attach at all
  EXPECT_TRUE(both([](Environment& e) { e.securityModules = std::vector<std::string>{"capability"}; e.yamaScope.reset(); }));
  EXPECT_FALSE(both([](Environment& e) { e.yamaScope.reset(); }));  // yama listed, its scope unreadable
  EXPECT_TRUE(both([](Environment& e) { e.securityModules.reset(); }));  // the list is unreadable (securityfs not mounted)
  EXPECT_FALSE(both([](Environment& e) { e.securityModules.reset(); e.yamaScope = 2; }));  // ... YAMA still counts
  EXPECT_FALSE(both([](Environment& e) { e.permittedCapabilities.reset(); }));
  {
    // ... and so do the capabilities
    Environment x = host(), y = host();
    x.securityModules.reset();
    y.securityModules.reset();
    y.permittedCapabilities = "0000000000080000";
    EXPECT_FALSE(predictedToWork(x, y));
  }
  EXPECT_TRUE(both([](Environment& e) { e.effectiveUid = 0; e.permittedCapabilities = "000001ffffffffff"; }));  // root in a privileged container
  std::string why;
  Environment bad = host();
  bad.dumpable = false;
  EXPECT_FALSE(describe(bad, &why).has_value());
  EXPECT_FALSE(why.empty());
}

namespace {
// Runs `prepare` in a forked child; the child then reports its facts and whether it can read a
// word of the parent, and stays alive until the parent has tried to read a word of the child.
struct ChildReport {
  bool prepared = false;
  bool hasDescriptor = false;
  char descriptor[512] = {};
  bool childReadsParent = false;
  uint64_t wordAddress = 0;
};

bool readWord(pid_t pid, uint64_t address, uint64_t expect) {
  uint64_t got = 0;
  iovec l{&got, sizeof(got)};
  iovec r{reinterpret_cast<void*>(address), sizeof(got)};
  return ::process_vm_readv(pid, &l, 1, &r, 1, 0) == static_cast<ssize_t>(sizeof(got)) && got == expect;
}

struct Outcome {
  bool prepared, predicted, parentReadsChild, childReadsParent;
};

Outcome tryPair(std::function<bool()> prepare) {
  static uint64_t parentWord = 0x1122334455667788ull;
  int up[2], down[2];
  if (::pipe(up) != 0 || ::pipe(down) != 0) throw TestFailure("pipe");
  const pid_t parent = ::getpid();
  pid_t pid = ::fork();
  if (pid == 0) {
    ChildReport rep;
    static uint64_t childWord = 0x8877665544332211ull;
    rep.prepared = prepare();
    if (rep.prepared) {
      auto d = describe(channel::cma::probeEnvironment(true));
      rep.hasDescriptor = d.has_value();
      if (d) std::snprintf(rep.descriptor, sizeof(rep.descriptor), "%s", d->c_str());
      rep.childReadsParent = readWord(parent, reinterpret_cast<uint64_t>(&parentWord), parentWord);
      rep.wordAddress = reinterpret_cast<uint64_t>(&childWord);
    }
    (void)!::write(up[1], &rep, sizeof(rep));
    char go;
    (void)!::read(down[0], &go, 1);
    ::_exit(0);
  }
  ChildReport rep;
  if (::read(up[0], &rep, sizeof(rep)) != static_cast<ssize_t>(sizeof(rep))) throw TestFailure("the child did not report");
  Outcome o{};
  o.prepared = rep.prepared;
  if (rep.prepared) {
    auto mine = describe(channel::cma::probeEnvironment(true));
    o.predicted = mine && rep.hasDescriptor && *mine == rep.descriptor;
    o.parentReadsChild = readWord(pid, rep.wordAddress, 0x8877665544332211ull);
    o.childReadsParent = rep.childReadsParent;
  }
  (void)!::write(down[1], "x", 1);
  int status = 0;
  ::waitpid(pid, &status, 0);
  for (int fd : {up[0], up[1], down[0], down[1]}) ::close(fd);
  return o;
}
}  // namespace

TPB_TEST(CmaMatrix, PredictionAgainstTheKernelForThePairsThisMachineAllows) {
  auto mine = describe(channel::cma::probeEnvironment(true));
  if (!mine) {
    std::cout << "  cma is not viable here at all; nothing to compare" << std::endl;
    return;
  }
  struct Case {
    const char* name;
    std::function<bool()> prepare;
    bool expectPrediction;
  };
  const std::vector<Case> cases = {
      {"a plain child", [] { return true; }, true},
      {"a child that made itself non-dumpable", [] { return ::prctl(PR_SET_DUMPABLE, 0, 0, 0, 0) == 0; }, false},
      {"a child running as another user", [] { return ::setgid(65534) == 0 && ::setuid(65534) == 0 && ::prctl(PR_SET_DUMPABLE, 1, 0, 0, 0) == 0; }, false},
      {"a child that dropped its capabilities",
       [] {
         __user_cap_header_struct hdr{_LINUX_CAPABILITY_VERSION_3, 0};
         __user_cap_data_struct data[2] = {};
         if (::syscall(SYS_capget, &hdr, data) != 0) return false;
         if (data[0].permitted == 0 && data[1].permitted == 0) return false;  // nothing to drop: same set as the parent
         __user_cap_data_struct none[2] = {};
         return ::syscall(SYS_capset, &hdr, none) == 0;
       },
       false},
      {"a child in a new user namespace", [] { return ::unshare(CLONE_NEWUSER) == 0; }, false},
  };
  int compared = 0;
  for (auto& c : cases) {
    Outcome o = tryPair(c.prepare);
    if (!o.prepared) {
      std::cout << "  " << c.name << ": cannot be set up here, skipped" << std::endl;
      continue;
    }
    ++compared;
    std::cout << "  " << c.name << ": predicted " << (o.predicted ? "yes" : "no") << ", parent reads child "
              << (o.parentReadsChild ? "yes" : "no") << ", child reads parent " << (o.childReadsParent ? "yes" : "no") << std::endl;
    if (o.predicted != c.expectPrediction) throw TestFailure(std::string("unexpected prediction for ") + c.name);
    // A yes must hold in both directions (either end may be the reader).
    if (o.predicted && !(o.parentReadsChild && o.childReadsParent))
      throw TestFailure(std::string("predicted to work but the kernel refused: ") + c.name);
    // And whenever the kernel refuses a direction, the prediction must have been no.
    if ((!o.parentReadsChild || !o.childReadsParent) && o.predicted)
      throw TestFailure(std::string("the kernel refused what was predicted to work: ") + c.name);
  }
  EXPECT_TRUE(compared >= 1);
}
