// Whether cross-memory attach (process_vm_readv) will work between two processes, decided from
// facts each of them can find out about itself. The facts go into the channel's device
// descriptor; two ends use the channel only if their descriptors are equal, so the prediction is
// symmetric and needs no probing of the peer. Kept apart from the channel so that the rules can be
// checked against a table of environments (containers, users, security modules) and against what
// the kernel really does for the pairs of processes a test can make.
//
// The rules restate tensorpipe/channel/cma/context_impl.cc:131-302; the reference checks them
// under a matrix of container set-ups (tensorpipe/test/channel/cma/docker_tests.sh:1-458).
#pragma once

#include <optional>
#include <string>
#include <vector>

namespace tpb {
namespace channel {
namespace cma {

struct Environment {
  std::optional<std::string> bootId;
  std::optional<std::string> pidNamespace, userNamespace;
  unsigned effectiveUid = 0, effectiveGid = 0;
  bool dumpable = true;                               // PR_GET_DUMPABLE == 1
  std::optional<std::vector<std::string>> securityModules;  // /sys/kernel/security/lsm, where readable
  std::optional<std::string> permittedCapabilities;  // always needed
  std::optional<int> yamaScope;                       // present iff YAMA is active
  bool canDeclareAnyTracer = true;                    // prctl(PR_SET_PTRACER, PR_SET_PTRACER_ANY) works
  bool selfProbeWorks = true;                         // the system call exists and is not filtered
};

// What this process is and may do, read from /proc, /sys and prctl. `declareTracer` makes the
// YAMA scope-1 declaration for real (the channel does; a test that only wants the facts does not).
Environment probeEnvironment(bool declareTracer);

// The device descriptor for `env`, or nullopt with the reason when the channel cannot work there.
std::optional<std::string> describe(const Environment& env, std::string* why = nullptr);

// Two ends select the channel iff both have a descriptor and the two are equal.
inline bool predictedToWork(const Environment& a, const Environment& b) {
  auto da = describe(a), db = describe(b);
  return da && db && *da == *db;
}

}  // namespace cma
}  // namespace channel
}  // namespace tpb
