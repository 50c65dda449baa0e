// cma: CPU tensors between two PROCESSES of one host; the receiver reads the sender's memory
// with process_vm_readv (cross-memory attach), so the bytes are copied once and never touch a
// socket. Whether that system call is allowed depends on many things, all of which go into the
// device descriptor so that two endpoints only pick this channel when it will work: same boot,
// same PID and user namespaces, same effective uid/gid, a ptrace policy that permits it (YAMA
// scope 0, or scope 1 after declaring PR_SET_PTRACER_ANY), and a successful self-probe
// (tensorpipe/channel/cma/context_impl.cc:131-302 explains the same checks).
#include <sys/prctl.h>
#include <sys/uio.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <sstream>

#include "channel/copy_channel.h"
#include "channel/nonviable.h"
#include "common/system.h"

namespace tpb {
namespace channel {
namespace cma {

namespace {

class BadReadError final : public BaseError {
 public:
  BadReadError(uint64_t expected, uint64_t actual) : expected_(expected), actual_(actual) {}
  std::string what() const override {
    return "Expected to read " + std::to_string(expected_) + ", got " + std::to_string(actual_);
  }

 private:
  uint64_t expected_, actual_;
};

Error copyFromProcess(uint64_t pid, const void* remote, void* local, size_t len) {
  // One call moves at most 0x7ffff000 bytes; loop for larger tensors and short reads.
  constexpr size_t kMaxPerCall = 0x7ffff000;
  size_t done = 0;
  while (done < len) {
    size_t n = std::min(kMaxPerCall, len - done);
    iovec l{static_cast<uint8_t*>(local) + done, n};
    iovec r{const_cast<uint8_t*>(static_cast<const uint8_t*>(remote)) + done, n};
    ssize_t got = ::process_vm_readv(static_cast<pid_t>(pid), &l, 1, &r, 1, 0);
    if (got < 0) return TPB_CREATE_ERROR(SystemError, "process_vm_readv", errno);
    if (got == 0) return TPB_CREATE_ERROR(ShortReadError, static_cast<ssize_t>(len), static_cast<ssize_t>(done));
    done += static_cast<size_t>(got);
  }
  return Error::kSuccess;
}

}  // namespace

std::shared_ptr<Context> create() {
  auto boot = getBootID();
  auto pidns = getLinuxNamespaceId(LinuxNamespace::kPid);
  auto userns = getLinuxNamespaceId(LinuxNamespace::kUser);
  if (!boot || !pidns || !userns) return std::make_shared<NonViableContext>();

  // A process that made itself non-dumpable cannot be read by its peers.
  if (::prctl(PR_GET_DUMPABLE, 0, 0, 0, 0) != 1) return std::make_shared<NonViableContext>();

  // The prefix differs from the reference's ("cma:", tensorpipe/channel/cma/context_impl.cc:236-243)
  // on purpose: this channel speaks its own protocol on one connection, the reference's speaks
  // another on two, so the two must never select each other.
  std::ostringstream d;
  d << "tpbcma1:" << *boot << "_" << *pidns << "_" << *userns << "_" << ::geteuid() << "_" << ::getegid();

  if (auto lsms = getLinuxSecurityModules()) {
    for (const auto& lsm : *lsms) {
      if (lsm == "capability") {
        // Reading needs the target's permitted capabilities to be a subset of ours: require equality.
        auto caps = getPermittedCapabilitiesID();
        if (!caps) return std::make_shared<NonViableContext>();
        d << "_" << *caps;
      } else if (lsm == "yama") {
        auto scope = getYamaPtraceScope();
        if (!scope) return std::make_shared<NonViableContext>();
        if (*scope == 1) {
          // "restricted": only declared tracers may attach. Declare everyone.
          if (::prctl(PR_SET_PTRACER, PR_SET_PTRACER_ANY, 0, 0, 0) != 0) return std::make_shared<NonViableContext>();
        } else if (*scope >= 2) {
          return std::make_shared<NonViableContext>();
        }
      }
    }
  }

  // Self-probe: the call may be filtered (seccomp) or missing.
  uint64_t probeSrc = 0x0123456789abcdefull, probeDst = 0;
  Error e = copyFromProcess(static_cast<uint64_t>(::getpid()), &probeSrc, &probeDst, sizeof(probeSrc));
  if (e || probeDst != probeSrc) {
    TPB_VLOG(4) << "cma not viable: " << (e ? e.what() : BadReadError(probeSrc, probeDst).what());
    return std::make_shared<NonViableContext>();
  }
  return std::make_shared<copy::ContextImpl>(d.str(), &copyFromProcess, "TP_CMA_loop");
}

}  // namespace cma
}  // namespace channel
}  // namespace tpb
