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

#include "channel/cma/environment.h"
#include "channel/copy_channel.h"
#include "channel/nonviable.h"
#include "common/system.h"

namespace tpb {
namespace channel {
namespace cma {

namespace {

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

Environment probeEnvironment(bool declareTracer) {
  Environment env;
  env.bootId = getBootID();
  env.pidNamespace = getLinuxNamespaceId(LinuxNamespace::kPid);
  env.userNamespace = getLinuxNamespaceId(LinuxNamespace::kUser);
  env.effectiveUid = ::geteuid();
  env.effectiveGid = ::getegid();
  env.dumpable = ::prctl(PR_GET_DUMPABLE, 0, 0, 0, 0) == 1;
  env.securityModules = getLinuxSecurityModules();
  env.permittedCapabilities = getPermittedCapabilitiesID();
  env.yamaScope = getYamaPtraceScope();
  if (declareTracer && env.yamaScope && *env.yamaScope == 1)
    env.canDeclareAnyTracer = ::prctl(PR_SET_PTRACER, PR_SET_PTRACER_ANY, 0, 0, 0) == 0;
  // Self-probe: the call may be filtered (seccomp) or missing.
  uint64_t probeSrc = 0x0123456789abcdefull, probeDst = 0;
  Error e = copyFromProcess(static_cast<uint64_t>(::getpid()), &probeSrc, &probeDst, sizeof(probeSrc));
  env.selfProbeWorks = !e && probeDst == probeSrc;
  return env;
}

std::optional<std::string> describe(const Environment& env, std::string* why) {
  auto no = [&](const char* reason) -> std::optional<std::string> {
    if (why) *why = reason;
    return std::nullopt;
  };
  if (!env.bootId || !env.pidNamespace || !env.userNamespace) return no("boot id or namespaces cannot be read");
  // A process that made itself non-dumpable cannot be read by its peers.
  if (!env.dumpable) return no("the process is not dumpable");
  // The prefix differs from the reference's ("cma:", tensorpipe/channel/cma/context_impl.cc:236-243)
  // on purpose: this channel speaks its own protocol on one connection, the reference's speaks
  // another on two, so the two must never select each other.
  std::ostringstream d;
  d << "tpbcma1:" << *env.bootId << "_" << *env.pidNamespace << "_" << *env.userNamespace << "_" << env.effectiveUid
    << "_" << env.effectiveGid;
  // Reading needs the target's permitted capabilities to be a subset of the reader's, and either
  // end may be the reader: require equality. The kernel makes this check whether or not the list
  // of security modules can be read (inside a container it often cannot), so the capabilities are
  // always part of the descriptor.
  if (!env.permittedCapabilities) return no("the permitted capabilities cannot be read");
  d << "_" << *env.permittedCapabilities;
  bool yamaListed = false;
  if (env.securityModules)
    for (const auto& lsm : *env.securityModules) yamaListed = yamaListed || lsm == "yama";
  if (yamaListed && !env.yamaScope) return no("the YAMA ptrace scope cannot be read");
  if (env.yamaScope) {
    // 1 = "restricted": only declared tracers may attach, so everyone is declared one.
    if (*env.yamaScope == 1 && !env.canDeclareAnyTracer) return no("YAMA restricts ptrace and no tracer can be declared");
    if (*env.yamaScope >= 2) return no("YAMA allows ptrace to administrators only, or to nobody");
  }
  if (!env.selfProbeWorks) return no("process_vm_readv is missing or filtered");
  return d.str();
}

std::shared_ptr<Context> create() {
  std::string why;
  auto descriptor = describe(probeEnvironment(true), &why);
  if (!descriptor) {
    TPB_VLOG(4) << "cma is not viable: " << why;
    return std::make_shared<NonViableContext>();
  }
  return std::make_shared<copy::ContextImpl>(*descriptor, &copyFromProcess, "TP_CMA_loop");
}

}  // namespace cma
}  // namespace channel
}  // namespace tpb
