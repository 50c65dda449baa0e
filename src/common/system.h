// Facts about the machine and the process that backends put in their domain / device
// descriptors to decide whether two endpoints can reach each other (same boot, same network or
// PID namespace, same user, ...). Counterpart of tensorpipe/common/system.h:29-127.
#pragma once

#include <cstdint>
#include <optional>
#include <string>
#include <vector>

namespace tpb {

// /proc/sys/kernel/random/boot_id, trimmed; nullopt if unreadable.
std::optional<std::string> getBootID();

enum class LinuxNamespace { kIpc, kNet, kPid, kUser };
// "<st_dev hex>_<st_ino hex>" of /proc/self/ns/<ns>: equal strings <=> same namespace.
std::optional<std::string> getLinuxNamespaceId(LinuxNamespace ns);

// Linux security modules listed in /sys/kernel/security/lsm.
std::optional<std::vector<std::string>> getLinuxSecurityModules();
// YAMA ptrace_scope: 0 classic, 1 restricted, 2 admin-only, 3 none; nullopt if YAMA is absent.
std::optional<int> getYamaPtraceScope();
// Hex string of the permitted capability set (raw capget).
std::optional<std::string> getPermittedCapabilitiesID();

bool isPow2(uint64_t n);
uint64_t nextPow2(uint64_t n);

}  // namespace tpb
