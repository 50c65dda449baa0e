#include "common/system.h"

#include <linux/capability.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <fstream>
#include <sstream>

namespace tpb {

std::optional<std::string> getBootID() {
  std::ifstream f("/proc/sys/kernel/random/boot_id");
  std::string s;
  if (!f.is_open() || !std::getline(f, s) || s.empty()) return std::nullopt;
  while (!s.empty() && (s.back() == '\n' || s.back() == ' ')) s.pop_back();
  return s;
}

std::optional<std::string> getLinuxNamespaceId(LinuxNamespace ns) {
  const char* name = nullptr;
  switch (ns) {
    case LinuxNamespace::kIpc: name = "ipc"; break;
    case LinuxNamespace::kNet: name = "net"; break;
    case LinuxNamespace::kPid: name = "pid"; break;
    case LinuxNamespace::kUser: name = "user"; break;
  }
  std::string path = std::string("/proc/self/ns/") + name;
  struct stat st;
  if (::stat(path.c_str(), &st) < 0) return std::nullopt;
  std::ostringstream ss;
  ss << std::hex << st.st_dev << '_' << st.st_ino;
  return ss.str();
}

std::optional<std::vector<std::string>> getLinuxSecurityModules() {
  std::ifstream f("/sys/kernel/security/lsm");
  if (!f.is_open()) return std::nullopt;
  std::string line;
  std::getline(f, line);
  std::vector<std::string> out;
  std::stringstream ss(line);
  std::string item;
  while (std::getline(ss, item, ',')) out.push_back(item);
  return out;
}

std::optional<int> getYamaPtraceScope() {
  std::ifstream f("/proc/sys/kernel/yama/ptrace_scope");
  int v;
  if (!f.is_open() || !(f >> v)) return std::nullopt;
  return v;
}

std::optional<std::string> getPermittedCapabilitiesID() {
  __user_cap_header_struct header{};
  header.version = _LINUX_CAPABILITY_VERSION_3;
  header.pid = 0;
  __user_cap_data_struct data[_LINUX_CAPABILITY_U32S_3] = {};
  if (::syscall(SYS_capget, &header, data) < 0) return std::nullopt;
  std::ostringstream ss;
  ss << std::hex;
  for (int i = _LINUX_CAPABILITY_U32S_3 - 1; i >= 0; --i) ss << data[i].permitted;
  return ss.str();
}

bool isPow2(uint64_t n) { return n != 0 && (n & (n - 1)) == 0; }
uint64_t nextPow2(uint64_t n) {
  uint64_t p = 1;
  while (p < n) p <<= 1;
  return p;
}

}  // namespace tpb
