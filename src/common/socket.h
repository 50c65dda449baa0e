// A socket that closes itself: UNIX-domain sockets in the abstract namespace (bootstrap of the shm
// transport, where file descriptors travel as SCM_RIGHTS ancillary data next to a small
// trivially-copyable value) and the few generic calls TCP users share. Role of
// tensorpipe/common/socket.h:63-255.
#pragma once

#include <fcntl.h>
#include <sys/socket.h>
#include <sys/un.h>

#include <algorithm>
#include <cstring>
#include <string>
#include <type_traits>

#include "common/fd.h"

namespace tpb {

class Socket final : public Fd {
 public:
  Socket() = default;
  explicit Socket(int fd) : Fd(fd) {}

  static std::pair<Error, Socket> createForFamily(int family, int extraFlags = 0) {
    int fd = ::socket(family, SOCK_STREAM | SOCK_CLOEXEC | extraFlags, 0);
    if (fd < 0) return {TPB_CREATE_ERROR(SystemError, "socket", errno), Socket()};
    return {Error::kSuccess, Socket(fd)};
  }

  Error setNonBlocking(bool on = true) {
    int flags = ::fcntl(fd_, F_GETFL, 0);
    if (flags < 0) return TPB_CREATE_ERROR(SystemError, "fcntl", errno);
    flags = on ? (flags | O_NONBLOCK) : (flags & ~O_NONBLOCK);
    if (::fcntl(fd_, F_SETFL, flags) < 0) return TPB_CREATE_ERROR(SystemError, "fcntl", errno);
    return Error::kSuccess;
  }

  // ---- abstract-namespace UNIX addresses (a leading NUL byte, no file on disk) ----
  static sockaddr_un abstractAddress(const std::string& name, socklen_t* len) {
    sockaddr_un sa{};
    sa.sun_family = AF_UNIX;
    const size_t n = std::min(name.size(), sizeof(sa.sun_path) - 1);
    std::memcpy(sa.sun_path + 1, name.data(), n);
    *len = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
    return sa;
  }
  // An empty name lets the kernel pick a unique one ("autobind").
  Error bindAbstract(const std::string& name) {
    if (name.empty()) {
      sockaddr_un sa{};
      sa.sun_family = AF_UNIX;
      if (::bind(fd_, reinterpret_cast<sockaddr*>(&sa), sizeof(sa_family_t)) < 0) return TPB_CREATE_ERROR(SystemError, "bind", errno);
      return Error::kSuccess;
    }
    socklen_t len;
    sockaddr_un sa = abstractAddress(name, &len);
    if (::bind(fd_, reinterpret_cast<sockaddr*>(&sa), len) < 0) return TPB_CREATE_ERROR(SystemError, "bind", errno);
    return Error::kSuccess;
  }
  Error connectAbstract(const std::string& name) {
    socklen_t len;
    sockaddr_un sa = abstractAddress(name, &len);
    for (;;) {
      if (::connect(fd_, reinterpret_cast<sockaddr*>(&sa), len) == 0) return Error::kSuccess;
      if (errno == EINTR) continue;
      return TPB_CREATE_ERROR(SystemError, "connect", errno);
    }
  }
  // The abstract name this socket is bound to (without the leading NUL).
  std::string boundAbstractName() const {
    sockaddr_un bound{};
    socklen_t len = sizeof(bound);
    if (::getsockname(fd_, reinterpret_cast<sockaddr*>(&bound), &len) < 0) return std::string();
    const size_t n = len - offsetof(sockaddr_un, sun_path);
    return n > 1 ? std::string(bound.sun_path + 1, n - 1) : std::string();
  }
  Error listen(int backlog) {
    if (::listen(fd_, backlog) < 0) return TPB_CREATE_ERROR(SystemError, "listen", errno);
    return Error::kSuccess;
  }
  // A connection waiting in the backlog; an empty socket and no error when there is none (the
  // listening socket is non-blocking).
  std::pair<Error, Socket> accept() {
    for (;;) {
      int fd = ::accept4(fd_, nullptr, nullptr, SOCK_CLOEXEC);
      if (fd >= 0) return {Error::kSuccess, Socket(fd)};
      if (errno == EINTR || errno == ECONNABORTED) continue;
      if (errno == EAGAIN || errno == EWOULDBLOCK) return {Error::kSuccess, Socket()};
      return {TPB_CREATE_ERROR(SystemError, "accept", errno), Socket()};
    }
  }

  // ---- a value plus file descriptors in one message ----
  template <typename T, size_t N>
  Error sendWithFds(const T& value, const int (&fds)[N]) {
    static_assert(std::is_trivially_copyable<T>::value, "the value travels as raw bytes");
    msghdr msg{};
    iovec iov{const_cast<T*>(&value), sizeof(T)};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int) * N)] = {};
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int) * N);
    std::memcpy(CMSG_DATA(c), fds, sizeof(int) * N);
    for (;;) {
      ssize_t n = ::sendmsg(fd_, &msg, MSG_NOSIGNAL);
      if (n < 0 && errno == EINTR) continue;
      if (n < 0) return TPB_CREATE_ERROR(SystemError, "sendmsg", errno);
      if (n != static_cast<ssize_t>(sizeof(T))) return TPB_CREATE_ERROR(ShortWriteError, sizeof(T), n);
      return Error::kSuccess;
    }
  }
  // `got` stays false (and no error is reported) when nothing has arrived yet on a non-blocking
  // socket. The received descriptors are owned by the caller.
  template <typename T, size_t N>
  Error recvWithFds(T& value, int (&fds)[N], bool& got) {
    static_assert(std::is_trivially_copyable<T>::value, "the value travels as raw bytes");
    got = false;
    msghdr msg{};
    iovec iov{&value, sizeof(T)};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int) * N)] = {};
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    ssize_t n = ::recvmsg(fd_, &msg, MSG_CMSG_CLOEXEC);
    if (n < 0) {
      if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) return Error::kSuccess;
      return TPB_CREATE_ERROR(SystemError, "recvmsg", errno);
    }
    if (n == 0) return TPB_CREATE_ERROR(EOFError);
    if (n != static_cast<ssize_t>(sizeof(T))) return TPB_CREATE_ERROR(ShortReadError, sizeof(T), n);
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    if (!c || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS || c->cmsg_len != CMSG_LEN(sizeof(int) * N))
      return TPB_CREATE_ERROR(ShortReadError, static_cast<ssize_t>(N), 0);
    std::memcpy(fds, CMSG_DATA(c), sizeof(int) * N);
    got = true;
    return Error::kSuccess;
  }
};

}  // namespace tpb
