// A file descriptor that closes itself, with the interrupted-call-safe transfers every user of
// raw descriptors ends up needing. Role of tensorpipe/common/fd.h:20-113.
#pragma once

#include <unistd.h>

#include <cerrno>
#include <cstddef>
#include <utility>

#include <tpb/error.h>

namespace tpb {

class Fd {
 public:
  Fd() = default;
  explicit Fd(int fd) : fd_(fd) {}
  Fd(Fd&& o) noexcept : fd_(o.fd_) { o.fd_ = -1; }
  Fd& operator=(Fd&& o) noexcept {
    if (this != &o) {
      reset();
      fd_ = o.fd_;
      o.fd_ = -1;
    }
    return *this;
  }
  Fd(const Fd&) = delete;
  Fd& operator=(const Fd&) = delete;
  virtual ~Fd() { reset(); }

  int fd() const { return fd_; }
  bool hasValue() const { return fd_ >= 0; }
  int release() {
    int fd = fd_;
    fd_ = -1;
    return fd;
  }
  void reset(int fd = -1) {
    if (fd_ >= 0) ::close(fd_);
    fd_ = fd;
  }

  // One read / write, restarted when a signal interrupts it. Return value as the system call's.
  ssize_t read(void* buf, size_t n) const {
    for (;;) {
      ssize_t r = ::read(fd_, buf, n);
      if (r < 0 && errno == EINTR) continue;
      return r;
    }
  }
  ssize_t write(const void* buf, size_t n) const {
    for (;;) {
      ssize_t r = ::write(fd_, buf, n);
      if (r < 0 && errno == EINTR) continue;
      return r;
    }
  }
  // Exactly n bytes or an error (end of file before n bytes is a ShortReadError).
  Error readFull(void* buf, size_t n) const {
    size_t done = 0;
    while (done < n) {
      ssize_t r = read(static_cast<char*>(buf) + done, n - done);
      if (r < 0) return TPB_CREATE_ERROR(SystemError, "read", errno);
      if (r == 0) return TPB_CREATE_ERROR(ShortReadError, static_cast<ssize_t>(n), static_cast<ssize_t>(done));
      done += static_cast<size_t>(r);
    }
    return Error::kSuccess;
  }
  Error writeFull(const void* buf, size_t n) const {
    size_t done = 0;
    while (done < n) {
      ssize_t r = write(static_cast<const char*>(buf) + done, n - done);
      if (r < 0) return TPB_CREATE_ERROR(SystemError, "write", errno);
      if (r == 0) return TPB_CREATE_ERROR(ShortWriteError, static_cast<ssize_t>(n), static_cast<ssize_t>(done));
      done += static_cast<size_t>(r);
    }
    return Error::kSuccess;
  }

 protected:
  int fd_ = -1;
};

}  // namespace tpb
