// An anonymous, fd-backed shared memory segment: created with memfd_create (falling back to an
// unlinked file in /dev/shm), sized with ftruncate, mapped MAP_SHARED, and shared with another
// process by passing the fd over a UNIX socket. Counterpart of
// tensorpipe/common/shm_segment.h:28-180.
#pragma once

#include <cstring>
#include <algorithm>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <cerrno>
#include <cstddef>
#include <utility>

#include <tpb/error.h>

namespace tpb {

class ShmSegment {
 public:
  ShmSegment() = default;
  ShmSegment(ShmSegment&& o) noexcept { *this = std::move(o); }
  ShmSegment& operator=(ShmSegment&& o) noexcept {
    reset();
    fd_ = o.fd_; ptr_ = o.ptr_; size_ = o.size_;
    o.fd_ = -1; o.ptr_ = nullptr; o.size_ = 0;
    return *this;
  }
  ShmSegment(const ShmSegment&) = delete;
  ShmSegment& operator=(const ShmSegment&) = delete;
  ~ShmSegment() { reset(); }

  static std::pair<Error, ShmSegment> create(size_t bytes) {
    ShmSegment s;
    int fd = static_cast<int>(::syscall(SYS_memfd_create, "tpb_shm", 1u /* MFD_CLOEXEC */));
    if (fd < 0) {
      fd = ::open("/dev/shm", O_TMPFILE | O_EXCL | O_RDWR | O_CLOEXEC, 0600);
      if (fd < 0) return {TPB_CREATE_ERROR(SystemError, "memfd_create", errno), std::move(s)};
    }
    if (::ftruncate(fd, static_cast<off_t>(bytes)) < 0) {
      int e = errno;
      ::close(fd);
      return {TPB_CREATE_ERROR(SystemError, "ftruncate", e), std::move(s)};
    }
    auto mapped = mapFd(fd, bytes);
    // The pages are not all touched up front (a pipe over shm has four connections with a 2 MiB
    // ring each, and zeroing 8 MiB made opening it take milliseconds): only the first ones,
    // which the first few hundred control frames will use; the rest are faulted in as the ring's
    // cursors reach them, once in the life of the segment.
    if (!mapped.first) std::memset(mapped.second.ptr(), 0, std::min<size_t>(bytes, kTouchedAtCreation));
    return mapped;
  }
  static constexpr size_t kTouchedAtCreation = 64 * 1024;
  // Takes ownership of fd. The size is read from the fd.
  static std::pair<Error, ShmSegment> load(int fd) {
    off_t n = ::lseek(fd, 0, SEEK_END);
    if (n <= 0) {
      int e = errno;
      ::close(fd);
      return {TPB_CREATE_ERROR(SystemError, "lseek", e ? e : EINVAL), ShmSegment()};
    }
    return mapFd(fd, static_cast<size_t>(n));
  }

  int fd() const { return fd_; }
  void* ptr() const { return ptr_; }
  size_t size() const { return size_; }
  explicit operator bool() const { return ptr_ != nullptr; }

 private:
  static std::pair<Error, ShmSegment> mapFd(int fd, size_t bytes) {
    ShmSegment s;
    void* p = ::mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    if (p == MAP_FAILED) {
      int e = errno;
      ::close(fd);
      return {TPB_CREATE_ERROR(SystemError, "mmap", e), std::move(s)};
    }
    s.fd_ = fd;
    s.ptr_ = p;
    s.size_ = bytes;
    return {Error::kSuccess, std::move(s)};
  }
  void reset() {
    if (ptr_) ::munmap(ptr_, size_);
    if (fd_ >= 0) ::close(fd_);
    ptr_ = nullptr;
    fd_ = -1;
    size_ = 0;
  }
  int fd_ = -1;
  void* ptr_ = nullptr;
  size_t size_ = 0;
};

}  // namespace tpb
