// A memory mapping that unmaps itself. Role of tensorpipe/common/memory.h:22-72: anonymous or
// fd-backed mappings for rings and shared segments.
#pragma once

#include <sys/mman.h>

#include <cerrno>
#include <cstddef>
#include <utility>

#include <tpb/error.h>

namespace tpb {

class MmappedPtr {
 public:
  MmappedPtr() = default;
  // fd < 0 with MAP_ANONYMOUS in `flags` maps fresh zeroed memory.
  static std::pair<Error, MmappedPtr> map(size_t length, int prot, int flags, int fd, off_t offset = 0) {
    MmappedPtr m;
    void* p = ::mmap(nullptr, length, prot, flags, fd, offset);
    if (p == MAP_FAILED) return {TPB_CREATE_ERROR(SystemError, "mmap", errno), std::move(m)};
    m.ptr_ = p;
    m.length_ = length;
    return {Error::kSuccess, std::move(m)};
  }
  MmappedPtr(MmappedPtr&& o) noexcept : ptr_(o.ptr_), length_(o.length_) {
    o.ptr_ = nullptr;
    o.length_ = 0;
  }
  MmappedPtr& operator=(MmappedPtr&& o) noexcept {
    if (this != &o) {
      reset();
      ptr_ = o.ptr_;
      length_ = o.length_;
      o.ptr_ = nullptr;
      o.length_ = 0;
    }
    return *this;
  }
  MmappedPtr(const MmappedPtr&) = delete;
  MmappedPtr& operator=(const MmappedPtr&) = delete;
  ~MmappedPtr() { reset(); }

  void* ptr() const { return ptr_; }
  size_t length() const { return length_; }
  explicit operator bool() const { return ptr_ != nullptr; }
  void reset() {
    if (ptr_) ::munmap(ptr_, length_);
    ptr_ = nullptr;
    length_ = 0;
  }

 private:
  void* ptr_ = nullptr;
  size_t length_ = 0;
};

}  // namespace tpb
