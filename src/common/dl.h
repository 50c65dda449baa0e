// A dynamically loaded library: dlopen on construction (lazily bound, local scope), dlclose on
// destruction, symbols by name. Failing to load is a state, not an exception, because "the
// library is not installed here" is how optional backends (CUDA driver, NVML, libibverbs) find
// out that they are not viable. Role of tensorpipe/common/dl.h:39-101.
#pragma once

#include <dlfcn.h>

#include <initializer_list>
#include <string>
#include <utility>

namespace tpb {

class DynamicLibraryHandle {
 public:
  DynamicLibraryHandle() = default;
  explicit DynamicLibraryHandle(const char* name, int flags = RTLD_LOCAL | RTLD_LAZY) {
    ::dlerror();
    handle_ = ::dlopen(name, flags);
    if (!handle_) {
      const char* e = ::dlerror();
      error_ = e ? e : std::string("dlopen(") + name + ") failed";
    }
  }
  DynamicLibraryHandle(DynamicLibraryHandle&& o) noexcept : handle_(o.handle_), error_(std::move(o.error_)) {
    o.handle_ = nullptr;
  }
  DynamicLibraryHandle& operator=(DynamicLibraryHandle&& o) noexcept {
    if (this != &o) {
      close();
      handle_ = o.handle_;
      error_ = std::move(o.error_);
      o.handle_ = nullptr;
    }
    return *this;
  }
  DynamicLibraryHandle(const DynamicLibraryHandle&) = delete;
  DynamicLibraryHandle& operator=(const DynamicLibraryHandle&) = delete;
  ~DynamicLibraryHandle() { close(); }

  bool loaded() const { return handle_ != nullptr; }
  const std::string& error() const { return error_; }

  // Address of the first of `names` that the library exports, or nullptr.
  void* symbol(std::initializer_list<const char*> names) const {
    if (!handle_) return nullptr;
    for (const char* n : names)
      if (void* p = ::dlsym(handle_, n)) return p;
    return nullptr;
  }
  // Fills `fn` (a function pointer) from the first exported name; false if none is.
  template <typename F>
  bool load(F& fn, std::initializer_list<const char*> names) const {
    void* p = symbol(names);
    if (!p) return false;
    fn = reinterpret_cast<F>(p);
    return true;
  }
  // Keeps the library mapped for the rest of the process (for libraries whose threads or
  // callbacks may outlive this object).
  void* release() {
    void* h = handle_;
    handle_ = nullptr;
    return h;
  }

 private:
  void close() {
    if (handle_) ::dlclose(handle_);
    handle_ = nullptr;
  }
  void* handle_ = nullptr;
  std::string error_;
};

}  // namespace tpb
