// Errors are values. An Error is a cheap handle on an immutable, polymorphic description plus
// the source location that created it; a default-constructed Error means success.
// Same taxonomy as the reference (tensorpipe/common/error.h:38-125, core/error.h:17-46,
// transport/error.h:18-44, channel/error.h:18-37) so callers can test `isOfType<T>()`.
#pragma once

#include <cstring>
#include <memory>
#include <sstream>
#include <string>

namespace tpb {

class BaseError {
 public:
  virtual ~BaseError() = default;
  virtual std::string what() const = 0;
};

class Error final {
 public:
  Error() = default;
  Error(std::shared_ptr<BaseError> e, const char* file, int line)
      : error_(std::move(e)), file_(file), line_(line) {}

  static const Error kSuccess;

  explicit operator bool() const { return static_cast<bool>(error_); }

  template <typename T>
  bool isOfType() const {
    return dynamic_cast<T*>(error_.get()) != nullptr;
  }
  template <typename T>
  std::shared_ptr<T> castToType() const {
    return std::dynamic_pointer_cast<T>(error_);
  }

  std::string what() const {
    if (!error_) return "success";
    std::ostringstream ss;
    const char* base = file_ ? std::strrchr(file_, '/') : nullptr;
    ss << error_->what() << " (this error originated at " << (base ? base + 1 : (file_ ? file_ : "?"))
       << ":" << line_ << ")";
    return ss.str();
  }

 private:
  std::shared_ptr<BaseError> error_;
  const char* file_ = nullptr;
  int line_ = 0;
};

#define TPB_CREATE_ERROR(T, ...) (::tpb::Error(std::make_shared<T>(__VA_ARGS__), __FILE__, __LINE__))

// ---- common -------------------------------------------------------------------------------
class SystemError final : public BaseError {
 public:
  SystemError(const char* syscall, int err) : syscall_(syscall), errno_(err) {}
  std::string what() const override {
    return std::string(syscall_) + ": " + std::strerror(errno_);
  }
  int errorCode() const { return errno_; }

 private:
  const char* syscall_;
  int errno_;
};

class ShortReadError final : public BaseError {
 public:
  ShortReadError(ssize_t expected, ssize_t actual) : expected_(expected), actual_(actual) {}
  std::string what() const override {
    return "short read: got " + std::to_string(actual_) + " bytes while expecting to read " +
        std::to_string(expected_) + " bytes";
  }

 private:
  ssize_t expected_, actual_;
};

class ShortWriteError final : public BaseError {
 public:
  ShortWriteError(ssize_t expected, ssize_t actual) : expected_(expected), actual_(actual) {}
  std::string what() const override {
    return "short write: wrote " + std::to_string(actual_) + " bytes while expecting to write " +
        std::to_string(expected_) + " bytes";
  }

 private:
  ssize_t expected_, actual_;
};

class EOFError final : public BaseError {
 public:
  std::string what() const override { return "eof"; }
};

#define TPB_SIMPLE_ERROR(Name, text)                     \
  class Name final : public ::tpb::BaseError {           \
   public:                                               \
    std::string what() const override { return text; }   \
  }

class MessageError final : public BaseError {  // free-form text (decode failures, CUDA strings, ...)
 public:
  explicit MessageError(std::string m) : m_(std::move(m)) {}
  std::string what() const override { return m_; }

 private:
  std::string m_;
};

TPB_SIMPLE_ERROR(AllocatorClosedError, "allocator closed");
TPB_SIMPLE_ERROR(CudaLoopClosedError, "CUDA loop already closed");
TPB_SIMPLE_ERROR(TimeoutError, "timeout");

class CudaError final : public BaseError {
 public:
  explicit CudaError(std::string m) : m_(std::move(m)) {}
  std::string what() const override { return m_; }

 private:
  std::string m_;
};

// A failed RDMA work request or verbs call, with the provider's text (ibv transport, cuda_gdr).
class IbvError final : public BaseError {
 public:
  explicit IbvError(std::string m) : m_(std::move(m)) {}
  std::string what() const override { return "ibv: " + m_; }

 private:
  std::string m_;
};

class DlError final : public BaseError {
 public:
  explicit DlError(std::string m) : m_(std::move(m)) {}
  std::string what() const override { return m_; }

 private:
  std::string m_;
};

// ---- core ---------------------------------------------------------------------------------
class LogicError final : public BaseError {
 public:
  explicit LogicError(std::string reason) : reason_(std::move(reason)) {}
  std::string what() const override { return "logic error: " + reason_; }

 private:
  std::string reason_;
};
TPB_SIMPLE_ERROR(ContextClosedError, "context closed");
TPB_SIMPLE_ERROR(ListenerClosedError, "listener closed");
TPB_SIMPLE_ERROR(PipeClosedError, "pipe closed");

// ---- transport ----------------------------------------------------------------------------
namespace transport {
TPB_SIMPLE_ERROR(ContextClosedError, "context closed");
TPB_SIMPLE_ERROR(ListenerClosedError, "listener closed");
TPB_SIMPLE_ERROR(ConnectionClosedError, "connection closed");
TPB_SIMPLE_ERROR(ContextNotViableError, "context not viable");
TPB_SIMPLE_ERROR(NoAddrFoundError, "no address found");
TPB_SIMPLE_ERROR(InjectedFaultError, "injected fault");
}  // namespace transport

// ---- channel ------------------------------------------------------------------------------
namespace channel {
TPB_SIMPLE_ERROR(ContextClosedError, "context closed");
TPB_SIMPLE_ERROR(ChannelClosedError, "channel closed");
TPB_SIMPLE_ERROR(ContextNotViableError, "context not viable");
}  // namespace channel

}  // namespace tpb
