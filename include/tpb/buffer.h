// Type-erased handle on "memory somewhere". A Buffer stores a small trivially-copyable
// descriptor (CpuBuffer or CudaBuffer) inline, remembers which one, and can report the device
// the memory lives on. Counterpart of tensorpipe/common/buffer.h:21-133, cpu_buffer.h:15-21 and
// cuda_buffer.h:17-22; the CUDA stream is carried as an opaque handle so this header does not
// need the CUDA toolkit.
#pragma once

#include <cstddef>
#include <cstdint>
#include <stdexcept>

#include <tpb/device.h>

namespace tpb {

struct CpuBuffer {
  void* ptr = nullptr;
};

// `stream` is a cudaStream_t / CUstream. All work the library enqueues for this buffer is
// ordered after what the user already enqueued on that stream, and the user must synchronise
// with that stream before touching received data from the host.
struct CudaBuffer {
  void* ptr = nullptr;
  void* stream = nullptr;
  int deviceIndex = -1;  // optional hint; -1 = derive from the pointer through the driver
};

// Looks the device of a CUDA pointer up through the driver (implemented in the CUDA part).
int cudaDeviceForPointerOrHint(const CudaBuffer& b);

class Buffer {
 public:
  enum class Kind : uint8_t { kNone, kCpu, kCuda };

  Buffer() : cuda_() {}
  /* implicit */ Buffer(CpuBuffer b) : kind_(Kind::kCpu), cpu_(b) {}
  /* implicit */ Buffer(CudaBuffer b) : kind_(Kind::kCuda), cuda_(b) {}

  Kind kind() const { return kind_; }
  bool isCpu() const { return kind_ == Kind::kCpu; }
  bool isCuda() const { return kind_ == Kind::kCuda; }

  Device device() const {
    switch (kind_) {
      case Kind::kCpu:
        return Device(kCpuDeviceType, 0);
      case Kind::kCuda:
        return Device(kCudaDeviceType, cudaDeviceForPointerOrHint(cuda_));
      default:
        throw std::runtime_error("Buffer::device() on an empty buffer");
    }
  }

  template <typename T>
  T& unwrap();
  template <typename T>
  const T& unwrap() const {
    return const_cast<Buffer*>(this)->unwrap<T>();
  }

 private:
  Kind kind_ = Kind::kNone;
  union {
    CpuBuffer cpu_;
    CudaBuffer cuda_;
  };
};

template <>
inline CpuBuffer& Buffer::unwrap<CpuBuffer>() {
  if (kind_ != Kind::kCpu) throw std::runtime_error("Buffer does not hold a CpuBuffer");
  return cpu_;
}
template <>
inline CudaBuffer& Buffer::unwrap<CudaBuffer>() {
  if (kind_ != Kind::kCuda) throw std::runtime_error("Buffer does not hold a CudaBuffer");
  return cuda_;
}

static_assert(sizeof(Buffer) <= 40, "Buffer is meant to stay a small value type");

}  // namespace tpb
