// Message / Descriptor / Allocation: what a pipe carries. Shape follows the reference
// (tensorpipe/core/message.h:27-102). A message is a metadata string, N small CPU payloads that
// travel on the transport connection, and N tensors that travel on channels.
//
// Extensions that the reference does not have (they never change the core wire structures; a
// channel that understands them carries them on its own control connection):
//   * Message::Tensor::view     — the source is a 2-D strided view (e.g. a transposed matrix);
//                                 `length` is the packed size rows*cols*elemSize.
//   * Allocation::Tensor::castTo — the receiver asks for the data to be converted to another
//                                 dtype while it is moved; its buffer holds rows*cols*dstElemSize.
#pragma once

#include <cstddef>
#include <cstdint>
#include <optional>
#include <string>
#include <vector>

#include <tpb/buffer.h>
#include <tpb/device.h>

namespace tpb {

enum class DType : uint8_t {
  kBytes = 0,  // opaque bytes, element size 1, no cast possible
  kF32 = 1,
  kBF16 = 2,
  kF16 = 3,
  kI64 = 4,
  kI32 = 5,
  kU8 = 6,
  kF64 = 7,
  kI16 = 8,
};

inline size_t dtypeSize(DType t) {
  switch (t) {
    case DType::kF32:
    case DType::kI32:
      return 4;
    case DType::kBF16:
    case DType::kF16:
    case DType::kI16:
      return 2;
    case DType::kI64:
    case DType::kF64:
      return 8;
    default:
      return 1;
  }
}

// 2-D strided view over the source buffer: element (r, c) lives at
// ptr + (r*rowStride + c*colStride)*dtypeSize(dtype). The packed (row-major) result is what is
// delivered. rows*cols*dtypeSize(dtype) must equal the tensor's `length`.
struct StridedView {
  DType dtype = DType::kBytes;
  int64_t rows = 0, cols = 0;
  int64_t rowStride = 0, colStride = 1;  // in elements
};

class Message final {
 public:
  std::string metadata;

  struct Payload {
    void* data = nullptr;
    size_t length = 0;
    std::string metadata;
  };
  std::vector<Payload> payloads;

  struct Tensor {
    Buffer buffer;
    size_t length = 0;
    std::optional<Device> targetDevice;  // pin the destination device, or let the receiver choose
    std::string metadata;
    DType dtype = DType::kBytes;       // extension: element type (needed for a cast)
    std::optional<StridedView> view;   // extension: non-contiguous source
  };
  std::vector<Tensor> tensors;
};

class Descriptor final {
 public:
  std::string metadata;

  struct Payload {
    size_t length = 0;
    std::string metadata;
  };
  std::vector<Payload> payloads;

  struct Tensor {
    size_t length = 0;
    Device sourceDevice;
    std::optional<Device> targetDevice;
    std::string metadata;
  };
  std::vector<Tensor> tensors;
};

class Allocation final {
 public:
  struct Payload {
    void* data = nullptr;
  };
  std::vector<Payload> payloads;

  struct Tensor {
    Buffer buffer;
    // Extension: receiver-requested dtype conversion. `sourceDtype` is the element type the
    // sender's data has (the receiver learns it from the tensor's metadata); the buffer holds
    // length / dtypeSize(sourceDtype) * dtypeSize(castTo) bytes.
    std::optional<DType> castTo;
    DType sourceDtype = DType::kBytes;
  };
  std::vector<Tensor> tensors;
};

}  // namespace tpb
