// CUDA helpers for the host side: error checks, RAII guards and events, lazily dlopen'ed driver
// (libcuda) and NVML entry points. The runtime is linked statically, the driver library is only
// opened on demand so the CPU-only parts work on machines without a driver, and "no driver / no
// device" degrades to "this channel is not viable" instead of an exception.
// Counterparts: tensorpipe/common/cuda.h:27-321, cuda_lib.h:45-145, nvml_lib.h:32-152.
#pragma once

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <array>
#include <cstdint>
#include <cstdio>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include <tpb/error.h>

#include "common/defs.h"

namespace tpb {

#define TPB_CUDA_CHECK(expr)                                                               \
  do {                                                                                     \
    cudaError_t tpb_e_ = (expr);                                                           \
    if (tpb_e_ != cudaSuccess) {                                                           \
      ::tpb::throwLogic(__FILE__, __LINE__,                                                \
                        std::string(#expr) + ": " + cudaGetErrorName(tpb_e_) + " (" +      \
                            cudaGetErrorString(tpb_e_) + ")");                             \
    }                                                                                      \
  } while (0)

inline Error cudaErrorToError(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return Error::kSuccess;
  return TPB_CREATE_ERROR(CudaError, std::string(what) + ": " + cudaGetErrorString(e));
}

// Makes `device` current for the scope and puts back what was current before. Implemented with the
// driver's context stack (push the device's primary context, pop it again), because restoring
// with cudaSetDevice(previous) CREATES a primary context on the previous device if the thread
// never used it (since CUDA 12 cudaSetDevice initialises the device): a library thread whose
// default device is 0 would quietly open a context on GPU 0 while only moving tensors of GPU 1.
// Falls back to the runtime calls when the driver entry points are missing.
class CudaDeviceGuard {
 public:
  explicit CudaDeviceGuard(int device);
  ~CudaDeviceGuard();
  CudaDeviceGuard(const CudaDeviceGuard&) = delete;
  CudaDeviceGuard& operator=(const CudaDeviceGuard&) = delete;

 private:
  int prev_ = -1;
  bool pushed_ = false;
  bool changed_ = false;
};

class CudaEvent {
 public:
  explicit CudaEvent(int device, bool interprocess = false) : device_(device) {
    CudaDeviceGuard g(device_);
    unsigned flags = cudaEventDisableTiming | (interprocess ? cudaEventInterprocess : 0);
    TPB_CUDA_CHECK(cudaEventCreateWithFlags(&ev_, flags));
  }
  ~CudaEvent() {
    if (ev_) {
      try {
        CudaDeviceGuard g(device_);
        cudaEventDestroy(ev_);
      } catch (...) {
        cudaEventDestroy(ev_);
      }
    }
  }
  CudaEvent(const CudaEvent&) = delete;
  CudaEvent& operator=(const CudaEvent&) = delete;
  void record(cudaStream_t s) {
    CudaDeviceGuard g(device_);
    TPB_CUDA_CHECK(cudaEventRecord(ev_, s));
  }
  void wait(cudaStream_t s, int streamDevice) {
    CudaDeviceGuard g(streamDevice);
    TPB_CUDA_CHECK(cudaStreamWaitEvent(s, ev_, 0));
  }
  bool query() const {
    cudaError_t e = cudaEventQuery(ev_);
    if (e == cudaErrorNotReady) return false;
    TPB_CUDA_CHECK(e);
    return true;
  }
  cudaEvent_t raw() const { return ev_; }
  int device() const { return device_; }

 private:
  cudaEvent_t ev_ = nullptr;
  int device_;
};

// ---- driver API through dlopen --------------------------------------------------------------
using CUdeviceptr_t = unsigned long long;
struct CudaLib {
  void* handle = nullptr;
  int (*cuInit)(unsigned) = nullptr;
  int (*cuDeviceGetCount)(int*) = nullptr;
  int (*cuPointerGetAttribute)(void*, int, CUdeviceptr_t) = nullptr;
  int (*cuMemGetAddressRange)(CUdeviceptr_t*, size_t*, CUdeviceptr_t) = nullptr;
  int (*cuStreamWaitValue32)(void* stream, CUdeviceptr_t addr, uint32_t value, unsigned flags) = nullptr;
  int (*cuStreamWriteValue32)(void* stream, CUdeviceptr_t addr, uint32_t value, unsigned flags) = nullptr;
  int (*cuGetErrorString)(int, const char**) = nullptr;
  int (*cuCtxGetCurrent)(void**) = nullptr;
  int (*cuDeviceGet)(int* device, int ordinal) = nullptr;
  int (*cuDevicePrimaryCtxRetain)(void** ctx, int device) = nullptr;
  int (*cuCtxPushCurrent)(void* ctx) = nullptr;
  int (*cuCtxPopCurrent)(void** ctx) = nullptr;
  int (*cuDevicePrimaryCtxGetState)(int device, unsigned* flags, int* active) = nullptr;
  bool ok = false;
  std::string why;

  // CU_POINTER_ATTRIBUTE_*
  static constexpr int kAttrDeviceOrdinal = 9;
  static constexpr int kAttrBufferId = 7;
  static constexpr int kAttrMemoryType = 2;
  // CU_STREAM_WAIT_VALUE_GEQ = 0, _EQ = 1, _FLUSH = 1<<30
  static constexpr unsigned kWaitGeq = 0, kWaitEq = 1, kWaitFlush = 1u << 30;

  static const CudaLib& get();  // loads once; `ok` says whether a usable driver + device exist
  std::string errorString(int rc) const {
    const char* s = nullptr;
    if (cuGetErrorString && cuGetErrorString(rc, &s) == 0 && s) return s;
    return "CUDA driver error " + std::to_string(rc);
  }
};

// ---- NVML through dlopen --------------------------------------------------------------------
struct NvmlLib {
  void* handle = nullptr;
  bool ok = false;
  int (*deviceGetHandleByUUID)(const char*, void**) = nullptr;
  int (*deviceGetP2PStatus)(void*, void*, int, int*) = nullptr;
  static const NvmlLib& get();
  // NVML_P2P_CAPS_INDEX_READ = 0, WRITE = 1; NVML_P2P_STATUS_OK = 0
  bool p2pOk(const std::string& uuidA, const std::string& uuidB) const;
};

// Number of visible CUDA devices, 0 when there is no driver or no device. Never throws.
int cudaDeviceCountNoThrow();
// "GPU-xxxxxxxx-xxxx-xxxx-xxxx-xxxxxxxxxxxx" for a visible device.
std::string cudaDeviceUuid(int device);
// Device index that owns a device pointer, or -1.
int cudaDeviceForPointer(const void* ptr);
// True when `ptr` is memory of `device` itself: the only source the bulk-copy (TMA) path of the
// push kernel is given. Another GPU's memory and pinned host memory are read with plain loads.
bool cudaIsLocalMemory(const void* ptr, int device);
// True when the driver positively says that `ptr` is NOT memory of `device`: another GPU's memory
// (own, peer-mapped or IPC-mapped) or host memory. False for memory of `device` and for pointers
// the driver knows nothing about.
bool cudaIsForeignMemory(const void* ptr, int device);
// True when `ptr` is page-locked host memory that CUDA knows about.
bool cudaIsPinnedHostMemory(const void* ptr);
// Base address, size and driver buffer id of the allocation containing ptr.
bool cudaAllocationInfo(const void* ptr, void** base, size_t* size, unsigned long long* bufferId);
// Enable peer access from `device` to `peer` once (idempotent). Returns false if impossible.
bool cudaEnablePeerAccessOnce(int device, int peer);
int cudaSmCount(int device);
// Whether this process has created (and not released) the primary context of `device`. Lets
// tests prove that moving tensors of one GPU never initialises another one. -1 if unknown.
int cudaPrimaryContextActive(int device);
// Zeroes device memory and returns only once that has happened, on a private stream: it neither
// waits for nor queues behind whatever the user's streams (or the legacy default stream) hold.
// For memory whose address is about to be handed to a peer that may write to it right away.
bool cudaZeroNow(void* ptr, size_t bytes, int device);

}  // namespace tpb
