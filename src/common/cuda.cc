#include "common/cuda.h"

#include <map>
#include <set>

#include <tpb/buffer.h>

#include "common/dl.h"

namespace tpb {

const CudaLib& CudaLib::get() {
  static CudaLib lib = [] {
    CudaLib l;
    DynamicLibraryHandle dl("libcuda.so.1");
    if (!dl.loaded()) {
      l.why = dl.error();
      TPB_VLOG(9) << "CUDA driver not loaded: " << l.why;
      return l;
    }
    bool all = dl.load(l.cuInit, {"cuInit"}) && dl.load(l.cuDeviceGetCount, {"cuDeviceGetCount"}) &&
        dl.load(l.cuPointerGetAttribute, {"cuPointerGetAttribute"}) &&
        dl.load(l.cuMemGetAddressRange, {"cuMemGetAddressRange_v2"}) &&
        dl.load(l.cuGetErrorString, {"cuGetErrorString"}) && dl.load(l.cuCtxGetCurrent, {"cuCtxGetCurrent"});
    dl.load(l.cuDeviceGet, {"cuDeviceGet"});
    dl.load(l.cuDevicePrimaryCtxRetain, {"cuDevicePrimaryCtxRetain"});
    dl.load(l.cuCtxPushCurrent, {"cuCtxPushCurrent_v2", "cuCtxPushCurrent"});
    dl.load(l.cuCtxPopCurrent, {"cuCtxPopCurrent_v2", "cuCtxPopCurrent"});
    dl.load(l.cuDevicePrimaryCtxGetState, {"cuDevicePrimaryCtxGetState"});
    // Stream memory operations are optional (the wait kernel is the fallback).
    dl.load(l.cuStreamWaitValue32, {"cuStreamWaitValue32_v2", "cuStreamWaitValue32"});
    dl.load(l.cuStreamWriteValue32, {"cuStreamWriteValue32_v2", "cuStreamWriteValue32"});
    // The driver stays mapped for the life of the process: the entry points above are kept.
    l.handle = dl.release();
    if (!all) {
      l.why = "libcuda.so.1 lacks required symbols";
      return l;
    }
    int rc = l.cuInit(0);
    if (rc != 0) {
      l.why = "cuInit: " + l.errorString(rc);
      return l;
    }
    int n = 0;
    if (l.cuDeviceGetCount(&n) != 0 || n == 0) {
      l.why = "no CUDA devices";
      return l;
    }
    l.ok = true;
    return l;
  }();
  return lib;
}

const NvmlLib& NvmlLib::get() {
  static NvmlLib lib = [] {
    NvmlLib l;
    DynamicLibraryHandle dl("libnvidia-ml.so.1");
    if (!dl.loaded()) return l;
    int (*init)() = nullptr;
    const bool all = dl.load(init, {"nvmlInit_v2"}) && dl.load(l.deviceGetHandleByUUID, {"nvmlDeviceGetHandleByUUID"}) &&
        dl.load(l.deviceGetP2PStatus, {"nvmlDeviceGetP2PStatus"});
    l.handle = dl.release();
    if (!all) return l;
    if (init() != 0) return l;
    l.ok = true;
    return l;
  }();
  return lib;
}

bool NvmlLib::p2pOk(const std::string& uuidA, const std::string& uuidB) const {
  if (!ok) return false;
  void *a = nullptr, *b = nullptr;
  if (deviceGetHandleByUUID(uuidA.c_str(), &a) != 0) return false;
  if (deviceGetHandleByUUID(uuidB.c_str(), &b) != 0) return false;
  int rd = -1, wr = -1;
  if (deviceGetP2PStatus(a, b, 0, &rd) != 0 || deviceGetP2PStatus(a, b, 1, &wr) != 0) return false;
  return rd == 0 && wr == 0;
}

namespace {
// The primary context of each device, retained once and kept for the life of the process.
void* primaryContext(int device) {
  static std::mutex m;
  static std::map<int, void*> cache;
  std::unique_lock<std::mutex> lock(m);
  auto it = cache.find(device);
  if (it != cache.end()) return it->second;
  const CudaLib& lib = CudaLib::get();
  void* ctx = nullptr;
  int dev = 0;
  if (!lib.ok || !lib.cuDeviceGet || !lib.cuDevicePrimaryCtxRetain || lib.cuDeviceGet(&dev, device) != 0 ||
      lib.cuDevicePrimaryCtxRetain(&ctx, dev) != 0)
    ctx = nullptr;
  cache[device] = ctx;
  return ctx;
}
}  // namespace

CudaDeviceGuard::CudaDeviceGuard(int device) {
  if (device < 0) return;
  const CudaLib& lib = CudaLib::get();
  if (lib.ok && lib.cuCtxPushCurrent && lib.cuCtxPopCurrent) {
    if (void* ctx = primaryContext(device)) {
      void* current = nullptr;
      lib.cuCtxGetCurrent(&current);
      if (current == ctx) return;
      if (lib.cuCtxPushCurrent(ctx) == 0) {
        pushed_ = true;
        return;
      }
    }
  }
  TPB_CUDA_CHECK(cudaGetDevice(&prev_));
  if (device != prev_) {
    TPB_CUDA_CHECK(cudaSetDevice(device));
    changed_ = true;
  }
}

CudaDeviceGuard::~CudaDeviceGuard() {
  if (pushed_) {
    void* popped = nullptr;
    CudaLib::get().cuCtxPopCurrent(&popped);
  } else if (changed_) {
    cudaSetDevice(prev_);
  }
}

int cudaDeviceCountNoThrow() {
  if (!CudaLib::get().ok) return 0;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

std::string cudaDeviceUuid(int device) {
  cudaDeviceProp prop;
  TPB_CUDA_CHECK(cudaGetDeviceProperties(&prop, device));
  const unsigned char* b = reinterpret_cast<const unsigned char*>(prop.uuid.bytes);
  char buf[64];
  std::snprintf(buf, sizeof(buf),
                "GPU-%02x%02x%02x%02x-%02x%02x-%02x%02x-%02x%02x-%02x%02x%02x%02x%02x%02x", b[0],
                b[1], b[2], b[3], b[4], b[5], b[6], b[7], b[8], b[9], b[10], b[11], b[12], b[13],
                b[14], b[15]);
  return buf;
}

int cudaDeviceForPointer(const void* ptr) {
  const CudaLib& lib = CudaLib::get();
  if (!lib.ok || ptr == nullptr) return -1;
  int ordinal = -1;
  int rc = lib.cuPointerGetAttribute(&ordinal, CudaLib::kAttrDeviceOrdinal,
                                     reinterpret_cast<CUdeviceptr_t>(ptr));
  if (rc != 0) return -1;
  return ordinal;
}

bool cudaIsLocalMemory(const void* ptr, int device) {
  const CudaLib& lib = CudaLib::get();
  if (!lib.ok) return false;
  unsigned type = 0;
  int ordinal = -1;
  const CUdeviceptr_t p = reinterpret_cast<CUdeviceptr_t>(ptr);
  if (lib.cuPointerGetAttribute(&type, CudaLib::kAttrMemoryType, p) != 0) return false;
  if (type != 2 /* CU_MEMORYTYPE_DEVICE */) return false;
  if (lib.cuPointerGetAttribute(&ordinal, CudaLib::kAttrDeviceOrdinal, p) != 0) return false;
  return ordinal == device;
}

bool cudaIsForeignMemory(const void* ptr, int device) {
  const CudaLib& lib = CudaLib::get();
  if (!lib.ok || ptr == nullptr) return false;
  unsigned type = 0;
  int ordinal = -1;
  const CUdeviceptr_t p = reinterpret_cast<CUdeviceptr_t>(ptr);
  if (lib.cuPointerGetAttribute(&type, CudaLib::kAttrMemoryType, p) != 0) return false;
  if (type == 1 /* CU_MEMORYTYPE_HOST */) return true;
  if (type != 2 /* CU_MEMORYTYPE_DEVICE */) return false;
  if (lib.cuPointerGetAttribute(&ordinal, CudaLib::kAttrDeviceOrdinal, p) != 0) return false;
  return ordinal != device;
}

bool cudaIsPinnedHostMemory(const void* ptr) {
  const CudaLib& lib = CudaLib::get();
  if (!lib.ok || ptr == nullptr) return false;
  unsigned type = 0;
  if (lib.cuPointerGetAttribute(&type, CudaLib::kAttrMemoryType, reinterpret_cast<CUdeviceptr_t>(ptr)) != 0) return false;
  return type == 1 /* CU_MEMORYTYPE_HOST */;
}

bool cudaAllocationInfo(const void* ptr, void** base, size_t* size, unsigned long long* bufferId) {
  const CudaLib& lib = CudaLib::get();
  if (!lib.ok) return false;
  CUdeviceptr_t b = 0;
  size_t s = 0;
  if (lib.cuMemGetAddressRange(&b, &s, reinterpret_cast<CUdeviceptr_t>(ptr)) != 0) return false;
  unsigned long long id = 0;
  if (lib.cuPointerGetAttribute(&id, CudaLib::kAttrBufferId, reinterpret_cast<CUdeviceptr_t>(ptr)) != 0)
    return false;
  *base = reinterpret_cast<void*>(b);
  *size = s;
  *bufferId = id;
  return true;
}

bool cudaEnablePeerAccessOnce(int device, int peer) {
  if (device == peer) return true;
  static std::mutex m;
  static std::map<std::pair<int, int>, bool> done;
  std::unique_lock<std::mutex> lock(m);
  auto it = done.find({device, peer});
  if (it != done.end()) return it->second;
  bool ok = false;
  int can = 0;
  if (cudaDeviceCanAccessPeer(&can, device, peer) == cudaSuccess && can) {
    CudaDeviceGuard g(device);
    cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
    if (e == cudaSuccess || e == cudaErrorPeerAccessAlreadyEnabled) ok = true;
    cudaGetLastError();
  }
  done[{device, peer}] = ok;
  return ok;
}

int cudaSmCount(int device) {
  static std::mutex m;
  static std::map<int, int> cache;
  std::unique_lock<std::mutex> lock(m);
  auto it = cache.find(device);
  if (it != cache.end()) return it->second;
  int n = 0;
  TPB_CUDA_CHECK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device));
  cache[device] = n;
  return n;
}

int cudaPrimaryContextActive(int device) {
  const CudaLib& lib = CudaLib::get();
  if (!lib.ok || !lib.cuDeviceGet || !lib.cuDevicePrimaryCtxGetState) return -1;
  int dev = 0;
  if (lib.cuDeviceGet(&dev, device) != 0) return -1;
  unsigned flags = 0;
  int active = 0;
  if (lib.cuDevicePrimaryCtxGetState(dev, &flags, &active) != 0) return -1;
  return active;
}

bool cudaZeroNow(void* ptr, size_t bytes, int device) {
  CudaDeviceGuard g(device);
  cudaStream_t s = nullptr;
  if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  bool ok = cudaMemsetAsync(ptr, 0, bytes, s) == cudaSuccess && cudaStreamSynchronize(s) == cudaSuccess;
  cudaStreamDestroy(s);
  if (!ok) cudaGetLastError();
  return ok;
}

int cudaDeviceForPointerOrHint(const CudaBuffer& b) {
  if (b.deviceIndex >= 0) return b.deviceIndex;
  int d = cudaDeviceForPointer(b.ptr);
  if (d < 0) {
    // A null pointer (legal for an empty tensor) belongs to the current device.
    if (cudaGetDevice(&d) != cudaSuccess) d = 0;
  }
  return d;
}

}  // namespace tpb
