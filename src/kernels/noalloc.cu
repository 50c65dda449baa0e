// Allocation-free variant of the push kernel: see include/tpb/noalloc.h for who needs it and the
// rules for using it. The scratch memory an ordinary launch gets from its caller (the table of
// copies and the arrive counter) lives here in one file-scope device array.
#include <tpb/noalloc.h>

#include <cuda_runtime.h>

#include <mutex>
#include <string>

namespace {

constexpr uint32_t kTileBytes = 8 * 1024;  // one warp's unit of work, as in the ordinary kernel
constexpr int kThreads = 256;
constexpr size_t kCounterBytes = 256;
constexpr int kMaxDevices = 64;

struct alignas(16) TableEntry {
  const void* src;
  void* dst;
  uint64_t bytes;
  uint32_t tileStart;
  uint32_t numTiles;
};
static_assert(sizeof(TableEntry) == 32, "table entry layout");

// [0, 256): arrive counter (first word used). [256, ...): the table. Every GPU that loads this
// library holds this array until the process exits. In HOST code the name is only a stand-in for
// the symbol; the device address comes from cudaGetSymbolAddress (see lookupScratch).
static __device__ __align__(256) unsigned char g_scratch[kCounterBytes + TPB_NOALLOC_MAX_ITEMS * sizeof(TableEntry)];

__device__ __forceinline__ void copyTile(const unsigned char* src, unsigned char* dst, uint32_t bytes, int lane) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst);
  if ((a & 15) == 0) {
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    const uint32_t n = bytes / 16;
    uint32_t i = lane;
    for (; i + 3 * 32 < n; i += 4 * 32) {
      uint4 r0 = s[i], r1 = s[i + 32], r2 = s[i + 64], r3 = s[i + 96];
      d[i] = r0;
      d[i + 32] = r1;
      d[i + 64] = r2;
      d[i + 96] = r3;
    }
    for (; i < n; i += 32) d[i] = s[i];
    for (uint32_t b = n * 16 + lane; b < bytes; b += 32) dst[b] = src[b];
  } else {
    for (uint32_t b = lane; b < bytes; b += 32) dst[b] = src[b];
  }
}

// `scratch` is the device address of g_scratch, looked up by the host.
__global__ void __launch_bounds__(kThreads) tpb_noalloc_push_kernel(unsigned char* scratch, uint32_t count,
                                                                    uint32_t totalTiles, uint32_t* flag,
                                                                    uint32_t flagValue) {
  const TableEntry* table = reinterpret_cast<const TableEntry*>(scratch + kCounterBytes);
  unsigned int* counter = reinterpret_cast<unsigned int*>(scratch);
  const uint32_t warpsPerCta = kThreads / 32;
  const uint32_t warp = blockIdx.x * warpsPerCta + threadIdx.x / 32;
  const uint32_t totalWarps = gridDim.x * warpsPerCta;
  const int lane = threadIdx.x & 31;
  for (uint32_t t = warp; t < totalTiles; t += totalWarps) {
    uint32_t e = 0;
    while (e + 1 < count && t - table[e].tileStart >= table[e].numTiles) ++e;
    const uint64_t off = static_cast<uint64_t>(t - table[e].tileStart) * kTileBytes;
    const uint64_t left = table[e].bytes - off;
    const uint32_t bytes = left > kTileBytes ? kTileBytes : static_cast<uint32_t>(left);
    copyTile(static_cast<const unsigned char*>(table[e].src) + off, static_cast<unsigned char*>(table[e].dst) + off,
             bytes, lane);
  }
  if (flag == nullptr) return;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int arrived = atomicAdd(counter, 1u);
    if (arrived == gridDim.x - 1) {
      __threadfence_system();
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(flagValue) : "memory");
    }
  }
}

thread_local std::string t_lastCudaError;

// Device address of g_scratch for the current device and that device's SM count; both resolved
// once per device.
int lookupScratch(unsigned char** out, int* smCount) {
  static std::mutex mu;
  static unsigned char* perDevice[kMaxDevices] = {};
  static int smsOf[kMaxDevices] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    t_lastCudaError = e != cudaSuccess ? cudaGetErrorString(e) : "device index out of range";
    return TPB_NOALLOC_CUDA_ERROR;
  }
  std::unique_lock<std::mutex> lock(mu);
  if (perDevice[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_scratch);
    if (e != cudaSuccess || p == nullptr) {
      t_lastCudaError = std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e);
      cudaGetLastError();
      return TPB_NOALLOC_CUDA_ERROR;
    }
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
      cudaGetLastError();
      sms = 1;
    }
    smsOf[dev] = sms;
    perDevice[dev] = static_cast<unsigned char*>(p);
  }
  *out = perDevice[dev];
  *smCount = smsOf[dev];
  return TPB_NOALLOC_OK;
}

}  // namespace

extern "C" int tpb_noalloc_push(const tpb_noalloc_item* items, size_t count, uint32_t* flag, uint32_t flag_value,
                                void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (count > TPB_NOALLOC_MAX_ITEMS) return TPB_NOALLOC_TOO_MANY;
  if (count > 0 && items == nullptr) return TPB_NOALLOC_BAD_ARGUMENT;

  // The table is built on the stack: no host allocation either.
  TableEntry table[TPB_NOALLOC_MAX_ITEMS];
  uint32_t n = 0, tiles = 0;
  for (size_t i = 0; i < count; ++i) {
    if (items[i].bytes == 0) continue;
    if (items[i].src == nullptr || items[i].dst == nullptr) return TPB_NOALLOC_BAD_ARGUMENT;
    if (items[i].bytes > UINT64_MAX - kTileBytes) return TPB_NOALLOC_BAD_ARGUMENT;  // rounding up would wrap
    const uint64_t t = (items[i].bytes + kTileBytes - 1) / kTileBytes;
    if (t > 0xffffffffull - tiles) return TPB_NOALLOC_BAD_ARGUMENT;
    table[n].src = items[i].src;
    table[n].dst = items[i].dst;
    table[n].bytes = items[i].bytes;
    table[n].tileStart = tiles;
    table[n].numTiles = static_cast<uint32_t>(t);
    tiles += static_cast<uint32_t>(t);
    ++n;
  }

  unsigned char* scratch = nullptr;
  int sms = 1;
  int rc = lookupScratch(&scratch, &sms);
  if (rc != TPB_NOALLOC_OK) return rc;

  cudaError_t e = cudaSuccess;
  // The array still holds the previous call's table and counter: rewrite both, in stream order.
  e = cudaMemsetAsync(scratch, 0, kCounterBytes, stream);
  if (e == cudaSuccess && n > 0) {
    // Pageable source: the runtime has consumed `table` by the time this returns.
    e = cudaMemcpyAsync(scratch + kCounterBytes, table, n * sizeof(TableEntry), cudaMemcpyHostToDevice, stream);
  }
  if (e == cudaSuccess) {
    const uint32_t warpsPerCta = kThreads / 32;
    uint32_t grid = (tiles + warpsPerCta - 1) / warpsPerCta;
    if (grid > static_cast<uint32_t>(sms) * 4) grid = static_cast<uint32_t>(sms) * 4;
    if (grid == 0) grid = 1;
    tpb_noalloc_push_kernel<<<grid, kThreads, 0, stream>>>(scratch, n, tiles, flag, flag_value);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    t_lastCudaError = cudaGetErrorString(e);
    return TPB_NOALLOC_CUDA_ERROR;
  }
  return TPB_NOALLOC_OK;
}

extern "C" const char* tpb_noalloc_strerror(int code) {
  switch (code) {
    case TPB_NOALLOC_OK: return "ok";
    case TPB_NOALLOC_TOO_MANY: return "more items than TPB_NOALLOC_MAX_ITEMS (256): split the request";
    case TPB_NOALLOC_BAD_ARGUMENT: return "null pointer for a non-empty item, or sizes that overflow";
    case TPB_NOALLOC_CUDA_ERROR: return t_lastCudaError.c_str();
    default: return "unknown code";
  }
}
