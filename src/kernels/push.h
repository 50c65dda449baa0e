// Host-visible interface of the device kernels.
//
//   K1/K6  tpb_push_pack   one persistent launch walks a table of copy entries (many tensors,
//                          contiguous or 2-D strided, optional dtype cast), moves them to their
//                          destinations — local memory or a peer GPU's memory mapped into this
//                          process — and finally publishes a release-ordered flag.
//   K2     tpb_wait_flag   bounded wait for such a flag on the receiver's stream.
//   K3     unpack          the same kernel as K1 with a local inbox as the source.
//   K7     tpb_delay       bounded busy kernel that scribbles over a buffer (stream-order tests).
//   K8     tpb_fill / tpb_verify   seeded pattern generator and on-device comparison.
//
// The reference has no device code of its own (its data path is cudaMemcpyAsync, see
// tensorpipe/channel/cuda_ipc/channel_impl.cc:238-252,453-463 and cuda_xth/channel_impl.cc:66-77);
// these kernels replace those call sites.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <vector>

#include <tpb/message.h>

namespace tpb {
namespace kernels {

enum EntryKind : uint32_t {
  kCopyBulk = 0,     // contiguous, src/dst/bytes all multiples of 16: TMA bulk pipeline
  kCopyPlain = 1,    // contiguous, any alignment: vectorised ld/st
  kCastPlain = 2,    // contiguous with dtype conversion
  kStrided = 3,      // 2-D strided source -> packed destination (optional conversion)
  kStridedWide16 = 4,  // transposed 2-byte elements, everything 4-byte aligned: 64x64 tiles moved as 32-bit words
  kStridedNarrow = 5,  // transposed matrix of at most 64 columns: a tile is 32 whole packed rows, written as one
                       // contiguous run with 16 bytes per lane (optional conversion)
  kStridedBand = 6,    // transposed matrix whose packed rows are at most 8 KiB, any alignment: a tile is a band of
                       // whole rows (as many as fit in 8 KiB), gathered down the source columns and written as
                       // ONE contiguous run (optional conversion)
};

struct alignas(16) PushEntry {
  const void* src;
  void* dst;
  uint64_t count;        // bytes for kCopy*, elements for kCast*/kStrided (= rows*cols)
  uint32_t kind;
  uint8_t srcDtype, dstDtype, srcElemSize, dstElemSize;
  int64_t rows, cols, rowStride, colStride;  // kStrided only, in elements
  uint32_t tileStart;    // first tile of this entry within its class (bulk / plain)
  uint32_t numTiles;
};
static_assert(sizeof(PushEntry) == 80, "entry layout");

constexpr int kMaxEntriesSmall = 8;
constexpr int kMaxEntriesLarge = 96;
constexpr uint32_t kPlainTileBytes = 8 * 1024;  // one warp's unit of work (destination bytes)
constexpr int kStridedTile = 32;                // a warp transposes 32x32 elements (16x32 for 8-byte ones)
constexpr int kWideTile = 64;                   // kStridedWide16: 64x64 two-byte elements per warp tile
constexpr int kNarrowMaxCols = 64;              // kStridedNarrow: 32 rows x (<= 64) columns per warp tile
constexpr uint32_t kBandBytes = 8 * 1024;       // kStridedBand: destination bytes of one band
// Rows of one band of a kStridedBand entry (host and device must agree).
constexpr inline uint32_t bandRows(uint64_t cols, uint32_t dstElemSize) {
  const uint64_t rowBytes = cols * dstElemSize;
  return rowBytes >= kBandBytes ? 1u : static_cast<uint32_t>(kBandBytes / rowBytes);
}
constexpr int kThreads = 512;                   // full kernel: warp 0 drives TMA, warps 1..15 use registers
constexpr int kLightThreads = 256;              // light kernel (no bulk pipeline, static shared memory only)
constexpr int kMaxBulkStages = 8;

// Shape of the TMA bulk pipeline; process-wide, read when a plan is built. The defaults are the
// measured optimum on B200 for HBM->HBM and HBM->NVLink streams.
struct PushTuning {
  uint32_t bulkTileBytes = 32 * 1024;  // multiple of 1024
  uint32_t bulkStages = 3;             // 2..kMaxBulkStages; stages * tile must fit in shared memory
  uint32_t bulkMinBytes = 512 * 1024;  // entries smaller than this take the plain path
  // Transposed matrices of at most 64 columns written as whole packed rows (kStridedNarrow):
  // 0 never, 1 for remote destinations (default), 2 always. TPB_PUSH_NARROW overrides the default.
  uint32_t narrowRows = 1;
  // Transposed matrices with packed rows of at most 8 KiB written as bands of whole rows
  // (kStridedBand), wherever the narrow form above does not apply: 0 never, 1 for remote
  // destinations (default), 2 always. TPB_PUSH_BAND overrides the default.
  uint32_t bandRows = 1;
};
void setPushTuning(const PushTuning& t);
PushTuning getPushTuning();

// Status word values written by kernels (0 = fine).
enum KernelStatus : uint32_t {
  kStatusOk = 0,
  kStatusWaitTimeout = 1,     // tpb_wait_flag gave up
  kStatusBarrierTimeout = 2,  // a bulk load never completed
};

struct PushPlan {
  std::vector<PushEntry> entries;
  uint32_t bulkTiles = 0;
  uint32_t plainTiles = 0;
  uint64_t totalBytesOut = 0;
  uint32_t bulkTileBytes = 0;  // fixed by the first bulk entry
  uint32_t bulkStages = 0;
};

struct CopyItem {
  const void* src = nullptr;
  void* dst = nullptr;
  uint64_t srcBytes = 0;            // packed bytes in the source dtype
  DType srcDtype = DType::kBytes;
  DType dstDtype = DType::kBytes;   // == srcDtype (or kBytes) when no conversion
  bool strided = false;
  StridedView view;
  // The destination is another GPU's memory: prefer the paths whose stores form long contiguous
  // runs (what NVLink wants) over the ones that are fastest against local HBM.
  bool remote = false;
};

// True if (src -> dst) is a conversion the kernels implement.
bool castSupported(DType src, DType dst);
uint64_t convertedBytes(uint64_t srcBytes, DType src, DType dst);

// Chooses the bulk tile of a plan that is still empty, for `bulkBytes` of bulk-path data spread
// over `ctas` CTAs: the largest tile not above the tuned one that leaves every CTA about the same
// number of tiles. A 1 MiB message then becomes 148 tiles of 7 KiB that move at once instead of 32
// tiles of 32 KiB on 32 SMs, and an 8 MiB message two full waves instead of one and three
// quarters. Without this call a plan uses the tuned tile size.
void chooseBulkTile(PushPlan& plan, uint64_t bulkBytes, int ctas);

// Splits items into kernel entries (aligned body for the bulk path, ragged head/tail for the
// plain path) and numbers their tiles. `useBulk=false` routes everything through the plain path.
void appendToPlan(PushPlan& plan, const CopyItem& item, bool useBulk);

// A launch may be told to hold back until a flag that another GPU writes has reached a value
// (cyclic comparison, as tpb_wait_flag does), for at most timeoutNs; on a timeout it copies
// nothing, reports kStatusWaitTimeout and does not publish its own flag. Only for producers on
// ANOTHER GPU: a kernel must not spin on something a different launch on its own GPU produces.
struct WaitBefore {
  const uint32_t* flag = nullptr;
  uint32_t value = 0;
  uint64_t timeoutNs = 0;
};

// A word in mapped host memory that the launch sets to `value` when all of its CTAs are through
// (also when the launch gave up): lets the host follow launches without events.
struct DoneSlot {
  uint32_t* slot = nullptr;
  uint32_t value = 0;
};

// Launches the plan on `stream` of the current device. `flag` may be null; when set, `counter`
// must point to a zeroed 32-bit word in this device's memory that is private to launches
// that cannot overlap on the GPU (the kernel leaves it zeroed again). `status` (device or mapped
// host memory) may be null; a launch that gives up writes a KernelStatus there and leaves the
// flag unpublished. Returns the number of kernel launches made (plans with many entries take
// several).
int launchPush(const PushPlan& plan, cudaStream_t stream, int maxCtas, uint32_t* flag,
               uint32_t flagValue, uint32_t* counter, uint32_t* status, WaitBefore wait = WaitBefore(),
               DoneSlot done = DoneSlot());

// Waits until *flag - value >= 0 (cyclic) or until timeoutNs elapsed; on a timeout writes
// kStatusWaitTimeout to *status (device or mapped host memory) and otherwise leaves it alone.
void launchWaitFlag(cudaStream_t stream, const uint32_t* flag, uint32_t value, uint64_t timeoutNs,
                    uint32_t* status);

// Keeps the stream busy for roughly `microseconds` (capped at 2 s) while scribbling into buf.
void launchDelay(cudaStream_t stream, void* buf, size_t bytes, uint32_t microseconds);

// buf[i] = pattern(seed, i) over 32-bit words (and trailing bytes).
void launchFill(cudaStream_t stream, void* buf, size_t bytes, uint64_t seed);
// Adds the number of mismatching bytes versus pattern(seed) to *mismatches (device memory).
void launchVerify(cudaStream_t stream, const void* buf, size_t bytes, uint64_t seed,
                  unsigned long long* mismatches);
// Host restatement of the pattern, for CPU-side checks.
uint8_t patternByte(uint64_t seed, uint64_t index);

// Total kernel launches made by this process (for benchmarks' accounting).
uint64_t launchCount();

// True when the library was built with -DTPB_DEBUG_KERNELS: the copy paths then compare every
// address they compute with the range its table entry declares, skip what lies outside and count it.
bool debugKernels();
// Violations counted so far, over every device this process has a context on (always 0 in a
// regular build).
uint64_t boundsViolations();

}  // namespace kernels
}  // namespace tpb
