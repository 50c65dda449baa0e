// sm_100a kernels of the device-to-device channel. See push.h for the interface.
//
// tpb_push_pack is ONE persistent launch (at most one CTA per SM) that serves a whole message:
//
//   * Warp 0 is a copy engine. Its elected lane drives a multi-stage pipeline of TMA bulk copies:
//     global -> shared (completion on an mbarrier) and shared -> global (bulk groups), for every
//     entry whose source, destination and size are 16-byte multiples. The loads only ever read
//     THIS GPU's memory; the stores may target a peer GPU's memory mapped over NVLink. No thread
//     touches the bytes. Tile size and depth are run-time parameters (PushTuning).
//   * The other warps handle what the bulk path cannot, one 8 KiB "warp tile" at a time and
//     without CTA-wide barriers: ragged heads and tails, relatively misaligned buffers, dtype
//     conversion (fp32 <-> bf16/fp16), and 2-D strided sources, which a warp transposes through
//     its private padded shared-memory tile so that both the strided reads and the packed writes
//     are coalesced (32x32 elements; 64x64 moved as 32-bit words for 2-byte elements; 32 whole
//     packed rows written as one contiguous run for matrices of at most 64 columns bound for
//     another GPU). A warp makes one call per tensor for all of its tiles.
//   * Tiles are dealt round-robin (bulk tile t to CTA t mod gridDim.x, warp tile t to warp
//     t mod #warps), so no scheduling state lives in global memory.
//   * Completion: every CTA makes its writes visible system-wide, then arrives on a counter;
//     the last CTA resets the counter and publishes the flag with a release store at system
//     scope. The flag lives in the receiver's memory; its stream waits on it.
//
// A "light" instantiation (256 threads, no bulk pipeline, shared memory only when a tensor is
// staged through it) serves messages without bulk work, where launch latency matters most.
//
// Built with -DTPB_DEBUG_KERNELS the copy paths check every address against its table entry,
// skip what lies outside and count it (boundsViolations()); nothing in here can trap.
//
// Every wait in here is bounded: a bulk load that does not complete within the limit makes the
// CTA record kStatusBarrierTimeout, drain its own outstanding stores and fall through to the
// completion protocol, so the kernel always terminates.
#include "kernels/push.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common/cuda.h"
#include "common/trace.h"

#include <atomic>
#include <cstdlib>
#include <mutex>
#include <stdexcept>
#include <string>

namespace tpb {
namespace kernels {

namespace {

std::atomic<uint64_t> gLaunches{0};
std::mutex gTuningMutex;
PushTuning initialTuning() {
  PushTuning t;
  if (const char* e = std::getenv("TPB_PUSH_BAND")) {
    if (e[0] >= '0' && e[0] <= '2' && e[1] == 0) t.bandRows = static_cast<uint32_t>(e[0] - '0');
  }
  if (const char* e = std::getenv("TPB_PUSH_NARROW")) {
    if (e[0] >= '0' && e[0] <= '2' && e[1] == 0) t.narrowRows = static_cast<uint32_t>(e[0] - '0');
  }
  // The shape of the bulk pipeline can be tried out without rebuilding; values that setPushTuning
  // would refuse are ignored.
  auto number = [](const char* name, uint32_t fallback) {
    const char* e = std::getenv(name);
    if (!e || !*e) return fallback;
    char* end = nullptr;
    const unsigned long v = std::strtoul(e, &end, 0);
    return end && *end == 0 ? static_cast<uint32_t>(v) : fallback;
  };
  const uint32_t tile = number("TPB_PUSH_TILE_BYTES", t.bulkTileBytes);
  const uint32_t stages = number("TPB_PUSH_STAGES", t.bulkStages);
  if (tile % 1024 == 0 && tile > 0 && stages >= 2 && stages <= static_cast<uint32_t>(kMaxBulkStages) &&
      static_cast<size_t>(tile) * stages <= 160 * 1024) {
    t.bulkTileBytes = tile;
    t.bulkStages = stages;
  }
  t.bulkMinBytes = number("TPB_PUSH_BULK_MIN_BYTES", t.bulkMinBytes);
  return t;
}
PushTuning gTuning = initialTuning();

constexpr uint32_t kWarpTileBytes = kStridedTile * (kStridedTile / 2 + 1) * 8;  // 4352 B per warp: 32 x 17 x 8-byte, or 32 x 33 x 4-byte
constexpr int kWidePitch = kWideTile + 2;                                        // 2-byte elements per staged column
constexpr uint32_t kWideWarpTileBytes = kWideTile * kWidePitch * 2;              // 8448 B per warp
constexpr size_t kMaxSmemPerCta = 227 * 1024;

// ---- PTX wrappers -----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smemAddr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbarInit(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarExpectTx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smemAddr(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbarTryWait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smemAddr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: ~2^22 polls, each of which may block for the hardware's time slice.
__device__ __forceinline__ bool mbarWaitBounded(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < (1u << 22); ++i) {
    if (mbarTryWait(bar, parity)) return true;
    if (i > 64) __nanosleep(64);
  }
  return false;
}
// Non-multicast bulk copy global -> this CTA's shared memory, completion on an mbarrier.
__device__ __forceinline__ void bulkLoad(void* smemDst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smemAddr(smemDst)),
      "l"(gsrc), "r"(bytes), "r"(smemAddr(bar))
      : "memory");
}
// Bulk copy this CTA's shared memory -> global (local or peer), tracked by bulk groups.
__device__ __forceinline__ void bulkStore(void* gdst, const void* smemSrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
               "r"(smemAddr(smemSrc)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulkCommit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulkWaitRead() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulkWaitAll() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fenceProxyAsync() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void storeReleaseSys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t loadAcquireSys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t globalTimerNs() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---- self-checking build ------------------------------------------------------------------------
// With -DTPB_DEBUG_KERNELS every address the copy paths compute is compared with the byte range
// its table entry declares before it is used; an address outside is counted and the access is
// skipped, so a wrong index shows up as a number the host can read (boundsViolations()) and never
// as a fault. compute-sanitizer plays this role elsewhere; here the kernel checks itself.
#ifdef TPB_DEBUG_KERNELS
__device__ unsigned long long gBoundsViolations = 0;
__device__ __forceinline__ bool dbgInside(const void* p, uint64_t n, const void* base, uint64_t span) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p), b = reinterpret_cast<uintptr_t>(base);
  if (a >= b && a - b <= span && n <= span - (a - b)) return true;
  atomicAdd(&gBoundsViolations, 1ull);
  return false;
}
#define TPB_DBG_INSIDE(p, n, base, span) dbgInside(p, n, base, span)
#else
#define TPB_DBG_INSIDE(p, n, base, span) true
#endif

// ---- parameters ---------------------------------------------------------------------------------
template <int N>
struct PushParams {
  PushEntry entries[N];
  uint32_t numEntries;
  uint32_t bulkTiles;
  uint32_t plainTiles;
  uint32_t flagValue;
  uint32_t* flag;
  uint32_t* counter;
  uint32_t* status;
  uint32_t bulkTileBytes;
  uint32_t bulkStages;
  uint32_t warpTileBytes;  // shared memory per register-path warp (0 when no entry needs staging)
  // Optional: nothing is read before *waitFlag has reached waitValue (cyclic comparison) or the
  // time limit has passed; used by a receiver that unpacks what another GPU is still delivering.
  const uint32_t* waitFlag;
  uint32_t waitValue;
  uint64_t waitTimeoutNs;
  // Optional: a word (mapped host memory) that receives doneValue once every CTA of the launch
  // has finished, whether the launch succeeded or gave up: the host's cheap way to learn that a
  // launch is over without an event.
  uint32_t* doneSlot;
  uint32_t doneValue;
  // When the kernel behind this one on the stream may be let go (see letDependentsLaunch):
  // 0 = at the start, 1 = when this CTA has issued all its work and is about to report in.
  uint32_t lateTrigger;
};

// The arrive counter of a launch doubles as its failure latch: the low half counts CTAs that
// have reported in, every CTA that gave up adds one to the high half.
constexpr uint32_t kArriveMask = 0xffffu;
constexpr uint32_t kArriveFailed = 0x10000u;

__device__ __forceinline__ void reportStatus(uint32_t* status, uint32_t code) {
  // The word may live in mapped host memory, where only a plain store is certain to be seen
  // by the CPU; codes are never cleared by a kernel, so the order of racing writers is moot.
  if (status) {
    *reinterpret_cast<volatile uint32_t*>(status) = code;
    __threadfence_system();
  }
}

template <int N>
__device__ __forceinline__ const PushEntry* findEntry(const PushParams<N>& p, uint32_t tile, bool bulk) {
  // Entries of one class have increasing tileStart; a linear scan over <=96 entries in the
  // constant bank (uniform across the warp) costs less than the tile it locates.
  for (uint32_t i = 0; i < p.numEntries; ++i) {
    const PushEntry& e = p.entries[i];
    if ((e.kind == kCopyBulk) != bulk) continue;
    if (tile - e.tileStart < e.numTiles) return &e;
  }
  return nullptr;
}

// ---- conversions --------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float toFloat(T v);
template <>
__device__ __forceinline__ float toFloat<float>(float v) { return v; }
template <>
__device__ __forceinline__ float toFloat<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float toFloat<__half>(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T fromFloat(float v);
template <>
__device__ __forceinline__ float fromFloat<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 fromFloat<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half fromFloat<__half>(float v) { return __float2half_rn(v); }

// ---- plain contiguous copy: one warp, one 8 KiB tile ----------------------------------------------
template <typename V>
__device__ __forceinline__ void copyVec(const uint8_t* src, uint8_t* dst, uint32_t bytes, int lane) {
  const V* s = reinterpret_cast<const V*>(src);
  V* d = reinterpret_cast<V*>(dst);
  const uint32_t n = bytes / sizeof(V);
  constexpr int kUnroll = 8;
  uint32_t i = lane;
  // Issue kUnroll independent loads before the first store: bytes in flight, not instructions,
  // are what fills an NVLink or HBM pipe.
  for (; i + (kUnroll - 1) * 32 < n; i += kUnroll * 32) {
    V r[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) r[u] = s[i + u * 32];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) d[i + u * 32] = r[u];
  }
  for (; i < n; i += 32) d[i] = s[i];
  const uint32_t done = n * sizeof(V);
  for (uint32_t b = done + lane; b < bytes; b += 32) dst[b] = src[b];
}

__device__ __forceinline__ void copyPlainTile(const PushEntry& e, uint32_t localTile, int lane) {
  const uint64_t off = static_cast<uint64_t>(localTile) * kPlainTileBytes;
  const uint64_t left = e.count - off;
  const uint32_t bytes = left > kPlainTileBytes ? kPlainTileBytes : static_cast<uint32_t>(left);
  const uint8_t* src = static_cast<const uint8_t*>(e.src) + off;
  uint8_t* dst = static_cast<uint8_t*>(e.dst) + off;
  if (!TPB_DBG_INSIDE(src, bytes, e.src, e.count) || !TPB_DBG_INSIDE(dst, bytes, e.dst, e.count)) return;
  const uintptr_t a = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst);
  if ((a & 15) == 0) copyVec<uint4>(src, dst, bytes, lane);
  else if ((a & 7) == 0) copyVec<uint2>(src, dst, bytes, lane);
  else if ((a & 3) == 0) copyVec<uint32_t>(src, dst, bytes, lane);
  else if ((a & 1) == 0) copyVec<uint16_t>(src, dst, bytes, lane);
  else copyVec<uint8_t>(src, dst, bytes, lane);
}

// ---- contiguous conversion ----------------------------------------------------------------------
template <typename S, typename D>
__device__ __forceinline__ void castTileTyped(const PushEntry& e, uint32_t localTile, int lane) {
  // A tile is kPlainTileBytes of DESTINATION bytes.
  constexpr uint32_t perTile = kPlainTileBytes / sizeof(D);
  const uint64_t first = static_cast<uint64_t>(localTile) * perTile;
  const uint64_t left = e.count - first;
  const uint32_t n = left > perTile ? perTile : static_cast<uint32_t>(left);
  const S* s = static_cast<const S*>(e.src) + first;
  D* d = static_cast<D*>(e.dst) + first;
  if (!TPB_DBG_INSIDE(s, uint64_t(n) * sizeof(S), e.src, e.count * sizeof(S)) ||
      !TPB_DBG_INSIDE(d, uint64_t(n) * sizeof(D), e.dst, e.count * sizeof(D)))
    return;
  constexpr int kVec = 16 / sizeof(D) < 16 / sizeof(S) ? 16 / sizeof(S) : 16 / sizeof(D);  // elements per step
  const bool aligned = ((reinterpret_cast<uintptr_t>(s) & 15) == 0) && ((reinterpret_cast<uintptr_t>(d) & 15) == 0);
  const uint32_t vecElems = aligned ? (n / kVec) * kVec : 0;
  for (uint32_t i = lane * kVec; i < vecElems; i += 32 * kVec) {
    alignas(16) S in[kVec];
    alignas(16) D out[kVec];
    constexpr int kInVecs = kVec * sizeof(S) / 16;
    constexpr int kOutVecs = kVec * sizeof(D) / 16;
#pragma unroll
    for (int v = 0; v < kInVecs; ++v) reinterpret_cast<uint4*>(in)[v] = reinterpret_cast<const uint4*>(s + i)[v];
#pragma unroll
    for (int k = 0; k < kVec; ++k) out[k] = fromFloat<D>(toFloat<S>(in[k]));
#pragma unroll
    for (int v = 0; v < kOutVecs; ++v) reinterpret_cast<uint4*>(d + i)[v] = reinterpret_cast<uint4*>(out)[v];
  }
  for (uint32_t i = vecElems + lane; i < n; i += 32) d[i] = fromFloat<D>(toFloat<S>(s[i]));
}

__device__ __noinline__ void castTile(const PushEntry& e, uint32_t localTile, int lane) {
  const uint32_t key = (static_cast<uint32_t>(e.srcDtype) << 8) | e.dstDtype;
  constexpr uint32_t F32 = static_cast<uint32_t>(DType::kF32), BF = static_cast<uint32_t>(DType::kBF16),
                     F16 = static_cast<uint32_t>(DType::kF16);
  switch (key) {
    case (F32 << 8) | BF: castTileTyped<float, __nv_bfloat16>(e, localTile, lane); break;
    case (F32 << 8) | F16: castTileTyped<float, __half>(e, localTile, lane); break;
    case (BF << 8) | F32: castTileTyped<__nv_bfloat16, float>(e, localTile, lane); break;
    case (F16 << 8) | F32: castTileTyped<__half, float>(e, localTile, lane); break;
    case (BF << 8) | F16: castTileTyped<__nv_bfloat16, __half>(e, localTile, lane); break;
    case (F16 << 8) | BF: castTileTyped<__half, __nv_bfloat16>(e, localTile, lane); break;
    default: break;  // rejected on the host
  }
}

// ---- 2-D strided source through a per-warp shared-memory tile ------------------------------------
// A warp stages TR x 32 raw source elements as tile[c][r] (row stride TR+1 words keeps both access
// patterns free of bank conflicts for 4-byte elements), reading along whichever source dimension is
// contiguous, then writes rows of the packed destination: 32 consecutive elements per store.
// The entry lives in the kernel's parameter block and is reached through a generic pointer inside
// the tile routines: its fields are read once per call into this pack, or every use inside the
// loops would become a load behind the tile stores.
struct StridedArgs {
  const void* src;
  void* dst;
  int64_t rows, cols, rowStride, colStride;
  uint32_t numTiles;
#ifdef TPB_DEBUG_KERNELS
  uint64_t srcSpan, dstSpan;  // bytes the view covers from src / the packed result covers from dst
#endif
};
__device__ __forceinline__ StridedArgs loadStridedArgs(const PushEntry& e) {
  StridedArgs a{e.src, e.dst, e.rows, e.cols, e.rowStride, e.colStride, e.numTiles};
#ifdef TPB_DEBUG_KERNELS
  // Views with non-negative strides only (what the host accepts): the last element is the farthest.
  a.srcSpan = static_cast<uint64_t>((e.rows - 1) * e.rowStride + (e.cols - 1) * e.colStride + 1) * e.srcElemSize;
  a.dstSpan = static_cast<uint64_t>(e.rows) * e.cols * e.dstElemSize;
#endif
  return a;
}
#ifdef TPB_DEBUG_KERNELS
#define TPB_DBG_SRC(a, p, n) dbgInside(p, n, (a).src, (a).srcSpan)
#define TPB_DBG_DST(a, p, n) dbgInside(p, n, (a).dst, (a).dstSpan)
#else
#define TPB_DBG_SRC(a, p, n) true
#define TPB_DBG_DST(a, p, n) true
#endif

template <typename S, typename D, bool kConvert>
__device__ __forceinline__ void stridedTileTyped(const StridedArgs& a, uint32_t localTile, int lane, uint8_t* tileMem) {
  constexpr int TC = kStridedTile;                                 // columns per tile
  constexpr int TR = sizeof(S) == 8 ? kStridedTile / 2 : kStridedTile;  // rows per tile
  S* tile = reinterpret_cast<S*>(tileMem);
  const int64_t rows = a.rows, cols = a.cols, rowStride = a.rowStride, colStride = a.colStride;
  const S* src = static_cast<const S*>(a.src);
  D* dst = static_cast<D*>(a.dst);
  const uint32_t tilesPerRow = static_cast<uint32_t>((cols + TC - 1) / TC);  // the tile count fits 32 bits
  const int64_t r0 = static_cast<int64_t>(localTile / tilesPerRow) * TR;
  const int64_t c0 = static_cast<int64_t>(localTile % tilesPerRow) * TC;
  const int nr = static_cast<int>(rows - r0 < TR ? rows - r0 : TR);
  const int nc = static_cast<int>(cols - c0 < TC ? cols - c0 : TC);
  const bool rowsFast = (rowStride == 1 || rows == 1) && colStride != 1;
  if (rowsFast && rowStride == 1 && nr == TR && nc == TC) {
    // Full tile of a transposed matrix: no predicates, pointers stepped instead of recomputed,
    // sixteen loads in flight per lane.
    constexpr int kWide = 16;
    const bool act = lane < TR;
    const S* colPtr = src + (r0 + lane) + c0 * colStride;
#pragma unroll 1
    for (int c = 0; c < TC; c += kWide) {
      S v[kWide];
#pragma unroll
      for (int k = 0; k < kWide; ++k)
        if (act && TPB_DBG_SRC(a, colPtr + k * colStride, sizeof(S))) v[k] = colPtr[k * colStride];
      colPtr += kWide * colStride;
#pragma unroll
      for (int k = 0; k < kWide; ++k)
        if (act) tile[(c + k) * (TR + 1) + lane] = v[k];
    }
    __syncwarp();
    D* outPtr = dst + r0 * cols + c0 + lane;
    const S* mine = tile + lane * (TR + 1);
#pragma unroll 1
    for (int r = 0; r < TR; r += kWide) {
      S v[kWide];
#pragma unroll
      for (int k = 0; k < kWide; ++k) v[k] = mine[r + k];
#pragma unroll
      for (int k = 0; k < kWide; ++k) {
        D out;
        if constexpr (kConvert) out = fromFloat<D>(toFloat<S>(v[k]));
        else out = v[k];
        if (TPB_DBG_DST(a, outPtr + k * cols, sizeof(D))) outPtr[k * cols] = out;
      }
      outPtr += kWide * cols;
    }
    __syncwarp();
    return;
  }
  constexpr int kBatch = 4;  // independent loads issued before their results are parked in the tile
  if (rowsFast) {
    // lanes walk down a source column: coalesced reads when the source is a transposed matrix
    for (int rb = 0; rb < nr; rb += 32) {
      const int r = rb + lane;
      const S* colPtr = src + (r0 + r) * rowStride + c0 * colStride;
      for (int c = 0; c < nc; c += kBatch) {
        S v[kBatch];
#pragma unroll
        for (int k = 0; k < kBatch; ++k)
          if (r < nr && c + k < nc && TPB_DBG_SRC(a, colPtr + static_cast<int64_t>(c + k) * colStride, sizeof(S)))
            v[k] = colPtr[static_cast<int64_t>(c + k) * colStride];
#pragma unroll
        for (int k = 0; k < kBatch; ++k)
          if (r < nr && c + k < nc) tile[(c + k) * (TR + 1) + r] = v[k];
      }
    }
  } else {
    for (int cb = 0; cb < nc; cb += 32) {
      const int c = cb + lane;
      const S* rowPtr = src + r0 * rowStride + (c0 + c) * colStride;
      for (int r = 0; r < nr; r += kBatch) {
        S v[kBatch];
#pragma unroll
        for (int k = 0; k < kBatch; ++k)
          if (c < nc && r + k < nr && TPB_DBG_SRC(a, rowPtr + static_cast<int64_t>(r + k) * rowStride, sizeof(S)))
            v[k] = rowPtr[static_cast<int64_t>(r + k) * rowStride];
#pragma unroll
        for (int k = 0; k < kBatch; ++k)
          if (c < nc && r + k < nr) tile[c * (TR + 1) + r + k] = v[k];
      }
    }
  }
  __syncwarp();
  {
    const int c = lane;  // TC == 32: one column per lane
    D* rowPtr = dst + r0 * cols + c0 + c;
    for (int r = 0; r < nr; r += kBatch) {
      S v[kBatch];
#pragma unroll
      for (int k = 0; k < kBatch; ++k)
        if (c < nc && r + k < nr) v[k] = tile[c * (TR + 1) + r + k];
#pragma unroll
      for (int k = 0; k < kBatch; ++k) {
        if (c < nc && r + k < nr) {
          D out;
          if constexpr (kConvert) out = fromFloat<D>(toFloat<S>(v[k]));
          else out = v[k];
          if (TPB_DBG_DST(a, rowPtr + static_cast<int64_t>(r + k) * cols, sizeof(D)))
            rowPtr[static_cast<int64_t>(r + k) * cols] = out;
        }
      }
    }
  }
  __syncwarp();  // the tile is reused by this warp's next strided tile
}

// Not inlined, one function per element type: inlined they would set the register budget of the
// whole kernel, including the copy loops that want many loads in flight. One call covers all
// of this warp's tiles of the entry (first, first + step, ...): a call saves and restores the
// registers it uses, which per tile would cost more local-memory traffic than the tile's payload.
template <typename S, typename D, bool kConvert>
__device__ __noinline__ void stridedTilesTyped(const PushEntry& a_, uint32_t first, uint32_t step, int lane,
                                               uint8_t* tileMem) {
  const StridedArgs a = loadStridedArgs(a_);
#pragma unroll 1
  for (uint32_t t = first; t < a.numTiles; t += step) stridedTileTyped<S, D, kConvert>(a, t, lane, tileMem);
}

__device__ __forceinline__ void stridedTiles(const PushEntry& a, uint32_t first, uint32_t step, int lane, uint8_t* tileMem) {
  const PushEntry& e = a;
  if (e.srcDtype == e.dstDtype || e.dstDtype == static_cast<uint8_t>(DType::kBytes)) {
    switch (e.srcElemSize) {
      case 1: stridedTilesTyped<uint8_t, uint8_t, false>(a, first, step, lane, tileMem); break;
      case 2: stridedTilesTyped<uint16_t, uint16_t, false>(a, first, step, lane, tileMem); break;
      case 4: stridedTilesTyped<uint32_t, uint32_t, false>(a, first, step, lane, tileMem); break;
      default: stridedTilesTyped<uint64_t, uint64_t, false>(a, first, step, lane, tileMem); break;
    }
    return;
  }
  const uint32_t key = (static_cast<uint32_t>(e.srcDtype) << 8) | e.dstDtype;
  constexpr uint32_t F32 = static_cast<uint32_t>(DType::kF32), BF = static_cast<uint32_t>(DType::kBF16),
                     F16 = static_cast<uint32_t>(DType::kF16);
  switch (key) {
    case (F32 << 8) | BF: stridedTilesTyped<float, __nv_bfloat16, true>(a, first, step, lane, tileMem); break;
    case (F32 << 8) | F16: stridedTilesTyped<float, __half, true>(a, first, step, lane, tileMem); break;
    case (BF << 8) | F32: stridedTilesTyped<__nv_bfloat16, float, true>(a, first, step, lane, tileMem); break;
    case (F16 << 8) | F32: stridedTilesTyped<__half, float, true>(a, first, step, lane, tileMem); break;
    case (BF << 8) | F16: stridedTilesTyped<__nv_bfloat16, __half, true>(a, first, step, lane, tileMem); break;
    case (F16 << 8) | BF: stridedTilesTyped<__half, __nv_bfloat16, true>(a, first, step, lane, tileMem); break;
    default: break;
  }
}

// Transposed matrix with few columns (cols <= 64, rowStride == 1): a tile is 32 whole rows of the
// packed result, i.e. ONE contiguous run of 32 * cols elements in the destination. Lanes read down
// the source columns as usual and park the (already converted) values in 32-bit slots tile[c][r];
// then every lane gathers the 16 bytes of its chunk of the run and stores them as one vector, so a
// warp writes 512 contiguous bytes per instruction instead of one 128-byte row segment. That is
// what a remote GPU's memory wants to see over NVLink. Needs cols * sizeof(D) to be a multiple of
// 16 and a 16-byte aligned destination.
template <typename S, typename D, bool kConvert>
__device__ __forceinline__ void stridedNarrowTile(const StridedArgs& a, uint32_t localTile, int lane, uint8_t* tileMem) {
  constexpr int TR = 32, P = TR + 1;
  constexpr int K = 16 / sizeof(D);  // destination elements per 16-byte chunk
  uint32_t* tile = reinterpret_cast<uint32_t*>(tileMem);
  const int64_t rows = a.rows, colStride = a.colStride;
  const int cols = static_cast<int>(a.cols);
  const S* src = static_cast<const S*>(a.src);
  D* dst = static_cast<D*>(a.dst);
  const int64_t r0 = static_cast<int64_t>(localTile) * TR;
  const int nr = static_cast<int>(rows - r0 < TR ? rows - r0 : TR);
  constexpr int kBatch = 16;
  {
    const bool act = lane < nr;
    const S* colPtr = src + (r0 + lane);
    for (int c = 0; c < cols; c += kBatch) {
      S v[kBatch];
#pragma unroll
      for (int k = 0; k < kBatch; ++k)
        if (act && c + k < cols && TPB_DBG_SRC(a, colPtr + static_cast<int64_t>(c + k) * colStride, sizeof(S)))
          v[k] = colPtr[static_cast<int64_t>(c + k) * colStride];
#pragma unroll
      for (int k = 0; k < kBatch; ++k) {
        if (act && c + k < cols) {
          D out;
          if constexpr (kConvert) out = fromFloat<D>(toFloat<S>(v[k]));
          else out = v[k];
          uint32_t bits = 0;
          if constexpr (sizeof(D) == 4) bits = *reinterpret_cast<const uint32_t*>(&out);
          else if constexpr (sizeof(D) == 2) bits = *reinterpret_cast<const uint16_t*>(&out);
          else bits = *reinterpret_cast<const uint8_t*>(&out);
          tile[(c + k) * P + lane] = bits;
        }
      }
    }
  }
  __syncwarp();
  {
    const int chunksPerRow = cols / K;
    const int chunks = nr * chunksPerRow;
    uint4* out = reinterpret_cast<uint4*>(dst + r0 * cols);
    // (r, c) of chunk q, advanced by 32 chunks per step without dividing in the loop.
    int r = lane / chunksPerRow;
    int cc = lane - r * chunksPerRow;  // chunk index within its row
    const int stepRows = 32 / chunksPerRow, stepChunks = 32 - stepRows * chunksPerRow;
    for (int q = lane; q < chunks; q += 32) {
      const int c = cc * K;
      alignas(16) D vals[K];
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const uint32_t bits = tile[(c + k) * P + r];
        if constexpr (sizeof(D) == 4) vals[k] = *reinterpret_cast<const D*>(&bits);
        else if constexpr (sizeof(D) == 2) {
          const uint16_t h = static_cast<uint16_t>(bits);
          vals[k] = *reinterpret_cast<const D*>(&h);
        } else {
          const uint8_t b = static_cast<uint8_t>(bits);
          vals[k] = *reinterpret_cast<const D*>(&b);
        }
      }
      if (TPB_DBG_DST(a, out + q, 16)) out[q] = *reinterpret_cast<const uint4*>(vals);
      r += stepRows;
      cc += stepChunks;
      if (cc >= chunksPerRow) {
        cc -= chunksPerRow;
        ++r;
      }
    }
  }
  __syncwarp();
}

template <typename S, typename D, bool kConvert>
__device__ __noinline__ void stridedNarrowTilesTyped(const PushEntry& e, uint32_t first, uint32_t step, int lane,
                                                     uint8_t* tileMem) {
  const StridedArgs a = loadStridedArgs(e);
#pragma unroll 1
  for (uint32_t t = first; t < a.numTiles; t += step) stridedNarrowTile<S, D, kConvert>(a, t, lane, tileMem);
}

__device__ __forceinline__ void stridedNarrowTiles(const PushEntry& e, uint32_t first, uint32_t step, int lane,
                                                   uint8_t* tileMem) {
  if (e.srcDtype == e.dstDtype || e.dstDtype == static_cast<uint8_t>(DType::kBytes)) {
    switch (e.srcElemSize) {
      case 1: stridedNarrowTilesTyped<uint8_t, uint8_t, false>(e, first, step, lane, tileMem); break;
      case 2: stridedNarrowTilesTyped<uint16_t, uint16_t, false>(e, first, step, lane, tileMem); break;
      default: stridedNarrowTilesTyped<uint32_t, uint32_t, false>(e, first, step, lane, tileMem); break;
    }
    return;
  }
  const uint32_t key = (static_cast<uint32_t>(e.srcDtype) << 8) | e.dstDtype;
  constexpr uint32_t F32 = static_cast<uint32_t>(DType::kF32), BF = static_cast<uint32_t>(DType::kBF16),
                     F16 = static_cast<uint32_t>(DType::kF16);
  switch (key) {
    case (F32 << 8) | BF: stridedNarrowTilesTyped<float, __nv_bfloat16, true>(e, first, step, lane, tileMem); break;
    case (F32 << 8) | F16: stridedNarrowTilesTyped<float, __half, true>(e, first, step, lane, tileMem); break;
    case (BF << 8) | F32: stridedNarrowTilesTyped<__nv_bfloat16, float, true>(e, first, step, lane, tileMem); break;
    case (F16 << 8) | F32: stridedNarrowTilesTyped<__half, float, true>(e, first, step, lane, tileMem); break;
    case (BF << 8) | F16: stridedNarrowTilesTyped<__nv_bfloat16, __half, true>(e, first, step, lane, tileMem); break;
    case (F16 << 8) | BF: stridedNarrowTilesTyped<__half, __nv_bfloat16, true>(e, first, step, lane, tileMem); break;
    default: break;
  }
}

// Transposed matrix (rowStride == 1) whose packed rows are at most 8 KiB, for destinations that
// want long contiguous writes (another GPU's memory over NVLink, where a 64-byte or misaligned
// 128-byte row segment costs a whole packet): a tile is a band of whole rows, as many as fit in
// 8 KiB. The band's elements are gathered down the source columns (consecutive rows of one column
// are adjacent in the source: coalesced, the more so the more rows a band has), converted, and laid
// out in shared memory exactly as the destination wants them, at the destination's own alignment
// modulo 16; the band then leaves as ONE contiguous run: bytes up to the first 16-byte boundary,
// 16-byte vectors, bytes after the last one. No alignment or divisibility is asked of anything.
template <typename S, typename D, bool kConvert>
__device__ __forceinline__ void stridedBandTile(const StridedArgs& a, uint32_t band, uint32_t bandRowsCount, int lane,
                                                uint8_t* tileMem) {
  const int64_t rows = a.rows, colStride = a.colStride;
  const uint32_t cols = static_cast<uint32_t>(a.cols);
  const S* src = static_cast<const S*>(a.src);
  const int64_t r0 = static_cast<int64_t>(band) * bandRowsCount;
  const uint32_t nr = static_cast<uint32_t>(rows - r0 < bandRowsCount ? rows - r0 : bandRowsCount);
  uint8_t* out = static_cast<uint8_t*>(a.dst) + static_cast<uint64_t>(r0) * cols * sizeof(D);
  const uint32_t skew = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(out) & 15);  // a multiple of sizeof(D)
  D* stage = reinterpret_cast<D*>(tileMem + skew);
  const uint32_t n = nr * cols;  // elements of this band
  // Gather: element q of the (c-major, r-minor) enumeration is (c, r) = (q / nr, q % nr); lanes take
  // q = lane, lane + 32, ... and keep (c, r) up to date without dividing in the loop.
  {
    constexpr int kBatch = 8;
    uint32_t c = lane / nr, r = lane - c * nr;
    const uint32_t stepC = 32 / nr, stepR = 32 - stepC * nr;
    for (uint32_t q = lane; q < n; q += 32 * kBatch) {
      S v[kBatch];
      uint32_t cs[kBatch], rs[kBatch];
#pragma unroll
      for (int k = 0; k < kBatch; ++k) {
        cs[k] = c;
        rs[k] = r;
        if (q + 32 * k < n && TPB_DBG_SRC(a, src + static_cast<int64_t>(c) * colStride + r0 + r, sizeof(S)))
          v[k] = src[static_cast<int64_t>(c) * colStride + r0 + r];
        c += stepC;
        r += stepR;
        if (r >= nr) {
          r -= nr;
          ++c;
        }
      }
#pragma unroll
      for (int k = 0; k < kBatch; ++k) {
        if (q + 32 * k < n) {
          D o;
          if constexpr (kConvert) o = fromFloat<D>(toFloat<S>(v[k]));
          else o = v[k];
          stage[rs[k] * cols + cs[k]] = o;
        }
      }
    }
  }
  __syncwarp();
  {
    const uint32_t bytes = n * static_cast<uint32_t>(sizeof(D));
    const uint8_t* from = tileMem + skew;
    // head: up to the first 16-byte boundary of the destination (and of the staging area: same skew)
    const uint32_t head = skew == 0 ? 0 : (16 - skew < bytes ? 16 - skew : bytes);
    if (static_cast<uint32_t>(lane) < head && TPB_DBG_DST(a, out + lane, 1)) out[lane] = from[lane];
    const uint32_t vectors = (bytes - head) / 16;
    const uint4* vfrom = reinterpret_cast<const uint4*>(from + head);
    uint4* vout = reinterpret_cast<uint4*>(out + head);
    for (uint32_t i = lane; i < vectors; i += 32)
      if (TPB_DBG_DST(a, vout + i, 16)) vout[i] = vfrom[i];
    const uint32_t done = head + vectors * 16;
    if (done + lane < bytes && TPB_DBG_DST(a, out + done + lane, 1)) out[done + lane] = from[done + lane];
  }
  __syncwarp();  // the staging area is reused by this warp's next band
}

template <typename S, typename D, bool kConvert>
__device__ __noinline__ void stridedBandTilesTyped(const PushEntry& e, uint32_t first, uint32_t step, int lane,
                                                   uint8_t* tileMem) {
  const StridedArgs a = loadStridedArgs(e);
  const uint32_t rowsPerBand = bandRows(static_cast<uint64_t>(e.cols), sizeof(D));
#pragma unroll 1
  for (uint32_t t = first; t < a.numTiles; t += step) stridedBandTile<S, D, kConvert>(a, t, rowsPerBand, lane, tileMem);
}

__device__ __forceinline__ void stridedBandTiles(const PushEntry& e, uint32_t first, uint32_t step, int lane,
                                                 uint8_t* tileMem) {
  if (e.srcDtype == e.dstDtype || e.dstDtype == static_cast<uint8_t>(DType::kBytes)) {
    switch (e.srcElemSize) {
      case 1: stridedBandTilesTyped<uint8_t, uint8_t, false>(e, first, step, lane, tileMem); break;
      case 2: stridedBandTilesTyped<uint16_t, uint16_t, false>(e, first, step, lane, tileMem); break;
      case 4: stridedBandTilesTyped<uint32_t, uint32_t, false>(e, first, step, lane, tileMem); break;
      default: stridedBandTilesTyped<uint64_t, uint64_t, false>(e, first, step, lane, tileMem); break;
    }
    return;
  }
  const uint32_t key = (static_cast<uint32_t>(e.srcDtype) << 8) | e.dstDtype;
  constexpr uint32_t F32 = static_cast<uint32_t>(DType::kF32), BF = static_cast<uint32_t>(DType::kBF16),
                     F16 = static_cast<uint32_t>(DType::kF16);
  switch (key) {
    case (F32 << 8) | BF: stridedBandTilesTyped<float, __nv_bfloat16, true>(e, first, step, lane, tileMem); break;
    case (F32 << 8) | F16: stridedBandTilesTyped<float, __half, true>(e, first, step, lane, tileMem); break;
    case (BF << 8) | F32: stridedBandTilesTyped<__nv_bfloat16, float, true>(e, first, step, lane, tileMem); break;
    case (F16 << 8) | F32: stridedBandTilesTyped<__half, float, true>(e, first, step, lane, tileMem); break;
    case (BF << 8) | F16: stridedBandTilesTyped<__nv_bfloat16, __half, true>(e, first, step, lane, tileMem); break;
    case (F16 << 8) | BF: stridedBandTilesTyped<__half, __nv_bfloat16, true>(e, first, step, lane, tileMem); break;
    default: break;
  }
}

// Transposed matrix of 2-byte elements (rowStride == 1), with the source, the destination, both
// extents and the column stride all even: a warp moves a 64x64 tile, reading 32-bit words down the
// source columns (128 B per instruction instead of 64) and writing 32-bit words along the packed
// rows. Staged as tile[c][r] with an even pitch, so a word of two rows lands on an aligned word.
__device__ __forceinline__ void stridedWide16Tile(const StridedArgs& a, uint32_t localTile, int lane, uint8_t* tileMem) {
  constexpr int T = kWideTile, P = kWidePitch;
  const uint16_t* tile = reinterpret_cast<const uint16_t*>(tileMem);
  uint32_t* tileWords = reinterpret_cast<uint32_t*>(tileMem);
  const int64_t rows = a.rows, cols = a.cols, colStride = a.colStride;
  const uint16_t* src = static_cast<const uint16_t*>(a.src);
  uint16_t* dst = static_cast<uint16_t*>(a.dst);
  const uint32_t tilesPerRow = static_cast<uint32_t>((cols + T - 1) / T);
  const int64_t r0 = static_cast<int64_t>(localTile / tilesPerRow) * T;
  const int64_t c0 = static_cast<int64_t>(localTile % tilesPerRow) * T;
  const int nr = static_cast<int>(rows - r0 < T ? rows - r0 : T);  // even
  const int nc = static_cast<int>(cols - c0 < T ? cols - c0 : T);  // even
  constexpr int kBatch = 16;
  const uint16_t* colPtr = src + (r0 + 2 * lane) + c0 * colStride;
  uint32_t* rowPtr = reinterpret_cast<uint32_t*>(dst + r0 * cols + c0) + lane;
  const int64_t rowWords = cols / 2;
  const uint16_t* lo = tile + (2 * lane) * P;
  const uint16_t* hi = lo + P;
  if (nr == T && nc == T) {
    // Full tile: no predicates, constant trip counts.
#pragma unroll 1
    for (int c = 0; c < T; c += kBatch) {
      uint32_t v[kBatch];
#pragma unroll
      for (int k = 0; k < kBatch; ++k)
        if (TPB_DBG_SRC(a, colPtr + k * colStride, 4)) v[k] = *reinterpret_cast<const uint32_t*>(colPtr + k * colStride);
      colPtr += kBatch * colStride;
#pragma unroll
      for (int k = 0; k < kBatch; ++k) tileWords[(c + k) * (P / 2) + lane] = v[k];
    }
    __syncwarp();
#pragma unroll 1
    for (int r = 0; r < T; r += kBatch) {
      uint32_t v[kBatch];
#pragma unroll
      for (int k = 0; k < kBatch; ++k) v[k] = static_cast<uint32_t>(lo[r + k]) | (static_cast<uint32_t>(hi[r + k]) << 16);
#pragma unroll
      for (int k = 0; k < kBatch; ++k)
        if (TPB_DBG_DST(a, rowPtr + k * rowWords, 4)) rowPtr[k * rowWords] = v[k];
      rowPtr += kBatch * rowWords;
    }
    __syncwarp();
    return;
  }
  {
    const bool active = 2 * lane < nr;
    for (int c = 0; c < nc; c += kBatch) {
      uint32_t v[kBatch];
#pragma unroll
      for (int k = 0; k < kBatch; ++k)
        if (active && c + k < nc && TPB_DBG_SRC(a, colPtr + static_cast<int64_t>(c + k) * colStride, 4))
          v[k] = *reinterpret_cast<const uint32_t*>(colPtr + static_cast<int64_t>(c + k) * colStride);
#pragma unroll
      for (int k = 0; k < kBatch; ++k)
        if (active && c + k < nc) tileWords[(c + k) * (P / 2) + lane] = v[k];
    }
  }
  __syncwarp();
  {
    const bool active = 2 * lane < nc;
    for (int r = 0; r < nr; r += kBatch) {
      uint32_t v[kBatch];
#pragma unroll
      for (int k = 0; k < kBatch; ++k)
        if (active && r + k < nr) v[k] = static_cast<uint32_t>(lo[r + k]) | (static_cast<uint32_t>(hi[r + k]) << 16);
#pragma unroll
      for (int k = 0; k < kBatch; ++k)
        if (active && r + k < nr && TPB_DBG_DST(a, rowPtr + static_cast<int64_t>(r + k) * rowWords, 4))
          rowPtr[static_cast<int64_t>(r + k) * rowWords] = v[k];
    }
  }
  __syncwarp();
}

__device__ __noinline__ void stridedWide16Tiles(const PushEntry& e, uint32_t first, uint32_t step, int lane,
                                                uint8_t* tileMem) {
  const StridedArgs a = loadStridedArgs(e);
#pragma unroll 1
  for (uint32_t t = first; t < a.numTiles; t += step) stridedWide16Tile(a, t, lane, tileMem);
}

// Warp tiles t = firstWarp, firstWarp + totalWarps, ... of the plain class.
template <int N>
__device__ __forceinline__ void runPlainWarp(const PushParams<N>& p, uint32_t firstWarp, uint32_t totalWarps, int lane,
                                             uint8_t* tileMem) {
  uint32_t t = firstWarp;
  while (t < p.plainTiles) {
    const PushEntry* e = findEntry(p, t, false);
    const uint32_t local = t - e->tileStart;
    if (e->kind == kCopyPlain) {
      copyPlainTile(*e, local, lane);
      t += totalWarps;
    } else if (e->kind == kCastPlain) {
      castTile(*e, local, lane);
      t += totalWarps;
    } else {
      // One call handles every tile of this entry that falls to this warp.
      if (e->kind == kStridedWide16) stridedWide16Tiles(*e, local, totalWarps, lane, tileMem);
      else if (e->kind == kStridedNarrow) stridedNarrowTiles(*e, local, totalWarps, lane, tileMem);
      else if (e->kind == kStridedBand) stridedBandTiles(*e, local, totalWarps, lane, tileMem);
      else stridedTiles(*e, local, totalWarps, lane, tileMem);
      t += (e->numTiles - local + totalWarps - 1) / totalWarps * totalWarps;
    }
  }
}

// One lane polls, the CTA learns the outcome. Bounded by the timer and by an iteration cap.
template <int N>
__device__ __forceinline__ bool waitForProducer(const PushParams<N>& p) {
  if (p.waitFlag == nullptr) return true;
  bool arrived = true;
  if (threadIdx.x == 0) {
    arrived = false;
    const uint64_t start = globalTimerNs();
    uint32_t backoff = 32;
    for (uint64_t i = 0; i < (1ull << 32); ++i) {
      if (static_cast<int32_t>(loadAcquireSys(p.waitFlag) - p.waitValue) >= 0) {
        arrived = true;
        break;
      }
      if (globalTimerNs() - start > p.waitTimeoutNs) break;
      __nanosleep(backoff);
      if (backoff < 1024) backoff <<= 1;
    }
    if (!arrived) reportStatus(p.status, kStatusWaitTimeout);
  }
  return __syncthreads_and(arrived) != 0;
}

// Last step of every launch. A launch that gave up anywhere (a bulk load that never completed,
// a producer that never arrived) does NOT publish its flag: whoever waits for it runs into its
// own time limit instead of reading half-written data.
// Programmatic dependent launch: a push kernel lets the kernel queued behind it on the stream start
// right away (its own blocks are on the SMs within microseconds, so "when every block has got
// going" is the moment), and itself waits for the kernel before it only where it first touches
// memory that kernel may have written. Two pushes queued back to back thus overlap the launch
// latency and the prologue of the second with the tail of the first; a kernel that is not launched
// with the attribute (anything of the user's) is serialised as always.
__device__ __forceinline__ void letDependentsLaunch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void waitForEarlierKernels() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <int N>
__device__ __forceinline__ void publish(const PushParams<N>& p, bool failedHere) {
  if (p.lateTrigger) letDependentsLaunch();
  if (p.flag == nullptr && p.doneSlot == nullptr) return;
  // Make this thread's writes visible system-wide before the CTA reports in.
  __threadfence_system();
  const bool ctaFailed = __syncthreads_or(failedHere) != 0;
  if (threadIdx.x == 0) {
    bool last = true, anyFailed = ctaFailed;
    if (gridDim.x > 1) {
      const uint32_t mine = 1u + (ctaFailed ? kArriveFailed : 0u);
      const uint32_t before = atomicAdd(p.counter, mine);
      last = (before & kArriveMask) == gridDim.x - 1;
      anyFailed = ((before + mine) & ~kArriveMask) != 0;
      if (last) {
        *p.counter = 0;  // ready for the next launch that is given this counter
        __threadfence_system();
      }
    }
    // With one CTA the barrier above already ordered every write of the launch before this.
    if (last) {
      if (p.flag != nullptr && !anyFailed) storeReleaseSys(p.flag, p.flagValue);
      if (p.doneSlot != nullptr) {
        *reinterpret_cast<volatile uint32_t*>(p.doneSlot) = p.doneValue;
        __threadfence_system();
      }
    }
  }
}

// ---- the kernels --------------------------------------------------------------------------------
template <int N>
__global__ void __launch_bounds__(kThreads, 1) tpb_push_pack(const __grid_constant__ PushParams<N> p) {
  extern __shared__ uint8_t smemRaw[];
  // Layout: [bulk stages][warp tiles][mbarriers]; dynamic shared memory is only guaranteed to be
  // 16-byte aligned, the bulk stages want 128.
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 127) & ~static_cast<uintptr_t>(127));
  uint8_t* stages = base;
  uint8_t* warpTiles = base + static_cast<size_t>(p.bulkStages) * p.bulkTileBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(warpTiles + (kThreads / 32 - 1) * p.warpTileBytes);

  const int tid = threadIdx.x;
  const int S = static_cast<int>(p.bulkStages);
  const bool haveBulk = p.bulkTiles > blockIdx.x;
  bool failed = false;

  if (!p.lateTrigger) letDependentsLaunch();
  if (tid == 0 && haveBulk) {
    for (int s = 0; s < S; ++s) mbarInit(&full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  waitForEarlierKernels();  // from here on memory is read and written
  if (!waitForProducer(p)) {
    publish(p, true);
    return;
  }

  if (tid < 32) {
    // ---- warp 0: the bulk copy pipeline, driven by one elected lane ----
    if (tid == 0 && haveBulk) {
      const uint32_t first = blockIdx.x, step = gridDim.x;
      const uint32_t mine = (p.bulkTiles - first + step - 1) / step;  // tiles this CTA owns
      const uint32_t tileBytes = p.bulkTileBytes;
#ifdef TPB_DEBUG_KERNELS
      // A bulk copy off the 16-byte grid is an illegal instruction: check the whole table first
      // and leave the pipeline alone if any entry is wrong.
      bool tableOk = true;
      for (uint32_t i = 0; i < p.numEntries; ++i) {
        const PushEntry& e = p.entries[i];
        if (e.kind != kCopyBulk) continue;
        if ((reinterpret_cast<uintptr_t>(e.src) | reinterpret_cast<uintptr_t>(e.dst) | e.count) & 15) {
          atomicAdd(&gBoundsViolations, 1ull);
          tableOk = false;
        }
      }
#else
      constexpr bool tableOk = true;
#endif
      auto describe = [&](uint32_t i, const uint8_t*& src, uint8_t*& dst, uint32_t& bytes) {
        const uint32_t t = first + i * step;
        const PushEntry* e = findEntry(p, t, true);
        const uint64_t off = static_cast<uint64_t>(t - e->tileStart) * tileBytes;
        const uint64_t left = e->count - off;
        bytes = left < tileBytes ? static_cast<uint32_t>(left) : tileBytes;
        src = static_cast<const uint8_t*>(e->src) + off;
        dst = static_cast<uint8_t*>(e->dst) + off;
      };
      auto issueLoad = [&](uint32_t i) {
        const uint8_t* src;
        uint8_t* dst;
        uint32_t bytes;
        describe(i, src, dst, bytes);
        const int s = i % S;
        mbarExpectTx(&full[s], bytes);
        bulkLoad(stages + static_cast<size_t>(s) * tileBytes, src, bytes, &full[s]);
      };
      const uint32_t prologue = !tableOk ? 0 : mine < static_cast<uint32_t>(S) ? mine : S;
      for (uint32_t i = 0; i < prologue; ++i) issueLoad(i);
      for (uint32_t c = 0; tableOk && c < mine; ++c) {
        const int s = c % S;
        if (!mbarWaitBounded(&full[s], (c / S) & 1)) {
          failed = true;
          break;
        }
        const uint8_t* src;
        uint8_t* dst;
        uint32_t bytes;
        describe(c, src, dst, bytes);
        fenceProxyAsync();
        bulkStore(dst, stages + static_cast<size_t>(s) * tileBytes, bytes);
        bulkCommit();
        // Refill the stage whose store was issued one iteration ago: by now it has most likely
        // finished reading shared memory, so this wait rarely stalls the pipeline.
        if (c >= 1 && (c - 1) + S < mine) {
          bulkWaitRead<1>();
          issueLoad((c - 1) + S);
        }
      }
      bulkWaitAll();  // stores are complete (not merely read out of shared memory)
      if (failed) reportStatus(p.status, kStatusBarrierTimeout);
    }
  } else {
    // ---- warps 1..: everything that needs registers ----
    constexpr uint32_t kPlainWarps = kThreads / 32 - 1;
    const uint32_t warp = tid / 32 - 1;
    runPlainWarp(p, blockIdx.x * kPlainWarps + warp, gridDim.x * kPlainWarps, tid & 31,
                 warpTiles + warp * p.warpTileBytes);
  }
  publish(p, failed);
}

template <int N>
__global__ void __launch_bounds__(kLightThreads, 2) tpb_push_pack_light(const __grid_constant__ PushParams<N> p) {
  extern __shared__ __align__(16) uint8_t lightTiles[];  // kWarps * p.warpTileBytes, none for plain copies
  constexpr uint32_t kWarps = kLightThreads / 32;
  const uint32_t warp = threadIdx.x / 32;
  if (!p.lateTrigger) letDependentsLaunch();
  waitForEarlierKernels();
  if (!waitForProducer(p)) {
    publish(p, true);
    return;
  }
  runPlainWarp(p, blockIdx.x * kWarps + warp, gridDim.x * kWarps, threadIdx.x & 31, lightTiles + warp * p.warpTileBytes);
  publish(p, false);
}

__global__ void tpb_wait_flag(const uint32_t* flag, uint32_t value, uint64_t timeoutNs, uint32_t* status) {
  if (threadIdx.x != 0) return;
  const uint64_t start = globalTimerNs();
  uint32_t backoff = 32;
  // Both limits bound the loop: the timer deadline and an iteration cap.
  for (uint64_t i = 0; i < (1ull << 32); ++i) {
    const uint32_t v = loadAcquireSys(flag);
    if (static_cast<int32_t>(v - value) >= 0) return;
    if (globalTimerNs() - start > timeoutNs) break;
    __nanosleep(backoff);
    if (backoff < 1024) backoff <<= 1;
  }
  // Only a failure is written: the word is shared with other waits and an earlier failure must
  // not be wiped out by a later success.
  reportStatus(status, kStatusWaitTimeout);
}

__global__ void tpb_delay(uint32_t* buf, size_t words, uint64_t ns) {
  const uint64_t start = globalTimerNs();
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  // Bounded by the deadline and by an iteration cap.
  for (uint32_t it = 0; it < (1u << 24); ++it) {
    for (size_t i = blockIdx.x * blockDim.x + threadIdx.x; i < words; i += stride) buf[i] = buf[i] * 1664525u + it;
    if (globalTimerNs() - start > ns) break;
    __nanosleep(1000);
  }
}

__host__ __device__ __forceinline__ uint32_t patternWord(uint64_t seed, uint64_t wordIndex) {
  // splitmix-style hash: cheap, seedable, identical on host and device
  uint64_t z = seed + (wordIndex + 1) * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return static_cast<uint32_t>(z ^ (z >> 31));
}

__global__ void tpb_fill(uint8_t* buf, size_t bytes, uint64_t seed) {
  const size_t words = bytes / 4;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  uint32_t* w = reinterpret_cast<uint32_t*>(buf);
  for (size_t i = blockIdx.x * blockDim.x + threadIdx.x; i < words; i += stride) w[i] = patternWord(seed, i);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (size_t b = words * 4; b < bytes; ++b) buf[b] = static_cast<uint8_t>(patternWord(seed, words) >> (8 * (b & 3)));
  }
}

__global__ void tpb_verify(const uint8_t* buf, size_t bytes, uint64_t seed, unsigned long long* mismatches) {
  const size_t words = bytes / 4;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const uint32_t* w = reinterpret_cast<const uint32_t*>(buf);
  unsigned long long bad = 0;
  for (size_t i = blockIdx.x * blockDim.x + threadIdx.x; i < words; i += stride) {
    const uint32_t x = w[i] ^ patternWord(seed, i);
    if (x) bad += ((x & 0xff) != 0) + ((x & 0xff00) != 0) + ((x & 0xff0000) != 0) + ((x & 0xff000000u) != 0);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (size_t b = words * 4; b < bytes; ++b)
      bad += buf[b] != static_cast<uint8_t>(patternWord(seed, words) >> (8 * (b & 3)));
  }
  if (bad) atomicAdd(mismatches, bad);
}

void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

// Launches with the programmatic-stream-serialization attribute (see letDependentsLaunch) where
// that pays: small launches that publish or await a flag, i.e. the eager pushes and unpacks
// between processes, which follow each other on a stream with no other work in between (measured
// across two GPUs: 9.1-10.9 us per message instead of 10.8-12.9 from 4 to 64 KiB; from 128 KiB
// to 4 MiB the attribute cost 2 us per message, beyond that it made no difference).
// TPB_PUSH_PDL=0 turns it off.
constexpr uint64_t kDependentLaunchMaxBytes = 64 * 1024;
// Larger launches up to TPB_PUSH_PDL_LATE_MAX_BYTES (default 0: none) are launched as dependents
// too, but let their own dependents go only when their work has been issued.
uint64_t lateDependentMaxBytes() {
  static const uint64_t v = [] {
    const char* e = std::getenv("TPB_PUSH_PDL_LATE_MAX_BYTES");
    return e && *e ? std::strtoull(e, nullptr, 0) : 0ull;
  }();
  return v;
}
bool programmaticLaunches() {
  static const bool on = [] {
    const char* e = std::getenv("TPB_PUSH_PDL");
    return !(e && e[0] == '0' && e[1] == 0);
  }();
  return on;
}

template <typename Kernel, typename Params>
void launchMaybeDependent(Kernel kernel, uint32_t grid, uint32_t threads, size_t smem, cudaStream_t stream, const Params& p,
                          bool dependent) {
  if (!dependent || !programmaticLaunches()) {
    kernel<<<grid, threads, smem, stream>>>(p);
    return;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, p);
}

template <int N>
void launchOne(const PushEntry* entries, uint32_t n, uint32_t bulkTiles, uint32_t plainTiles, uint32_t bulkTileBytes,
               uint32_t bulkStages, cudaStream_t stream, int maxCtas, uint32_t* flag, uint32_t flagValue,
               uint32_t* counter, uint32_t* status, const WaitBefore& wait, const DoneSlot& done, uint64_t bytesOut) {
  const bool publishes = flag != nullptr || wait.flag != nullptr || done.slot != nullptr;
  const bool early = bytesOut <= kDependentLaunchMaxBytes;
  const bool dependent = publishes && (early || bytesOut <= lateDependentMaxBytes());
  PushParams<N> p;
  p.lateTrigger = early ? 0 : 1;
  for (uint32_t i = 0; i < n; ++i) p.entries[i] = entries[i];
  p.numEntries = n;
  p.bulkTiles = bulkTiles;
  p.plainTiles = plainTiles;
  p.flagValue = flagValue;
  p.flag = flag;
  p.counter = counter;
  p.status = status;
  p.waitFlag = wait.flag;
  p.waitValue = wait.value;
  p.waitTimeoutNs = wait.timeoutNs;
  p.doneSlot = done.slot;
  p.doneValue = done.value;
  p.bulkTileBytes = bulkTileBytes;
  p.bulkStages = bulkStages;
  p.warpTileBytes = 0;
  for (uint32_t i = 0; i < n; ++i) {
    const uint32_t need = entries[i].kind == kStridedWide16 || entries[i].kind == kStridedNarrow ||
            entries[i].kind == kStridedBand
        ? kWideWarpTileBytes
        : entries[i].kind == kStrided                                                            ? kWarpTileBytes
                                                                                                 : 0;
    if (need > p.warpTileBytes) p.warpTileBytes = need;
  }
  int dev = 0;
  check(cudaGetDevice(&dev), "cudaGetDevice");
  if (bulkTiles == 0) {
    // Light kernel: 8 warps per CTA, shared memory only when an entry is staged through it.
    constexpr uint32_t kWarps = kLightThreads / 32;
    uint32_t grid = (plainTiles + kWarps - 1) / kWarps;
    if (grid > static_cast<uint32_t>(maxCtas) * 2) grid = static_cast<uint32_t>(maxCtas) * 2;
    if (grid == 0) grid = 1;
    const size_t lightSmem = static_cast<size_t>(kWarps) * p.warpTileBytes;
    static size_t lightConfigured[64] = {};
    if (lightSmem > 48 * 1024 && dev < 64 && lightConfigured[dev] < lightSmem) {
      check(cudaFuncSetAttribute(tpb_push_pack_light<N>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(lightSmem)),
            "cudaFuncSetAttribute");
      lightConfigured[dev] = lightSmem;
    }
    launchMaybeDependent(tpb_push_pack_light<N>, grid, kLightThreads, lightSmem, stream, p, dependent);
    check(cudaGetLastError(), "tpb_push_pack_light launch");
    ++gLaunches;
    return;
  }
  const size_t smem = static_cast<size_t>(bulkStages) * bulkTileBytes + (kThreads / 32 - 1) * p.warpTileBytes +
      kMaxBulkStages * sizeof(uint64_t) + 128;
  if (smem > kMaxSmemPerCta) throw std::runtime_error("push plan needs more shared memory than a CTA has");
  static size_t configured[64] = {};
  if (dev < 64 && configured[dev] < smem) {
    check(cudaFuncSetAttribute(tpb_push_pack<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)),
          "cudaFuncSetAttribute");
    configured[dev] = smem;
  }
  constexpr uint32_t kPlainWarps = kThreads / 32 - 1;
  uint32_t want = bulkTiles;
  const uint32_t plainCtas = (plainTiles + kPlainWarps - 1) / kPlainWarps;
  if (plainCtas > want) want = plainCtas;
  uint32_t grid = want < static_cast<uint32_t>(maxCtas) ? want : static_cast<uint32_t>(maxCtas);
  if (grid == 0) grid = 1;
  launchMaybeDependent(tpb_push_pack<N>, grid, kThreads, smem, stream, p, dependent);
  check(cudaGetLastError(), "tpb_push_pack launch");
  ++gLaunches;
}

}  // namespace

void setPushTuning(const PushTuning& t) {
  if (t.bulkStages < 2 || t.bulkStages > static_cast<uint32_t>(kMaxBulkStages) || t.bulkTileBytes % 1024 != 0 ||
      t.bulkTileBytes == 0 || static_cast<size_t>(t.bulkStages) * t.bulkTileBytes > 160 * 1024)
    throw std::runtime_error("invalid bulk pipeline tuning");
  std::unique_lock<std::mutex> l(gTuningMutex);
  gTuning = t;
}
PushTuning getPushTuning() {
  std::unique_lock<std::mutex> l(gTuningMutex);
  return gTuning;
}

// ---- host-side planning -------------------------------------------------------------------------
bool castSupported(DType s, DType d) {
  auto isFloat = [](DType t) { return t == DType::kF32 || t == DType::kBF16 || t == DType::kF16; };
  return s == d || (isFloat(s) && isFloat(d));
}

uint64_t convertedBytes(uint64_t srcBytes, DType s, DType d) {
  if (s == d || d == DType::kBytes) return srcBytes;
  return srcBytes / dtypeSize(s) * dtypeSize(d);
}

namespace {
void pushEntry(PushPlan& plan, PushEntry e) {
  if (e.count == 0) return;
  if (e.kind == kCopyBulk) {
    e.numTiles = static_cast<uint32_t>((e.count + plan.bulkTileBytes - 1) / plan.bulkTileBytes);
    e.tileStart = plan.bulkTiles;
    plan.bulkTiles += e.numTiles;
  } else if (e.kind == kCopyPlain) {
    e.numTiles = static_cast<uint32_t>((e.count + kPlainTileBytes - 1) / kPlainTileBytes);
    e.tileStart = plan.plainTiles;
    plan.plainTiles += e.numTiles;
  } else if (e.kind == kCastPlain) {
    const uint64_t perTile = kPlainTileBytes / e.dstElemSize;
    e.numTiles = static_cast<uint32_t>((e.count + perTile - 1) / perTile);
    e.tileStart = plan.plainTiles;
    plan.plainTiles += e.numTiles;
  } else if (e.kind == kStridedBand) {
    const uint32_t perBand = bandRows(static_cast<uint64_t>(e.cols), e.dstElemSize);
    e.numTiles = static_cast<uint32_t>((e.rows + perBand - 1) / perBand);
    e.tileStart = plan.plainTiles;
    plan.plainTiles += e.numTiles;
  } else if (e.kind == kStridedNarrow) {
    e.numTiles = static_cast<uint32_t>((e.rows + kStridedTile - 1) / kStridedTile);
    e.tileStart = plan.plainTiles;
    plan.plainTiles += e.numTiles;
  } else if (e.kind == kStridedWide16) {
    const uint64_t tr = (e.rows + kWideTile - 1) / kWideTile, tc = (e.cols + kWideTile - 1) / kWideTile;
    e.numTiles = static_cast<uint32_t>(tr * tc);
    e.tileStart = plan.plainTiles;
    plan.plainTiles += e.numTiles;
  } else {
    const int tileRows = e.srcElemSize == 8 ? kStridedTile / 2 : kStridedTile;
    const uint64_t tr = (e.rows + tileRows - 1) / tileRows, tc = (e.cols + kStridedTile - 1) / kStridedTile;
    e.numTiles = static_cast<uint32_t>(tr * tc);
    e.tileStart = plan.plainTiles;
    plan.plainTiles += e.numTiles;
  }
  plan.entries.push_back(e);
}
}  // namespace

void chooseBulkTile(PushPlan& plan, uint64_t bulkBytes, int ctas) {
  const PushTuning t = getPushTuning();
  plan.bulkStages = t.bulkStages;
  plan.bulkTileBytes = t.bulkTileBytes;
  if (!plan.entries.empty() || bulkBytes == 0 || ctas <= 0) return;
  const uint64_t perWave = static_cast<uint64_t>(ctas) * t.bulkTileBytes;
  const uint64_t waves = (bulkBytes + perWave - 1) / perWave;
  uint64_t tile = (bulkBytes + waves * ctas - 1) / (waves * ctas);
  tile = (tile + 1023) / 1024 * 1024;
  if (tile < 4096) tile = 4096;
  if (tile > t.bulkTileBytes) tile = t.bulkTileBytes;
  plan.bulkTileBytes = static_cast<uint32_t>(tile);
}

void appendToPlan(PushPlan& plan, const CopyItem& item, bool useBulk) {
  if (plan.bulkTileBytes == 0) {
    const PushTuning t = getPushTuning();
    plan.bulkTileBytes = t.bulkTileBytes;
    plan.bulkStages = t.bulkStages;
  }
  PushEntry e{};
  e.srcDtype = static_cast<uint8_t>(item.srcDtype);
  const DType dstDtype = item.dstDtype == DType::kBytes ? item.srcDtype : item.dstDtype;
  e.dstDtype = static_cast<uint8_t>(dstDtype);
  e.srcElemSize = static_cast<uint8_t>(dtypeSize(item.srcDtype));
  e.dstElemSize = static_cast<uint8_t>(dtypeSize(dstDtype));
  const bool convert = dstDtype != item.srcDtype;
  if (convert && !castSupported(item.srcDtype, dstDtype)) throw std::runtime_error("unsupported dtype conversion");
  plan.totalBytesOut += convertedBytes(item.srcBytes, item.srcDtype, dstDtype);

  if (item.strided) {
    const StridedView& v = item.view;
    if (static_cast<uint64_t>(v.rows) * v.cols * dtypeSize(v.dtype) != item.srcBytes)
      throw std::runtime_error("strided view does not match the tensor length");
    e.srcDtype = static_cast<uint8_t>(v.dtype);
    e.srcElemSize = static_cast<uint8_t>(dtypeSize(v.dtype));
    if (!convert) {
      e.dstDtype = e.srcDtype;
      e.dstElemSize = e.srcElemSize;
    }
    e.src = item.src;
    e.dst = item.dst;
    e.kind = kStrided;
    {
      // The word-wide variant needs even everything; it also needs its larger staging area to fit
      // next to the bulk stages this plan was sized with.
      const uintptr_t both = reinterpret_cast<uintptr_t>(item.src) | reinterpret_cast<uintptr_t>(item.dst);
      const size_t smemWithWide = static_cast<size_t>(plan.bulkStages) * plan.bulkTileBytes +
          (kThreads / 32 - 1) * kWideWarpTileBytes + kMaxBulkStages * sizeof(uint64_t) + 128;
      if (!convert && e.srcElemSize == 2 && v.rowStride == 1 && v.colStride != 1 && v.rows >= kWideTile &&
          v.cols >= kWideTile && v.rows % 2 == 0 && v.cols % 2 == 0 && v.colStride % 2 == 0 && (both & 3) == 0 &&
          smemWithWide <= kMaxSmemPerCta)
        e.kind = kStridedWide16;
      // Few columns: whole packed rows per tile, written as one contiguous run (wins over the above).
      const uint64_t dstRowBytes = static_cast<uint64_t>(v.cols) * e.dstElemSize;
      const uint32_t narrowRows = getPushTuning().narrowRows;
      if ((narrowRows == 2 || (narrowRows == 1 && item.remote)) && v.rowStride == 1 && v.colStride != 1 &&
          v.cols <= kNarrowMaxCols && e.srcElemSize <= 4 && e.dstElemSize <= 4 &&
          dstRowBytes % 16 == 0 && (reinterpret_cast<uintptr_t>(item.dst) & 15) == 0 && v.rows > 1 &&
          smemWithWide <= kMaxSmemPerCta)
        e.kind = kStridedNarrow;
      // Any other transposed matrix with rows of at most 8 KiB: bands of whole rows, each written
      // as one contiguous run whatever its alignment.
      const uint32_t bands = getPushTuning().bandRows;
      if (e.kind != kStridedNarrow && (bands == 2 || (bands == 1 && item.remote)) && v.rowStride == 1 &&
          v.colStride != 1 && v.rows > 1 && dstRowBytes <= kBandBytes && smemWithWide <= kMaxSmemPerCta)
        e.kind = kStridedBand;
    }
    e.rows = v.rows;
    e.cols = v.cols;
    e.rowStride = v.rowStride;
    e.colStride = v.colStride;
    e.count = static_cast<uint64_t>(v.rows) * v.cols;
    pushEntry(plan, e);
    return;
  }
  if (convert) {
    e.src = item.src;
    e.dst = item.dst;
    e.kind = kCastPlain;
    e.count = item.srcBytes / dtypeSize(item.srcDtype);
    pushEntry(plan, e);
    return;
  }
  // Contiguous copy: aligned body on the bulk path, ragged head and tail on the plain path.
  const uint8_t* src = static_cast<const uint8_t*>(item.src);
  uint8_t* dst = static_cast<uint8_t*>(item.dst);
  uint64_t bytes = item.srcBytes;
  const uintptr_t sa = reinterpret_cast<uintptr_t>(src), da = reinterpret_cast<uintptr_t>(dst);
  const bool sameSkew = ((sa ^ da) & 15) == 0;
  if (useBulk && sameSkew && bytes >= getPushTuning().bulkMinBytes) {
    // Bulk (TMA) loads read the launching GPU's own memory only. Whatever the caller asked for, a
    // source that the driver places on another GPU or in host memory goes through plain loads.
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess) {
      cudaGetLastError();
      device = -1;
    }
    if (device >= 0 && cudaIsForeignMemory(src, device)) useBulk = false;
  }
  if (!useBulk || !sameSkew || bytes < getPushTuning().bulkMinBytes) {
    e.src = src;
    e.dst = dst;
    e.kind = kCopyPlain;
    e.count = bytes;
    pushEntry(plan, e);
    return;
  }
  const uint64_t head = (16 - (sa & 15)) & 15;
  if (head) {
    PushEntry h = e;
    h.src = src;
    h.dst = dst;
    h.kind = kCopyPlain;
    h.count = head;
    pushEntry(plan, h);
    src += head;
    dst += head;
    bytes -= head;
  }
  const uint64_t body = bytes & ~static_cast<uint64_t>(15);
  PushEntry b = e;
  b.src = src;
  b.dst = dst;
  b.kind = kCopyBulk;
  b.count = body;
  pushEntry(plan, b);
  if (bytes - body) {
    PushEntry t = e;
    t.src = src + body;
    t.dst = dst + body;
    t.kind = kCopyPlain;
    t.count = bytes - body;
    pushEntry(plan, t);
  }
}

int launchPush(const PushPlan& plan, cudaStream_t stream, int maxCtas, uint32_t* flag, uint32_t flagValue,
               uint32_t* counter, uint32_t* status, WaitBefore wait, DoneSlot done) {
  if ((flag != nullptr || done.slot != nullptr) && counter == nullptr && maxCtas > 1)
    throw std::runtime_error("a launch that publishes a flag or a completion word from several CTAs needs an arrive counter");
  const size_t n = plan.entries.size();
  trace::Scope traced("tpb_push_pack launch", plan.totalBytesOut);
  if (maxCtas <= 0) maxCtas = 1;
  const uint32_t tileBytes = plan.bulkTileBytes ? plan.bulkTileBytes : 32768;
  const uint32_t stages = plan.bulkStages ? plan.bulkStages : 4;
  if (n <= static_cast<size_t>(kMaxEntriesLarge)) {
    if (n <= static_cast<size_t>(kMaxEntriesSmall))
      launchOne<kMaxEntriesSmall>(plan.entries.data(), static_cast<uint32_t>(n), plan.bulkTiles, plan.plainTiles,
                                  tileBytes, stages, stream, maxCtas, flag, flagValue, counter, status, wait, done,
                                  plan.totalBytesOut);
    else
      launchOne<kMaxEntriesLarge>(plan.entries.data(), static_cast<uint32_t>(n), plan.bulkTiles, plan.plainTiles,
                                  tileBytes, stages, stream, maxCtas, flag, flagValue, counter, status, wait, done,
                                  plan.totalBytesOut);
    return 1;
  }
  // More entries than one parameter block holds: several launches on the same stream, each with
  // its own tile numbering; only the last publishes the flag (stream order covers the others).
  int launches = 0;
  for (size_t first = 0; first < n; first += kMaxEntriesLarge) {
    const size_t cnt = n - first < static_cast<size_t>(kMaxEntriesLarge) ? n - first : kMaxEntriesLarge;
    std::vector<PushEntry> part(plan.entries.begin() + first, plan.entries.begin() + first + cnt);
    uint32_t bulk = 0, plain = 0;
    for (auto& e : part) {
      if (e.kind == kCopyBulk) {
        e.tileStart = bulk;
        bulk += e.numTiles;
      } else {
        e.tileStart = plain;
        plain += e.numTiles;
      }
    }
    const bool last = first + cnt == n;
    // Only the first launch waits for the producer; stream order covers the rest.
    launchOne<kMaxEntriesLarge>(part.data(), static_cast<uint32_t>(cnt), bulk, plain, tileBytes, stages, stream,
                                maxCtas, last ? flag : nullptr, flagValue, counter, status,
                                first == 0 ? wait : WaitBefore(), last ? done : DoneSlot(), plan.totalBytesOut);
    ++launches;
  }
  return launches;
}

void launchWaitFlag(cudaStream_t stream, const uint32_t* flag, uint32_t value, uint64_t timeoutNs, uint32_t* status) {
  tpb_wait_flag<<<1, 32, 0, stream>>>(flag, value, timeoutNs, status);
  check(cudaGetLastError(), "tpb_wait_flag launch");
  ++gLaunches;
}

void launchDelay(cudaStream_t stream, void* buf, size_t bytes, uint32_t microseconds) {
  uint64_t ns = static_cast<uint64_t>(microseconds) * 1000;
  if (ns > 2'000'000'000ull) ns = 2'000'000'000ull;
  tpb_delay<<<8, 128, 0, stream>>>(static_cast<uint32_t*>(buf), bytes / 4, ns);
  check(cudaGetLastError(), "tpb_delay launch");
  ++gLaunches;
}

void launchFill(cudaStream_t stream, void* buf, size_t bytes, uint64_t seed) {
  if (bytes == 0) return;
  size_t blocks = (bytes / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks == 0) blocks = 1;
  tpb_fill<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<uint8_t*>(buf), bytes, seed);
  check(cudaGetLastError(), "tpb_fill launch");
  ++gLaunches;
}

void launchVerify(cudaStream_t stream, const void* buf, size_t bytes, uint64_t seed, unsigned long long* mismatches) {
  if (bytes == 0) return;
  size_t blocks = (bytes / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks == 0) blocks = 1;
  tpb_verify<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<const uint8_t*>(buf), bytes, seed,
                                                                mismatches);
  check(cudaGetLastError(), "tpb_verify launch");
  ++gLaunches;
}

uint8_t patternByte(uint64_t seed, uint64_t index) {
  return static_cast<uint8_t>(patternWord(seed, index / 4) >> (8 * (index & 3)));
}

uint64_t launchCount() { return gLaunches.load(); }

bool debugKernels() {
#ifdef TPB_DEBUG_KERNELS
  return true;
#else
  return false;
#endif
}

uint64_t boundsViolations() {
#ifdef TPB_DEBUG_KERNELS
  // Summed over the devices this process has a context on (and only those: asking a device
  // without one would create it).
  unsigned long long total = 0;
  const int n = cudaDeviceCountNoThrow();
  for (int d = 0; d < n; ++d) {
    if (cudaPrimaryContextActive(d) != 1) continue;
    CudaDeviceGuard g(d);
    unsigned long long v = 0;
    check(cudaMemcpyFromSymbol(&v, gBoundsViolations, sizeof(v)), "reading the violation counter");
    total += v;
  }
  return total;
#else
  return 0;
#endif
}

}  // namespace kernels
}  // namespace tpb
