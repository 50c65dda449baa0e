// sm_100a kernels of the device-to-device channel. See push.h for the interface.
//
// tpb_push_pack is ONE persistent launch (at most one CTA per SM) that serves a whole message:
//
//   * Warp 0 is a copy engine. Its elected lane drives a 4-stage pipeline of TMA bulk copies:
//     global -> shared (completion on an mbarrier) and shared -> global (bulk groups), 32 KiB
//     per stage, for every entry whose source, destination and size are 16-byte multiples.
//     The loads only ever read THIS GPU's memory; the stores may target a peer GPU's memory
//     mapped over NVLink. No thread touches the bytes.
//   * Warps 1..15 handle what the bulk path cannot: ragged heads and tails, relatively
//     misaligned buffers, dtype conversion (fp32 <-> bf16/fp16) and 2-D strided sources, which
//     go through a padded shared-memory tile so that both the strided reads and the packed
//     writes are coalesced.
//   * Tiles are dealt round-robin to CTAs (tile t belongs to CTA t mod gridDim.x), so no
//     scheduling state lives in global memory.
//   * Completion: every CTA makes its writes visible system-wide, then arrives on a counter;
//     the last CTA resets the counter and publishes the flag with a release store at system
//     scope. The flag lives in the receiver's memory; its stream waits on it.
//
// Every wait in here is bounded: a bulk load that does not complete within the limit makes the
// CTA record kStatusBarrierTimeout, drain its own outstanding stores and fall through to the
// completion protocol, so the kernel always terminates.
#include "kernels/push.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <stdexcept>
#include <string>

namespace tpb {
namespace kernels {

namespace {

std::atomic<uint64_t> gLaunches{0};

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
__device__ __forceinline__ void plainBarrier(int nthreads) {
  asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}

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
};

struct SharedStorage {
  alignas(128) uint8_t stages[kBulkStages][kBulkTileBytes];
  alignas(16) uint8_t tile[kStridedTile * (kStridedTile + 1) * 8];
  alignas(8) uint64_t full[kBulkStages];
};

template <int N>
__device__ __forceinline__ const PushEntry* findEntry(const PushParams<N>& p, uint32_t tile, bool bulk) {
  // Entries of one class have increasing tileStart; a linear scan over <=96 entries in the
  // constant bank costs less than the tile it locates.
  const PushEntry* found = nullptr;
  for (uint32_t i = 0; i < p.numEntries; ++i) {
    const PushEntry& e = p.entries[i];
    bool isBulk = e.kind == kCopyBulk;
    if (isBulk != bulk) continue;
    if (tile >= e.tileStart && tile < e.tileStart + e.numTiles) {
      found = &e;
      break;
    }
  }
  return found;
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

// ---- plain contiguous copy ----------------------------------------------------------------------
template <typename V>
__device__ __forceinline__ void copyVec(const uint8_t* src, uint8_t* dst, uint64_t bytes, int tid, int nthr) {
  const V* s = reinterpret_cast<const V*>(src);
  V* d = reinterpret_cast<V*>(dst);
  const uint64_t n = bytes / sizeof(V);
  constexpr int kUnroll = 8;
  uint64_t i = tid;
  // Issue kUnroll independent loads before the first store: bytes in flight, not instructions,
  // are what fills an NVLink or HBM pipe.
  for (; i + static_cast<uint64_t>(kUnroll - 1) * nthr < n; i += static_cast<uint64_t>(kUnroll) * nthr) {
    V r[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) r[u] = s[i + static_cast<uint64_t>(u) * nthr];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) d[i + static_cast<uint64_t>(u) * nthr] = r[u];
  }
  for (; i < n; i += nthr) d[i] = s[i];
  // Trailing bytes that do not fill a vector.
  const uint64_t done = n * sizeof(V);
  for (uint64_t b = done + tid; b < bytes; b += nthr) dst[b] = src[b];
}

__device__ __forceinline__ void copyPlainTile(const PushEntry& e, uint32_t localTile, int tid, int nthr) {
  const uint64_t off = static_cast<uint64_t>(localTile) * kPlainTileBytes;
  uint64_t bytes = e.count - off;
  if (bytes > kPlainTileBytes) bytes = kPlainTileBytes;
  const uint8_t* src = static_cast<const uint8_t*>(e.src) + off;
  uint8_t* dst = static_cast<uint8_t*>(e.dst) + off;
  const uintptr_t a = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst);
  if ((a & 15) == 0) copyVec<uint4>(src, dst, bytes, tid, nthr);
  else if ((a & 7) == 0) copyVec<uint2>(src, dst, bytes, tid, nthr);
  else if ((a & 3) == 0) copyVec<uint32_t>(src, dst, bytes, tid, nthr);
  else if ((a & 1) == 0) copyVec<uint16_t>(src, dst, bytes, tid, nthr);
  else copyVec<uint8_t>(src, dst, bytes, tid, nthr);
}

// ---- contiguous conversion ----------------------------------------------------------------------
template <typename S, typename D>
__device__ __forceinline__ void castTileTyped(const PushEntry& e, uint32_t localTile, int tid, int nthr) {
  // A tile is kPlainTileBytes of DESTINATION bytes.
  const uint64_t perTile = kPlainTileBytes / sizeof(D);
  const uint64_t first = static_cast<uint64_t>(localTile) * perTile;
  uint64_t n = e.count - first;
  if (n > perTile) n = perTile;
  const S* s = static_cast<const S*>(e.src) + first;
  D* d = static_cast<D*>(e.dst) + first;
  constexpr int kVec = 16 / sizeof(D) < 16 / sizeof(S) ? 16 / sizeof(S) : 16 / sizeof(D);  // elems per step
  const bool aligned = ((reinterpret_cast<uintptr_t>(s) & 15) == 0) && ((reinterpret_cast<uintptr_t>(d) & 15) == 0);
  uint64_t vecElems = aligned ? (n / kVec) * kVec : 0;
  for (uint64_t i = static_cast<uint64_t>(tid) * kVec; i < vecElems; i += static_cast<uint64_t>(nthr) * kVec) {
    alignas(16) S in[kVec];
    alignas(16) D out[kVec];
    constexpr int kInVecs = kVec * sizeof(S) / 16;
    constexpr int kOutVecs = (kVec * sizeof(D) + 15) / 16;
#pragma unroll
    for (int v = 0; v < kInVecs; ++v)
      reinterpret_cast<uint4*>(in)[v] = reinterpret_cast<const uint4*>(s + i)[v];
#pragma unroll
    for (int k = 0; k < kVec; ++k) out[k] = fromFloat<D>(toFloat<S>(in[k]));
    if (kVec * sizeof(D) >= 16) {
#pragma unroll
      for (int v = 0; v < kOutVecs; ++v) reinterpret_cast<uint4*>(d + i)[v] = reinterpret_cast<uint4*>(out)[v];
    } else {
      *reinterpret_cast<uint2*>(d + i) = *reinterpret_cast<uint2*>(out);
    }
  }
  for (uint64_t i = vecElems + tid; i < n; i += nthr) d[i] = fromFloat<D>(toFloat<S>(s[i]));
}

__device__ __forceinline__ void castTile(const PushEntry& e, uint32_t localTile, int tid, int nthr) {
  const uint32_t key = (static_cast<uint32_t>(e.srcDtype) << 8) | e.dstDtype;
  constexpr uint32_t F32 = static_cast<uint32_t>(DType::kF32), BF = static_cast<uint32_t>(DType::kBF16),
                     F16 = static_cast<uint32_t>(DType::kF16);
  switch (key) {
    case (F32 << 8) | BF: castTileTyped<float, __nv_bfloat16>(e, localTile, tid, nthr); break;
    case (F32 << 8) | F16: castTileTyped<float, __half>(e, localTile, tid, nthr); break;
    case (BF << 8) | F32: castTileTyped<__nv_bfloat16, float>(e, localTile, tid, nthr); break;
    case (F16 << 8) | F32: castTileTyped<__half, float>(e, localTile, tid, nthr); break;
    case (BF << 8) | F16: castTileTyped<__nv_bfloat16, __half>(e, localTile, tid, nthr); break;
    case (F16 << 8) | BF: castTileTyped<__half, __nv_bfloat16>(e, localTile, tid, nthr); break;
    default: break;  // rejected on the host
  }
}

// ---- 2-D strided source through a shared-memory tile ----------------------------------------------
// The tile is staged as raw source elements: smem[c][r] when the source is contiguous along rows
// (a transposed matrix), smem[r][c] otherwise. Writes are always coalesced along dst columns.
template <typename S, typename D, bool kConvert>
__device__ __forceinline__ void stridedTileTyped(const PushEntry& e, uint32_t localTile, int tid, int nthr,
                                                 uint8_t* tileMem) {
  constexpr int T = kStridedTile;
  S* tile = reinterpret_cast<S*>(tileMem);
  const int64_t tilesPerRow = (e.cols + T - 1) / T;
  const int64_t r0 = (localTile / tilesPerRow) * T;
  const int64_t c0 = (localTile % tilesPerRow) * T;
  const int nr = static_cast<int>(e.rows - r0 < T ? e.rows - r0 : T);
  const int nc = static_cast<int>(e.cols - c0 < T ? e.cols - c0 : T);
  const S* src = static_cast<const S*>(e.src);
  D* dst = static_cast<D*>(e.dst);
  const bool rowsFast = (e.rowStride == 1 || e.rows == 1) && e.colStride != 1;
  if (rowsFast) {
    // consecutive threads walk down a source column: coalesced reads
    for (int idx = tid; idx < nr * nc; idx += nthr) {
      const int c = idx / nr, r = idx % nr;
      tile[c * (T + 1) + r] = src[(r0 + r) * e.rowStride + (c0 + c) * e.colStride];
    }
  } else {
    for (int idx = tid; idx < nr * nc; idx += nthr) {
      const int r = idx / nc, c = idx % nc;
      tile[c * (T + 1) + r] = src[(r0 + r) * e.rowStride + (c0 + c) * e.colStride];
    }
  }
  plainBarrier(nthr);
  for (int idx = tid; idx < nr * nc; idx += nthr) {
    const int r = idx / nc, c = idx % nc;
    const S v = tile[c * (T + 1) + r];
    D out;
    if constexpr (kConvert) out = fromFloat<D>(toFloat<S>(v));
    else out = v;
    dst[(r0 + r) * e.cols + (c0 + c)] = out;
  }
  plainBarrier(nthr);  // the tile is reused by the next strided tile
}

__device__ __forceinline__ void stridedTile(const PushEntry& e, uint32_t localTile, int tid, int nthr,
                                            uint8_t* tileMem) {
  if (e.srcDtype == e.dstDtype || e.dstDtype == static_cast<uint8_t>(DType::kBytes)) {
    switch (e.srcElemSize) {
      case 1: stridedTileTyped<uint8_t, uint8_t, false>(e, localTile, tid, nthr, tileMem); break;
      case 2: stridedTileTyped<uint16_t, uint16_t, false>(e, localTile, tid, nthr, tileMem); break;
      case 4: stridedTileTyped<uint32_t, uint32_t, false>(e, localTile, tid, nthr, tileMem); break;
      default: stridedTileTyped<uint64_t, uint64_t, false>(e, localTile, tid, nthr, tileMem); break;
    }
    return;
  }
  const uint32_t key = (static_cast<uint32_t>(e.srcDtype) << 8) | e.dstDtype;
  constexpr uint32_t F32 = static_cast<uint32_t>(DType::kF32), BF = static_cast<uint32_t>(DType::kBF16),
                     F16 = static_cast<uint32_t>(DType::kF16);
  switch (key) {
    case (F32 << 8) | BF: stridedTileTyped<float, __nv_bfloat16, true>(e, localTile, tid, nthr, tileMem); break;
    case (F32 << 8) | F16: stridedTileTyped<float, __half, true>(e, localTile, tid, nthr, tileMem); break;
    case (BF << 8) | F32: stridedTileTyped<__nv_bfloat16, float, true>(e, localTile, tid, nthr, tileMem); break;
    case (F16 << 8) | F32: stridedTileTyped<__half, float, true>(e, localTile, tid, nthr, tileMem); break;
    case (BF << 8) | F16: stridedTileTyped<__nv_bfloat16, __half, true>(e, localTile, tid, nthr, tileMem); break;
    case (F16 << 8) | BF: stridedTileTyped<__half, __nv_bfloat16, true>(e, localTile, tid, nthr, tileMem); break;
    default: break;
  }
}

// ---- the kernel ---------------------------------------------------------------------------------
template <int N>
__global__ void __launch_bounds__(kThreads, 1) tpb_push_pack(const __grid_constant__ PushParams<N> p) {
  extern __shared__ uint8_t smemRaw[];
  // dynamic shared memory is only guaranteed 16-byte aligned: round up for the bulk stages
  SharedStorage& sm = *reinterpret_cast<SharedStorage*>(
      (reinterpret_cast<uintptr_t>(smemRaw) + 127) & ~static_cast<uintptr_t>(127));

  const int tid = threadIdx.x;
  const bool haveBulk = p.bulkTiles > blockIdx.x;

  if (tid == 0 && haveBulk) {
    for (int s = 0; s < kBulkStages; ++s) mbarInit(&sm.full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (tid < 32) {
    // ---- warp 0: the bulk copy pipeline, driven by one elected lane ----
    if (tid == 0 && haveBulk) {
      const uint32_t first = blockIdx.x, step = gridDim.x;
      const uint32_t mine = (p.bulkTiles - first + step - 1) / step;  // tiles this CTA owns
      bool failed = false;
      // Describe my i-th tile.
      auto describe = [&](uint32_t i, const uint8_t*& src, uint8_t*& dst, uint32_t& bytes) {
        const uint32_t t = first + i * step;
        const PushEntry* e = findEntry(p, t, true);
        const uint64_t off = static_cast<uint64_t>(t - e->tileStart) * kBulkTileBytes;
        const uint64_t left = e->count - off;
        bytes = left < kBulkTileBytes ? static_cast<uint32_t>(left) : kBulkTileBytes;
        src = static_cast<const uint8_t*>(e->src) + off;
        dst = static_cast<uint8_t*>(e->dst) + off;
      };
      auto issueLoad = [&](uint32_t i) {
        const uint8_t* src;
        uint8_t* dst;
        uint32_t bytes;
        describe(i, src, dst, bytes);
        const int s = i % kBulkStages;
        mbarExpectTx(&sm.full[s], bytes);
        bulkLoad(sm.stages[s], src, bytes, &sm.full[s]);
      };
      const uint32_t prologue = mine < static_cast<uint32_t>(kBulkStages) ? mine : kBulkStages;
      for (uint32_t i = 0; i < prologue; ++i) issueLoad(i);
      for (uint32_t c = 0; c < mine; ++c) {
        const int s = c % kBulkStages;
        if (!mbarWaitBounded(&sm.full[s], (c / kBulkStages) & 1)) {
          failed = true;
          break;
        }
        const uint8_t* src;
        uint8_t* dst;
        uint32_t bytes;
        describe(c, src, dst, bytes);
        fenceProxyAsync();
        bulkStore(dst, sm.stages[s], bytes);
        bulkCommit();
        // Refill the stage whose store was issued one iteration ago: by now it has most likely
        // finished reading shared memory, so this wait rarely stalls the pipeline.
        if (c >= 1 && (c - 1) + kBulkStages < mine) {
          bulkWaitRead<1>();
          issueLoad((c - 1) + kBulkStages);
        }
      }
      bulkWaitAll();  // stores are complete (not merely read out of shared memory)
      if (failed && p.status) atomicMax(p.status, static_cast<uint32_t>(kStatusBarrierTimeout));
    }
  } else {
    // ---- warps 1..: everything that needs registers ----
    const int ptid = tid - 32;
    const int pn = kThreads - 32;
    for (uint32_t t = blockIdx.x; t < p.plainTiles; t += gridDim.x) {
      const PushEntry* e = findEntry(p, t, false);
      const uint32_t local = t - e->tileStart;
      if (e->kind == kCopyPlain) copyPlainTile(*e, local, ptid, pn);
      else if (e->kind == kCastPlain) castTile(*e, local, ptid, pn);
      else stridedTile(*e, local, ptid, pn, sm.tile);
    }
  }

  if (p.flag == nullptr) return;
  // Make this thread's writes visible system-wide before the CTA reports in.
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    const uint32_t arrived = atomicAdd(p.counter, 1u);
    if (arrived == gridDim.x - 1) {
      *p.counter = 0;  // ready for the next launch on this stream
      __threadfence_system();
      storeReleaseSys(p.flag, p.flagValue);
    }
  }
}

__global__ void tpb_wait_flag(const uint32_t* flag, uint32_t value, uint64_t timeoutNs, uint32_t* status) {
  if (threadIdx.x != 0) return;
  const uint64_t start = globalTimerNs();
  uint32_t backoff = 32;
  uint32_t result = kStatusWaitTimeout;
  // Both limits bound the loop: the timer deadline and an iteration cap.
  for (uint64_t i = 0; i < (1ull << 32); ++i) {
    const uint32_t v = loadAcquireSys(flag);
    if (static_cast<int32_t>(v - value) >= 0) {
      result = kStatusOk;
      break;
    }
    if (globalTimerNs() - start > timeoutNs) break;
    __nanosleep(backoff);
    if (backoff < 1024) backoff <<= 1;
  }
  if (status) *status = result;
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

template <int N>
void launchOne(const PushEntry* entries, uint32_t n, uint32_t bulkTiles, uint32_t plainTiles, cudaStream_t stream,
               int maxCtas, uint32_t* flag, uint32_t flagValue, uint32_t* counter, uint32_t* status) {
  static const size_t kSmem = sizeof(SharedStorage) + 128;
  static bool configured[64] = {};
  int dev = 0;
  check(cudaGetDevice(&dev), "cudaGetDevice");
  if (dev < 64 && !configured[dev]) {
    check(cudaFuncSetAttribute(tpb_push_pack<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmem)),
          "cudaFuncSetAttribute");
    configured[dev] = true;
  }
  PushParams<N> p;
  for (uint32_t i = 0; i < n; ++i) p.entries[i] = entries[i];
  p.numEntries = n;
  p.bulkTiles = bulkTiles;
  p.plainTiles = plainTiles;
  p.flagValue = flagValue;
  p.flag = flag;
  p.counter = counter;
  p.status = status;
  uint32_t tiles = bulkTiles > plainTiles ? bulkTiles : plainTiles;
  uint32_t grid = tiles < static_cast<uint32_t>(maxCtas) ? tiles : static_cast<uint32_t>(maxCtas);
  if (grid == 0) grid = 1;
  tpb_push_pack<N><<<grid, kThreads, kSmem, stream>>>(p);
  check(cudaGetLastError(), "tpb_push_pack launch");
  ++gLaunches;
}

}  // namespace

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
    e.numTiles = static_cast<uint32_t>((e.count + kBulkTileBytes - 1) / kBulkTileBytes);
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
  } else {
    const uint64_t tr = (e.rows + kStridedTile - 1) / kStridedTile, tc = (e.cols + kStridedTile - 1) / kStridedTile;
    e.numTiles = static_cast<uint32_t>(tr * tc);
    e.tileStart = plan.plainTiles;
    plan.plainTiles += e.numTiles;
  }
  plan.entries.push_back(e);
}
}  // namespace

void appendToPlan(PushPlan& plan, const CopyItem& item, bool useBulk) {
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
  if (!useBulk || !sameSkew || bytes < 2048) {
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
               uint32_t* counter, uint32_t* status) {
  const size_t n = plan.entries.size();
  if (maxCtas <= 0) maxCtas = 1;
  if (n <= static_cast<size_t>(kMaxEntriesLarge)) {
    if (n <= static_cast<size_t>(kMaxEntriesSmall))
      launchOne<kMaxEntriesSmall>(plan.entries.data(), static_cast<uint32_t>(n), plan.bulkTiles, plan.plainTiles,
                                  stream, maxCtas, flag, flagValue, counter, status);
    else
      launchOne<kMaxEntriesLarge>(plan.entries.data(), static_cast<uint32_t>(n), plan.bulkTiles, plan.plainTiles,
                                  stream, maxCtas, flag, flagValue, counter, status);
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
    launchOne<kMaxEntriesLarge>(part.data(), static_cast<uint32_t>(cnt), bulk, plain, stream, maxCtas,
                                last ? flag : nullptr, flagValue, counter, status);
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

}  // namespace kernels
}  // namespace tpb
