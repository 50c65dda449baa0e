// Host-side planning of the push kernel (no GPU needed): how tensors are split into entries, how
// tiles are numbered, and which path each entry takes. The device side of the same cases is in
// kernel_gpu_test.cc.
#include "kernels/push.h"
#include "test_util.h"

using namespace tpb;
using namespace tpb::kernels;

namespace {
uint8_t* at(uintptr_t a) { return reinterpret_cast<uint8_t*>(a); }

CopyItem contiguous(uintptr_t src, uintptr_t dst, uint64_t bytes) {
  CopyItem c;
  c.src = at(src);
  c.dst = at(dst);
  c.srcBytes = bytes;
  return c;
}
}  // namespace

TPB_TEST(Plan, AlignedTensorTakesTheBulkPathInWholeTiles) {
  PushPlan plan;
  appendToPlan(plan, contiguous(0x10000000, 0x20000000, 3 * 1024 * 1024), true);
  EXPECT_EQ(plan.entries.size(), size_t(1));
  EXPECT_EQ(int(plan.entries[0].kind), int(kCopyBulk));
  const PushTuning t = getPushTuning();
  EXPECT_EQ(plan.bulkTiles, uint32_t(3 * 1024 * 1024 / t.bulkTileBytes));
  EXPECT_EQ(plan.plainTiles, uint32_t(0));
  EXPECT_EQ(plan.totalBytesOut, uint64_t(3 * 1024 * 1024));
}

TPB_TEST(Plan, RaggedEndsGoToThePlainPathAndTheBodyStaysAligned) {
  PushPlan plan;
  // Both addresses are 5 bytes past a 16-byte boundary: head of 11 bytes, aligned body, ragged tail.
  const uint64_t bytes = 2 * 1024 * 1024 + 11 + 7;
  appendToPlan(plan, contiguous(0x10000005, 0x20000005, bytes), true);
  EXPECT_EQ(plan.entries.size(), size_t(3));
  EXPECT_EQ(int(plan.entries[0].kind), int(kCopyPlain));
  EXPECT_EQ(plan.entries[0].count, uint64_t(11));
  EXPECT_EQ(int(plan.entries[1].kind), int(kCopyBulk));
  EXPECT_EQ(reinterpret_cast<uintptr_t>(plan.entries[1].src) % 16, uintptr_t(0));
  EXPECT_EQ(reinterpret_cast<uintptr_t>(plan.entries[1].dst) % 16, uintptr_t(0));
  EXPECT_EQ(plan.entries[1].count % 16, uint64_t(0));
  EXPECT_EQ(int(plan.entries[2].kind), int(kCopyPlain));
  EXPECT_EQ(plan.entries[0].count + plan.entries[1].count + plan.entries[2].count, bytes);
  // Tile numbering is per class and contiguous.
  EXPECT_EQ(plan.entries[0].tileStart, uint32_t(0));
  EXPECT_EQ(plan.entries[2].tileStart, plan.entries[0].numTiles);
  EXPECT_EQ(plan.plainTiles, plan.entries[0].numTiles + plan.entries[2].numTiles);
}

TPB_TEST(Plan, DifferentMisalignmentOrSmallOrNoBulkMeansPlain) {
  {
    PushPlan plan;  // source and destination disagree modulo 16: no bulk copy can serve both
    appendToPlan(plan, contiguous(0x10000004, 0x20000008, 4 * 1024 * 1024), true);
    EXPECT_EQ(plan.entries.size(), size_t(1));
    EXPECT_EQ(int(plan.entries[0].kind), int(kCopyPlain));
    EXPECT_EQ(plan.entries[0].numTiles, uint32_t(4 * 1024 * 1024 / kPlainTileBytes));
  }
  {
    PushPlan plan;  // below the bulk threshold
    appendToPlan(plan, contiguous(0x10000000, 0x20000000, 4096), true);
    EXPECT_EQ(int(plan.entries[0].kind), int(kCopyPlain));
    EXPECT_EQ(plan.bulkTiles, uint32_t(0));
  }
  {
    PushPlan plan;  // bulk path switched off by the caller
    appendToPlan(plan, contiguous(0x10000000, 0x20000000, 8 * 1024 * 1024), false);
    EXPECT_EQ(int(plan.entries[0].kind), int(kCopyPlain));
  }
  {
    PushPlan plan;  // empty tensors leave no entry behind
    appendToPlan(plan, contiguous(0x10000000, 0x20000000, 0), true);
    EXPECT_EQ(plan.entries.size(), size_t(0));
  }
}

TPB_TEST(Plan, ConversionsAndViews) {
  PushPlan plan;
  CopyItem c = contiguous(0x10000000, 0x20000000, 1000 * 4);
  c.srcDtype = DType::kF32;
  c.dstDtype = DType::kBF16;
  appendToPlan(plan, c, true);
  EXPECT_EQ(int(plan.entries[0].kind), int(kCastPlain));
  EXPECT_EQ(plan.entries[0].count, uint64_t(1000));  // elements
  EXPECT_EQ(plan.totalBytesOut, uint64_t(2000));
  EXPECT_EQ(plan.entries[0].numTiles, uint32_t(1));  // 2000 destination bytes fit one 8 KiB tile

  CopyItem v = contiguous(0x30000000, 0x40000000, 100 * 70 * 4);
  v.srcDtype = v.dstDtype = DType::kF32;
  v.strided = true;
  v.view = StridedView{DType::kF32, 100, 70, 1, 100};
  appendToPlan(plan, v, true);
  EXPECT_EQ(int(plan.entries[1].kind), int(kStrided));
  EXPECT_EQ(plan.entries[1].numTiles, uint32_t(4 * 3));  // ceil(100/32) x ceil(70/32)
  EXPECT_EQ(plan.entries[1].tileStart, plan.entries[0].numTiles);

  CopyItem w = contiguous(0x50000000, 0x60000000, 128 * 192 * 2);
  w.srcDtype = w.dstDtype = DType::kBF16;
  w.strided = true;
  w.view = StridedView{DType::kBF16, 128, 192, 1, 128};
  appendToPlan(plan, w, true);
  EXPECT_EQ(int(plan.entries[2].kind), int(kStridedWide16));
  EXPECT_EQ(plan.entries[2].numTiles, uint32_t(2 * 3));  // 64 x 64 tiles

  CopyItem i64 = contiguous(0x70000000, 0x78000000, 64 * 64 * 8);
  i64.srcDtype = i64.dstDtype = DType::kI64;
  i64.strided = true;
  i64.view = StridedView{DType::kI64, 64, 64, 1, 64};
  appendToPlan(plan, i64, true);
  EXPECT_EQ(plan.entries[3].numTiles, uint32_t(4 * 2));  // 16-row x 32-column tiles for 8-byte elements

  bool threw = false;
  try {
    CopyItem bad = contiguous(0x10000000, 0x20000000, 64);
    bad.srcDtype = DType::kI64;
    bad.dstDtype = DType::kF32;
    appendToPlan(plan, bad, true);
  } catch (const std::exception&) {
    threw = true;
  }
  EXPECT_TRUE(threw);  // integer -> float is not a conversion the kernel offers
  threw = false;
  try {
    CopyItem bad = contiguous(0x10000000, 0x20000000, 100);
    bad.srcDtype = bad.dstDtype = DType::kF32;
    bad.strided = true;
    bad.view = StridedView{DType::kF32, 10, 10, 1, 10};  // 400 bytes, not 100
    appendToPlan(plan, bad, true);
  } catch (const std::exception&) {
    threw = true;
  }
  EXPECT_TRUE(threw);
}

TPB_TEST(Plan, CastTableAndSizes) {
  EXPECT_TRUE(castSupported(DType::kF32, DType::kBF16));
  EXPECT_TRUE(castSupported(DType::kF16, DType::kBF16));
  EXPECT_TRUE(castSupported(DType::kI64, DType::kI64));
  EXPECT_FALSE(castSupported(DType::kI32, DType::kF32));
  EXPECT_EQ(convertedBytes(4000, DType::kF32, DType::kBF16), uint64_t(2000));
  EXPECT_EQ(convertedBytes(2000, DType::kF16, DType::kF32), uint64_t(4000));
  EXPECT_EQ(convertedBytes(123, DType::kU8, DType::kBytes), uint64_t(123));
  EXPECT_EQ(int(patternByte(7, 5)), int(patternByte(7, 5)));
  EXPECT_TRUE(patternByte(7, 0) != patternByte(8, 0) || patternByte(7, 1) != patternByte(8, 1));
}

TPB_TEST(Plan, NarrowMatricesFollowTheDestinationAndTheTuning) {
  auto kindOf = [](bool remote) {
    PushPlan plan;
    CopyItem v = contiguous(0x30000000, 0x40000000, 1000 * 64 * 4);
    v.srcDtype = v.dstDtype = DType::kF32;
    v.strided = true;
    v.view = StridedView{DType::kF32, 1000, 64, 1, 1000};
    v.remote = remote;
    appendToPlan(plan, v, true);
    return int(plan.entries.back().kind);
  };
  const PushTuning before = getPushTuning();
  PushTuning t = before;
  t.narrowRows = 1;  // the default: whole packed rows only towards another GPU
  setPushTuning(t);
  EXPECT_EQ(kindOf(true), int(kStridedNarrow));
  EXPECT_EQ(kindOf(false), int(kStrided));
  t.narrowRows = 0;  // without the narrow form such a matrix goes in bands of whole rows
  setPushTuning(t);
  EXPECT_EQ(kindOf(true), int(kStridedBand));
  t.bandRows = 0;
  setPushTuning(t);
  EXPECT_EQ(kindOf(true), int(kStrided));
  t.bandRows = 2;    // bands for local destinations too
  setPushTuning(t);
  EXPECT_EQ(kindOf(false), int(kStridedBand));
  t.narrowRows = 2;
  setPushTuning(t);
  EXPECT_EQ(kindOf(false), int(kStridedNarrow));
  setPushTuning(before);
  // 1000 rows in tiles of 32 whole rows.
  PushPlan plan;
  CopyItem v = contiguous(0x30000000, 0x40000000, 1000 * 64 * 4);
  v.srcDtype = v.dstDtype = DType::kF32;
  v.strided = true;
  v.view = StridedView{DType::kF32, 1000, 64, 1, 1000};
  v.remote = true;
  appendToPlan(plan, v, true);
  EXPECT_EQ(plan.entries.back().numTiles, uint32_t(32));
}

// ---- the cache of opened IPC mappings (bookkeeping only: the two driver calls are counters) ----
#include "channel/cuda_p2p/mapping_cache.h"

TPB_TEST(Plan, MappingsAreKeyedByHandleAndAccessingDeviceAndIdleOnesAreClosed) {
  using tpb::channel::cuda_p2p::MappingCache;
  MappingCache cache;
  std::vector<std::pair<uintptr_t, int>> opened, closed;
  uintptr_t next = 0x1000;
  cache.setBackendForTesting(
      [&](const MappingCache::Handle&, int device, size_t* size) {
        *size = 4096;
        opened.emplace_back(next, device);
        void* p = reinterpret_cast<void*>(next);
        next += 0x1000;
        return p;
      },
      [&](void* base, int device) { closed.emplace_back(reinterpret_cast<uintptr_t>(base), device); });
  cache.setLimits(4, 0);  // at most four mappings; anything not in use this instant counts as idle
  MappingCache::Handle a{}, b{};
  a[0] = 1;
  b[0] = 2;
  size_t size = 0;
  std::string why;
  // The same allocation seen from two GPUs is two mappings: peer access is enabled per accessing
  // device when a mapping is opened.
  void* a0 = cache.open(a, 0, &size, &why);
  void* a1 = cache.open(a, 1, &size, &why);
  EXPECT_TRUE(a0 != nullptr && a1 != nullptr && a0 != a1);
  EXPECT_EQ(size, size_t(4096));
  EXPECT_EQ(opened.size(), size_t(2));
  EXPECT_TRUE(cache.open(a, 0, &size, &why) == a0);  // a hit: nothing is opened again
  EXPECT_EQ(opened.size(), size_t(2));
  // A pinned mapping (a channel's arena) survives any eviction.
  void* pinned = cache.open(b, 0, nullptr, &why, /*pin=*/true);
  const uint64_t before = cache.generation();
  MappingCache::Handle more{};
  for (int i = 0; i < 6; ++i) {
    more[1] = static_cast<uint8_t>(10 + i);
    EXPECT_TRUE(cache.open(more, 0, nullptr, &why) != nullptr);
  }
  EXPECT_TRUE(cache.size() <= 5);
  EXPECT_TRUE(!closed.empty());
  EXPECT_TRUE(cache.generation() != before);  // holders of old addresses must look them up again
  for (auto& c : closed) EXPECT_TRUE(c.first != reinterpret_cast<uintptr_t>(pinned));
  EXPECT_TRUE(cache.open(b, 0, nullptr, &why) == pinned);
  EXPECT_EQ(cache.closedCount(), uint64_t(closed.size()));
}
