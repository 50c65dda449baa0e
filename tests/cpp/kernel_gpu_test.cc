// GPU tests of the device kernels against plain CPU restatements of the same operations:
// memcpy, a strided 2-D gather and IEEE float -> bfloat16 round-to-nearest-even. Shapes include
// the adversarial ones (0, 1, 15, 16, 17 bytes, odd offsets, sizes that straddle tile edges,
// many tensors in one launch), and every destination is fenced by canary bytes.
#include <cuda_runtime.h>

#include <cstring>
#include <random>

#include "common/cuda.h"
#include "kernels/push.h"
#include "test_util.h"

using namespace tpb;
using namespace tpb::kernels;

namespace {

#define CK(x) TPB_CUDA_CHECK(x)

constexpr size_t kGuard = 256;

struct DeviceBuf {
  uint8_t* p = nullptr;
  size_t n = 0;
  explicit DeviceBuf(size_t bytes) : n(bytes) { CK(cudaMalloc(&p, bytes ? bytes : 1)); }
  ~DeviceBuf() { cudaFree(p); }
};

std::vector<uint8_t> download(const uint8_t* p, size_t n) {
  std::vector<uint8_t> v(n);
  if (n) CK(cudaMemcpy(v.data(), p, n, cudaMemcpyDeviceToHost));
  return v;
}

uint16_t f32ToBf16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  if ((x & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((x >> 16) | 0x40);  // quiet NaN
  uint32_t lsb = (x >> 16) & 1;
  x += 0x7fffu + lsb;
  return static_cast<uint16_t>(x >> 16);
}
float bf16ToF32(uint16_t h) {
  uint32_t x = static_cast<uint32_t>(h) << 16;
  float f;
  std::memcpy(&f, &x, 4);
  return f;
}

// Runs one plan with a single contiguous copy and checks bytes + canaries.
void checkCopy(size_t bytes, size_t srcOff, size_t dstOff, bool bulk, int ctas) {
  DeviceBuf src(bytes + srcOff + 64), dst(bytes + dstOff + 2 * kGuard);
  std::vector<uint8_t> host(bytes + srcOff + 64);
  std::mt19937 rng(static_cast<uint32_t>(bytes * 31 + srcOff * 7 + dstOff));
  for (auto& b : host) b = static_cast<uint8_t>(rng());
  CK(cudaMemcpy(src.p, host.data(), host.size(), cudaMemcpyHostToDevice));
  CK(cudaMemset(dst.p, 0xCD, dst.n));
  PushPlan plan;
  CopyItem it;
  it.src = src.p + srcOff;
  it.dst = dst.p + kGuard + dstOff;
  it.srcBytes = bytes;
  appendToPlan(plan, it, bulk);
  if (!plan.entries.empty()) launchPush(plan, nullptr, ctas, nullptr, 0, nullptr, nullptr);
  CK(cudaDeviceSynchronize());
  auto out = download(dst.p, dst.n);
  for (size_t i = 0; i < kGuard + dstOff; ++i)
    if (out[i] != 0xCD) throw tpbtest::TestFailure("front canary overwritten, bytes=" + std::to_string(bytes));
  for (size_t i = 0; i < bytes; ++i)
    if (out[kGuard + dstOff + i] != host[srcOff + i])
      throw tpbtest::TestFailure("mismatch at byte " + std::to_string(i) + " of " + std::to_string(bytes) +
                                 " (srcOff " + std::to_string(srcOff) + ", dstOff " + std::to_string(dstOff) +
                                 ", bulk " + std::to_string(bulk) + ")");
  for (size_t i = kGuard + dstOff + bytes; i < out.size(); ++i)
    if (out[i] != 0xCD) throw tpbtest::TestFailure("back canary overwritten, bytes=" + std::to_string(bytes));
}

}  // namespace

TPB_GPU_TEST(Kernel, ContiguousCopySmallAndRagged, 1) {
  for (bool bulk : {false, true})
    for (size_t bytes : {size_t(0), size_t(1), size_t(15), size_t(16), size_t(17), size_t(255), size_t(2047),
                         size_t(2048), size_t(4096), size_t(4099), size_t(65536), size_t(65537), size_t(100000)})
      for (size_t so : {size_t(0), size_t(1), size_t(8)})
        for (size_t d : {size_t(0), size_t(1), size_t(8), size_t(13)}) checkCopy(bytes, so, d, bulk, 148);
}

TPB_GPU_TEST(Kernel, ContiguousCopyLarge, 1) {
  // Tile-edge sizes and more tiles than CTAs (and fewer CTAs than tiles, on purpose).
  for (bool bulk : {false, true}) {
    checkCopy((32u << 10) * 4 * 3 + 48, 0, 0, bulk, 2);
    checkCopy((1u << 20) + 16, 16, 16, bulk, 148);
    checkCopy((64u << 20) + 5, 3, 3, bulk, 148);
    checkCopy((8u << 20), 0, 16, bulk, 7);
  }
}

TPB_GPU_TEST(Kernel, CastFloat32ToBfloat16MatchesRoundToNearestEven, 1) {
  for (size_t n : {size_t(1), size_t(7), size_t(8), size_t(1000), size_t(65536 / 2 + 3), size_t(1 << 20)}) {
    std::vector<float> host(n);
    std::mt19937 rng(static_cast<uint32_t>(n));
    std::normal_distribution<float> dist(0.f, 1.f);
    for (auto& f : host) f = dist(rng);
    if (n > 6) {
      host[0] = 1.00390625f;  // exactly halfway between two bf16 values (ties to even)
      host[1] = 1.01171875f;
      host[2] = -0.f;
      host[3] = 3.4e38f;
      host[4] = 1e-40f;  // denormal
      host[5] = std::numeric_limits<float>::infinity();
    }
    DeviceBuf src(n * 4), dst(n * 2 + 2 * kGuard);
    CK(cudaMemcpy(src.p, host.data(), n * 4, cudaMemcpyHostToDevice));
    CK(cudaMemset(dst.p, 0xCD, dst.n));
    PushPlan plan;
    CopyItem it;
    it.src = src.p;
    it.dst = dst.p + kGuard;
    it.srcBytes = n * 4;
    it.srcDtype = DType::kF32;
    it.dstDtype = DType::kBF16;
    appendToPlan(plan, it, true);
    launchPush(plan, nullptr, 148, nullptr, 0, nullptr, nullptr);
    CK(cudaDeviceSynchronize());
    auto out = download(dst.p, dst.n);
    for (size_t i = 0; i < n; ++i) {
      uint16_t got;
      std::memcpy(&got, &out[kGuard + 2 * i], 2);
      EXPECT_EQ(got, f32ToBf16(host[i]));
    }
    EXPECT_EQ(int(out[kGuard - 1]), 0xCD);
    EXPECT_EQ(int(out[kGuard + 2 * n]), 0xCD);

    // and back: bf16 -> fp32 is exact
    DeviceBuf back(n * 4);
    PushPlan plan2;
    CopyItem it2;
    it2.src = dst.p + kGuard;
    it2.dst = back.p;
    it2.srcBytes = n * 2;
    it2.srcDtype = DType::kBF16;
    it2.dstDtype = DType::kF32;
    appendToPlan(plan2, it2, true);
    launchPush(plan2, nullptr, 148, nullptr, 0, nullptr, nullptr);
    CK(cudaDeviceSynchronize());
    auto outBack = download(back.p, n * 4);
    for (size_t i = 0; i < n; ++i) {
      float got;
      std::memcpy(&got, &outBack[4 * i], 4);
      float want = bf16ToF32(f32ToBf16(host[i]));
      EXPECT_TRUE(std::memcmp(&got, &want, 4) == 0);
    }
  }
}

TPB_GPU_TEST(Kernel, StridedViewsPackLikeACpuGather, 1) {
  struct Case {
    int64_t rows, cols;
    bool transposed;
    size_t es;
  };
  for (Case c : {Case{1, 1, true, 4}, Case{3, 5, true, 2}, Case{100, 37, true, 4}, Case{64, 64, true, 8},
                 Case{257, 129, true, 2}, Case{1000, 64, true, 4}, Case{33, 70, false, 4}, Case{128, 200, false, 1}}) {
    // Source storage: transposed => a [cols, rows] row-major matrix viewed as [rows, cols];
    // otherwise a [rows, 2*cols] matrix of which we take every other column (colStride 2).
    const int64_t storageElems = c.transposed ? c.rows * c.cols : c.rows * c.cols * 2;
    std::vector<uint8_t> host(storageElems * c.es);
    std::mt19937 rng(static_cast<uint32_t>(c.rows * 131 + c.cols));
    for (auto& b : host) b = static_cast<uint8_t>(rng());
    StridedView v;
    v.dtype = c.es == 1 ? DType::kU8 : c.es == 2 ? DType::kBF16 : c.es == 4 ? DType::kF32 : DType::kI64;
    v.rows = c.rows;
    v.cols = c.cols;
    v.rowStride = c.transposed ? 1 : c.cols * 2;
    v.colStride = c.transposed ? c.rows : 2;
    const size_t packed = c.rows * c.cols * c.es;
    DeviceBuf src(host.size()), dst(packed + 2 * kGuard);
    CK(cudaMemcpy(src.p, host.data(), host.size(), cudaMemcpyHostToDevice));
    CK(cudaMemset(dst.p, 0xCD, dst.n));
    PushPlan plan;
    CopyItem it;
    it.src = src.p;
    it.dst = dst.p + kGuard;
    it.srcBytes = packed;
    it.srcDtype = v.dtype;
    it.dstDtype = v.dtype;
    it.strided = true;
    it.view = v;
    appendToPlan(plan, it, true);
    launchPush(plan, nullptr, 148, nullptr, 0, nullptr, nullptr);
    CK(cudaDeviceSynchronize());
    auto out = download(dst.p, dst.n);
    for (int64_t r = 0; r < c.rows; ++r)
      for (int64_t col = 0; col < c.cols; ++col) {
        const uint8_t* want = &host[(r * v.rowStride + col * v.colStride) * c.es];
        const uint8_t* got = &out[kGuard + (r * c.cols + col) * c.es];
        if (std::memcmp(want, got, c.es) != 0)
          throw tpbtest::TestFailure("strided mismatch at (" + std::to_string(r) + "," + std::to_string(col) +
                                     ") of " + std::to_string(c.rows) + "x" + std::to_string(c.cols));
      }
    EXPECT_EQ(int(out[kGuard - 1]), 0xCD);
    EXPECT_EQ(int(out[kGuard + packed]), 0xCD);
  }
}

// Even-sized transposed matrices of 2-byte elements take the word-wide 64x64 tile path; alone they
// run in the light kernel, next to a large contiguous tensor in the full kernel (bulk pipeline on
// warp 0, the transposition on the other warps with the larger staging area).
TPB_GPU_TEST(Kernel, WideTransposeOfTwoByteElements, 1) {
  struct Case {
    int64_t rows, cols;
    bool withBulk;
  };
  for (Case c : {Case{64, 66, false}, Case{130, 198, false}, Case{1024, 258, false}, Case{2050, 514, true},
                 Case{66, 4096, true}}) {
    std::vector<uint16_t> host(c.rows * c.cols);
    std::mt19937 rng(static_cast<uint32_t>(c.rows * 7 + c.cols));
    for (auto& b : host) b = static_cast<uint16_t>(rng());
    const size_t packed = host.size() * 2;
    const size_t bulkBytes = 3 * 1024 * 1024 + 16;
    DeviceBuf src(packed), dst(packed + 2 * kGuard), bsrc(bulkBytes), bdst(bulkBytes);
    CK(cudaMemcpy(src.p, host.data(), packed, cudaMemcpyHostToDevice));
    CK(cudaMemset(dst.p, 0xCD, dst.n));
    launchFill(nullptr, bsrc.p, bulkBytes, 99);
    CK(cudaMemset(bdst.p, 0, bulkBytes));
    PushPlan plan;
    if (c.withBulk) {
      CopyItem b;
      b.src = bsrc.p;
      b.dst = bdst.p;
      b.srcBytes = bulkBytes;
      appendToPlan(plan, b, true);
    }
    CopyItem it;
    it.src = src.p;
    it.dst = dst.p + kGuard;
    it.srcBytes = packed;
    it.srcDtype = DType::kF16;
    it.dstDtype = DType::kF16;
    it.strided = true;
    it.view = StridedView{DType::kF16, c.rows, c.cols, 1, c.rows};
    appendToPlan(plan, it, true);
    EXPECT_EQ(int(plan.entries.back().kind), int(kStridedWide16));
    if (c.withBulk) EXPECT_TRUE(plan.bulkTiles > 0);
    launchPush(plan, nullptr, 148, nullptr, 0, nullptr, nullptr);
    CK(cudaDeviceSynchronize());
    auto out = download(dst.p, dst.n);
    for (int64_t r = 0; r < c.rows; ++r)
      for (int64_t col = 0; col < c.cols; ++col) {
        uint16_t got;
        std::memcpy(&got, &out[kGuard + (r * c.cols + col) * 2], 2);
        if (got != host[col * c.rows + r])
          throw tpbtest::TestFailure("wide transpose mismatch at (" + std::to_string(r) + "," + std::to_string(col) +
                                     ") of " + std::to_string(c.rows) + "x" + std::to_string(c.cols));
      }
    EXPECT_EQ(int(out[kGuard - 1]), 0xCD);
    EXPECT_EQ(int(out[kGuard + packed]), 0xCD);
    if (c.withBulk) {
      DeviceBuf bad(8);
      CK(cudaMemset(bad.p, 0, 8));
      launchVerify(nullptr, bdst.p, bulkBytes, 99, reinterpret_cast<unsigned long long*>(bad.p));
      CK(cudaDeviceSynchronize());
      auto n = download(bad.p, 8);
      unsigned long long mism;
      std::memcpy(&mism, n.data(), 8);
      EXPECT_EQ(mism, 0ull);
    }
  }
  // Odd extents, an odd column stride or a misaligned destination fall back to the element-wise tiles.
  {
    PushPlan plan;
    DeviceBuf src(65 * 66 * 2), dst(65 * 66 * 2 + 64);
    CopyItem it;
    it.src = src.p;
    it.dst = dst.p;
    it.srcBytes = 65 * 66 * 2;
    it.srcDtype = it.dstDtype = DType::kBF16;
    it.strided = true;
    it.view = StridedView{DType::kBF16, 65, 66, 1, 65};
    appendToPlan(plan, it, true);
    EXPECT_EQ(int(plan.entries.back().kind), int(kStrided));
    it.srcBytes = 64 * 64 * 2;
    it.view = StridedView{DType::kBF16, 64, 64, 1, 64};
    it.dst = dst.p + 2;
    appendToPlan(plan, it, true);
    EXPECT_EQ(int(plan.entries.back().kind), int(kStrided));
  }
}

// Transposed matrices of at most 64 columns take the narrow path: 32 whole packed rows per tile,
// written as one contiguous run; with and without conversion, odd row counts, several widths.
TPB_GPU_TEST(Kernel, NarrowTransposeWritesWholeRows, 1) {
  struct Case {
    int64_t rows, cols;
    size_t es;     // source element size
    bool toBf16;   // fp32 -> bf16 on the way (es == 4 only)
  };
  for (Case c : {Case{2, 64, 4, false}, Case{33, 64, 4, false}, Case{1000, 64, 4, false}, Case{4097, 32, 4, false},
                 Case{77, 4, 4, false}, Case{300, 64, 2, false}, Case{129, 8, 2, false}, Case{65, 16, 1, false},
                 Case{999, 64, 4, true}, Case{64, 8, 4, true}, Case{31, 48, 2, false}}) {
    const size_t srcBytes = c.rows * c.cols * c.es;
    const size_t des = c.toBf16 ? 2 : c.es;
    const size_t packed = c.rows * c.cols * des;
    std::vector<uint8_t> host(srcBytes);
    std::mt19937 rng(static_cast<uint32_t>(c.rows * 31 + c.cols + c.es));
    if (c.toBf16) {
      auto* f = reinterpret_cast<float*>(host.data());
      std::normal_distribution<float> dist(0.f, 100.f);
      for (size_t i = 0; i < srcBytes / 4; ++i) f[i] = dist(rng);
    } else {
      for (auto& b : host) b = static_cast<uint8_t>(rng());
    }
    DeviceBuf src(srcBytes), dst(packed + 2 * kGuard);
    CK(cudaMemcpy(src.p, host.data(), srcBytes, cudaMemcpyHostToDevice));
    CK(cudaMemset(dst.p, 0xCD, dst.n));
    PushPlan plan;
    CopyItem it;
    it.src = src.p;
    it.dst = dst.p + kGuard;
    it.srcBytes = srcBytes;
    const DType dt = c.es == 1 ? DType::kU8 : c.es == 2 ? DType::kF16 : DType::kF32;
    it.srcDtype = dt;
    it.dstDtype = c.toBf16 ? DType::kBF16 : dt;
    it.strided = true;
    it.view = StridedView{dt, c.rows, c.cols, 1, c.rows};
    it.remote = true;  // the path is chosen for destinations on another GPU; its result is the same anywhere
    appendToPlan(plan, it, true);
    EXPECT_EQ(int(plan.entries.back().kind), int(kStridedNarrow));
    EXPECT_EQ(plan.entries.back().numTiles, uint32_t((c.rows + 31) / 32));
    launchPush(plan, nullptr, 148, nullptr, 0, nullptr, nullptr);
    CK(cudaDeviceSynchronize());
    auto out = download(dst.p, dst.n);
    for (int64_t r = 0; r < c.rows; ++r)
      for (int64_t col = 0; col < c.cols; ++col) {
        const uint8_t* want = &host[(col * c.rows + r) * c.es];
        const uint8_t* got = &out[kGuard + (r * c.cols + col) * des];
        bool same;
        if (c.toBf16) {
          float f;
          std::memcpy(&f, want, 4);
          uint16_t g;
          std::memcpy(&g, got, 2);
          same = g == f32ToBf16(f);
        } else {
          same = std::memcmp(want, got, c.es) == 0;
        }
        if (!same)
          throw tpbtest::TestFailure("narrow transpose mismatch at (" + std::to_string(r) + "," + std::to_string(col) +
                                     ") of " + std::to_string(c.rows) + "x" + std::to_string(c.cols) + " es=" +
                                     std::to_string(c.es));
      }
    EXPECT_EQ(int(out[kGuard - 1]), 0xCD);
    EXPECT_EQ(int(out[kGuard + packed]), 0xCD);
  }
  // Rows that are not whole 16-byte chunks, a misaligned destination or 8-byte elements go in bands
  // of whole rows when bound for another GPU, and keep the 32x32 tiles otherwise.
  {
    DeviceBuf src(4096), dst(4096 + 64);
    auto kindOf = [&](int64_t rows, int64_t cols, DType dt, uint8_t* d, bool remote = true) {
      PushPlan plan;
      CopyItem it;
      it.src = src.p;
      it.dst = d;
      it.srcBytes = rows * cols * dtypeSize(dt);
      it.srcDtype = it.dstDtype = dt;
      it.strided = true;
      it.view = StridedView{dt, rows, cols, 1, rows};
      it.remote = remote;
      appendToPlan(plan, it, true);
      return int(plan.entries.back().kind);
    };
    EXPECT_EQ(kindOf(10, 6, DType::kF32, dst.p), int(kStridedBand));        // 24-byte rows
    EXPECT_EQ(kindOf(10, 8, DType::kF32, dst.p + 4), int(kStridedBand));    // destination off the 16-byte grid
    EXPECT_EQ(kindOf(10, 8, DType::kI64, dst.p), int(kStridedBand));        // 8-byte elements
    EXPECT_EQ(kindOf(10, 8, DType::kF32, dst.p), int(kStridedNarrow));
    EXPECT_EQ(kindOf(10, 8, DType::kF32, dst.p, false), int(kStrided));  // local destination: the 32x32 tiles are faster
    EXPECT_EQ(kindOf(10, 6, DType::kF32, dst.p, false), int(kStrided));
    EXPECT_EQ(kindOf(2, 2049, DType::kF32, dst.p), int(kStrided));          // rows longer than a band
    EXPECT_EQ(kindOf(1, 100, DType::kF32, dst.p), int(kStrided));           // a single row is contiguous anyway
  }
}

// Bulk (TMA) loads are planned for sources in the launching GPU's own memory only, whatever the
// caller asks for: pinned host memory and another GPU's memory fall back to plain loads.
TPB_GPU_TEST(Kernel, BulkLoadsAreOnlyPlannedForLocalSources, 1) {
  constexpr size_t kBytes = 4u << 20;
  DeviceBuf local(kBytes), dst(kBytes);
  auto kinds = [&](const void* src) {
    PushPlan plan;
    CopyItem it;
    it.src = src;
    it.dst = dst.p;
    it.srcBytes = kBytes;
    appendToPlan(plan, it, true);
    int bulk = 0;
    for (auto& e : plan.entries) bulk += e.kind == kCopyBulk;
    return bulk;
  };
  EXPECT_EQ(kinds(local.p), 1);
  uint8_t* pinned = nullptr;
  CK(cudaHostAlloc(reinterpret_cast<void**>(&pinned), kBytes, cudaHostAllocPortable));
  EXPECT_EQ(kinds(pinned), 0);
  // ... and the plan still moves the bytes
  for (size_t i = 0; i < kBytes; ++i) pinned[i] = static_cast<uint8_t>(i * 7);
  PushPlan plan;
  CopyItem it;
  it.src = pinned;
  it.dst = dst.p;
  it.srcBytes = kBytes;
  appendToPlan(plan, it, true);
  launchPush(plan, nullptr, 148, nullptr, 0, nullptr, nullptr);
  CK(cudaDeviceSynchronize());
  auto out = download(dst.p, kBytes);
  EXPECT_TRUE(std::memcmp(out.data(), pinned, kBytes) == 0);
  CK(cudaFreeHost(pinned));
  int devices = 0;
  CK(cudaGetDeviceCount(&devices));
  if (devices >= 2) {
    CK(cudaSetDevice(1));
    uint8_t* other = nullptr;
    CK(cudaMalloc(&other, kBytes));
    CK(cudaSetDevice(0));
    EXPECT_EQ(kinds(other), 0);
    CK(cudaSetDevice(1));
    CK(cudaFree(other));
    CK(cudaSetDevice(0));
  }
}

// Transposed matrices bound for another GPU whose packed rows fit 8 KiB go in bands of whole rows,
// each written as one contiguous run: any element size, any alignment of the destination, odd
// extents, rows so long that a band is a single row, with and without conversion.
TPB_GPU_TEST(Kernel, BandTransposeWritesOneRunPerBand, 1) {
  struct Case {
    int64_t rows, cols;
    size_t es;      // source element size
    bool toBf16;    // fp32 -> bf16 on the way (es == 4 only)
    size_t skew;    // destination offset from a 256-byte boundary, a multiple of the element size
  };
  for (Case c : {Case{167, 14, 2, false, 0}, Case{627, 132, 2, false, 2}, Case{1199, 10, 2, false, 6},
                 Case{55, 428, 2, false, 10}, Case{35, 635, 2, false, 14}, Case{678, 56, 4, false, 4},
                 Case{2, 2048, 4, false, 12}, Case{381, 10, 4, false, 8}, Case{6, 611, 4, false, 0},
                 Case{144, 1478, 4, false, 4}, Case{582, 63, 8, false, 8}, Case{12, 381, 8, false, 0},
                 Case{17, 824, 8, false, 8}, Case{3, 1024, 8, false, 0}, Case{1086, 14, 8, false, 8},
                 Case{500, 7, 1, false, 3}, Case{40, 8191, 1, false, 1}, Case{999, 65, 4, true, 2},
                 Case{64, 9, 4, true, 6}, Case{5, 4096, 4, true, 0}, Case{33, 3, 4, true, 14}}) {
    const size_t srcBytes = c.rows * c.cols * c.es;
    const size_t des = c.toBf16 ? 2 : c.es;
    const size_t packed = c.rows * c.cols * des;
    std::vector<uint8_t> host(srcBytes);
    std::mt19937 rng(static_cast<uint32_t>(c.rows * 131 + c.cols * 7 + c.es));
    if (c.toBf16) {
      auto* f = reinterpret_cast<float*>(host.data());
      std::normal_distribution<float> dist(0.f, 100.f);
      for (size_t i = 0; i < srcBytes / 4; ++i) f[i] = dist(rng);
    } else {
      for (auto& b : host) b = static_cast<uint8_t>(rng());
    }
    DeviceBuf src(srcBytes), dst(packed + 2 * kGuard + 16);
    CK(cudaMemcpy(src.p, host.data(), srcBytes, cudaMemcpyHostToDevice));
    CK(cudaMemset(dst.p, 0xCD, dst.n));
    PushPlan plan;
    CopyItem it;
    it.src = src.p;
    it.dst = dst.p + kGuard + c.skew;
    it.srcBytes = srcBytes;
    const DType dt = c.es == 1 ? DType::kU8 : c.es == 2 ? DType::kF16 : c.es == 4 ? DType::kF32 : DType::kI64;
    it.srcDtype = dt;
    it.dstDtype = c.toBf16 ? DType::kBF16 : dt;
    it.strided = true;
    it.view = StridedView{dt, c.rows, c.cols, 1, c.rows};
    it.remote = true;
    appendToPlan(plan, it, true);
    EXPECT_EQ(int(plan.entries.back().kind), int(kStridedBand));
    const uint32_t perBand = bandRows(c.cols, static_cast<uint32_t>(des));
    EXPECT_TRUE(perBand >= 1 && static_cast<uint64_t>(perBand) * c.cols * des <= kBandBytes);
    EXPECT_EQ(plan.entries.back().numTiles, uint32_t((c.rows + perBand - 1) / perBand));
    launchPush(plan, nullptr, 148, nullptr, 0, nullptr, nullptr);
    CK(cudaDeviceSynchronize());
    auto out = download(dst.p, dst.n);
    const size_t at = kGuard + c.skew;
    for (int64_t r = 0; r < c.rows; ++r)
      for (int64_t col = 0; col < c.cols; ++col) {
        const uint8_t* want = &host[(col * c.rows + r) * c.es];
        const uint8_t* got = &out[at + (r * c.cols + col) * des];
        bool same;
        if (c.toBf16) {
          float f;
          std::memcpy(&f, want, 4);
          uint16_t g;
          std::memcpy(&g, got, 2);
          same = g == f32ToBf16(f);
        } else {
          same = std::memcmp(want, got, c.es) == 0;
        }
        if (!same)
          throw tpbtest::TestFailure("band transpose mismatch at (" + std::to_string(r) + "," + std::to_string(col) +
                                     ") of " + std::to_string(c.rows) + "x" + std::to_string(c.cols) + " es=" +
                                     std::to_string(c.es) + " skew=" + std::to_string(c.skew));
      }
    // nothing before the first byte or after the last one was touched
    for (size_t i = 0; i < at; ++i)
      if (out[i] != 0xCD) throw tpbtest::TestFailure("band transpose wrote before its destination");
    for (size_t i = at + packed; i < out.size(); ++i)
      if (out[i] != 0xCD) throw tpbtest::TestFailure("band transpose wrote past its destination");
  }
}

TPB_GPU_TEST(Kernel, StridedWithCast, 1) {
  const int64_t rows = 130, cols = 70;
  std::vector<float> host(rows * cols);
  std::mt19937 rng(5);
  std::normal_distribution<float> dist(0.f, 3.f);
  for (auto& f : host) f = dist(rng);
  DeviceBuf src(host.size() * 4), dst(rows * cols * 2);
  CK(cudaMemcpy(src.p, host.data(), host.size() * 4, cudaMemcpyHostToDevice));
  PushPlan plan;
  CopyItem it;
  it.src = src.p;
  it.dst = dst.p;
  it.srcBytes = rows * cols * 4;
  it.srcDtype = DType::kF32;
  it.dstDtype = DType::kBF16;
  it.strided = true;
  it.view = StridedView{DType::kF32, rows, cols, 1, rows};
  appendToPlan(plan, it, true);
  launchPush(plan, nullptr, 148, nullptr, 0, nullptr, nullptr);
  CK(cudaDeviceSynchronize());
  auto out = download(dst.p, rows * cols * 2);
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c) {
      uint16_t got;
      std::memcpy(&got, &out[(r * cols + c) * 2], 2);
      EXPECT_EQ(got, f32ToBf16(host[c * rows + r]));
    }
}

TPB_GPU_TEST(Kernel, ManyTensorsInOneLaunchAndAcrossLaunchLimit, 1) {
  for (int count : {3, 8, 9, 64, 150}) {
    std::mt19937 rng(count);
    struct T {
      size_t bytes, srcOff, dstOff;
    };
    std::vector<T> ts;
    size_t srcTotal = 0, dstTotal = 0;
    for (int i = 0; i < count; ++i) {
      size_t bytes = 1 + rng() % (i % 5 == 0 ? 300000 : 5000);
      size_t skew = i % 3 == 0 ? 0 : (rng() % 16);
      ts.push_back({bytes, srcTotal + skew, dstTotal + (i % 2 ? skew : 0)});
      srcTotal += bytes + 64;
      dstTotal += bytes + 64;
    }
    std::vector<uint8_t> host(srcTotal);
    for (auto& b : host) b = static_cast<uint8_t>(rng());
    DeviceBuf src(srcTotal), dst(dstTotal);
    CK(cudaMemcpy(src.p, host.data(), srcTotal, cudaMemcpyHostToDevice));
    CK(cudaMemset(dst.p, 0xCD, dstTotal));
    PushPlan plan;
    for (auto& t : ts) {
      CopyItem it;
      it.src = src.p + t.srcOff;
      it.dst = dst.p + t.dstOff;
      it.srcBytes = t.bytes;
      appendToPlan(plan, it, true);
    }
    int launches = launchPush(plan, nullptr, 148, nullptr, 0, nullptr, nullptr);
    EXPECT_TRUE(launches >= 1);
    CK(cudaDeviceSynchronize());
    auto out = download(dst.p, dstTotal);
    std::vector<uint8_t> want(dstTotal, 0xCD);
    for (auto& t : ts) std::memcpy(&want[t.dstOff], &host[t.srcOff], t.bytes);
    EXPECT_TRUE(out == want);
  }
}

TPB_GPU_TEST(Kernel, FlagIsPublishedAndCounterResets, 1) {
  DeviceBuf src(1 << 20), dst(1 << 20), words(256);
  CK(cudaMemset(words.p, 0, 256));
  uint32_t* flag = reinterpret_cast<uint32_t*>(words.p);
  uint32_t* counter = flag + 16;
  uint32_t* status = flag + 32;
  launchFill(nullptr, src.p, 1 << 20, 77);
  for (uint32_t round = 1; round <= 3; ++round) {
    PushPlan plan;
    CopyItem it;
    it.src = src.p;
    it.dst = dst.p;
    it.srcBytes = 1 << 20;
    appendToPlan(plan, it, round != 2);
    launchPush(plan, nullptr, 148, flag, round, counter, status);
    // The flag is already set when the wait kernel starts (same stream): it must return OK.
    launchWaitFlag(nullptr, flag, round, 1'000'000'000ull, status + 1);
    CK(cudaDeviceSynchronize());
    auto w = download(words.p, 256);
    uint32_t f, c, s0, s1;
    std::memcpy(&f, &w[0], 4);
    std::memcpy(&c, &w[64], 4);
    std::memcpy(&s0, &w[128], 4);
    std::memcpy(&s1, &w[132], 4);
    EXPECT_EQ(f, round);
    EXPECT_EQ(c, 0u);
    EXPECT_EQ(s0, 0u);
    EXPECT_EQ(s1, uint32_t(kStatusOk));
  }
  unsigned long long* bad;
  CK(cudaMalloc(&bad, 8));
  CK(cudaMemset(bad, 0, 8));
  launchVerify(nullptr, dst.p, 1 << 20, 77, bad);
  unsigned long long h = 1;
  CK(cudaMemcpy(&h, bad, 8, cudaMemcpyDeviceToHost));
  EXPECT_EQ(h, 0ull);
  cudaFree(bad);
}

TPB_GPU_TEST(Kernel, WaitGivesUpWithATimeoutStatus, 1) {
  // A flag that nothing sets: the wait must end by itself and say so, leaving the context usable.
  DeviceBuf words(64);
  CK(cudaMemset(words.p, 0, 64));
  uint32_t* flag = reinterpret_cast<uint32_t*>(words.p);
  auto t0 = std::chrono::steady_clock::now();
  launchWaitFlag(nullptr, flag, 5, 50'000'000ull /* 50 ms */, flag + 1);
  CK(cudaDeviceSynchronize());
  double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
  auto w = download(words.p, 64);
  uint32_t status;
  std::memcpy(&status, &w[4], 4);
  EXPECT_EQ(status, uint32_t(kStatusWaitTimeout));
  EXPECT_TRUE(ms >= 40 && ms < 5000);
  // The context still works.
  launchFill(nullptr, words.p, 64, 1);
  CK(cudaDeviceSynchronize());
}

TPB_GPU_TEST(Kernel, FillAndVerifyAgreeWithTheHostPattern, 1) {
  for (size_t bytes : {size_t(1), size_t(7), size_t(4096), size_t(100003)}) {
    DeviceBuf buf(bytes);
    launchFill(nullptr, buf.p, bytes, 99);
    CK(cudaDeviceSynchronize());
    auto out = download(buf.p, bytes);
    for (size_t i = 0; i < bytes; ++i) EXPECT_EQ(int(out[i]), int(patternByte(99, i)));
    unsigned long long* bad;
    CK(cudaMalloc(&bad, 8));
    CK(cudaMemset(bad, 0, 8));
    launchVerify(nullptr, buf.p, bytes, 99, bad);
    CK(cudaMemset(buf.p + bytes / 2, out[bytes / 2] ^ 0xff, 1));
    launchVerify(nullptr, buf.p, bytes, 99, bad);
    unsigned long long h = 0;
    CK(cudaMemcpy(&h, bad, 8, cudaMemcpyDeviceToHost));
    EXPECT_EQ(h, 1ull);
    cudaFree(bad);
  }
}
