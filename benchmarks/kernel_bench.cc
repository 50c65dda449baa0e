// Micro-benchmark of the push/pack kernel on one GPU, without any pipe around it: HBM -> HBM copy
// bandwidth for several shapes of the TMA bulk pipeline, the register (plain) path, conversion and
// strided packing, against cudaMemcpyAsync device-to-device as the yardstick the reference's
// channels use (tensorpipe/channel/cuda_xth/channel_impl.cc:66-77). Timed with CUDA events after
// warm-up; buffers larger than L2; prints one line per case.
//
//   kernel_bench [--bytes N] [--iters K] [--case substring]
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cmath>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "common/cuda.h"
#include "kernels/push.h"

using namespace tpb;
using namespace tpb::kernels;

#define CK(x) TPB_CUDA_CHECK(x)

struct Timer {
  cudaEvent_t a, b;
  Timer() {
    CK(cudaEventCreate(&a));
    CK(cudaEventCreate(&b));
  }
  template <typename F>
  double run(int warm, int iters, F&& f) {
    for (int i = 0; i < warm; ++i) f();
    CK(cudaDeviceSynchronize());
    CK(cudaEventRecord(a));
    for (int i = 0; i < iters; ++i) f();
    CK(cudaEventRecord(b));
    CK(cudaEventSynchronize(b));
    float ms = 0;
    CK(cudaEventElapsedTime(&ms, a, b));
    return ms / iters;
  }
};

int main(int argc, char** argv) {
  size_t bytes = 1ull << 30;
  int iters = 20;
  std::string only;
  for (int i = 1; i + 1 < argc; i += 2) {
    std::string k = argv[i];
    if (k == "--bytes") bytes = std::strtoull(argv[i + 1], nullptr, 10);
    else if (k == "--iters") iters = std::atoi(argv[i + 1]);
    else if (k == "--case") only = argv[i + 1];
  }
  CK(cudaSetDevice(0));
  int sms = cudaSmCount(0);
  uint8_t *src, *dst;
  CK(cudaMalloc(&src, bytes + 256));
  CK(cudaMalloc(&dst, bytes + 256));
  CK(cudaMemset(src, 1, bytes + 256));
  CK(cudaMemset(dst, 2, bytes + 256));
  uint32_t* words;
  CK(cudaMalloc(&words, 256));
  CK(cudaMemset(words, 0, 256));
  Timer timer;
  auto report = [&](const std::string& name, size_t movedBytes, double ms) {
    std::printf("%-44s %10.1f us  %8.1f GB/s payload  %8.1f GB/s read+write\n", name.c_str(), ms * 1e3,
                movedBytes / (ms * 1e-3) / 1e9, 2.0 * movedBytes / (ms * 1e-3) / 1e9);
    std::fflush(stdout);
  };
  auto want = [&](const std::string& name) { return only.empty() || name.find(only) != std::string::npos; };

  if (want("memcpy")) {
    double ms = timer.run(3, iters, [&] { CK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, nullptr)); });
    report("cudaMemcpyAsync D2D", bytes, ms);
  }
  struct Shape {
    uint32_t tile, stages;
  };
  for (Shape sh : {Shape{16384, 4}, Shape{16384, 8}, Shape{32768, 2}, Shape{32768, 3}, Shape{32768, 4},
                   Shape{49152, 3}, Shape{65536, 2}, Shape{24576, 6}}) {
    char name[96];
    std::snprintf(name, sizeof(name), "bulk tile=%uK stages=%u", sh.tile / 1024, sh.stages);
    if (!want(name) && !want("bulk")) continue;
    PushTuning t;
    t.bulkTileBytes = sh.tile;
    t.bulkStages = sh.stages;
    setPushTuning(t);
    for (int ctas : {sms, sms / 2}) {
      PushPlan plan;
      CopyItem it;
      it.src = src;
      it.dst = dst;
      it.srcBytes = bytes;
      appendToPlan(plan, it, true);
      double ms = timer.run(3, iters, [&] { launchPush(plan, nullptr, ctas, words, 1, words + 16, nullptr); });
      report(std::string(name) + " ctas=" + std::to_string(ctas), bytes, ms);
    }
  }
  setPushTuning(PushTuning());
  if (want("plain")) {
    PushPlan plan;
    CopyItem it;
    it.src = src;
    it.dst = dst;
    it.srcBytes = bytes;
    appendToPlan(plan, it, false);
    double ms = timer.run(3, iters, [&] { launchPush(plan, nullptr, sms, words, 1, words + 16, nullptr); });
    report("plain ld/st (light kernel)", bytes, ms);
    PushPlan skew;
    it.src = src + 4;
    it.dst = dst + 8;
    appendToPlan(skew, it, true);
    ms = timer.run(3, iters, [&] { launchPush(skew, nullptr, sms, nullptr, 0, nullptr, nullptr); });
    report("plain, relatively misaligned by 4 bytes", bytes, ms);
  }
  if (want("cast")) {
    PushPlan plan;
    CopyItem it;
    it.src = src;
    it.dst = dst;
    it.srcBytes = bytes;
    it.srcDtype = DType::kF32;
    it.dstDtype = DType::kBF16;
    appendToPlan(plan, it, true);
    double ms = timer.run(3, iters, [&] { launchPush(plan, nullptr, sms, nullptr, 0, nullptr, nullptr); });
    std::printf("%-44s %10.1f us  %8.1f GB/s read, %8.1f GB/s read+write\n", "cast fp32 -> bf16", ms * 1e3,
                bytes / (ms * 1e-3) / 1e9, 1.5 * bytes / (ms * 1e-3) / 1e9);
  }
  if (want("strided")) {
    for (size_t es : {size_t(2), size_t(4), size_t(8)}) {
      const int64_t cols = 4096;
      const int64_t rows = static_cast<int64_t>(bytes / es / cols);
      PushPlan plan;
      CopyItem it;
      it.src = src;
      it.dst = dst;
      it.srcBytes = static_cast<uint64_t>(rows) * cols * es;
      it.strided = true;
      it.view = StridedView{es == 2 ? DType::kBF16 : es == 4 ? DType::kF32 : DType::kI64, rows, cols, 1, rows};
      it.srcDtype = it.dstDtype = it.view.dtype;
      appendToPlan(plan, it, true);
      double ms = timer.run(2, iters / 2 + 1, [&] { launchPush(plan, nullptr, sms, nullptr, 0, nullptr, nullptr); });
      report("transposed view, " + std::to_string(es) + "-byte elements", it.srcBytes, ms);
    }
  }
  if (want("band")) {
    // Transposed matrices in the form chosen for another GPU's memory (bands of whole rows, one
    // contiguous run each), here against local memory: shapes of the mixed message.
    struct Shape {
      int64_t cols;
      size_t es;
    };
    for (Shape sh : {Shape{14, 2}, Shape{132, 2}, Shape{1478, 4}, Shape{63, 8}}) {
      const int64_t rows = static_cast<int64_t>(std::min<size_t>(bytes, 256u << 20) / sh.es / sh.cols);
      for (bool band : {false, true}) {
        PushPlan plan;
        CopyItem it;
        it.src = src;
        it.dst = dst;
        it.srcBytes = static_cast<uint64_t>(rows) * sh.cols * sh.es;
        it.strided = true;
        it.view = StridedView{sh.es == 2 ? DType::kBF16 : sh.es == 4 ? DType::kF32 : DType::kI64, rows, sh.cols, 1, rows};
        it.srcDtype = it.dstDtype = it.view.dtype;
        it.remote = band;
        appendToPlan(plan, it, true);
        double ms = timer.run(2, iters / 2 + 1, [&] { launchPush(plan, nullptr, sms, nullptr, 0, nullptr, nullptr); });
        report(std::string(band ? "band" : "32x32 tiles") + ", transposed [rows, " + std::to_string(sh.cols) + "] of " +
                   std::to_string(sh.es) + "-byte elements",
               it.srcBytes, ms);
      }
    }
  }
  if (want("hoststage")) {
    // What the staged channel (cuda_basic) launches: device memory -> mapped pinned host memory
    // and back, 2 MiB pieces, sixteen pieces per launch, against the copy engine.
    const size_t total = std::min<size_t>(bytes, 32u << 20);
    uint8_t* pinned = nullptr;
    CK(cudaHostAlloc(reinterpret_cast<void**>(&pinned), total, cudaHostAllocMapped | cudaHostAllocPortable));
    auto planOf = [&](bool out) {
      PushPlan plan;
      for (size_t off = 0; off < total; off += 2u << 20) {
        CopyItem it;
        it.src = out ? src + off : pinned + off;
        it.dst = out ? pinned + off : dst + off;
        it.srcBytes = std::min<size_t>(2u << 20, total - off);
        it.remote = out;
        appendToPlan(plan, it, out);  // bulk loads read device memory only
      }
      return plan;
    };
    PushPlan outPlan = planOf(true), inPlan = planOf(false);
    double ms = timer.run(3, iters, [&] { launchPush(outPlan, nullptr, sms, words, 1, words + 16, nullptr); });
    report("stage-out: device -> pinned host, one launch", total, ms);
    ms = timer.run(3, iters, [&] { CK(cudaMemcpyAsync(pinned, src, total, cudaMemcpyDeviceToHost, nullptr)); });
    report("cudaMemcpyAsync device -> pinned host", total, ms);
    ms = timer.run(3, iters, [&] { launchPush(inPlan, nullptr, sms, words, 1, words + 16, nullptr); });
    report("stage-in: pinned host -> device, one launch", total, ms);
    ms = timer.run(3, iters, [&] { CK(cudaMemcpyAsync(dst, pinned, total, cudaMemcpyHostToDevice, nullptr)); });
    report("cudaMemcpyAsync pinned host -> device", total, ms);
    cudaFreeHost(pinned);
  }
  if (want("mixed")) {
    // The 64-tensor message of the pipe benchmarks as ONE launch of the full kernel on one GPU:
    // dtype cycles fp32 / bf16 / int64, sizes log-uniform in [1 KiB, 16 MiB], every fourth tensor a
    // transposed [rows, 64] view, every other fp32 tensor converted to bf16. The bulk pipeline and
    // the register paths run side by side in the same CTAs.
    std::mt19937_64 rng(1);
    PushPlan plan;
    uint64_t srcOff = 0, dstOff = 0, delivered = 0, read = 0;
    int fp32Count = 0;
    for (int i = 0; i < 64; ++i) {
      const DType dt = i % 3 == 0 ? DType::kF32 : (i % 3 == 1 ? DType::kBF16 : DType::kI64);
      const double lg = std::log(1024.0) + (std::log(16.0 * 1024 * 1024) - std::log(1024.0)) *
                                                (static_cast<double>(rng() % 100000) / 100000.0);
      const uint64_t es = dtypeSize(dt);
      const int64_t rows = static_cast<int64_t>(std::max<uint64_t>(1, static_cast<uint64_t>(std::exp(lg)) / es / 64));
      const uint64_t elems = static_cast<uint64_t>(rows) * 64;
      const bool cast = dt == DType::kF32 && (fp32Count++ % 2) == 0;
      CopyItem it;
      it.src = src + srcOff;
      it.dst = dst + dstOff;
      it.srcBytes = elems * es;
      it.srcDtype = dt;
      it.dstDtype = cast ? DType::kBF16 : dt;
      if (i % 4 == 3) {
        it.strided = true;
        it.view = StridedView{dt, rows, 64, 1, rows};
      }
      appendToPlan(plan, it, true);
      srcOff += (it.srcBytes + 255) / 256 * 256;
      const uint64_t out = cast ? elems * 2 : elems * es;
      dstOff += (out + 255) / 256 * 256;
      delivered += out;
      read += it.srcBytes;
    }
    if (srcOff <= bytes && dstOff <= bytes) {
      double ms = timer.run(3, iters, [&] { launchPush(plan, nullptr, sms, words, 1, words + 16, nullptr); });
      std::printf("%-44s %10.1f us  %8.1f GB/s delivered  %8.1f GB/s read+write  (%zu entries, %u bulk + %u warp tiles)\n",
                  "64-tensor mixed message, one launch", ms * 1e3, delivered / (ms * 1e-3) / 1e9,
                  (read + delivered) / (ms * 1e-3) / 1e9, plan.entries.size(), plan.bulkTiles, plan.plainTiles);
    }
  }
  if (want("small")) {
    // Launch-bound regime: back-to-back launches of a 4 KiB copy.
    for (bool bulk : {false, true}) {
      PushTuning t;
      t.bulkMinBytes = bulk ? 1024 : 512 * 1024;
      setPushTuning(t);
      PushPlan plan;
      CopyItem it;
      it.src = src;
      it.dst = dst;
      it.srcBytes = 4096;
      appendToPlan(plan, it, true);
      double ms = timer.run(20, 200, [&] { launchPush(plan, nullptr, sms, words, 1, words + 16, nullptr); });
      report(bulk ? "4 KiB, full kernel (bulk path)" : "4 KiB, light kernel", 4096, ms);
    }
    setPushTuning(PushTuning());
    double ms = timer.run(20, 200, [&] { CK(cudaMemcpyAsync(dst, src, 4096, cudaMemcpyDeviceToDevice, nullptr)); });
    report("4 KiB, cudaMemcpyAsync D2D", 4096, ms);
  }
  if (want("unpack")) {
    // The receiving side of a small message whose data has already landed: the stand-alone wait
    // kernel, and the unpack launch that looks at the flag itself before it copies 4 KiB and
    // 64 KiB out of the inbox. The flag is set beforehand, so nothing here spins.
    const uint32_t arrived = 7;
    CK(cudaMemcpy(words + 32, &arrived, sizeof(arrived), cudaMemcpyHostToDevice));
    double ms = timer.run(20, 200, [&] { launchWaitFlag(nullptr, words + 32, arrived, 1'000'000'000ull, words + 40); });
    report("wait kernel, flag already set", 0, ms);
    for (size_t n : {size_t(4096), size_t(65536)}) {
      PushPlan plan;
      CopyItem it;
      it.src = src;
      it.dst = dst;
      it.srcBytes = n;
      appendToPlan(plan, it, false);
      WaitBefore w;
      w.flag = words + 32;
      w.value = arrived;
      w.timeoutNs = 1'000'000'000ull;
      ms = timer.run(20, 200, [&] { launchPush(plan, nullptr, sms, nullptr, 0, words + 16, words + 40, w); });
      report(std::to_string(n >> 10) + " KiB unpack with the wait fused in", n, ms);
    }
  }
  return 0;
}
