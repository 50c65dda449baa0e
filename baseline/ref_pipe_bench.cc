// Benchmark harness over the REFERENCE library's public C++ API (tensorpipe::Context, Listener,
// Pipe, Message) as shipped inside PyTorch: headers from torch/include/tensorpipe, code from
// libtorch_cpu.so / libtorch_cuda.so. Nothing from this repository's library is linked in.
//
// It runs the same ring as the native benchmark: every rank owns a sending context that dials the
// next rank and a receiving context that the previous rank dials (one rank: the two talk to each
// other in-process, which selects the reference's cuda_xth channel; several ranks: cuda_ipc).
// Commands arrive on stdin, one per line, and each prints one line on stdout:
//   stream <bytes> <steps> <depth>       -> "ok <device_ms> <host_ms>"
//   latency <bytes> <laps>               -> "ok <n> <sample_us>..."   (rank 0 only has samples)
//   e2e <bytes> <steps>                  -> "ok <host_ms>"  (H2D from pinned memory every step,
//                                            D2H of a 4-byte result every step)
//   mixed <steps> <depth> <seed>         -> "ok <device_ms> <bytes_per_message>"  (64 tensors per
//                                            message with the sizes the native mixed message
//                                            DELIVERS; all contiguous and unconverted, because
//                                            the reference has neither views nor casts: the layout
//                                            work is left out in the reference's favour)
//   quit
// Protocol per step and timing points are the same as in src/tools/ring_bench.cc.
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <functional>
#include <future>
#include <iostream>
#include <cmath>
#include <mutex>
#include <random>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#include <tensorpipe/tensorpipe.h>
#include <tensorpipe/tensorpipe_cuda.h>

namespace tp = tensorpipe;
using Clock = std::chrono::steady_clock;

#define CK(x)                                                                              \
  do {                                                                                     \
    cudaError_t e_ = (x);                                                                  \
    if (e_ != cudaSuccess) {                                                               \
      std::cerr << "CUDA error " << cudaGetErrorString(e_) << " at " << __LINE__ << "\n";  \
      std::exit(2);                                                                        \
    }                                                                                      \
  } while (0)

struct Args {
  int rank = 0, world = 1, device = 0, nextDevice = 0, basePort = 29700;
  size_t maxBytes = 1ull << 30;
  std::string channels = "all";  // or "cuda_basic": only the staged CUDA channel (and basic)
};

std::shared_ptr<tp::Context> makeContext(const std::string& name, const std::string& channels) {
  auto ctx = std::make_shared<tp::Context>(tp::ContextOptions().name(name));
  ctx->registerTransport(0, "uv", tp::transport::uv::create());
  ctx->registerTransport(10, "shm", tp::transport::shm::create());
  ctx->registerChannel(0, "basic", tp::channel::basic::create());
  ctx->registerChannel(101, "cuda_basic", tp::channel::cuda_basic::create(tp::channel::basic::create()));
  if (channels != "cuda_basic") {
    ctx->registerChannel(300, "cuda_ipc", tp::channel::cuda_ipc::create());
    ctx->registerChannel(400, "cuda_xth", tp::channel::cuda_xth::create());
  }
  return ctx;
}

struct Bench {
  Args args;
  std::shared_ptr<tp::Context> sendCtx, recvCtx;
  std::shared_ptr<tp::Listener> listener;
  std::shared_ptr<tp::Pipe> sendPipe, recvPipe;
  cudaStream_t sendStream, recvStream;
  uint8_t* src;
  uint8_t* dst[2];
  cudaEvent_t evStart, evEnd;

  void setup() {
    CK(cudaSetDevice(args.device));
    CK(cudaStreamCreateWithFlags(&sendStream, cudaStreamNonBlocking));
    CK(cudaStreamCreateWithFlags(&recvStream, cudaStreamNonBlocking));
    CK(cudaMalloc(&src, args.maxBytes));
    CK(cudaMalloc(&dst[0], args.maxBytes));
    CK(cudaMalloc(&dst[1], args.maxBytes));
    CK(cudaMemset(src, 1, args.maxBytes));
    CK(cudaEventCreate(&evStart));
    CK(cudaEventCreate(&evEnd));
    sendCtx = makeContext("send" + std::to_string(args.rank), args.channels);
    recvCtx = makeContext("recv" + std::to_string(args.rank), args.channels);
    const std::string myAddr = "uv://127.0.0.1:" + std::to_string(args.basePort + args.rank);
    listener = recvCtx->listen({myAddr, "shm://tpref-" + std::to_string(args.basePort + args.rank)});
    std::promise<std::shared_ptr<tp::Pipe>> accepted;
    listener->accept([&](const tp::Error& e, std::shared_ptr<tp::Pipe> p) {
      if (e) {
        std::cerr << "accept: " << e.what() << "\n";
        std::exit(3);
      }
      accepted.set_value(std::move(p));
    });
    // The next rank may not be listening yet: dial until the handshake goes through.
    const std::string next = "uv://127.0.0.1:" + std::to_string(args.basePort + (args.rank + 1) % args.world);
    std::this_thread::sleep_for(std::chrono::milliseconds(args.world > 1 ? 1500 : 10));
    sendPipe = sendCtx->connect(next);
    recvPipe = accepted.get_future().get();
  }

  struct Segment {
    size_t offset, bytes;
  };

  double stream(size_t bytes, int steps, int depth, double* hostMs) {
    return streamSegments({Segment{0, bytes}}, steps, depth, hostMs);
  }

  // The sizes of the 64-tensor mixed message as delivered: dtype cycles fp32, bf16, int64; sizes
  // log-uniform in [1 KiB, 16 MiB] rounded to whole rows (64 columns, or for every fourth tensor a
  // column count log-uniform in [8, 4096], the transposed views of the native message); every other
  // fp32 tensor arrives as bf16. Same generator and seed as the native benchmark, so both sides
  // move the same bytes.
  static std::vector<Segment> mixedSegments(uint64_t seed, size_t* delivered) {
    std::vector<Segment> segs;
    std::mt19937_64 rng(seed);
    int fp32Count = 0;
    size_t offset = 0;
    *delivered = 0;
    for (int i = 0; i < 64; ++i) {
      const size_t es = i % 3 == 0 ? 4 : (i % 3 == 1 ? 2 : 8);
      const double lg = std::log(1024.0) + (std::log(16.0 * 1024 * 1024) - std::log(1024.0)) *
                                                (static_cast<double>(rng() % 100000) / 100000.0);
      const uint64_t bytes = static_cast<uint64_t>(std::exp(lg));
      uint64_t cols = 64;
      if (i % 4 == 3) {
        const double lc = std::log(8.0) + (std::log(4096.0) - std::log(8.0)) * (static_cast<double>(rng() % 100000) / 100000.0);
        cols = static_cast<uint64_t>(std::exp(lc));
      }
      const uint64_t rows = std::max<uint64_t>(1, bytes / es / cols);
      const uint64_t elems = rows * cols;
      bool cast = false;
      if (es == 4) cast = (fp32Count++ % 2) == 0;
      const size_t out = cast ? elems * 2 : elems * es;
      segs.push_back(Segment{offset, out});
      offset += (out + 255) / 256 * 256;
      *delivered += out;
    }
    return segs;
  }

  double streamSegments(std::vector<Segment> segs, int steps, int depth, double* hostMs) {
    struct State {
      std::mutex mu;
      int sent = 0, inflight = 0, received = 0, armed = 0, descs = 0;
      std::promise<void> recvDone, sendDone;
    };
    auto st = std::make_shared<State>();
    auto armRead = std::make_shared<std::function<void()>>();
    *armRead = [=]() {
      {
        std::unique_lock<std::mutex> l(st->mu);
        if (st->armed >= steps) return;
        ++st->armed;
      }
      recvPipe->readDescriptor([=](const tp::Error& e, tp::Descriptor d) {
        if (e) { std::cerr << "readDescriptor: " << e.what() << "\n"; std::exit(4); }
        int k;
        { std::unique_lock<std::mutex> l(st->mu); k = st->descs++; }
        tp::Allocation a;
        for (const Segment& seg : segs) {
          tp::Allocation::Tensor t;
          t.buffer = tp::CudaBuffer{dst[k & 1] + seg.offset, recvStream};
          a.tensors.push_back(t);
        }
        recvPipe->read(std::move(a), [=](const tp::Error& e2) {
          if (e2) { std::cerr << "read: " << e2.what() << "\n"; std::exit(4); }
          bool last;
          { std::unique_lock<std::mutex> l(st->mu); last = ++st->received == steps; }
          if (last) {
            cudaSetDevice(args.device);
            cudaEventRecord(evEnd, recvStream);
            st->recvDone.set_value();
          }
        });
        (*armRead)();
      });
    };
    auto pump = std::make_shared<std::function<void()>>();
    *pump = [=]() {
      for (;;) {
        {
          std::unique_lock<std::mutex> l(st->mu);
          if (st->inflight >= depth || st->sent >= steps) return;
          ++st->sent;
          ++st->inflight;
        }
        tp::Message m;
        for (const Segment& seg : segs) {
          tp::Message::Tensor t;
          t.buffer = tp::CudaBuffer{src + seg.offset, sendStream};
          t.length = seg.bytes;
          t.targetDevice = tp::Device(tp::kCudaDeviceType, args.nextDevice);
          m.tensors.push_back(t);
        }
        sendPipe->write(std::move(m), [=](const tp::Error& e) {
          if (e) { std::cerr << "write: " << e.what() << "\n"; std::exit(4); }
          bool done;
          {
            std::unique_lock<std::mutex> l(st->mu);
            --st->inflight;
            done = st->sent >= steps && st->inflight == 0;
          }
          if (done) st->sendDone.set_value();
          else (*pump)();
        });
      }
    };
    auto t0 = Clock::now();
    CK(cudaEventRecord(evStart, recvStream));
    (*armRead)();
    (*pump)();
    st->recvDone.get_future().wait();
    st->sendDone.get_future().wait();
    *armRead = nullptr;
    *pump = nullptr;
    CK(cudaEventSynchronize(evEnd));
    *hostMs = std::chrono::duration<double, std::milli>(Clock::now() - t0).count();
    float ms = 0;
    CK(cudaEventElapsedTime(&ms, evStart, evEnd));
    CK(cudaStreamSynchronize(sendStream));
    return ms;
  }

  std::vector<double> latency(size_t bytes, int laps) {
    struct State {
      std::mutex mu;
      int lapsDone = 0;
      std::vector<double> samples;
      Clock::time_point t0;
      std::promise<void> done;
    };
    auto st = std::make_shared<State>();
    const bool starter = args.rank == 0;
    const int world = args.world;
    auto sendToken = std::make_shared<std::function<void()>>();
    *sendToken = [=]() {
      tp::Message m;
      tp::Message::Tensor t;
      t.buffer = tp::CudaBuffer{src, sendStream};
      t.length = bytes;
      t.targetDevice = tp::Device(tp::kCudaDeviceType, args.nextDevice);
      m.tensors.push_back(t);
      if (starter) st->t0 = Clock::now();
      sendPipe->write(std::move(m), [](const tp::Error& e) {
        if (e) { std::cerr << "write: " << e.what() << "\n"; std::exit(4); }
      });
    };
    auto armRead = std::make_shared<std::function<void()>>();
    *armRead = [=]() {
      recvPipe->readDescriptor([=](const tp::Error& e, tp::Descriptor) {
        if (e) { std::cerr << "readDescriptor: " << e.what() << "\n"; std::exit(4); }
        tp::Allocation a;
        tp::Allocation::Tensor t;
        t.buffer = tp::CudaBuffer{dst[0], recvStream};
        a.tensors.push_back(t);
        recvPipe->read(std::move(a), [=](const tp::Error& e2) {
          if (e2) { std::cerr << "read: " << e2.what() << "\n"; std::exit(4); }
          cudaSetDevice(args.device);
          cudaStreamSynchronize(recvStream);
          int done;
          {
            std::unique_lock<std::mutex> l(st->mu);
            if (starter)
              st->samples.push_back(std::chrono::duration<double, std::micro>(Clock::now() - st->t0).count() / world);
            done = ++st->lapsDone;
          }
          if (done < laps) {
            (*armRead)();
            (*sendToken)();
          } else {
            if (!starter) (*sendToken)();
            st->done.set_value();
          }
        });
      });
    };
    (*armRead)();
    if (starter) (*sendToken)();
    st->done.get_future().wait();
    CK(cudaStreamSynchronize(sendStream));
    std::this_thread::sleep_for(std::chrono::milliseconds(20));
    *armRead = nullptr;
    *sendToken = nullptr;
    return st->samples;
  }

  // Host-driven steps: H2D from pinned memory, send, receive, read a 4-byte result back.
  double e2e(size_t bytes, int steps) {
    uint8_t* hostIn;
    uint32_t* hostOut;
    CK(cudaMallocHost(&hostIn, bytes));
    CK(cudaMallocHost(&hostOut, 4));
    for (size_t i = 0; i < bytes; i += 4096) hostIn[i] = static_cast<uint8_t>(i);
    auto step = [&](int i) {
      CK(cudaMemcpyAsync(src, hostIn, bytes, cudaMemcpyHostToDevice, sendStream));
      std::promise<void> wrote, got;
      tp::Message m;
      tp::Message::Tensor t;
      t.buffer = tp::CudaBuffer{src, sendStream};
      t.length = bytes;
      t.targetDevice = tp::Device(tp::kCudaDeviceType, args.nextDevice);
      m.tensors.push_back(t);
      sendPipe->write(std::move(m), [&](const tp::Error& e) {
        if (e) { std::cerr << "write: " << e.what() << "\n"; std::exit(4); }
        wrote.set_value();
      });
      recvPipe->readDescriptor([&, i](const tp::Error& e, tp::Descriptor) {
        if (e) { std::cerr << "readDescriptor: " << e.what() << "\n"; std::exit(4); }
        tp::Allocation a;
        tp::Allocation::Tensor at;
        at.buffer = tp::CudaBuffer{dst[i & 1], recvStream};
        a.tensors.push_back(at);
        recvPipe->read(std::move(a), [&](const tp::Error& e2) {
          if (e2) { std::cerr << "read: " << e2.what() << "\n"; std::exit(4); }
          got.set_value();
        });
      });
      got.get_future().wait();
      wrote.get_future().wait();
      CK(cudaMemcpyAsync(hostOut, dst[i & 1], 4, cudaMemcpyDeviceToHost, recvStream));
      CK(cudaStreamSynchronize(recvStream));
      CK(cudaStreamSynchronize(sendStream));
    };
    for (int i = 0; i < 3; ++i) step(i);
    std::cout << "ready" << std::endl;  // the driver puts a barrier here
    std::string go;
    std::getline(std::cin, go);
    auto t0 = Clock::now();
    for (int i = 0; i < steps; ++i) step(i);
    double ms = std::chrono::duration<double, std::milli>(Clock::now() - t0).count();
    cudaFreeHost(hostIn);
    cudaFreeHost(hostOut);
    return ms;
  }
};

int main(int argc, char** argv) {
  Args args;
  for (int i = 1; i + 1 < argc; i += 2) {
    std::string k = argv[i];
    std::string v = argv[i + 1];
    if (k == "--rank") args.rank = std::stoi(v);
    else if (k == "--world") args.world = std::stoi(v);
    else if (k == "--device") args.device = std::stoi(v);
    else if (k == "--next-device") args.nextDevice = std::stoi(v);
    else if (k == "--base-port") args.basePort = std::stoi(v);
    else if (k == "--max-bytes") args.maxBytes = std::stoull(v);
    else if (k == "--channels") args.channels = v;
  }
  Bench b;
  b.args = args;
  b.setup();
  std::cout << "up" << std::endl;
  std::string line;
  while (std::getline(std::cin, line)) {
    std::istringstream in(line);
    std::string cmd;
    in >> cmd;
    if (cmd == "quit") break;
    if (cmd == "stream") {
      size_t bytes;
      int steps, depth;
      in >> bytes >> steps >> depth;
      double host = 0;
      double ms = b.stream(bytes, steps, depth, &host);
      std::cout << "ok " << ms << " " << host << std::endl;
    } else if (cmd == "mixed") {
      int steps, depth;
      uint64_t seed;
      in >> steps >> depth >> seed;
      size_t delivered = 0;
      auto segs = Bench::mixedSegments(seed, &delivered);
      double host = 0;
      double ms = b.streamSegments(segs, steps, depth, &host);
      std::cout << "ok " << ms << " " << delivered << std::endl;
    } else if (cmd == "latency") {
      size_t bytes;
      int laps;
      in >> bytes >> laps;
      auto s = b.latency(bytes, laps);
      std::cout << "ok " << s.size();
      for (double v : s) std::cout << " " << v;
      std::cout << std::endl;
    } else if (cmd == "e2e") {
      size_t bytes;
      int steps;
      in >> bytes >> steps;
      double ms = b.e2e(bytes, steps);
      std::cout << "ok " << ms << std::endl;
    } else {
      std::cout << "error unknown command" << std::endl;
    }
  }
  b.sendPipe.reset();
  b.recvPipe.reset();
  b.listener.reset();
  b.sendCtx->join();
  b.recvCtx->join();
  return 0;
}
