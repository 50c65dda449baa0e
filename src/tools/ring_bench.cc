#include "tools/ring_bench.h"

#include <atomic>
#include <chrono>
#include <cmath>
#include <future>
#include <mutex>
#include <random>
#include <thread>

#include <tpb/tpb.h>

#include "common/cuda.h"
#include "kernels/push.h"

namespace tpb {
namespace tools {

namespace {
using Clock = std::chrono::steady_clock;
double msSince(Clock::time_point t0) {
  return std::chrono::duration<double, std::milli>(Clock::now() - t0).count();
}
void failOn(const Error& e, const char* what) {
  if (e) throw std::runtime_error(std::string(what) + ": " + e.what());
}
template <typename T>
T waitOrThrow(std::future<T>& f, int seconds, const char* what) {
  if (f.wait_for(std::chrono::seconds(seconds)) != std::future_status::ready)
    throw std::runtime_error(std::string("timed out: ") + what);
  return f.get();
}
}  // namespace

struct RingBench::Impl {
  RingBenchOptions opts;
  std::shared_ptr<Context> sendCtx, recvCtx;
  std::shared_ptr<Listener> listener;
  std::shared_ptr<Pipe> sendPipe, recvPipe;
  int nextDevice = 0;
  cudaStream_t sendStream = nullptr, recvStream = nullptr;
  uint8_t* src = nullptr;
  uint8_t* dst[2] = {nullptr, nullptr};
  unsigned long long* mismatches = nullptr;
  cudaEvent_t evStart = nullptr, evEnd = nullptr;
  uint64_t srcSeed = 0;
  std::vector<std::shared_ptr<Pipe>> meshSend, meshRecv;  // all-pairs mode
  std::vector<int> meshSendDevice;
  std::vector<cudaStream_t> meshSendStream;  // one stream per destination so pushes overlap
  uint8_t* hostIn = nullptr;   // end-to-end mode: the pinned source ...
  size_t hostInBytes = 0;
  uint32_t* hostOut = nullptr;  // ... and where the step's result lands

  PhaseResult runMixedOn(const std::vector<std::shared_ptr<Pipe>>& sendPipes, const std::vector<int>& sendDevices,
                         const std::vector<cudaStream_t>& sendStreams,
                         const std::vector<std::shared_ptr<Pipe>>& recvPipes, int steps, uint64_t seed,
                         uint64_t* bytesPerMessage);
  uint64_t verifyMixed(uint64_t seed);

  std::shared_ptr<Context> makeContext(const std::string& name) {
    auto ctx = std::make_shared<Context>(ContextOptions().name(name));
    ctx->registerTransport(0, "uv", transport::uv::create());
    if (opts.useShm) ctx->registerTransport(10, "shm", transport::shm::create());
    auto basic = channel::basic::create();
    ctx->registerChannel(0, "basic", basic);
    if (opts.channel == "cuda_basic") {
      ctx->registerChannel(5, "cuda_basic", channel::cuda_basic::create(channel::basic::create()));
    } else {
      channel::cuda_p2p::Options o;
      o.useBulkCopy = opts.useBulkCopy;
      o.waitWithKernel = opts.waitWithKernel;
      o.eagerThreshold = opts.eagerThreshold;
      o.maxCtas = opts.maxCtas;
      ctx->registerChannel(10, "cuda_p2p", channel::cuda_p2p::create(o));
    }
    return ctx;
  }

  // A tensor-less message to the next rank and one from the previous rank: lines neighbouring
  // ranks up to within one message latency before a timed region starts (a collective barrier
  // leaves them hundreds of microseconds apart).
  void syncNeighbours() { syncOn(sendPipe, recvPipe); }
  void syncOn(const std::shared_ptr<Pipe>& sendPipe, const std::shared_ptr<Pipe>& recvPipe) {
    std::promise<Error> wrote, got;
    Message m;
    m.metadata = "sync";
    sendPipe->write(std::move(m), [&](const Error& e) { wrote.set_value(e); });
    recvPipe->readDescriptor([&](const Error& e, Descriptor) {
      if (e) return got.set_value(e);
      recvPipe->read(Allocation(), [&](const Error& e2) { got.set_value(e2); });
    });
    auto fg = got.get_future();
    auto fw = wrote.get_future();
    failOn(waitOrThrow(fg, 120, "sync message from the previous rank"), "sync read");
    failOn(waitOrThrow(fw, 120, "sync message to the next rank"), "sync write");
  }

  void fillSource(size_t bytes, uint64_t seed) {
    kernels::launchFill(sendStream, src, bytes, seed);
    TPB_CUDA_CHECK(cudaStreamSynchronize(sendStream));
    srcSeed = seed;
  }
};

RingBench::RingBench(RingBenchOptions opts) : impl_(new Impl) {
  Impl& m = *impl_;
  m.opts = opts;
  TPB_CUDA_CHECK(cudaSetDevice(opts.device));
  TPB_CUDA_CHECK(cudaStreamCreateWithFlags(&m.sendStream, cudaStreamNonBlocking));
  TPB_CUDA_CHECK(cudaStreamCreateWithFlags(&m.recvStream, cudaStreamNonBlocking));
  TPB_CUDA_CHECK(cudaMalloc(&m.src, opts.maxBytes));
  TPB_CUDA_CHECK(cudaMalloc(&m.dst[0], opts.maxBytes));
  TPB_CUDA_CHECK(cudaMalloc(&m.dst[1], opts.maxBytes));
  TPB_CUDA_CHECK(cudaMalloc(&m.mismatches, sizeof(unsigned long long)));
  TPB_CUDA_CHECK(cudaMemset(m.mismatches, 0, sizeof(unsigned long long)));
  TPB_CUDA_CHECK(cudaEventCreate(&m.evStart));
  TPB_CUDA_CHECK(cudaEventCreate(&m.evEnd));
  m.sendCtx = m.makeContext("send" + std::to_string(opts.device));
  m.recvCtx = m.makeContext("recv" + std::to_string(opts.device));
  std::vector<std::string> urls = {"uv://127.0.0.1"};
  if (opts.useShm) urls.push_back("shm://");
  m.listener = m.recvCtx->listen(urls);
}

RingBench::~RingBench() {
  Impl& m = *impl_;
  m.sendPipe.reset();
  m.recvPipe.reset();
  m.meshSend.clear();
  m.meshRecv.clear();
  m.listener.reset();
  if (m.sendCtx) m.sendCtx->join();
  if (m.recvCtx) m.recvCtx->join();
  cudaSetDevice(m.opts.device);
  cudaDeviceSynchronize();
  if (m.hostIn) cudaFreeHost(m.hostIn);
  if (m.hostOut) cudaFreeHost(m.hostOut);
  cudaFree(m.src);
  cudaFree(m.dst[0]);
  cudaFree(m.dst[1]);
  cudaFree(m.mismatches);
  cudaEventDestroy(m.evStart);
  cudaEventDestroy(m.evEnd);
  cudaStreamDestroy(m.sendStream);
  cudaStreamDestroy(m.recvStream);
}

std::string RingBench::listenUrl() const { return impl_->listener->url("uv"); }

void RingBench::connect(const std::string& nextUrl) {
  Impl& m = *impl_;
  std::promise<std::pair<Error, std::shared_ptr<Pipe>>> accepted;
  m.listener->accept([&](const Error& e, std::shared_ptr<Pipe> p) { accepted.set_value({e, std::move(p)}); });
  // "url|device": the device index the next rank receives on.
  std::string url = nextUrl;
  m.nextDevice = m.opts.device;
  auto bar = nextUrl.rfind('|');
  if (bar != std::string::npos) {
    url = nextUrl.substr(0, bar);
    m.nextDevice = std::stoi(nextUrl.substr(bar + 1));
  }
  m.sendPipe = m.sendCtx->connect(url);
  auto f = accepted.get_future();
  auto [e, p] = waitOrThrow(f, 60, "accepting the previous rank's pipe");
  failOn(e, "accept");
  m.recvPipe = std::move(p);
}

PhaseResult RingBench::runStream(size_t bytes, int steps, int depth, bool verify) {
  Impl& m = *impl_;
  if (bytes > m.opts.maxBytes) throw std::runtime_error("tensor larger than the benchmark's buffers");
  TPB_CUDA_CHECK(cudaSetDevice(m.opts.device));
  if (verify) {
    m.fillSource(bytes, 0x5eed0000 + bytes);
    TPB_CUDA_CHECK(cudaMemsetAsync(m.mismatches, 0, sizeof(unsigned long long), m.recvStream));
    TPB_CUDA_CHECK(cudaMemsetAsync(m.dst[0], 0, bytes, m.recvStream));
    TPB_CUDA_CHECK(cudaMemsetAsync(m.dst[1], 0, bytes, m.recvStream));
    TPB_CUDA_CHECK(cudaStreamSynchronize(m.recvStream));
    depth = 1;
  }
  const uint64_t launches0 = kernels::launchCount();

  struct State {
    std::mutex mu;
    int sent = 0, inflight = 0, received = 0, armed = 0, descs = 0;
    Error error;
    std::promise<void> recvDone, sendDone;
    bool recvSet = false, sendSet = false;
  };
  auto st = std::make_shared<State>();
  Impl* mp = &m;

  // ---- receiver: descriptor -> allocation -> read, re-armed as soon as the read is issued ----
  auto armRead = std::make_shared<std::function<void()>>();
  *armRead = [=]() {
    {
      std::unique_lock<std::mutex> l(st->mu);
      if (st->armed >= steps || st->error) return;
      ++st->armed;
    }
    mp->recvPipe->readDescriptor([=](const Error& e, Descriptor d) {
      if (e) {
        std::unique_lock<std::mutex> l(st->mu);
        st->error = e;
        if (!st->recvSet) { st->recvSet = true; st->recvDone.set_value(); }
        return;
      }
      int k;
      {
        std::unique_lock<std::mutex> l(st->mu);
        k = st->descs++;
      }
      Allocation a;
      Allocation::Tensor t;
      t.buffer = CudaBuffer{mp->dst[k & 1], mp->recvStream, mp->opts.device};
      a.tensors.push_back(t);
      mp->recvPipe->read(std::move(a), [=](const Error& e2) {
        bool last = false;
        {
          std::unique_lock<std::mutex> l(st->mu);
          if (e2) st->error = e2;
          ++st->received;
          last = st->received == steps || bool(st->error);
        }
        if (!e2 && verify) {
          cudaSetDevice(mp->opts.device);
          kernels::launchVerify(mp->recvStream, mp->dst[k & 1], bytes, mp->srcSeed, mp->mismatches);
          cudaStreamSynchronize(mp->recvStream);
        }
        if (last) {
          cudaSetDevice(mp->opts.device);
          cudaEventRecord(mp->evEnd, mp->recvStream);
          std::unique_lock<std::mutex> l(st->mu);
          if (!st->recvSet) { st->recvSet = true; st->recvDone.set_value(); }
        } else if (verify) {
          (*armRead)();
        }
      });
      if (!verify) (*armRead)();
    });
  };

  // ---- sender: keep `depth` writes in flight ----
  auto pump = std::make_shared<std::function<void()>>();
  *pump = [=]() {
    for (;;) {
      {
        std::unique_lock<std::mutex> l(st->mu);
        if (st->error || st->inflight >= depth || st->sent >= steps) {
          if ((st->sent >= steps && st->inflight == 0) || st->error) {
            if (!st->sendSet) { st->sendSet = true; st->sendDone.set_value(); }
          }
          return;
        }
        ++st->sent;
        ++st->inflight;
      }
      Message msg;
      Message::Tensor t;
      t.buffer = CudaBuffer{mp->src, mp->sendStream, mp->opts.device};
      t.length = bytes;
      t.targetDevice = Device(kCudaDeviceType, mp->nextDevice);
      t.dtype = DType::kBF16;
      msg.tensors.push_back(t);
      mp->sendPipe->write(std::move(msg), [=](const Error& e) {
        {
          std::unique_lock<std::mutex> l(st->mu);
          if (e) st->error = e;
          --st->inflight;
        }
        (*pump)();
      });
    }
  };

  m.syncNeighbours();
  auto t0 = Clock::now();
  TPB_CUDA_CHECK(cudaEventRecord(m.evStart, m.recvStream));
  (*armRead)();
  (*pump)();
  auto fr = st->recvDone.get_future();
  auto fs = st->sendDone.get_future();
  waitOrThrow(fr, 300, "receiving");
  waitOrThrow(fs, 300, "sending");
  // Break the self-references of the recursive closures.
  *armRead = nullptr;
  *pump = nullptr;
  failOn(st->error, "ring stream");
  TPB_CUDA_CHECK(cudaEventSynchronize(m.evEnd));
  PhaseResult r;
  r.hostMs = msSince(t0);
  float ms = 0;
  TPB_CUDA_CHECK(cudaEventElapsedTime(&ms, m.evStart, m.evEnd));
  r.deviceMs = ms;
  TPB_CUDA_CHECK(cudaStreamSynchronize(m.sendStream));
  if (verify) {
    unsigned long long bad = 0;
    TPB_CUDA_CHECK(cudaMemcpy(&bad, m.mismatches, sizeof(bad), cudaMemcpyDeviceToHost));
    r.mismatches = bad;
  }
  r.kernelLaunches = kernels::launchCount() - launches0;
  return r;
}

PhaseResult RingBench::runEndToEnd(size_t bytes, int steps, bool verify) {
  Impl& m = *impl_;
  if (bytes > m.opts.maxBytes) throw std::runtime_error("tensor larger than the benchmark's buffers");
  TPB_CUDA_CHECK(cudaSetDevice(m.opts.device));
  constexpr uint64_t kSeed = 0xe2e0000;
  if (m.hostInBytes < bytes) {
    if (m.hostIn) cudaFreeHost(m.hostIn);
    m.hostIn = nullptr;
    TPB_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&m.hostIn), bytes, cudaHostAllocPortable));
    m.hostInBytes = bytes;
    // Pinned memory is addressable from the device: the fill kernel writes the pattern into it.
    kernels::launchFill(m.sendStream, m.hostIn, bytes, kSeed);
    TPB_CUDA_CHECK(cudaStreamSynchronize(m.sendStream));
  }
  if (!m.hostOut) TPB_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&m.hostOut), 64, cudaHostAllocPortable));
  const uint64_t launches0 = kernels::launchCount();
  auto step = [&](int i) {
    std::promise<Error> wrote, got;
    Message msg;
    Message::Tensor t;
    t.buffer = CudaBuffer{m.hostIn, m.sendStream, m.opts.device};
    t.length = bytes;
    t.targetDevice = Device(kCudaDeviceType, m.nextDevice);
    msg.tensors.push_back(t);
    m.sendPipe->write(std::move(msg), [&](const Error& e) { wrote.set_value(e); });
    m.recvPipe->readDescriptor([&, i](const Error& e, Descriptor) {
      if (e) return got.set_value(e);
      Allocation a;
      Allocation::Tensor at;
      at.buffer = CudaBuffer{m.dst[i & 1], m.recvStream, m.opts.device};
      a.tensors.push_back(at);
      m.recvPipe->read(std::move(a), [&](const Error& e2) { got.set_value(e2); });
    });
    auto fg = got.get_future();
    auto fw = wrote.get_future();
    failOn(waitOrThrow(fg, 120, "end-to-end read"), "read");
    failOn(waitOrThrow(fw, 120, "end-to-end write"), "write");
    TPB_CUDA_CHECK(cudaMemcpyAsync(m.hostOut, m.dst[i & 1], 4, cudaMemcpyDeviceToHost, m.recvStream));
    TPB_CUDA_CHECK(cudaStreamSynchronize(m.recvStream));
    TPB_CUDA_CHECK(cudaStreamSynchronize(m.sendStream));
  };
  PhaseResult r;
  auto t0 = Clock::now();
  for (int i = 0; i < steps; ++i) step(i);
  r.hostMs = msSince(t0);
  r.deviceMs = r.hostMs;
  r.kernelLaunches = kernels::launchCount() - launches0;
  if (verify && steps > 0) {
    TPB_CUDA_CHECK(cudaMemsetAsync(m.mismatches, 0, sizeof(unsigned long long), m.recvStream));
    kernels::launchVerify(m.recvStream, m.dst[(steps - 1) & 1], bytes, kSeed, m.mismatches);
    unsigned long long bad = 0;
    TPB_CUDA_CHECK(cudaMemcpyAsync(&bad, m.mismatches, sizeof(bad), cudaMemcpyDeviceToHost, m.recvStream));
    TPB_CUDA_CHECK(cudaStreamSynchronize(m.recvStream));
    r.mismatches = bad;
  }
  return r;
}

std::vector<double> RingBench::runLatency(size_t bytes, int laps, int rank, int world) {
  Impl& m = *impl_;
  TPB_CUDA_CHECK(cudaSetDevice(m.opts.device));
  struct State {
    std::mutex mu;
    int lapsDone = 0;
    Error error;
    std::vector<double> samples;
    Clock::time_point t0;
    std::promise<void> done;
    bool set = false;
  };
  auto st = std::make_shared<State>();
  Impl* mp = &m;
  const bool starter = rank == 0;

  auto finish = [=]() {
    std::unique_lock<std::mutex> l(st->mu);
    if (!st->set) { st->set = true; st->done.set_value(); }
  };
  auto sendToken = std::make_shared<std::function<void()>>();
  *sendToken = [=]() {
    Message msg;
    Message::Tensor t;
    t.buffer = CudaBuffer{mp->src, mp->sendStream, mp->opts.device};
    t.length = bytes;
    t.targetDevice = Device(kCudaDeviceType, mp->nextDevice);
    msg.tensors.push_back(t);
    if (starter) st->t0 = Clock::now();
    mp->sendPipe->write(std::move(msg), [=](const Error& e) {
      if (e) {
        { std::unique_lock<std::mutex> l(st->mu); st->error = e; }
        finish();
      }
    });
  };
  auto armRead = std::make_shared<std::function<void()>>();
  *armRead = [=]() {
    mp->recvPipe->readDescriptor([=](const Error& e, Descriptor) {
      if (e) {
        { std::unique_lock<std::mutex> l(st->mu); st->error = e; }
        return finish();
      }
      Allocation a;
      Allocation::Tensor t;
      t.buffer = CudaBuffer{mp->dst[0], mp->recvStream, mp->opts.device};
      a.tensors.push_back(t);
      mp->recvPipe->read(std::move(a), [=](const Error& e2) {
        if (e2) {
          { std::unique_lock<std::mutex> l(st->mu); st->error = e2; }
          return finish();
        }
        cudaSetDevice(mp->opts.device);
        cudaStreamSynchronize(mp->recvStream);  // the data is on the device now
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
          if (!starter) (*sendToken)();  // pass the last token on so the starter finishes its lap
          finish();
        }
      });
    });
  };
  (*armRead)();
  if (starter) (*sendToken)();
  auto f = st->done.get_future();
  waitOrThrow(f, 300, "latency laps");
  // Let the final write of a non-starter complete before tearing the closures down.
  TPB_CUDA_CHECK(cudaStreamSynchronize(m.sendStream));
  std::this_thread::sleep_for(std::chrono::milliseconds(20));
  *armRead = nullptr;
  *sendToken = nullptr;
  failOn(st->error, "ring latency");
  return st->samples;
}

namespace {
// 64 tensors: dtype cycles fp32, bf16, int64; sizes log-uniform in [1 KiB, 16 MiB]; every 4th is a
// transposed 2-D view whose column count is drawn log-uniformly from [8, 4096] (so that no single
// code path of the kernel is favoured); every other fp32 tensor is cast to bf16 by the receiver.
struct MixedSpec {
  DType dtype;
  bool transposed;
  bool cast;
  int64_t rows, cols;
  uint64_t srcOff, dstOff, srcBytes, dstBytes;
};
struct MixedLayout {
  std::vector<MixedSpec> specs;
  uint64_t srcTotal = 0, dstTotal = 0, delivered = 0;
};
MixedLayout makeMixedLayout(uint64_t seed) {
  MixedLayout L;
  std::mt19937_64 rng(seed);
  int fp32Count = 0;
  for (int i = 0; i < 64; ++i) {
    MixedSpec s{};
    s.dtype = i % 3 == 0 ? DType::kF32 : (i % 3 == 1 ? DType::kBF16 : DType::kI64);
    const double lg = std::log(1024.0) + (std::log(16.0 * 1024 * 1024) - std::log(1024.0)) *
                                              (static_cast<double>(rng() % 100000) / 100000.0);
    const uint64_t bytes = static_cast<uint64_t>(std::exp(lg));
    const uint64_t es = dtypeSize(s.dtype);
    s.transposed = i % 4 == 3;
    s.cols = 64;
    if (s.transposed) {
      const double lc = std::log(8.0) + (std::log(4096.0) - std::log(8.0)) * (static_cast<double>(rng() % 100000) / 100000.0);
      s.cols = static_cast<int64_t>(std::exp(lc));
    }
    s.rows = static_cast<int64_t>(std::max<uint64_t>(1, bytes / es / s.cols));
    const uint64_t elems = static_cast<uint64_t>(s.rows) * s.cols;
    s.srcBytes = elems * es;
    if (s.dtype == DType::kF32) s.cast = (fp32Count++ % 2) == 0;
    s.dstBytes = s.cast ? elems * 2 : s.srcBytes;
    s.srcOff = L.srcTotal;
    s.dstOff = L.dstTotal;
    L.srcTotal += (s.srcBytes + 255) / 256 * 256;
    L.dstTotal += (s.dstBytes + 255) / 256 * 256;
    L.delivered += s.dstBytes;
    L.specs.push_back(s);
  }
  return L;
}
}  // namespace

void RingBench::connectMesh(const std::vector<std::string>& urls, int rank) {
  Impl& m = *impl_;
  const int world = static_cast<int>(urls.size());
  std::mutex mu;
  std::vector<std::shared_ptr<Pipe>> accepted;
  std::promise<void> all;
  std::function<void()> arm = [&]() {
    m.listener->accept([&](const Error& e, std::shared_ptr<Pipe> p) {
      if (e) return;
      bool done;
      {
        std::unique_lock<std::mutex> l(mu);
        accepted.push_back(std::move(p));
        done = static_cast<int>(accepted.size()) == world - 1;
      }
      if (done) all.set_value();
      else arm();
    });
  };
  if (world > 1) arm();
  // Peers in rotation order (rank+1, rank+2, ...): the sends of one round are launched in this
  // order, so at any moment the ranks target distinct receivers instead of all converging on rank 0
  // first (an all-to-all's usual schedule; with every rank starting at peer 0 the receivers' links
  // take turns being oversubscribed sevenfold while the others idle).
  for (int d = 1; d < world; ++d) {
    const int j = (rank + d) % world;
    std::string url = urls[j];
    int dev = m.opts.device;
    auto bar = url.rfind('|');
    if (bar != std::string::npos) {
      dev = std::stoi(url.substr(bar + 1));
      url = url.substr(0, bar);
    }
    m.meshSend.push_back(m.sendCtx->connect(url));
    m.meshSendDevice.push_back(dev);
    cudaStream_t st = nullptr;
    TPB_CUDA_CHECK(cudaSetDevice(m.opts.device));
    TPB_CUDA_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    m.meshSendStream.push_back(st);
  }
  if (world > 1) {
    auto f = all.get_future();
    waitOrThrow(f, 120, "accepting the mesh's pipes");
  }
  m.meshRecv = accepted;
}

PhaseResult RingBench::runMixedMesh(int steps, uint64_t seed, uint64_t* bytesPerMessage) {
  Impl& m = *impl_;
  return m.runMixedOn(m.meshSend, m.meshSendDevice, m.meshSendStream, m.meshRecv, steps, seed, bytesPerMessage);
}

namespace {
uint16_t toBf16(uint32_t bits) {
  if ((bits & 0x7f800000u) == 0x7f800000u && (bits & 0x007fffffu)) return 0x7fff;  // NaN (compared loosely)
  const uint32_t lsb = (bits >> 16) & 1;
  return static_cast<uint16_t>((bits + 0x7fffu + lsb) >> 16);
}
bool isNanBf16(uint16_t v) { return (v & 0x7f80) == 0x7f80 && (v & 0x7f); }
}  // namespace

// One message from a source filled with the seeded pattern, then every delivered tensor against
// a CPU restatement of what the sender's kernel must have done with it: gather of the transposed
// views, round-to-nearest-even conversion of the fp32 tensors the receiver wanted as bf16, plain
// bytes for the rest. Returns the number of elements that differ.
uint64_t RingBench::Impl::verifyMixed(uint64_t seed) {
  Impl& m = *this;
  TPB_CUDA_CHECK(cudaSetDevice(m.opts.device));
  const MixedLayout layout = makeMixedLayout(seed);
  const uint64_t fillSeed = 0xfeed0000 + seed;
  kernels::launchFill(m.sendStream, m.src, layout.srcTotal, fillSeed);
  TPB_CUDA_CHECK(cudaStreamSynchronize(m.sendStream));
  TPB_CUDA_CHECK(cudaMemsetAsync(m.dst[0], 0xA5, layout.dstTotal, m.recvStream));
  TPB_CUDA_CHECK(cudaStreamSynchronize(m.recvStream));
  uint64_t bytes = 0;
  runMixedOn({m.sendPipe}, {m.nextDevice}, {m.sendStream}, {m.recvPipe}, 1, seed, &bytes);
  TPB_CUDA_CHECK(cudaStreamSynchronize(m.recvStream));
  std::vector<uint8_t> got(layout.dstTotal);
  TPB_CUDA_CHECK(cudaMemcpy(got.data(), m.dst[0], got.size(), cudaMemcpyDeviceToHost));
  // The source as the sender saw it (every rank fills the same pattern).
  std::vector<uint32_t> src((layout.srcTotal + 3) / 4);
  for (size_t w = 0; w < src.size(); ++w) {
    uint32_t v = 0;
    for (int b = 0; b < 4; ++b) v |= static_cast<uint32_t>(kernels::patternByte(fillSeed, w * 4 + b)) << (8 * b);
    src[w] = v;
  }
  const uint8_t* srcBytes = reinterpret_cast<const uint8_t*>(src.data());
  uint64_t bad = 0;
  for (const MixedSpec& s : layout.specs) {
    const size_t es = dtypeSize(s.dtype);
    const uint8_t* in = srcBytes + s.srcOff;
    const uint8_t* out = got.data() + s.dstOff;
    const uint64_t elems = static_cast<uint64_t>(s.rows) * s.cols;
    for (uint64_t i = 0; i < elems; ++i) {
      // element i of the delivered (packed, row-major [rows, cols]) tensor
      uint64_t from = i;
      if (s.transposed) from = (i % s.cols) * static_cast<uint64_t>(s.rows) + i / s.cols;
      if (s.cast) {
        uint32_t bits;
        std::memcpy(&bits, in + from * 4, 4);
        uint16_t want = toBf16(bits), have;
        std::memcpy(&have, out + i * 2, 2);
        if (want != have && !(isNanBf16(want) && isNanBf16(have))) ++bad;
      } else if (std::memcmp(in + from * es, out + i * es, es) != 0) {
        ++bad;
      }
    }
  }
  return bad;
}

PhaseResult RingBench::runMixed(int steps, uint64_t seed, uint64_t* bytesPerStep, bool verify) {
  Impl& m = *impl_;
  if (verify) {
    PhaseResult r;
    r.mismatches = m.verifyMixed(seed);
    if (bytesPerStep) *bytesPerStep = makeMixedLayout(seed).delivered;
    return r;
  }
  return m.runMixedOn({m.sendPipe}, {m.nextDevice}, {m.sendStream}, {m.recvPipe}, steps, seed, bytesPerStep);
}

PhaseResult RingBench::Impl::runMixedOn(const std::vector<std::shared_ptr<Pipe>>& sendPipes,
                                        const std::vector<int>& sendDevices,
                                        const std::vector<cudaStream_t>& sendStreams,
                                        const std::vector<std::shared_ptr<Pipe>>& recvPipes, int steps,
                                        uint64_t seed, uint64_t* bytesPerMessage) {
  Impl& m = *this;
  TPB_CUDA_CHECK(cudaSetDevice(m.opts.device));
  auto layout = std::make_shared<MixedLayout>(makeMixedLayout(seed));
  if (layout->srcTotal > m.opts.maxBytes || layout->dstTotal * recvPipes.size() > m.opts.maxBytes)
    throw std::runtime_error("mixed messages larger than the benchmark's buffers");
  if (bytesPerMessage) *bytesPerMessage = layout->delivered;
  const uint64_t launches0 = kernels::launchCount();
  const int totalRecv = steps * static_cast<int>(recvPipes.size());
  const int totalSend = steps * static_cast<int>(sendPipes.size());

  struct State {
    std::mutex mu;
    int received = 0, sent = 0;
    Error error;
    std::promise<void> recvDone, sendDone;
    bool recvSet = false, sendSet = false;
  };
  auto st = std::make_shared<State>();
  Impl* mp = &m;

  // Two receive chains per incoming pipe (two messages in flight, like the single-tensor stream),
  // alternating between the two destination buffers; each pipe has its own region in both.
  auto readsIssued = std::make_shared<std::vector<int>>(recvPipes.size(), 0);
  auto armRead = std::make_shared<std::function<void(size_t, int)>>();
  *armRead = [=](size_t k, int remaining) {
    if (remaining == 0) return;
    auto pipe = recvPipes[k];
    pipe->readDescriptor([=](const Error& e, Descriptor d) {
      auto fail = [&](const Error& err) {
        std::unique_lock<std::mutex> l(st->mu);
        st->error = err;
        if (!st->recvSet) { st->recvSet = true; st->recvDone.set_value(); }
      };
      if (e) return fail(e);
      // Descriptor callbacks of one context run one at a time: no lock needed for the counter.
      uint8_t* base = mp->dst[(*readsIssued)[k]++ & 1] + k * layout->dstTotal;
      Allocation a;
      for (const MixedSpec& s : layout->specs) {
        Allocation::Tensor t;
        t.buffer = CudaBuffer{base + s.dstOff, mp->recvStream, mp->opts.device};
        if (s.cast) {
          t.castTo = DType::kBF16;
          t.sourceDtype = DType::kF32;
        }
        a.tensors.push_back(t);
      }
      pipe->read(std::move(a), [=](const Error& e2) {
        bool last;
        {
          std::unique_lock<std::mutex> l(st->mu);
          if (e2) st->error = e2;
          last = ++st->received == totalRecv || bool(st->error);
        }
        if (last) {
          cudaSetDevice(mp->opts.device);
          cudaEventRecord(mp->evEnd, mp->recvStream);
          std::unique_lock<std::mutex> l(st->mu);
          if (!st->recvSet) { st->recvSet = true; st->recvDone.set_value(); }
        } else {
          (*armRead)(k, remaining - 1);
        }
      });
    });
  };
  // Two send chains per outgoing pipe; all of them read the same source tensors.
  auto sendOne = std::make_shared<std::function<void(size_t, int)>>();
  *sendOne = [=](size_t k, int remaining) {
    if (remaining == 0) return;
    Message msg;
    for (const MixedSpec& s : layout->specs) {
      Message::Tensor t;
      t.buffer = CudaBuffer{mp->src + s.srcOff, sendStreams[k], mp->opts.device};
      t.length = s.srcBytes;
      t.dtype = s.dtype;
      t.targetDevice = Device(kCudaDeviceType, sendDevices[k]);
      if (s.transposed) {
        // The buffer holds a [cols, rows] row-major matrix; we send its transpose [rows, cols].
        StridedView v;
        v.dtype = s.dtype;
        v.rows = s.rows;
        v.cols = s.cols;
        v.rowStride = 1;
        v.colStride = s.rows;
        t.view = v;
      }
      msg.tensors.push_back(t);
    }
    sendPipes[k]->write(std::move(msg), [=](const Error& e) {
      bool done;
      {
        std::unique_lock<std::mutex> l(st->mu);
        if (e) st->error = e;
        done = ++st->sent == totalSend || bool(st->error);
        if (done && !st->sendSet) { st->sendSet = true; st->sendDone.set_value(); }
      }
      if (!e) (*sendOne)(k, remaining - 1);
    });
  };

  if (recvPipes.size() == 1 && sendPipes.size() == 1) m.syncOn(sendPipes[0], recvPipes[0]);
  auto t0 = Clock::now();
  TPB_CUDA_CHECK(cudaEventRecord(m.evStart, m.recvStream));
  for (int chain = 0; chain < 2; ++chain) {
    const int share = chain == 0 ? (steps + 1) / 2 : steps / 2;
    for (size_t k = 0; k < recvPipes.size(); ++k) (*armRead)(k, share);
  }
  for (int chain = 0; chain < 2; ++chain) {
    const int share = chain == 0 ? (steps + 1) / 2 : steps / 2;
    for (size_t k = 0; k < sendPipes.size(); ++k) (*sendOne)(k, share);
  }
  auto fr = st->recvDone.get_future();
  auto fs = st->sendDone.get_future();
  if (totalRecv > 0) waitOrThrow(fr, 300, "receiving");
  if (totalSend > 0) waitOrThrow(fs, 300, "sending");
  *armRead = nullptr;
  *sendOne = nullptr;
  failOn(st->error, "mixed messages");
  PhaseResult r;
  if (totalRecv > 0) {
    TPB_CUDA_CHECK(cudaEventSynchronize(m.evEnd));
    float ms = 0;
    TPB_CUDA_CHECK(cudaEventElapsedTime(&ms, m.evStart, m.evEnd));
    r.deviceMs = ms;
  }
  r.hostMs = msSince(t0);
  for (cudaStream_t st : sendStreams) TPB_CUDA_CHECK(cudaStreamSynchronize(st));
  r.kernelLaunches = kernels::launchCount() - launches0;
  return r;
}

}  // namespace tools
}  // namespace tpb
