// Two-process ping-pong over a full pipe with the command line of the reference's benchmark
// (tensorpipe/benchmark/benchmark_pipe.cc:173-740, options.cc): start one process with
// --mode listen and one with --mode connect, same remaining flags on both.
//
//   benchmark_pipe --mode listen|connect --transport uv|shm --channel NAME --address URL
//                  --num-round-trips N [--num-payloads N --payload-size B]
//                  [--num-tensors N --tensor-size B --tensor-type cpu|cuda]
//                  [--metadata-size B] [--cuda-sync-period N]
//
// Channels by name: basic, xth, cma, mpt_uv (4 TCP lanes), cuda_basic (over basic), cuda_p2p
// (cuda_xth and cuda_ipc are aliases of it). The client sends a message, the server echoes one of
// the same shape; the client reports round-trip percentiles. With CUDA tensors the client
// synchronises its stream every --cuda-sync-period round trips and reports host-side and
// device-complete latencies separately. Contents are a fixed pattern checked by both sides on the
// first and last round trip.
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <future>
#include <iostream>
#include <memory>
#include <string>
#include <vector>

#include <tpb/tpb.h>

namespace {

using namespace tpb;
using Clock = std::chrono::steady_clock;

struct Options {
  std::string mode, transport = "uv", channel = "basic", address;
  int numRoundTrips = 0;
  size_t numPayloads = 0, payloadSize = 0, numTensors = 0, tensorSize = 0, metadataSize = 0, cudaSyncPeriod = 1;
  bool cuda = false;
};

[[noreturn]] void usage(const std::string& why) {
  std::cerr << "benchmark_pipe: " << why << "\n"
            << "  --mode listen|connect --transport uv|shm --channel NAME --address URL --num-round-trips N\n"
            << "  [--num-payloads N] [--payload-size B] [--num-tensors N] [--tensor-size B]\n"
            << "  [--tensor-type cpu|cuda] [--metadata-size B] [--cuda-sync-period N]\n";
  std::exit(2);
}

Options parse(int argc, char** argv) {
  Options o;
  for (int i = 1; i < argc; ++i) {
    std::string k = argv[i];
    std::string v;
    auto eq = k.find('=');
    if (eq != std::string::npos) {
      v = k.substr(eq + 1);
      k = k.substr(0, eq);
    } else {
      if (i + 1 >= argc) usage("missing value for " + k);
      v = argv[++i];
    }
    if (k == "--mode") o.mode = v;
    else if (k == "--transport") o.transport = v;
    else if (k == "--channel") o.channel = v;
    else if (k == "--address") o.address = v;
    else if (k == "--num-round-trips") o.numRoundTrips = std::stoi(v);
    else if (k == "--num-payloads") o.numPayloads = std::stoull(v);
    else if (k == "--payload-size") o.payloadSize = std::stoull(v);
    else if (k == "--num-tensors") o.numTensors = std::stoull(v);
    else if (k == "--tensor-size") o.tensorSize = std::stoull(v);
    else if (k == "--tensor-type") {
      if (v != "cpu" && v != "cuda") usage("--tensor-type must be cpu or cuda");
      o.cuda = v == "cuda";
    } else if (k == "--metadata-size") o.metadataSize = std::stoull(v);
    else if (k == "--cuda-sync-period") o.cudaSyncPeriod = std::max<size_t>(1, std::stoull(v));
    else usage("unknown flag " + k);
  }
  if (o.mode != "listen" && o.mode != "connect") usage("--mode must be listen or connect");
  if (o.address.empty()) usage("--address is required");
  if (o.numRoundTrips <= 0) usage("--num-round-trips must be positive");
  return o;
}

// String -> factory tables (the reference keeps c10-style registries: benchmark/channel_registry.cc,
// transport_registry.cc).
std::shared_ptr<transport::Context> makeTransport(const std::string& name) {
  if (name == "uv") return transport::uv::create();
  if (name == "shm") return transport::shm::create();
  if (name == "ibv") return transport::ibv::create();
  usage("unknown transport " + name);
}

std::shared_ptr<channel::Context> makeChannel(const std::string& name) {
  if (name == "basic") return channel::basic::create();
  if (name == "xth") return channel::xth::create();
  if (name == "cma") return channel::cma::create();
  if (name == "mpt_uv") {
    std::vector<std::shared_ptr<transport::Context>> ctxs;
    std::vector<std::shared_ptr<transport::Listener>> listeners;
    for (int i = 0; i < 4; ++i) {
      ctxs.push_back(transport::uv::create());
      listeners.push_back(ctxs.back()->listen("127.0.0.1"));
    }
    return channel::mpt::create(std::move(ctxs), std::move(listeners));
  }
  if (name == "cuda_basic") return channel::cuda_basic::create(channel::basic::create());
  if (name == "cuda_p2p" || name == "cuda_xth" || name == "cuda_ipc") return channel::cuda_p2p::create();
  if (name == "cuda_gdr") return channel::cuda_gdr::create();
  usage("unknown channel " + name);
}

uint8_t patternAt(size_t i) { return static_cast<uint8_t>((i >> 8) ^ (i & 0xff) ^ 0x5a); }

void checkCuda(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    std::cerr << what << ": " << cudaGetErrorString(e) << std::endl;
    std::exit(3);
  }
}

// Buffers of one side: what it sends (patterned) and where it receives.
struct Data {
  std::string metadata;
  std::vector<std::vector<uint8_t>> payloadsOut, payloadsIn;
  std::vector<std::vector<uint8_t>> cpuOut, cpuIn;
  std::vector<uint8_t*> cudaOut, cudaIn;
  cudaStream_t stream = nullptr;

  explicit Data(const Options& o) {
    metadata.assign(o.metadataSize, 'm');
    std::vector<uint8_t> pattern(std::max(o.payloadSize, o.tensorSize));
    for (size_t i = 0; i < pattern.size(); ++i) pattern[i] = patternAt(i);
    for (size_t i = 0; i < o.numPayloads; ++i) {
      payloadsOut.emplace_back(pattern.begin(), pattern.begin() + o.payloadSize);
      payloadsIn.emplace_back(o.payloadSize);
    }
    if (o.cuda) {
      checkCuda(cudaSetDevice(0), "cudaSetDevice");
      checkCuda(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "cudaStreamCreate");
      for (size_t i = 0; i < o.numTensors; ++i) {
        uint8_t *a = nullptr, *b = nullptr;
        checkCuda(cudaMalloc(&a, std::max<size_t>(o.tensorSize, 1)), "cudaMalloc");
        checkCuda(cudaMalloc(&b, std::max<size_t>(o.tensorSize, 1)), "cudaMalloc");
        checkCuda(cudaMemcpy(a, pattern.data(), o.tensorSize, cudaMemcpyHostToDevice), "cudaMemcpy");
        checkCuda(cudaMemset(b, 0, o.tensorSize), "cudaMemset");
        cudaOut.push_back(a);
        cudaIn.push_back(b);
      }
    } else {
      for (size_t i = 0; i < o.numTensors; ++i) {
        cpuOut.emplace_back(pattern.begin(), pattern.begin() + o.tensorSize);
        cpuIn.emplace_back(o.tensorSize);
      }
    }
  }

  Message message(const Options& o) {
    Message m;
    m.metadata = metadata;
    for (auto& p : payloadsOut) {
      Message::Payload mp;
      mp.data = p.data();
      mp.length = p.size();
      m.payloads.push_back(mp);
    }
    for (size_t i = 0; i < o.numTensors; ++i) {
      Message::Tensor t;
      if (o.cuda) {
        t.buffer = CudaBuffer{cudaOut[i], stream, 0};
        t.targetDevice = Device(kCudaDeviceType, 0);
      } else {
        t.buffer = CpuBuffer{cpuOut[i].data()};
        t.targetDevice = Device(kCpuDeviceType, 0);
      }
      t.length = o.tensorSize;
      m.tensors.push_back(t);
    }
    return m;
  }

  Allocation allocation(const Options& o, const Descriptor& d) {
    if (d.payloads.size() != o.numPayloads || d.tensors.size() != o.numTensors || d.metadata.size() != o.metadataSize) {
      std::cerr << "peer sent a message of a different shape: are both sides using the same flags?" << std::endl;
      std::exit(3);
    }
    Allocation a;
    for (auto& p : payloadsIn) a.payloads.push_back({p.data()});
    for (size_t i = 0; i < o.numTensors; ++i) {
      Allocation::Tensor t;
      if (o.cuda) t.buffer = CudaBuffer{cudaIn[i], stream, 0};
      else t.buffer = CpuBuffer{cpuIn[i].data()};
      a.tensors.push_back(t);
    }
    return a;
  }

  void verify(const Options& o) {
    if (o.cuda) checkCuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    auto bad = [](const uint8_t* p, size_t n) {
      for (size_t i = 0; i < n; ++i)
        if (p[i] != patternAt(i)) return true;
      return false;
    };
    bool wrong = false;
    for (auto& p : payloadsIn) wrong |= bad(p.data(), p.size());
    std::vector<uint8_t> host(o.tensorSize);
    for (size_t i = 0; i < o.numTensors; ++i) {
      if (o.cuda) {
        checkCuda(cudaMemcpy(host.data(), cudaIn[i], o.tensorSize, cudaMemcpyDeviceToHost), "cudaMemcpy");
        wrong |= bad(host.data(), host.size());
      } else {
        wrong |= bad(cpuIn[i].data(), cpuIn[i].size());
      }
    }
    if (wrong) {
      std::cerr << "received bytes differ from the pattern" << std::endl;
      std::exit(4);
    }
  }

  void clearInputs(const Options& o) {
    for (auto& p : payloadsIn) std::fill(p.begin(), p.end(), 0);
    for (auto& t : cpuIn) std::fill(t.begin(), t.end(), 0);
    for (auto* t : cudaIn) checkCuda(cudaMemset(t, 0, o.tensorSize), "cudaMemset");
  }
};

void fail(const char* what, const Error& e) {
  std::cerr << what << ": " << e.what() << std::endl;
  std::exit(3);
}

void writeSync(Pipe& pipe, Message m) {
  std::promise<Error> done;
  pipe.write(std::move(m), [&](const Error& e) { done.set_value(e); });
  Error e = done.get_future().get();
  if (e) fail("write", e);
}

void readSync(Pipe& pipe, Data& data, const Options& o) {
  std::promise<Error> done;
  pipe.readDescriptor([&](const Error& e, Descriptor d) {
    if (e) return done.set_value(e);
    pipe.read(data.allocation(o, d), [&](const Error& e2) { done.set_value(e2); });
  });
  Error e = done.get_future().get();
  if (e) fail("read", e);
}

void report(const char* what, std::vector<double> us, size_t bytes) {
  std::sort(us.begin(), us.end());
  auto pct = [&](double q) { return us[std::min(us.size() - 1, static_cast<size_t>(q * us.size()))]; };
  double sum = 0;
  for (double v : us) sum += v;
  std::fprintf(stderr, "%-10s %-15s %-15s %-12s %-9s %-9s %-9s %-9s %-9s\n", "", "bytes/message", "# ping-pong",
               "avg (usec)", "p50", "p75", "p90", "p95", "p99");
  std::fprintf(stderr, "%-10s %-15zu %-15zu %-12.3f %-9.3f %-9.3f %-9.3f %-9.3f %-9.3f\n", what, bytes, us.size(),
               sum / us.size(), pct(0.50), pct(0.75), pct(0.90), pct(0.95), pct(0.99));
}

constexpr int kWarmUps = 5;  // as the reference: benchmark_pipe.cc:56

int run(const Options& o) {
  auto ctx = std::make_shared<Context>(ContextOptions().name(o.mode == "listen" ? "server" : "client"));
  ctx->registerTransport(0, o.transport, makeTransport(o.transport));
  ctx->registerChannel(0, o.channel, makeChannel(o.channel));
  Data data(o);
  const size_t bytes = o.metadataSize + o.numPayloads * o.payloadSize + o.numTensors * o.tensorSize;
  const int total = o.numRoundTrips + kWarmUps;

  if (o.mode == "listen") {
    auto listener = ctx->listen({o.address});
    std::promise<std::shared_ptr<Pipe>> accepted;
    listener->accept([&](const Error& e, std::shared_ptr<Pipe> p) {
      if (e) fail("accept", e);
      accepted.set_value(std::move(p));
    });
    std::cerr << "listening on " << listener->url(o.transport) << std::endl;
    auto pipe = accepted.get_future().get();
    for (int i = 0; i < total; ++i) {
      readSync(*pipe, data, o);
      if (i == 0 || i == total - 1) data.verify(o);
      writeSync(*pipe, data.message(o));
    }
    if (o.cuda) checkCuda(cudaStreamSynchronize(data.stream), "cudaStreamSynchronize");
    // Keep the pipe up until the client has taken the last reply and hung up.
    std::promise<void> gone;
    pipe->readDescriptor([&](const Error&, Descriptor) { gone.set_value(); });
    gone.get_future().wait();
    ctx->join();
    return 0;
  }

  auto pipe = ctx->connect(o.address);
  std::vector<double> hostUs, deviceUs;
  Clock::time_point windowStart;
  for (int i = 0; i < total; ++i) {
    const bool timed = i >= kWarmUps;
    const int k = i - kWarmUps;
    if (i == total - 1) data.clearInputs(o);
    if (timed && o.cuda && k % o.cudaSyncPeriod == 0) windowStart = Clock::now();
    auto t0 = Clock::now();
    writeSync(*pipe, data.message(o));
    readSync(*pipe, data, o);
    auto t1 = Clock::now();
    if (timed) hostUs.push_back(std::chrono::duration<double, std::micro>(t1 - t0).count());
    if (o.cuda && timed && ((k + 1) % o.cudaSyncPeriod == 0 || i == total - 1)) {
      checkCuda(cudaStreamSynchronize(data.stream), "cudaStreamSynchronize");
      const size_t n = k % o.cudaSyncPeriod + 1;
      deviceUs.push_back(std::chrono::duration<double, std::micro>(Clock::now() - windowStart).count() / n);
    }
    if (i == 0 || i == total - 1) data.verify(o);
  }
  report(o.cuda ? "host" : "cpu", hostUs, bytes);
  if (o.cuda) report("device", deviceUs, bytes);
  pipe->close();
  ctx->join();
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  try {
    return run(parse(argc, argv));
  } catch (const std::exception& e) {
    std::cerr << "benchmark_pipe: " << e.what() << std::endl;
    return 3;
  }
}
