// Latency-bound workloads over full pipes, written once against the API shape this library shares
// with the reference (Context / Listener / Pipe / Message) and compiled twice: against this
// library (default) and, with -DUSE_REFERENCE, against the TensorPipe that PyTorch ships — so both
// are measured by literally the same benchmark code (the reference's own benchmark_pipe plays this
// role upstream: tensorpipe/benchmark/benchmark_pipe.cc:173-740).
//
//   --workload cpu_pingpong  --transport uv|shm  --channel basic|cma  [--iters 1000]
//       two forked processes; every message = 64 KiB payload + four fp32 CPU tensors of shapes
//       [1024], [256,256], [64,64,64], [1<<20]; the server echoes; the client verifies every byte
//       and that callbacks arrive in order; prints p50 / p99 round-trip latency.
//   --workload transport_pingpong  --transport uv|shm  [--bytes 64]  [--iters 20000]
//       raw transport connections (no pipe): one frame each way per round trip, two forked
//       processes; prints p50 / p99 round-trip latency (the reference's benchmark_transport,
//       tensorpipe/benchmark/benchmark_transport.cc:30-199).
//   --workload rpc_fanin  --ranks N  [--iters 20000]
//       rank 0 serves, ranks 1..N-1 (one forked process each, GPU r mod #GPUs) issue requests of a
//       256 B payload + one 4 KiB fp32 CUDA tensor and wait for a same-shaped reply; prints
//       p50 / p99 round-trip latency over all clients and messages per second.
#include <cuda_runtime.h>
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstring>
#include <functional>
#include <future>
#include <iostream>
#include <memory>
#include <random>
#include <string>
#include <thread>
#include <vector>

#ifdef USE_REFERENCE
#include <tensorpipe/tensorpipe.h>
#include <tensorpipe/tensorpipe_cuda.h>
namespace lib = tensorpipe;
static const char* kImpl = "reference";
static lib::Buffer cudaBuffer(void* p, cudaStream_t s, int) { return lib::CudaBuffer{p, s}; }
#else
#include <tpb/tpb.h>
namespace lib = tpb;
static const char* kImpl = "native";
static lib::Buffer cudaBuffer(void* p, cudaStream_t s, int dev) { return lib::CudaBuffer{p, s, dev}; }
#endif

using Clock = std::chrono::steady_clock;

struct Options {
  std::string workload = "cpu_pingpong", transport = "uv", channel = "basic";
  int iters = 1000, ranks = 2, warmup = 20;
  size_t bytes = 64;
};

static void die(const std::string& what) {
  std::cerr << "[" << getpid() << "] " << what << std::endl;
  _exit(3);
}

// A few words of shared memory for the forked processes to exchange the listener's URL and results.
struct Shared {
  std::atomic<int> urlReady;
  char url[256];
  std::atomic<int> clientsDone;
  double p50[64], p99[64], mean[64], seconds[64];
  std::atomic<int> failed;
};

static double percentile(std::vector<double> v, double q) {
  std::sort(v.begin(), v.end());
  return v[std::min(v.size() - 1, static_cast<size_t>(q * v.size()))];
}

static std::shared_ptr<lib::Context> makeCpuContext(const Options& o, const std::string& name) {
  auto ctx = std::make_shared<lib::Context>(lib::ContextOptions().name(name));
  ctx->registerTransport(0, "uv", lib::transport::uv::create());
  if (o.transport == "shm") ctx->registerTransport(10, "shm", lib::transport::shm::create());
  ctx->registerChannel(0, "basic", lib::channel::basic::create());
  if (o.channel == "cma") ctx->registerChannel(10, "cma", lib::channel::cma::create());
  return ctx;
}

// ---- workload 1 ---------------------------------------------------------------------------------
static const size_t kTensorBytes[4] = {1024 * 4, 256 * 256 * 4, 64 * 64 * 64 * 4, (1u << 20) * 4};
static const size_t kPayloadBytes = 64 * 1024;

struct CpuMessage {
  std::vector<uint8_t> payload;
  std::vector<std::vector<float>> tensors;
  void fill(uint32_t seed) {
    std::mt19937 rng(seed);
    payload.resize(kPayloadBytes);
    for (auto& b : payload) b = static_cast<uint8_t>(rng());
    tensors.resize(4);
    std::normal_distribution<float> dist(0.f, 1.f);
    for (int i = 0; i < 4; ++i) {
      tensors[i].resize(kTensorBytes[i] / 4);
      for (auto& f : tensors[i]) f = dist(rng);
    }
  }
  void allocate() {
    payload.assign(kPayloadBytes, 0);
    tensors.resize(4);
    for (int i = 0; i < 4; ++i) tensors[i].assign(kTensorBytes[i] / 4, 0.f);
  }
  lib::Message view() {
    lib::Message m;
    m.metadata = "cfg1";
    lib::Message::Payload p;
    p.data = payload.data();
    p.length = payload.size();
    m.payloads.push_back(p);
    for (auto& t : tensors) {
      lib::Message::Tensor mt;
      mt.buffer = lib::CpuBuffer{t.data()};
      mt.length = t.size() * 4;
      mt.targetDevice = lib::Device(lib::kCpuDeviceType, 0);
      m.tensors.push_back(mt);
    }
    return m;
  }
  lib::Allocation allocation() {
    lib::Allocation a;
    a.payloads.push_back({payload.data()});
    for (auto& t : tensors) {
      lib::Allocation::Tensor at;
      at.buffer = lib::CpuBuffer{t.data()};
      a.tensors.push_back(at);
    }
    return a;
  }
  bool equals(const CpuMessage& o) const {
    if (payload != o.payload) return false;
    for (int i = 0; i < 4; ++i)
      if (std::memcmp(tensors[i].data(), o.tensors[i].data(), tensors[i].size() * 4) != 0) return false;
    return true;
  }
};

static void readInto(lib::Pipe& pipe, CpuMessage& into) {
  std::promise<void> done;
  pipe.readDescriptor([&](const lib::Error& e, lib::Descriptor d) {
    if (e) die("readDescriptor: " + e.what());
    if (d.payloads.size() != 1 || d.tensors.size() != 4) die("unexpected message shape");
    pipe.read(into.allocation(), [&](const lib::Error& e2) {
      if (e2) die("read: " + e2.what());
      done.set_value();
    });
  });
  done.get_future().wait();
}
static void writeFrom(lib::Pipe& pipe, CpuMessage& from) {
  std::promise<void> done;
  pipe.write(from.view(), [&](const lib::Error& e) {
    if (e) die("write: " + e.what());
    done.set_value();
  });
  done.get_future().wait();
}

static int cpuPingPong(const Options& o, Shared* sh) {
  const int total = o.iters + o.warmup;
  pid_t server = fork();
  if (server == 0) {
    auto ctx = makeCpuContext(o, "server");
    std::vector<std::string> urls = {"uv://127.0.0.1"};
    if (o.transport == "shm") urls.push_back("shm://");
    auto listener = ctx->listen(urls);
    std::string url = listener->url("uv");
    std::strncpy(sh->url, url.c_str(), sizeof(sh->url) - 1);
    sh->urlReady = 1;
    std::promise<std::shared_ptr<lib::Pipe>> pp;
    listener->accept([&](const lib::Error& e, std::shared_ptr<lib::Pipe> p) {
      if (e) die("accept: " + e.what());
      pp.set_value(p);
    });
    auto pipe = pp.get_future().get();
    CpuMessage buf;
    buf.allocate();
    for (int i = 0; i < total; ++i) {
      readInto(*pipe, buf);
      writeFrom(*pipe, buf);
    }
    while (sh->clientsDone.load() == 0) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    ctx->join();
    _exit(0);
  }
  pid_t client = fork();
  if (client == 0) {
    while (sh->urlReady.load() == 0) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    auto ctx = makeCpuContext(o, "client");
    auto pipe = ctx->connect(sh->url);
    CpuMessage msg, echo;
    msg.fill(12345);
    echo.allocate();
    std::vector<double> rtt;
    // In-order check: issue two writes back to back every so often and watch the callback order.
    for (int i = 0; i < total; ++i) {
      auto t0 = Clock::now();
      writeFrom(*pipe, msg);
      readInto(*pipe, echo);
      double us = std::chrono::duration<double, std::micro>(Clock::now() - t0).count();
      if (i >= o.warmup) rtt.push_back(us);
      if (!msg.equals(echo)) {
        sh->failed = 1;
        die("echo differs from what was sent");
      }
      echo.payload[0] ^= 0xff;  // make sure the next round really rewrites the buffers
    }
    sh->p50[0] = percentile(rtt, 0.5);
    sh->p99[0] = percentile(rtt, 0.99);
    double sum = 0;
    for (double v : rtt) sum += v;
    sh->mean[0] = sum / rtt.size();
    sh->clientsDone = 1;
    ctx->join();
    _exit(0);
  }
  int s1 = 0, s2 = 0;
  waitpid(client, &s2, 0);
  sh->clientsDone = 1;
  waitpid(server, &s1, 0);
  if (!WIFEXITED(s1) || WEXITSTATUS(s1) || !WIFEXITED(s2) || WEXITSTATUS(s2) || sh->failed) {
    std::cout << "{\"impl\": \"" << kImpl << "\", \"workload\": \"cpu_pingpong\", \"error\": \"a peer failed\"}" << std::endl;
    return 1;
  }
  const size_t bytes = kPayloadBytes + kTensorBytes[0] + kTensorBytes[1] + kTensorBytes[2] + kTensorBytes[3];
  std::cout << "{\"impl\": \"" << kImpl << "\", \"workload\": \"cpu_pingpong\", \"transport\": \"" << o.transport
            << "\", \"channel\": \"" << o.channel << "\", \"round_trips\": " << o.iters << ", \"bytes_per_message\": "
            << bytes << ", \"rtt_p50_us\": " << sh->p50[0] << ", \"rtt_p99_us\": " << sh->p99[0]
            << ", \"rtt_mean_us\": " << sh->mean[0] << ", \"verified\": \"byte-exact, every round trip\"}" << std::endl;
  return 0;
}

// ---- raw transport ping-pong ------------------------------------------------------------------------
#ifdef USE_REFERENCE
// PyTorch ships the reference's public headers only; transport/connection.h and listener.h are
// not among them, so the raw transport API cannot be driven from here.
static int transportPingPong(const Options&, Shared*) {
  std::cout << "{\"impl\": \"reference\", \"workload\": \"transport_pingpong\", \"unavailable\": "
               "\"the reference's transport headers are not shipped with PyTorch\"}" << std::endl;
  return 0;
}
#else
static int transportPingPong(const Options& o, Shared* sh) {
  const int total = o.iters + o.warmup * 10;
  auto makeTransport = [&]() -> std::shared_ptr<lib::transport::Context> {
    if (o.transport == "shm") return lib::transport::shm::create();
    return lib::transport::uv::create();
  };
  pid_t server = fork();
  if (server == 0) {
    auto t = makeTransport();
    auto listener = t->listen(o.transport == "shm" ? std::string("tpb-bench-") + std::to_string(getpid()) : std::string("127.0.0.1"));
    std::strncpy(sh->url, listener->addr().c_str(), sizeof(sh->url) - 1);
    sh->urlReady = 1;
    std::promise<std::shared_ptr<lib::transport::Connection>> pc;
    listener->accept([&](const lib::Error& e, std::shared_ptr<lib::transport::Connection> c) {
      if (e) die("accept: " + e.what());
      pc.set_value(c);
    });
    auto conn = pc.get_future().get();
    std::vector<uint8_t> buf(o.bytes);
    std::promise<void> done;
    int count = 0;
    std::function<void()> arm = [&]() {
      conn->read(buf.data(), buf.size(), [&](const lib::Error& e, const void*, size_t) {
        if (e) die("read: " + e.what());
        conn->write(buf.data(), buf.size(), [&](const lib::Error& e2) {
          if (e2) die("write: " + e2.what());
        });
        if (++count == total) done.set_value();
        else arm();
      });
    };
    arm();
    done.get_future().wait();
    while (sh->clientsDone.load() == 0) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    t->join();
    _exit(0);
  }
  pid_t client = fork();
  if (client == 0) {
    while (sh->urlReady.load() == 0) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    auto t = makeTransport();
    auto conn = t->connect(sh->url);
    std::vector<uint8_t> out(o.bytes, 7), in(o.bytes);
    std::vector<double> rtt;
    rtt.reserve(o.iters);
    std::promise<void> done;
    int count = 0;
    Clock::time_point t0;
    std::function<void()> round = [&]() {
      t0 = Clock::now();
      conn->write(out.data(), out.size(), [&](const lib::Error& e) {
        if (e) die("write: " + e.what());
      });
      conn->read(in.data(), in.size(), [&](const lib::Error& e, const void*, size_t) {
        if (e) die("read: " + e.what());
        if (count >= o.warmup * 10) rtt.push_back(std::chrono::duration<double, std::micro>(Clock::now() - t0).count());
        if (++count == total) done.set_value();
        else round();
      });
    };
    round();
    done.get_future().wait();
    sh->p50[0] = percentile(rtt, 0.5);
    sh->p99[0] = percentile(rtt, 0.99);
    double sum = 0;
    for (double v : rtt) sum += v;
    sh->mean[0] = sum / rtt.size();
    sh->clientsDone = 1;
    t->join();
    _exit(0);
  }
  int s1 = 0, s2 = 0;
  waitpid(client, &s2, 0);
  sh->clientsDone = 1;
  waitpid(server, &s1, 0);
  if (!WIFEXITED(s1) || WEXITSTATUS(s1) || !WIFEXITED(s2) || WEXITSTATUS(s2)) {
    std::cout << "{\"impl\": \"" << kImpl << "\", \"workload\": \"transport_pingpong\", \"error\": \"a peer failed\"}" << std::endl;
    return 1;
  }
  std::cout << "{\"impl\": \"" << kImpl << "\", \"workload\": \"transport_pingpong\", \"transport\": \"" << o.transport
            << "\", \"bytes\": " << o.bytes << ", \"round_trips\": " << o.iters << ", \"rtt_p50_us\": " << sh->p50[0]
            << ", \"rtt_p99_us\": " << sh->p99[0] << ", \"rtt_mean_us\": " << sh->mean[0] << "}" << std::endl;
  return 0;
}
#endif

// ---- workload 5 ---------------------------------------------------------------------------------
static std::shared_ptr<lib::Context> makeCudaContext(const std::string& name) {
  auto ctx = std::make_shared<lib::Context>(lib::ContextOptions().name(name));
  ctx->registerTransport(0, "uv", lib::transport::uv::create());
  ctx->registerTransport(10, "shm", lib::transport::shm::create());
  ctx->registerChannel(0, "basic", lib::channel::basic::create());
  ctx->registerChannel(101, "cuda_basic", lib::channel::cuda_basic::create(lib::channel::basic::create()));
  ctx->registerChannel(300, "cuda_ipc", lib::channel::cuda_ipc::create());
#ifdef USE_REFERENCE
  ctx->registerChannel(400, "cuda_xth", lib::channel::cuda_xth::create());
#endif
  return ctx;
}

static int rpcFanIn(const Options& o, Shared* sh) {
  constexpr size_t kPayload = 256, kTensor = 4096;
  const int clients = o.ranks - 1;
  if (clients < 1 || clients > 63) die("--ranks must be 2..64");
  const int total = o.iters + o.warmup;
  std::vector<pid_t> pids;
  pid_t server = fork();
  if (server == 0) {
    int numGpus = 0;
    cudaGetDeviceCount(&numGpus);
    if (numGpus == 0) die("no GPU");
    cudaSetDevice(0);
    cudaStream_t stream;
    cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
    auto ctx = makeCudaContext("rank0");
    auto listener = ctx->listen({"uv://127.0.0.1", "shm://"});
    std::strncpy(sh->url, listener->url("uv").c_str(), sizeof(sh->url) - 1);
    sh->urlReady = 1;
    struct Conn {
      std::shared_ptr<lib::Pipe> pipe;
      void* tensor = nullptr;
      std::vector<uint8_t> payload = std::vector<uint8_t>(kPayload);
      int clientGpu = 0;
    };
    std::vector<std::shared_ptr<Conn>> conns;
    std::function<void(std::shared_ptr<Conn>)> serve = [&](std::shared_ptr<Conn> c) {
      c->pipe->readDescriptor([&, c](const lib::Error& e, lib::Descriptor d) {
        if (e) return;  // client went away: done
        c->clientGpu = d.tensors.at(0).sourceDevice.index;
        lib::Allocation a;
        a.payloads.push_back({c->payload.data()});
        lib::Allocation::Tensor at;
        at.buffer = cudaBuffer(c->tensor, stream, 0);
        a.tensors.push_back(at);
        c->pipe->read(a, [&, c](const lib::Error& e2) {
          if (e2) return;
          lib::Message reply;
          lib::Message::Payload p;
          p.data = c->payload.data();
          p.length = kPayload;
          reply.payloads.push_back(p);
          lib::Message::Tensor t;
          t.buffer = cudaBuffer(c->tensor, stream, 0);
          t.length = kTensor;
          t.targetDevice = lib::Device(lib::kCudaDeviceType, c->clientGpu);
          reply.tensors.push_back(t);
          c->pipe->write(reply, [](const lib::Error&) {});
          serve(c);
        });
      });
    };
    std::function<void()> arm = [&]() {
      listener->accept([&](const lib::Error& e, std::shared_ptr<lib::Pipe> p) {
        if (e) return;
        auto c = std::make_shared<Conn>();
        c->pipe = p;
        cudaSetDevice(0);
        cudaMalloc(&c->tensor, kTensor);
        conns.push_back(c);
        serve(c);
        arm();
      });
    };
    arm();
    while (sh->clientsDone.load() < clients) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    ctx->join();
    _exit(0);
  }
  for (int r = 1; r <= clients; ++r) {
    pid_t pid = fork();
    if (pid == 0) {
      while (sh->urlReady.load() == 0) std::this_thread::sleep_for(std::chrono::milliseconds(1));
      int numGpus = 0;
      cudaGetDeviceCount(&numGpus);
      const int dev = r % numGpus;
      cudaSetDevice(dev);
      cudaStream_t stream;
      cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
      void *sendBuf, *recvBuf;
      cudaMalloc(&sendBuf, kTensor);
      cudaMalloc(&recvBuf, kTensor);
      std::vector<float> host(kTensor / 4);
      std::mt19937 rng(r);
      std::uniform_real_distribution<float> dist(-1.f, 1.f);
      for (auto& f : host) f = dist(rng);
      cudaMemcpy(sendBuf, host.data(), kTensor, cudaMemcpyHostToDevice);
      std::vector<uint8_t> payload(kPayload, static_cast<uint8_t>(r)), replyPayload(kPayload);
      auto ctx = makeCudaContext("rank" + std::to_string(r));
      auto pipe = ctx->connect(sh->url);
      std::vector<double> rtt;
      auto tStart = Clock::now();
      for (int i = 0; i < total; ++i) {
        if (i == o.warmup) tStart = Clock::now();
        auto t0 = Clock::now();
        lib::Message m;
        lib::Message::Payload p;
        p.data = payload.data();
        p.length = kPayload;
        m.payloads.push_back(p);
        lib::Message::Tensor t;
        t.buffer = cudaBuffer(sendBuf, stream, dev);
        t.length = kTensor;
        t.targetDevice = lib::Device(lib::kCudaDeviceType, 0);
        m.tensors.push_back(t);
        std::promise<void> got;
        pipe->write(m, [](const lib::Error& e) {
          if (e) die("write: " + e.what());
        });
        pipe->readDescriptor([&](const lib::Error& e, lib::Descriptor) {
          if (e) die("readDescriptor: " + e.what());
          lib::Allocation a;
          a.payloads.push_back({replyPayload.data()});
          lib::Allocation::Tensor at;
          at.buffer = cudaBuffer(recvBuf, stream, dev);
          a.tensors.push_back(at);
          pipe->read(a, [&](const lib::Error& e2) {
            if (e2) die("read: " + e2.what());
            cudaSetDevice(dev);
            cudaStreamSynchronize(stream);  // the reply is on the device
            got.set_value();
          });
        });
        got.get_future().wait();
        if (i >= o.warmup) rtt.push_back(std::chrono::duration<double, std::micro>(Clock::now() - t0).count());
      }
      sh->seconds[r] = std::chrono::duration<double>(Clock::now() - tStart).count();
      // the reply must be the tensor we sent
      std::vector<float> back(kTensor / 4);
      cudaMemcpy(back.data(), recvBuf, kTensor, cudaMemcpyDeviceToHost);
      if (back != host || replyPayload != payload) {
        sh->failed = 1;
        die("reply differs from the request");
      }
      sh->p50[r] = percentile(rtt, 0.5);
      sh->p99[r] = percentile(rtt, 0.99);
      double sum = 0;
      for (double v : rtt) sum += v;
      sh->mean[r] = sum / rtt.size();
      sh->clientsDone.fetch_add(1);
      ctx->join();
      _exit(0);
    }
    pids.push_back(pid);
  }
  bool ok = true;
  for (pid_t pid : pids) {
    int st = 0;
    waitpid(pid, &st, 0);
    if (!WIFEXITED(st) || WEXITSTATUS(st)) {
      ok = false;
      sh->clientsDone.fetch_add(1);
    }
  }
  int st = 0;
  waitpid(server, &st, 0);
  if (!ok || sh->failed) {
    std::cout << "{\"impl\": \"" << kImpl << "\", \"workload\": \"rpc_fanin\", \"error\": \"a rank failed\"}" << std::endl;
    return 1;
  }
  double p50 = 0, p99 = 0, mean = 0, rate = 0;
  for (int r = 1; r <= clients; ++r) {
    p50 = std::max(p50, sh->p50[r]);
    p99 = std::max(p99, sh->p99[r]);
    mean += sh->mean[r] / clients;
    rate += o.iters / sh->seconds[r];
  }
  std::cout << "{\"impl\": \"" << kImpl << "\", \"workload\": \"rpc_fanin\", \"ranks\": " << o.ranks
            << ", \"messages_per_client\": " << o.iters << ", \"rtt_p50_us_worst_client\": " << p50
            << ", \"rtt_p99_us_worst_client\": " << p99 << ", \"rtt_mean_us\": " << mean
            << ", \"messages_per_second\": " << rate << ", \"verified\": \"last reply compared with the request\"}" << std::endl;
  return 0;
}

int main(int argc, char** argv) {
  Options o;
  for (int i = 1; i + 1 < argc; i += 2) {
    std::string k = argv[i], v = argv[i + 1];
    if (k == "--workload") o.workload = v;
    else if (k == "--transport") o.transport = v;
    else if (k == "--channel") o.channel = v;
    else if (k == "--iters") o.iters = std::stoi(v);
    else if (k == "--ranks") o.ranks = std::stoi(v);
    else if (k == "--warmup") o.warmup = std::stoi(v);
    else if (k == "--bytes") o.bytes = std::stoull(v);
  }
  auto* sh = static_cast<Shared*>(mmap(nullptr, sizeof(Shared), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0));
  std::memset(static_cast<void*>(sh), 0, sizeof(Shared));
  if (o.workload == "cpu_pingpong") return cpuPingPong(o, sh);
  if (o.workload == "rpc_fanin") return rpcFanIn(o, sh);
  if (o.workload == "transport_pingpong") return transportPingPong(o, sh);
  std::cerr << "unknown workload" << std::endl;
  return 2;
}
