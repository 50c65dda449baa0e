// Latency-bound workloads over full pipes, written once against the API shape this library shares
// with the reference (Context / Listener / Pipe / Message) and compiled twice: against this
// library (default) and, with -DUSE_REFERENCE, against the TensorPipe that PyTorch ships — so both
// are measured by literally the same benchmark code (the reference's own benchmark_pipe plays this
// role upstream: tensorpipe/benchmark/benchmark_pipe.cc:173-740).
//
//   --workload cpu_pingpong  --transport uv|shm  --channel basic|cma|mpt  [--iters 1000]
//       two forked processes; every message = 64 KiB payload + four fp32 CPU tensors of shapes
//       [1024], [256,256], [64,64,64], [1<<20]; the server echoes; the client verifies every byte
//       and that callbacks arrive in order; prints p50 / p99 round-trip latency.
//   --workload cpu_small  --transport uv|shm  [--bytes 64]  [--iters 20000]
//       the same two processes exchanging a message that is one payload of --bytes and nothing
//       else (what the reference's benchmark_pipe does by default): the pipe's own cost per
//       message (descriptor, payload, callbacks), no channel involved.
//   --workload cpu_stream  --transport uv|shm  [--bytes 64]  [--iters 100000]  [--depth 16]
//       one way: the client keeps --depth payload-only messages in flight, the server reads them
//       and answers once at the end; prints microseconds per message and messages per second.
//   --workload pipe_setup  --transport uv|shm  --channel basic|cma|mpt  [--iters 200]
//       the client opens --iters pipes one after the other; for each, the time from connect() to
//       the answer to its first message (handshake, transport upgrade, channel connections).
//   --workload transport_pingpong  --transport uv|shm  [--bytes 64]  [--iters 20000]
//       raw transport connections (no pipe): one frame each way per round trip, two forked
//       processes; prints p50 / p99 round-trip latency (the reference's benchmark_transport,
//       tensorpipe/benchmark/benchmark_transport.cc:30-199).
//   --workload rpc_fanin  --ranks N  [--iters 20000]
//       rank 0 serves, ranks 1..N-1 (one forked process each, GPU r mod #GPUs) issue requests of a
//       256 B payload + one 4 KiB fp32 CUDA tensor and wait for a same-shaped reply; prints
//       p50 / p99 round-trip latency over all clients and messages per second.
//   --workload all_pairs  --ranks N  [--iters 10]
//       N forked processes, one per GPU; every rank sends every other rank a message of 64 CUDA
//       tensors (fp32 / bf16 / int64, 1 KiB - 16 MiB log-uniform), two messages in flight per
//       pipe, all pipes at once. Against this library a quarter of the tensors are transposed 2-D
//       views and half of the fp32 tensors are converted to bf16 on the way; the reference has
//       neither, so it moves contiguous tensors of the delivered sizes (its layout work is left
//       out, in its favour). Prints aggregate and per-GPU GB/s of delivered bytes, device-timed.
//   --workload pp_1f1b  --ranks S  [--iters 5] [--micro-batches 32] [--fwd-us 600] [--bwd-us 1200]
//       S pipeline stages, one process and GPU each; 16 MiB activations forward and 16 MiB
//       gradients backward between neighbours through pipes, 1F1B schedule, `micro-batches` per
//       step; the stage's compute is a device memset calibrated to last fwd-us / bwd-us, the same
//       for both libraries. Prints steps per second.
#include <cuda_runtime.h>
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <mutex>
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
  int microBatches = 32, fwdUs = 600, bwdUs = 1200;
  int depth = 16;
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
  // multi-rank workloads: every rank's listener URL, a reusable barrier, per-rank results
  char urls[64][128];
  std::atomic<int> urlsReady;
  std::atomic<int> barrierCount;
  std::atomic<int> barrierPhase;
  double deviceMs[64], hostMs[64];
  uint64_t delivered;
};

// All `n` ranks meet here; a rank that failed elsewhere makes the others give up instead of hanging.
static void rankBarrier(Shared* sh, int n) {
  const int phase = sh->barrierPhase.load();
  if (sh->barrierCount.fetch_add(1) + 1 == n) {
    sh->barrierCount = 0;
    sh->barrierPhase.fetch_add(1);
    return;
  }
  auto t0 = Clock::now();
  while (sh->barrierPhase.load() == phase) {
    if (sh->failed.load() || std::chrono::duration<double>(Clock::now() - t0).count() > 300) die("a peer rank failed");
    std::this_thread::yield();
  }
}

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
  if (o.channel == "mpt") {
    // Four lanes, each a TCP transport context (and thread) of its own, as PyTorch's agent sets
    // its "mpt_uv" channel up with more.
    std::vector<std::shared_ptr<lib::transport::Context>> contexts;
    std::vector<std::shared_ptr<lib::transport::Listener>> listeners;
    for (int lane = 0; lane < 4; ++lane) {
      auto c = lib::transport::uv::create();
      listeners.push_back(c->listen("127.0.0.1"));
      contexts.push_back(std::move(c));
    }
    ctx->registerChannel(10, "mpt", lib::channel::mpt::create(std::move(contexts), std::move(listeners)));
  }
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
    CpuMessage second;
    second.fill(54321);
    for (int i = 0; i < total; ++i) {
      // In-order check, every hundredth round trip (not timed): two different messages written
      // back to back; their write callbacks and their echoes must come in the order of the calls.
      if (i % 100 == 50 && i + 1 < total) {
        std::atomic<int> calls{0};
        int firstAt = -1, secondAt = -1;
        std::promise<void> w1, w2;
        pipe->write(msg.view(), [&](const lib::Error& e) {
          if (e) die("write: " + e.what());
          firstAt = calls++;
          w1.set_value();
        });
        pipe->write(second.view(), [&](const lib::Error& e) {
          if (e) die("write: " + e.what());
          secondAt = calls++;
          w2.set_value();
        });
        readInto(*pipe, echo);
        const bool firstOk = msg.equals(echo);
        readInto(*pipe, echo);
        const bool secondOk = second.equals(echo);
        w1.get_future().wait();
        w2.get_future().wait();
        if (!firstOk || !secondOk || firstAt != 0 || secondAt != 1) {
          sh->failed = 1;
          die("two messages written back to back did not come back, or call back, in order");
        }
        echo.payload[0] ^= 0xff;
        ++i;  // two of the server's round trips are used up
        continue;
      }
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
            << ", \"rtt_mean_us\": " << sh->mean[0]
            << ", \"verified\": \"byte-exact, every round trip; every hundredth, two messages back to back: callbacks and echoes in order\"}" << std::endl;
  return 0;
}

// ---- workload 1b: payload-only ping-pong (the default shape of the reference's benchmark_pipe) -----
static int cpuSmallPingPong(const Options& o, Shared* sh) {
  const int total = o.iters + o.warmup;
  // Everything runs from the library's callbacks, as in the reference's benchmark_pipe
  // (tensorpipe/benchmark/benchmark_pipe.cc:341-427): no thread of the benchmark stands between
  // a message's arrival and the answer to it.
  struct Side {
    std::shared_ptr<lib::Pipe> pipe;
    std::vector<uint8_t> out, in;
    int left = 0;
    bool client = false;
    int warmup = 0;
    Clock::time_point t0;
    std::vector<double> rtt;
    std::promise<void> finished;
    bool mismatch = false;
    void write() {
      lib::Message m;
      lib::Message::Payload p;
      p.data = out.data();
      p.length = out.size();
      m.payloads.push_back(p);
      pipe->write(std::move(m), [](const lib::Error& e) {
        if (e) die("write: " + e.what());
      });
    }
    void armRead() {
      pipe->readDescriptor([this](const lib::Error& e, lib::Descriptor d) {
        if (e) die("readDescriptor: " + e.what());
        if (d.payloads.size() != 1 || d.payloads[0].length != in.size()) die("unexpected message shape");
        lib::Allocation a;
        a.payloads.push_back({in.data()});
        pipe->read(std::move(a), [this](const lib::Error& e2) {
          if (e2) die("read: " + e2.what());
          arrived();
        });
      });
    }
    void arrived() {
      if (client) {
        const double us = std::chrono::duration<double, std::micro>(Clock::now() - t0).count();
        if (static_cast<int>(rtt.size()) + left <= 0) return;
        if (warmup > 0) --warmup;
        else rtt.push_back(us);
        mismatch = mismatch || in != out;
        if (--left == 0) return finished.set_value();
        out[0] = static_cast<uint8_t>(left);
        t0 = Clock::now();
        armRead();
        write();
      } else {
        out = in;  // echo what came
        if (--left > 0) armRead();
        write();
        if (left == 0) finished.set_value();
      }
    }
  };
  pid_t server = fork();
  if (server == 0) {
    auto ctx = makeCpuContext(o, "server");
    std::vector<std::string> urls = {"uv://127.0.0.1"};
    if (o.transport == "shm") urls.push_back("shm://");
    auto listener = ctx->listen(urls);
    std::strncpy(sh->url, listener->url("uv").c_str(), sizeof(sh->url) - 1);
    sh->urlReady = 1;
    std::promise<std::shared_ptr<lib::Pipe>> pp;
    listener->accept([&](const lib::Error& e, std::shared_ptr<lib::Pipe> p) {
      if (e) die("accept: " + e.what());
      pp.set_value(p);
    });
    Side side;
    side.pipe = pp.get_future().get();
    side.out.resize(o.bytes);
    side.in.resize(o.bytes);
    side.left = total;
    side.armRead();
    side.finished.get_future().wait();
    while (sh->clientsDone.load() == 0) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    ctx->join();
    _exit(0);
  }
  pid_t client = fork();
  if (client == 0) {
    while (sh->urlReady.load() == 0) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    auto ctx = makeCpuContext(o, "client");
    Side side;
    side.pipe = ctx->connect(sh->url);
    side.client = true;
    side.warmup = o.warmup;
    side.out.resize(o.bytes);
    side.in.resize(o.bytes);
    for (size_t k = 0; k < side.out.size(); ++k) side.out[k] = static_cast<uint8_t>(k * 31 + 7);
    side.left = total;
    side.t0 = Clock::now();
    side.armRead();
    side.write();
    side.finished.get_future().wait();
    if (side.mismatch) {
      sh->failed = 1;
      die("echo differs from what was sent");
    }
    sh->p50[0] = percentile(side.rtt, 0.5);
    sh->p99[0] = percentile(side.rtt, 0.99);
    double sum = 0;
    for (double v : side.rtt) sum += v;
    sh->mean[0] = sum / side.rtt.size();
    sh->clientsDone = 1;
    ctx->join();
    _exit(0);
  }
  int s1 = 0, s2 = 0;
  waitpid(client, &s2, 0);
  sh->clientsDone = 1;
  waitpid(server, &s1, 0);
  if (!WIFEXITED(s1) || WEXITSTATUS(s1) || !WIFEXITED(s2) || WEXITSTATUS(s2) || sh->failed) {
    std::cout << "{\"impl\": \"" << kImpl << "\", \"workload\": \"cpu_small\", \"error\": \"a peer failed\"}" << std::endl;
    return 1;
  }
  std::cout << "{\"impl\": \"" << kImpl << "\", \"workload\": \"cpu_small\", \"transport\": \"" << o.transport
            << "\", \"payload_bytes\": " << o.bytes << ", \"round_trips\": " << o.iters << ", \"rtt_p50_us\": "
            << sh->p50[0] << ", \"rtt_p99_us\": " << sh->p99[0] << ", \"rtt_mean_us\": " << sh->mean[0]
            << ", \"verified\": \"byte-exact, every round trip\"}" << std::endl;
  return 0;
}

// ---- workload 1c: a stream of payload-only messages, `depth` writes in flight -----------------------
static int cpuStream(const Options& o, Shared* sh) {
  const int total = o.iters;
  pid_t server = fork();
  if (server == 0) {
    auto ctx = makeCpuContext(o, "server");
    std::vector<std::string> urls = {"uv://127.0.0.1"};
    if (o.transport == "shm") urls.push_back("shm://");
    auto listener = ctx->listen(urls);
    std::strncpy(sh->url, listener->url("uv").c_str(), sizeof(sh->url) - 1);
    sh->urlReady = 1;
    std::promise<std::shared_ptr<lib::Pipe>> pp;
    listener->accept([&](const lib::Error& e, std::shared_ptr<lib::Pipe> p) {
      if (e) die("accept: " + e.what());
      pp.set_value(p);
    });
    auto pipe = pp.get_future().get();
    std::vector<uint8_t> in(o.bytes);
    std::promise<void> all;
    int left = total;
    uint64_t sum = 0;
    std::function<void()> arm = [&]() {
      pipe->readDescriptor([&](const lib::Error& e, lib::Descriptor d) {
        if (e) die("readDescriptor: " + e.what());
        if (d.payloads.size() != 1 || d.payloads[0].length != in.size()) die("unexpected message shape");
        lib::Allocation a;
        a.payloads.push_back({in.data()});
        pipe->read(std::move(a), [&](const lib::Error& e2) {
          if (e2) die("read: " + e2.what());
          sum += in[0];
          if (--left == 0) return all.set_value();
          arm();
        });
      });
    };
    arm();
    all.get_future().wait();
    // One message back tells the client that everything has arrived, and what arrived.
    std::promise<void> acked;
    lib::Message m;
    m.metadata = std::to_string(sum);
    pipe->write(std::move(m), [&](const lib::Error& e) {
      if (e) die("ack: " + e.what());
      acked.set_value();
    });
    acked.get_future().wait();
    while (sh->clientsDone.load() == 0) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    ctx->join();
    _exit(0);
  }
  pid_t client = fork();
  if (client == 0) {
    while (sh->urlReady.load() == 0) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    auto ctx = makeCpuContext(o, "client");
    auto pipe = ctx->connect(sh->url);
    const int depth = std::max(1, o.depth);
    std::vector<std::vector<uint8_t>> out(depth, std::vector<uint8_t>(o.bytes, 1));
    std::mutex mu;
    int issued = 0;
    uint64_t expected = 0;
    std::function<void(int)> writeNext = [&](int slot) {
      {
        std::lock_guard<std::mutex> lock(mu);
        if (issued == total) return;
        out[slot][0] = static_cast<uint8_t>(issued);
        expected += out[slot][0];
        ++issued;
      }
      lib::Message m;
      lib::Message::Payload p;
      p.data = out[slot].data();
      p.length = out[slot].size();
      m.payloads.push_back(p);
      pipe->write(std::move(m), [&, slot](const lib::Error& e) {
        if (e) die("write: " + e.what());
        writeNext(slot);
      });
    };
    std::promise<std::string> ack;
    pipe->readDescriptor([&](const lib::Error& e, lib::Descriptor d) {
      if (e) die("readDescriptor: " + e.what());
      std::string meta = d.metadata;
      pipe->read(lib::Allocation(), [&, meta](const lib::Error& e2) {
        if (e2) die("read: " + e2.what());
        ack.set_value(meta);
      });
    });
    auto t0 = Clock::now();
    for (int slot = 0; slot < depth; ++slot) writeNext(slot);
    const std::string got = ack.get_future().get();
    sh->seconds[0] = std::chrono::duration<double>(Clock::now() - t0).count();
    if (got != std::to_string(expected)) {
      sh->failed = 1;
      die("the server saw other bytes than were sent");
    }
    sh->clientsDone = 1;
    ctx->join();
    _exit(0);
  }
  int s1 = 0, s2 = 0;
  waitpid(client, &s2, 0);
  sh->clientsDone = 1;
  waitpid(server, &s1, 0);
  if (!WIFEXITED(s1) || WEXITSTATUS(s1) || !WIFEXITED(s2) || WEXITSTATUS(s2) || sh->failed) {
    std::cout << "{\"impl\": \"" << kImpl << "\", \"workload\": \"cpu_stream\", \"error\": \"a peer failed\"}" << std::endl;
    return 1;
  }
  std::cout << "{\"impl\": \"" << kImpl << "\", \"workload\": \"cpu_stream\", \"transport\": \"" << o.transport
            << "\", \"payload_bytes\": " << o.bytes << ", \"messages\": " << total << ", \"depth\": " << o.depth
            << ", \"us_per_message\": " << sh->seconds[0] / total * 1e6 << ", \"messages_per_second\": "
            << total / sh->seconds[0] << ", \"MBps\": " << static_cast<double>(total) * o.bytes / sh->seconds[0] / 1e6
            << ", \"verified\": \"checksum of the first byte of every message, kept by the server\"}" << std::endl;
  return 0;
}

// ---- workload 1d: how long a new pipe takes from connect() to its first answered message -----------
static int pipeSetup(const Options& o, Shared* sh) {
  const int total = o.iters;
  pid_t server = fork();
  if (server == 0) {
    auto ctx = makeCpuContext(o, "server");
    std::vector<std::string> urls = {"uv://127.0.0.1"};
    if (o.transport == "shm") urls.push_back("shm://");
    auto listener = ctx->listen(urls);
    std::strncpy(sh->url, listener->url("uv").c_str(), sizeof(sh->url) - 1);
    sh->urlReady = 1;
    // Every accepted pipe answers one message with one message; pipes are kept until the end.
    std::mutex mu;
    std::vector<std::shared_ptr<lib::Pipe>> pipes;
    std::function<void()> arm = [&]() {
      listener->accept([&](const lib::Error& e, std::shared_ptr<lib::Pipe> p) {
        if (e) return;  // the listener is closing
        {
          std::lock_guard<std::mutex> lock(mu);
          pipes.push_back(p);
        }
        lib::Pipe* raw = p.get();
        raw->readDescriptor([raw](const lib::Error& e2, lib::Descriptor) {
          if (e2) return;
          raw->read(lib::Allocation(), [raw](const lib::Error& e3) {
            if (e3) return;
            lib::Message m;
            m.metadata = "ok";
            raw->write(std::move(m), [](const lib::Error&) {});
          });
        });
        arm();
      });
    };
    arm();
    while (sh->clientsDone.load() == 0) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    listener.reset();
    pipes.clear();
    ctx->join();
    _exit(0);
  }
  pid_t client = fork();
  if (client == 0) {
    while (sh->urlReady.load() == 0) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    auto ctx = makeCpuContext(o, "client");
    std::vector<double> us;
    std::vector<std::shared_ptr<lib::Pipe>> pipes;
    for (int i = 0; i < total + 5; ++i) {
      auto t0 = Clock::now();
      auto pipe = ctx->connect(sh->url);
      std::promise<void> answered;
      pipe->readDescriptor([&](const lib::Error& e, lib::Descriptor d) {
        if (e) die("readDescriptor: " + e.what());
        if (d.metadata != "ok") die("unexpected answer");
        pipe->read(lib::Allocation(), [&](const lib::Error& e2) {
          if (e2) die("read: " + e2.what());
          answered.set_value();
        });
      });
      lib::Message m;
      m.metadata = "hello";
      pipe->write(std::move(m), [](const lib::Error& e) {
        if (e) die("write: " + e.what());
      });
      answered.get_future().wait();
      if (i >= 5) us.push_back(std::chrono::duration<double, std::micro>(Clock::now() - t0).count());
      pipes.push_back(std::move(pipe));
    }
    sh->p50[0] = percentile(us, 0.5);
    sh->p99[0] = percentile(us, 0.99);
    pipes.clear();
    sh->clientsDone = 1;
    ctx->join();
    _exit(0);
  }
  int s1 = 0, s2 = 0;
  waitpid(client, &s2, 0);
  sh->clientsDone = 1;
  waitpid(server, &s1, 0);
  if (!WIFEXITED(s1) || WEXITSTATUS(s1) || !WIFEXITED(s2) || WEXITSTATUS(s2) || sh->failed) {
    std::cout << "{\"impl\": \"" << kImpl << "\", \"workload\": \"pipe_setup\", \"error\": \"a peer failed\"}" << std::endl;
    return 1;
  }
  std::cout << "{\"impl\": \"" << kImpl << "\", \"workload\": \"pipe_setup\", \"transport\": \"" << o.transport
            << "\", \"channel\": \"" << o.channel << "\", \"pipes\": " << total << ", \"connect_to_first_answer_p50_us\": "
            << sh->p50[0] << ", \"p99_us\": " << sh->p99[0] << "}" << std::endl;
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


// ---- workload 3: all pairs ----------------------------------------------------------------------
namespace mesh {

struct Spec {
  int dtype;  // 0 fp32, 1 bf16, 2 int64
  bool transposed, cast;
  int64_t rows, cols;
  uint64_t srcOff, dstOff, srcBytes, dstBytes;
};
struct Layout {
  std::vector<Spec> specs;
  uint64_t srcTotal = 0, dstTotal = 0, delivered = 0;
};
// Same generator as the library's own ring benchmark: 64 tensors, dtype cycling fp32 / bf16 / int64,
// sizes log-uniform in [1 KiB, 16 MiB], every fourth a transposed view of 8 - 4096 columns, every
// other fp32 tensor delivered as bf16.
static Layout makeLayout(uint64_t seed) {
  Layout L;
  std::mt19937_64 rng(seed);
  int fp32Count = 0;
  for (int i = 0; i < 64; ++i) {
    Spec s{};
    s.dtype = i % 3;
    const uint64_t es = s.dtype == 0 ? 4 : (s.dtype == 1 ? 2 : 8);
    const double lg = std::log(1024.0) + (std::log(16.0 * 1024 * 1024) - std::log(1024.0)) *
                                              (static_cast<double>(rng() % 100000) / 100000.0);
    const uint64_t bytes = static_cast<uint64_t>(std::exp(lg));
    s.transposed = i % 4 == 3;
    s.cols = 64;
    if (s.transposed) {
      const double lc = std::log(8.0) + (std::log(4096.0) - std::log(8.0)) * (static_cast<double>(rng() % 100000) / 100000.0);
      s.cols = static_cast<int64_t>(std::exp(lc));
    }
    s.rows = static_cast<int64_t>(std::max<uint64_t>(1, bytes / es / s.cols));
    const uint64_t elems = static_cast<uint64_t>(s.rows) * s.cols;
    s.srcBytes = elems * es;
    if (s.dtype == 0) s.cast = (fp32Count++ % 2) == 0;
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

}  // namespace mesh

static int allPairs(const Options& o, Shared* sh) {
  const int world = o.ranks;
  if (world < 2 || world > 64) die("--ranks must be 2..64");
  const mesh::Layout layout = mesh::makeLayout(1234);
  sh->delivered = layout.delivered;
  std::vector<pid_t> pids;
  for (int rank = 0; rank < world; ++rank) {
    pid_t pid = fork();
    if (pid != 0) {
      pids.push_back(pid);
      continue;
    }
    int numGpus = 0;
    cudaGetDeviceCount(&numGpus);
    if (numGpus == 0) die("no GPU");
    const int dev = rank % numGpus;
    cudaSetDevice(dev);
    cudaStream_t recvStream;
    cudaStreamCreateWithFlags(&recvStream, cudaStreamNonBlocking);
    std::vector<cudaStream_t> sendStreams(world, nullptr);
    for (int j = 0; j < world; ++j)
      if (j != rank) cudaStreamCreateWithFlags(&sendStreams[j], cudaStreamNonBlocking);
    uint8_t* src = nullptr;
    uint8_t* dst[2] = {nullptr, nullptr};
    // Against the reference the source holds contiguous tensors of the delivered sizes.
#ifdef USE_REFERENCE
    const uint64_t srcTotal = layout.dstTotal;
#else
    const uint64_t srcTotal = layout.srcTotal;
#endif
    if (cudaMalloc(&src, srcTotal) != cudaSuccess) die("cudaMalloc");
    cudaMemset(src, 0x3c, srcTotal);
    for (auto& d : dst)
      if (cudaMalloc(&d, layout.dstTotal * (world - 1)) != cudaSuccess) die("cudaMalloc");
    cudaDeviceSynchronize();
    cudaEvent_t evStart, evEnd;
    cudaEventCreate(&evStart);
    cudaEventCreate(&evEnd);

    auto ctx = makeCudaContext("rank" + std::to_string(rank));
    auto listener = ctx->listen({"uv://127.0.0.1", "shm://"});
    std::strncpy(sh->urls[rank], listener->url("uv").c_str(), sizeof(sh->urls[rank]) - 1);
    sh->urlsReady.fetch_add(1);
    while (sh->urlsReady.load() < world) std::this_thread::sleep_for(std::chrono::milliseconds(1));

    // Pipes: one outgoing per peer (rotation order, so that the ranks do not all start with the
    // same receiver), one incoming per peer.
    std::mutex mu;
    std::vector<std::shared_ptr<lib::Pipe>> incoming;
    std::promise<void> allIn;
    std::function<void()> arm = [&]() {
      listener->accept([&](const lib::Error& e, std::shared_ptr<lib::Pipe> p) {
        if (e) return;
        bool done;
        {
          std::unique_lock<std::mutex> l(mu);
          incoming.push_back(std::move(p));
          done = static_cast<int>(incoming.size()) == world - 1;
        }
        if (done) allIn.set_value();
        else arm();
      });
    };
    arm();
    std::vector<std::shared_ptr<lib::Pipe>> outgoing;
    std::vector<int> outRank;
    for (int d = 1; d < world; ++d) {
      const int j = (rank + d) % world;
      outgoing.push_back(ctx->connect(sh->urls[j]));
      outRank.push_back(j);
    }
    if (allIn.get_future().wait_for(std::chrono::seconds(120)) != std::future_status::ready) die("mesh did not come up");

    auto runRound = [&](int iters, double* deviceMs, double* hostMs) {
      const int totalRecv = iters * (world - 1), totalSend = iters * (world - 1);
      std::atomic<int> received{0}, sent{0};
      std::promise<void> recvDone, sendDone;
      std::vector<int> readsIssued(world, 0);
      std::function<void(size_t, int)> armRead = [&](size_t k, int remaining) {
        if (remaining == 0) return;
        auto pipe = incoming[k];
        pipe->readDescriptor([&, k, remaining, pipe](const lib::Error& e, lib::Descriptor d) {
          if (e) die("readDescriptor: " + e.what());
          if (d.tensors.size() != layout.specs.size()) die("unexpected message shape");
          uint8_t* base = dst[readsIssued[k]++ & 1] + k * layout.dstTotal;
          lib::Allocation a;
          for (const auto& s : layout.specs) {
            lib::Allocation::Tensor t;
            t.buffer = cudaBuffer(base + s.dstOff, recvStream, dev);
#ifndef USE_REFERENCE
            if (s.cast) {
              t.castTo = lib::DType::kBF16;
              t.sourceDtype = lib::DType::kF32;
            }
#endif
            a.tensors.push_back(t);
          }
          pipe->read(std::move(a), [&, k, remaining](const lib::Error& e2) {
            if (e2) die("read: " + e2.what());
            if (received.fetch_add(1) + 1 == totalRecv) {
              cudaSetDevice(dev);
              cudaEventRecord(evEnd, recvStream);
              recvDone.set_value();
            } else {
              armRead(k, remaining - 1);
            }
          });
        });
      };
      std::function<void(size_t, int)> sendOne = [&](size_t k, int remaining) {
        if (remaining == 0) return;
        int targetDev = outRank[k] % numGpus;
        lib::Message msg;
        for (const auto& s : layout.specs) {
          lib::Message::Tensor t;
#ifdef USE_REFERENCE
          t.buffer = cudaBuffer(src + s.dstOff, sendStreams[outRank[k]], dev);
          t.length = s.dstBytes;
#else
          t.buffer = cudaBuffer(src + s.srcOff, sendStreams[outRank[k]], dev);
          t.length = s.srcBytes;
          t.dtype = s.dtype == 0 ? lib::DType::kF32 : (s.dtype == 1 ? lib::DType::kBF16 : lib::DType::kI64);
          if (s.transposed) {
            lib::StridedView v;
            v.dtype = t.dtype;
            v.rows = s.rows;
            v.cols = s.cols;
            v.rowStride = 1;
            v.colStride = s.rows;
            t.view = v;
          }
#endif
          t.targetDevice = lib::Device(lib::kCudaDeviceType, targetDev);
          msg.tensors.push_back(t);
        }
        outgoing[k]->write(std::move(msg), [&, k, remaining](const lib::Error& e) {
          if (e) die("write: " + e.what());
          if (sent.fetch_add(1) + 1 == totalSend) sendDone.set_value();
          sendOne(k, remaining - 1);
        });
      };
      rankBarrier(sh, world);
      auto t0 = Clock::now();
      cudaEventRecord(evStart, recvStream);
      for (int chain = 0; chain < 2; ++chain) {
        const int share = chain == 0 ? (iters + 1) / 2 : iters / 2;
        for (size_t k = 0; k < incoming.size(); ++k) armRead(k, share);
      }
      for (int chain = 0; chain < 2; ++chain) {
        const int share = chain == 0 ? (iters + 1) / 2 : iters / 2;
        for (size_t k = 0; k < outgoing.size(); ++k) sendOne(k, share);
      }
      if (recvDone.get_future().wait_for(std::chrono::seconds(300)) != std::future_status::ready) die("receiving timed out");
      if (sendDone.get_future().wait_for(std::chrono::seconds(300)) != std::future_status::ready) die("sending timed out");
      cudaEventSynchronize(evEnd);
      float ms = 0;
      cudaEventElapsedTime(&ms, evStart, evEnd);
      *deviceMs = ms;
      *hostMs = std::chrono::duration<double, std::milli>(Clock::now() - t0).count();
      for (int j = 0; j < world; ++j)
        if (sendStreams[j]) cudaStreamSynchronize(sendStreams[j]);
    };
    double dms = 0, hms = 0;
    runRound(std::max(2, o.warmup > 10 ? 3 : o.warmup), &dms, &hms);
    runRound(o.iters, &dms, &hms);
    sh->deviceMs[rank] = dms;
    sh->hostMs[rank] = hms;
    rankBarrier(sh, world);
    outgoing.clear();
    incoming.clear();
    ctx->join();
    _exit(0);
  }
  bool ok = true;
  for (pid_t pid : pids) {
    int st = 0;
    waitpid(pid, &st, 0);
    if (!WIFEXITED(st) || WEXITSTATUS(st)) {
      ok = false;
      sh->failed = 1;
    }
  }
  if (!ok) {
    std::cout << "{\"impl\": \"" << kImpl << "\", \"workload\": \"all_pairs\", \"error\": \"a rank failed\"}" << std::endl;
    return 1;
  }
  double ms = 0;
  for (int r = 0; r < world; ++r) ms = std::max(ms, sh->deviceMs[r]);
  ms /= o.iters;
  const double perGpu = static_cast<double>(sh->delivered) * (world - 1) / (ms * 1e-3) / 1e9;
  std::cout << "{\"impl\": \"" << kImpl << "\", \"workload\": \"all_pairs\", \"ranks\": " << world
            << ", \"tensors_per_message\": 64, \"bytes_per_message\": " << sh->delivered
            << ", \"ms_per_round\": " << ms << ", \"per_gpu_egress_GBps\": " << perGpu
            << ", \"aggregate_GBps\": " << perGpu * world << ", \"per_gpu_fraction_of_900\": " << perGpu / 900.0
            << ", \"layout_work\": \""
#ifdef USE_REFERENCE
            << "none: contiguous tensors of the delivered sizes"
#else
            << "16 transposed views of 8-4096 columns, 11 fp32->bf16 conversions"
#endif
            << "\"}" << std::endl;
  return 0;
}

// ---- workload 4: 1F1B pipeline --------------------------------------------------------------------
static int pipeline1F1B(const Options& o, Shared* sh) {
  const int stages = o.ranks;
  if (stages < 2 || stages > 64) die("--ranks must be 2..64");
  constexpr size_t kActivation = 16u << 20;  // 8 x 1024 tokens x 1024 features, bf16
  const int M = o.microBatches;
  std::vector<pid_t> pids;
  for (int s = 0; s < stages; ++s) {
    pid_t pid = fork();
    if (pid != 0) {
      pids.push_back(pid);
      continue;
    }
    int numGpus = 0;
    cudaGetDeviceCount(&numGpus);
    if (numGpus == 0) die("no GPU");
    const int dev = s % numGpus;
    cudaSetDevice(dev);
    cudaStream_t stream;
    cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
    // Activation / gradient buffers: one per micro-batch in flight (at most `stages` of them).
    const int slots = stages + 1;
    std::vector<uint8_t*> actIn(slots), actOut(slots), gradIn(slots), gradOut(slots);
    for (int i = 0; i < slots; ++i) {
      cudaMalloc(&actIn[i], kActivation);
      cudaMalloc(&actOut[i], kActivation);
      cudaMalloc(&gradIn[i], kActivation);
      cudaMalloc(&gradOut[i], kActivation);
    }
    // "Compute": a memset sized so that it lasts the requested time on this GPU.
    uint8_t* scratch = nullptr;
    const size_t scratchBytes = 1ull << 30;
    if (cudaMalloc(&scratch, scratchBytes) != cudaSuccess) die("cudaMalloc scratch");
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    for (int i = 0; i < 3; ++i) cudaMemsetAsync(scratch, i, scratchBytes, stream);
    cudaEventRecord(e0, stream);
    cudaMemsetAsync(scratch, 7, scratchBytes, stream);
    cudaEventRecord(e1, stream);
    cudaEventSynchronize(e1);
    float msPerGiB = 0;
    cudaEventElapsedTime(&msPerGiB, e0, e1);
    auto compute = [&](int us) {
      size_t bytes = static_cast<size_t>(static_cast<double>(us) * 1e-3 / msPerGiB * scratchBytes);
      while (bytes > 0) {
        const size_t n = std::min(bytes, scratchBytes);
        cudaMemsetAsync(scratch, 1, n, stream);
        bytes -= n;
      }
    };

    auto ctx = makeCudaContext("stage" + std::to_string(s));
    auto listener = ctx->listen({"uv://127.0.0.1", "shm://"});
    std::strncpy(sh->urls[s], listener->url("uv").c_str(), sizeof(sh->urls[s]) - 1);
    sh->urlsReady.fetch_add(1);
    while (sh->urlsReady.load() < stages) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    // One pipe per neighbour pair: stage s dials stage s+1; activations go down it, gradients come back up.
    std::shared_ptr<lib::Pipe> next, prev;
    std::promise<std::shared_ptr<lib::Pipe>> accepted;
    if (s > 0)
      listener->accept([&](const lib::Error& e, std::shared_ptr<lib::Pipe> p) {
        if (e) die("accept: " + e.what());
        accepted.set_value(std::move(p));
      });
    if (s < stages - 1) next = ctx->connect(sh->urls[s + 1]);
    if (s > 0) prev = accepted.get_future().get();
    const int nextDev = (s + 1) % numGpus, prevDev = (s + stages - 1) % numGpus;

    auto sendTensor = [&](lib::Pipe& pipe, uint8_t* p, int targetDev) {
      lib::Message m;
      lib::Message::Tensor t;
      t.buffer = cudaBuffer(p, stream, dev);
      t.length = kActivation;
      t.targetDevice = lib::Device(lib::kCudaDeviceType, targetDev);
      m.tensors.push_back(t);
      pipe.write(std::move(m), [](const lib::Error& e) {
        if (e) die("write: " + e.what());
      });
    };
    auto recvTensor = [&](lib::Pipe& pipe, uint8_t* p) {
      std::promise<void> got;
      pipe.readDescriptor([&](const lib::Error& e, lib::Descriptor) {
        if (e) die("readDescriptor: " + e.what());
        lib::Allocation a;
        lib::Allocation::Tensor t;
        t.buffer = cudaBuffer(p, stream, dev);
        a.tensors.push_back(t);
        pipe.read(std::move(a), [&](const lib::Error& e2) {
          if (e2) die("read: " + e2.what());
          got.set_value();
        });
      });
      if (got.get_future().wait_for(std::chrono::seconds(120)) != std::future_status::ready) die("a stage stopped answering");
    };
    auto forward = [&](int mb) {
      if (s > 0) recvTensor(*prev, actIn[mb % slots]);
      compute(o.fwdUs);
      if (s < stages - 1) sendTensor(*next, actOut[mb % slots], nextDev);
    };
    auto backward = [&](int mb) {
      if (s < stages - 1) recvTensor(*next, gradIn[mb % slots]);
      compute(o.bwdUs);
      if (s > 0) sendTensor(*prev, gradOut[mb % slots], prevDev);
    };
    auto step = [&]() {
      // 1F1B: warm up with as many forwards as there are stages behind this one, then alternate,
      // then drain the backwards.
      const int warm = std::min(M, stages - 1 - s);
      int f = 0, b = 0;
      for (; f < warm; ++f) forward(f);
      while (f < M) {
        forward(f++);
        backward(b++);
      }
      while (b < M) backward(b++);
      cudaStreamSynchronize(stream);
    };
    for (int i = 0; i < std::max(1, std::min(o.warmup, 2)); ++i) step();
    rankBarrier(sh, stages);
    auto t0 = Clock::now();
    for (int i = 0; i < o.iters; ++i) step();
    sh->seconds[s] = std::chrono::duration<double>(Clock::now() - t0).count();
    rankBarrier(sh, stages);
    next.reset();
    prev.reset();
    ctx->join();
    _exit(0);
  }
  bool ok = true;
  for (pid_t pid : pids) {
    int st = 0;
    waitpid(pid, &st, 0);
    if (!WIFEXITED(st) || WEXITSTATUS(st)) {
      ok = false;
      sh->failed = 1;
    }
  }
  if (!ok) {
    std::cout << "{\"impl\": \"" << kImpl << "\", \"workload\": \"pp_1f1b\", \"error\": \"a stage failed\"}" << std::endl;
    return 1;
  }
  double seconds = 0;
  for (int s = 0; s < stages; ++s) seconds = std::max(seconds, sh->seconds[s]);
  // What the schedule costs with free communication: (M + stages - 1) slots of (fwd + bwd).
  const double ideal = (o.microBatches + stages - 1) * (o.fwdUs + o.bwdUs) * 1e-6;
  std::cout << "{\"impl\": \"" << kImpl << "\", \"workload\": \"pp_1f1b\", \"stages\": " << stages
            << ", \"micro_batches\": " << o.microBatches << ", \"activation_bytes\": " << kActivation
            << ", \"fwd_us\": " << o.fwdUs << ", \"bwd_us\": " << o.bwdUs << ", \"steps\": " << o.iters
            << ", \"steps_per_second\": " << o.iters / seconds << ", \"seconds_per_step\": " << seconds / o.iters
            << ", \"compute_only_seconds_per_step\": " << ideal << "}" << std::endl;
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
    else if (k == "--depth") o.depth = std::stoi(v);
    else if (k == "--micro-batches") o.microBatches = std::stoi(v);
    else if (k == "--fwd-us") o.fwdUs = std::stoi(v);
    else if (k == "--bwd-us") o.bwdUs = std::stoi(v);
  }
  auto* sh = static_cast<Shared*>(mmap(nullptr, sizeof(Shared), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0));
  std::memset(static_cast<void*>(sh), 0, sizeof(Shared));
  if (o.workload == "cpu_pingpong") return cpuPingPong(o, sh);
  if (o.workload == "cpu_small") return cpuSmallPingPong(o, sh);
  if (o.workload == "cpu_stream") return cpuStream(o, sh);
  if (o.workload == "pipe_setup") return pipeSetup(o, sh);
  if (o.workload == "rpc_fanin") return rpcFanIn(o, sh);
  if (o.workload == "transport_pingpong") return transportPingPong(o, sh);
  if (o.workload == "all_pairs") return allPairs(o, sh);
  if (o.workload == "pp_1f1b") return pipeline1F1B(o, sh);
  std::cerr << "unknown workload" << std::endl;
  return 2;
}
