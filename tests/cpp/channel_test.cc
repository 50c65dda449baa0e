// Generic channel suite: one body, every CPU channel, on raw transport connections (no pipe), the
// way the reference organises its channel tests (tensorpipe/test/channel/channel_test.cc:18-336,
// channel_test_cpu.cc:19-109): the two peers open N TCP connections tagged with an index, hand
// them to createChannel on both sides, and exchange tensors.
#include <tpb/tpb.h>

#include <mutex>
#include <random>

#include "channel/copy_channel.h"
#include "channel_wiring.h"
#include "test_util.h"

using namespace tpb;
using namespace tpbtest;

namespace {

struct Backend {
  const char* name;
  std::function<std::shared_ptr<channel::Context>()> make;
  bool needsProcesses;  // endpoints must be different processes
};

std::shared_ptr<channel::Context> makeMpt() {
  std::vector<std::shared_ptr<transport::Context>> ctxs;
  std::vector<std::shared_ptr<transport::Listener>> listeners;
  for (int i = 0; i < 3; ++i) {
    auto c = transport::uv::create();
    listeners.push_back(c->listen("127.0.0.1"));
    ctxs.push_back(std::move(c));
  }
  return channel::mpt::create(std::move(ctxs), std::move(listeners));
}

const Backend kBackends[] = {
    {"basic", [] { return channel::basic::create(); }, false},
    {"xth", [] { return channel::xth::create(); }, false},
    {"mpt", [] { return makeMpt(); }, false},
    {"cma", [] { return channel::cma::create(); }, true},
};

void sendSync(channel::Channel& ch, void* p, size_t n) {
  std::promise<Error> pr;
  ch.send(CpuBuffer{p}, n, [&](const Error& e) { pr.set_value(e); });
  auto f = pr.get_future();
  Error e = waitFor(f);
  if (e) throw TestFailure("send: " + e.what());
}
void recvSync(channel::Channel& ch, void* p, size_t n) {
  std::promise<Error> pr;
  ch.recv(CpuBuffer{p}, n, [&](const Error& e) { pr.set_value(e); });
  auto f = pr.get_future();
  Error e = waitFor(f);
  if (e) throw TestFailure("recv: " + e.what());
}
std::vector<uint8_t> pattern(size_t n, uint32_t seed) {
  std::vector<uint8_t> v(n);
  std::mt19937 rng(seed);
  for (auto& b : v) b = static_cast<uint8_t>(rng());
  return v;
}

using Body = std::function<void(channel::Channel&)>;

// Runs server/client bodies over one channel of the backend, as threads or as processes.
void runChannel(const Backend& b, Body server, Body client) {
  auto serverSide = [&](std::function<void(std::string)> tell, std::function<std::string()> hear) {
    auto cctx = b.make();
    if (!cctx->isViable()) {
      tell("skip");
      return;
    }
    Wiring w;
    tell(w.listen());
    auto conns = w.acceptAll(cctx->numConnectionsNeeded());
    auto ch = cctx->createChannel(std::move(conns), channel::Endpoint::kListen);
    server(*ch);
    hear();
    ch->close();
    ch.reset();
    cctx->join();
    w.tctx->join();
  };
  auto clientSide = [&](std::function<void(std::string)> tell, std::function<std::string()> hear) {
    std::string addr = hear();
    if (addr == "skip") return;
    auto cctx = b.make();
    Wiring w;
    auto conns = w.connectAll(addr, cctx->numConnectionsNeeded());
    auto ch = cctx->createChannel(std::move(conns), channel::Endpoint::kConnect);
    client(*ch);
    tell("done");
    ch->close();
    ch.reset();
    cctx->join();
    w.tctx->join();
  };
  if (b.needsProcesses) {
    ProcessPeers::run(
        [&](const ProcessPeers::Side& me) { serverSide([&](std::string s) { me.send(s); }, [&] { return me.recv(); }); },
        [&](const ProcessPeers::Side& me) { clientSide([&](std::string s) { me.send(s); }, [&] { return me.recv(); }); });
  } else {
    ThreadPeers peers;
    peers.run(
        [&](ThreadPeers& pg) { serverSide([&](std::string s) { pg.sendToClient(s); }, [&] { return pg.recvFromClient(); }); },
        [&](ThreadPeers& pg) { clientSide([&](std::string s) { pg.sendToServer(s); }, [&] { return pg.recvFromServer(); }); });
  }
}

void forEachBackend(std::function<void(const Backend&)> body) {
  for (const auto& b : kBackends) {
    try {
      body(b);
    } catch (const TestFailure& e) {
      throw TestFailure(std::string("[") + b.name + "] " + e.what());
    }
  }
}

}  // namespace

TPB_TEST(Channel, DeviceDescriptors) {
  forEachBackend([](const Backend& b) {
    auto a = b.make();
    auto c = b.make();
    if (!a->isViable()) return;
    const auto& da = a->deviceDescriptors();
    const auto& dc = c->deviceDescriptors();
    EXPECT_TRUE(da.count(Device(kCpuDeviceType, 0)) == 1);
    for (const auto& d : da) {
      EXPECT_FALSE(d.second.empty());
      // Two contexts of one process describe the same endpoint.
      EXPECT_TRUE(a->canCommunicateWithRemote(d.second, dc.at(d.first)));
      EXPECT_FALSE(a->canCommunicateWithRemote(d.second, "nonsense"));
    }
    a->join();
    c->join();
  });
}

TPB_TEST(Channel, ClientToServerAndBack) {
  forEachBackend([](const Backend& b) {
    auto data = pattern(300007, 1);
    runChannel(
        b,
        [&](channel::Channel& ch) {
          std::vector<uint8_t> got(data.size());
          recvSync(ch, got.data(), got.size());
          EXPECT_TRUE(got == data);
          sendSync(ch, got.data(), got.size());
        },
        [&](channel::Channel& ch) {
          auto copy = data;
          sendSync(ch, copy.data(), copy.size());
          std::vector<uint8_t> back(data.size());
          recvSync(ch, back.data(), back.size());
          EXPECT_TRUE(back == data);
        });
  });
}

TPB_TEST(Channel, SendMultipleTensorsKeepsOrder) {
  forEachBackend([](const Backend& b) {
    constexpr int kN = 20;
    runChannel(
        b,
        [&](channel::Channel& ch) {
          std::vector<std::vector<uint8_t>> got(kN);
          std::vector<std::promise<Error>> done(kN);
          for (int i = 0; i < kN; ++i) {
            got[i].resize(1000 + i * 997);
            ch.recv(CpuBuffer{got[i].data()}, got[i].size(), [&, i](const Error& e) { done[i].set_value(e); });
          }
          for (int i = 0; i < kN; ++i) {
            auto f = done[i].get_future();
            EXPECT_FALSE(bool(waitFor(f)));
            EXPECT_TRUE(got[i] == pattern(1000 + i * 997, 50 + i));
          }
        },
        [&](channel::Channel& ch) {
          std::vector<std::vector<uint8_t>> data(kN);
          std::vector<std::promise<Error>> done(kN);
          for (int i = 0; i < kN; ++i) {
            data[i] = pattern(1000 + i * 997, 50 + i);
            ch.send(CpuBuffer{data[i].data()}, data[i].size(), [&, i](const Error& e) { done[i].set_value(e); });
          }
          for (int i = 0; i < kN; ++i) {
            auto f = done[i].get_future();
            EXPECT_FALSE(bool(waitFor(f)));
          }
        });
  });
}

// Large tensors (sliced over several copy threads where the channel has them) between small ones:
// the bytes are right and the callbacks on both sides come in the order of the calls, although
// the small copies finish long before the large ones ahead of them.
TPB_TEST(Channel, LargeAndSmallTensorsCompleteInOrder) {
  forEachBackend([](const Backend& b) {
    const std::vector<size_t> sizes = {6u << 20, 100, (3u << 20) + 17, 4096, 5u << 20, 1, (1u << 20) + 1, 64};
    const int n = static_cast<int>(sizes.size());
    runChannel(
        b,
        [&](channel::Channel& ch) {
          std::vector<std::vector<uint8_t>> got(n);
          std::vector<std::promise<Error>> done(n);
          std::mutex mu;
          std::vector<int> order;
          for (int i = 0; i < n; ++i) {
            got[i].resize(sizes[i]);
            ch.recv(CpuBuffer{got[i].data()}, got[i].size(), [&, i](const Error& e) {
              {
                std::lock_guard<std::mutex> lock(mu);
                order.push_back(i);
              }
              done[i].set_value(e);
            });
          }
          for (int i = 0; i < n; ++i) {
            auto f = done[i].get_future();
            EXPECT_FALSE(bool(waitFor(f)));
            EXPECT_TRUE(got[i] == pattern(sizes[i], 900 + i));
          }
          std::lock_guard<std::mutex> lock(mu);
          for (int i = 0; i < n; ++i) EXPECT_EQ(order[i], i);
        },
        [&](channel::Channel& ch) {
          std::vector<std::vector<uint8_t>> data(n);
          std::vector<std::promise<Error>> done(n);
          std::mutex mu;
          std::vector<int> order;
          for (int i = 0; i < n; ++i) {
            data[i] = pattern(sizes[i], 900 + i);
            ch.send(CpuBuffer{data[i].data()}, data[i].size(), [&, i](const Error& e) {
              {
                std::lock_guard<std::mutex> lock(mu);
                order.push_back(i);
              }
              done[i].set_value(e);
            });
          }
          for (int i = 0; i < n; ++i) {
            auto f = done[i].get_future();
            EXPECT_FALSE(bool(waitFor(f)));
          }
          std::lock_guard<std::mutex> lock(mu);
          for (int i = 0; i < n; ++i) EXPECT_EQ(order[i], i);
        });
  });
}

// One slice of a sliced copy fails (a copy function that refuses one address range stands in for
// process_vm_readv on memory that has gone away): that receive reports the error, the one before
// it succeeds, the ones after it fail, all in the order of the calls, and the sender's pending
// callbacks end with an error instead of hanging.
TPB_TEST(Channel, AFailedSliceFailsItsReceiveAndThoseBehindIt) {
  static std::atomic<uintptr_t> poisonBegin{0}, poisonEnd{0};
  static auto copyFn = [](uint64_t, const void* remote, void* local, size_t len) -> Error {
    const uintptr_t a = reinterpret_cast<uintptr_t>(remote);
    if (a < poisonEnd.load() && a + len > poisonBegin.load()) return TPB_CREATE_ERROR(SystemError, "process_vm_readv", EFAULT);
    std::memcpy(local, remote, len);
    return Error::kSuccess;
  };
  Backend sliced{"sliced copy",
                 [] {
                   ::setenv("TPB_COPY_THREADS", "4", 1);
                   auto ctx = std::make_shared<channel::copy::ContextImpl>(
                       "tpbtest:any", +[](uint64_t pid, const void* r, void* l, size_t n) { return copyFn(pid, r, l, n); },
                       "TP_TEST_copy");
                   ::unsetenv("TPB_COPY_THREADS");
                   return std::static_pointer_cast<channel::Context>(ctx);
                 },
                 false};
  constexpr size_t kBytes = 4u << 20;
  std::vector<std::vector<uint8_t>> data(3);
  for (int i = 0; i < 3; ++i) data[i] = pattern(kBytes, 70 + i);
  // the third quarter of the second tensor cannot be read
  poisonBegin = reinterpret_cast<uintptr_t>(data[1].data()) + kBytes / 2;
  poisonEnd = poisonBegin.load() + 4096;
  runChannel(
      sliced,
      [&](channel::Channel& ch) {
        std::vector<std::vector<uint8_t>> got(3, std::vector<uint8_t>(kBytes));
        std::vector<std::promise<Error>> done(3);
        std::mutex mu;
        std::vector<int> order;
        for (int i = 0; i < 3; ++i)
          ch.recv(CpuBuffer{got[i].data()}, kBytes, [&, i](const Error& e) {
            {
              std::lock_guard<std::mutex> lock(mu);
              order.push_back(i);
            }
            done[i].set_value(e);
          });
        std::vector<Error> results;
        for (int i = 0; i < 3; ++i) {
          auto f = done[i].get_future();
          results.push_back(waitFor(f));
        }
        EXPECT_FALSE(bool(results[0]));
        EXPECT_TRUE(got[0] == data[0]);
        EXPECT_TRUE(bool(results[1]));
        EXPECT_TRUE(bool(results[2]));
        std::lock_guard<std::mutex> lock(mu);
        for (int i = 0; i < 3; ++i) EXPECT_EQ(order[i], i);
      },
      [&](channel::Channel& ch) {
        std::vector<std::promise<Error>> done(3);
        for (int i = 0; i < 3; ++i)
          ch.send(CpuBuffer{data[i].data()}, kBytes, [&, i](const Error& e) { done[i].set_value(e); });
        auto f0 = done[0].get_future();
        EXPECT_FALSE(bool(waitFor(f0)));
        for (int i = 1; i < 3; ++i) {
          auto f = done[i].get_future();
          EXPECT_TRUE(bool(waitFor(f)));
        }
      });
  poisonBegin = 0;
  poisonEnd = 0;
}

// The last reference to a copy context may die on one of its own worker threads (the job holds
// one while it runs): the context then winds down from there without waiting for that thread.
TPB_TEST(Channel, ACopyContextMayDieOnItsOwnWorker) {
  static std::atomic<int> copies{0};
  for (size_t bytes : {size_t(64), size_t(4u << 20)}) {
    auto ctx = std::make_shared<channel::copy::ContextImpl>(
        "tpbtest:any",
        +[](uint64_t, const void* r, void* l, size_t n) -> Error {
          std::this_thread::sleep_for(std::chrono::milliseconds(30));
          std::memcpy(l, r, n);
          ++copies;
          return Error::kSuccess;
        },
        "TP_TEST_copy");
    auto src = std::make_shared<std::vector<uint8_t>>(pattern(bytes, 5));
    auto dst = std::make_shared<std::vector<uint8_t>>(bytes);
    auto finished = std::make_shared<std::promise<Error>>();
    auto f = finished->get_future();
    ctx->requestCopy(0, src->data(), dst->data(), bytes, [finished, src, dst](const Error& e) { finished->set_value(e); });
    ctx.reset();  // the jobs hold the only references now
    EXPECT_FALSE(bool(waitFor(f)));
    EXPECT_TRUE(*src == *dst);
  }
  std::this_thread::sleep_for(std::chrono::milliseconds(100));  // let the workers run out
  EXPECT_TRUE(copies.load() >= 2);
}

TPB_TEST(Channel, SendTensorsBothWaysAtOnce) {
  forEachBackend([](const Backend& b) {
    auto a = pattern(123457, 7), c = pattern(76543, 8);
    auto side = [&](const std::vector<uint8_t>& mine, const std::vector<uint8_t>& theirs) {
      return [&](channel::Channel& ch) {
        auto out = mine;
        std::vector<uint8_t> in(theirs.size());
        std::promise<Error> ps, pr;
        ch.send(CpuBuffer{out.data()}, out.size(), [&](const Error& e) { ps.set_value(e); });
        ch.recv(CpuBuffer{in.data()}, in.size(), [&](const Error& e) { pr.set_value(e); });
        auto fs = ps.get_future(), fr = pr.get_future();
        EXPECT_FALSE(bool(waitFor(fs)));
        EXPECT_FALSE(bool(waitFor(fr)));
        EXPECT_TRUE(in == theirs);
      };
    };
    runChannel(b, side(a, c), side(c, a));
  });
}

TPB_TEST(Channel, EmptyAndNullTensors) {
  forEachBackend([](const Backend& b) {
    auto data = pattern(4096, 9);
    runChannel(
        b,
        [&](channel::Channel& ch) {
          std::vector<uint8_t> got(data.size());
          recvSync(ch, nullptr, 0);  // a null pointer with length 0 is legal
          recvSync(ch, got.data(), got.size());
          recvSync(ch, got.data(), 0);
          EXPECT_TRUE(got == data);
        },
        [&](channel::Channel& ch) {
          auto copy = data;
          sendSync(ch, nullptr, 0);
          sendSync(ch, copy.data(), copy.size());
          sendSync(ch, copy.data(), 0);
        });
  });
}

TPB_TEST(Channel, CallbacksAreDeferred) {
  // The copy must not happen inside recv()/send(): the mutex is held across the call and taken
  // inside the callback, so a callback that runs inline deadlocks (the reference's check,
  // tensorpipe/test/channel/channel_test_cpu.cc:45-109).
  forEachBackend([](const Backend& b) {
    if (b.needsProcesses) return;
    auto data = pattern(100000, 3);
    runChannel(
        b,
        [&](channel::Channel& ch) {
          std::vector<uint8_t> got(data.size());
          std::mutex m;
          std::promise<Error> done;
          {
            std::unique_lock<std::mutex> lock(m);
            ch.recv(CpuBuffer{got.data()}, got.size(), [&](const Error& e) {
              std::unique_lock<std::mutex> inner(m);
              done.set_value(e);
            });
            std::this_thread::sleep_for(std::chrono::milliseconds(2));
          }
          auto f = done.get_future();
          EXPECT_FALSE(bool(waitFor(f)));
          EXPECT_TRUE(got == data);
        },
        [&](channel::Channel& ch) {
          auto copy = data;
          std::mutex m;
          std::promise<Error> done;
          {
            std::unique_lock<std::mutex> lock(m);
            ch.send(CpuBuffer{copy.data()}, copy.size(), [&](const Error& e) {
              std::unique_lock<std::mutex> inner(m);
              done.set_value(e);
            });
            std::this_thread::sleep_for(std::chrono::milliseconds(2));
          }
          auto f = done.get_future();
          EXPECT_FALSE(bool(waitFor(f)));
        });
  });
}

TPB_TEST(Channel, ClosingFailsPendingOperations) {
  forEachBackend([](const Backend& b) {
    runChannel(
        b,
        [&](channel::Channel& ch) {
          std::vector<uint8_t> buf(100);
          std::promise<Error> pr;
          ch.recv(CpuBuffer{buf.data()}, buf.size(), [&](const Error& e) { pr.set_value(e); });
          ch.close();
          auto f = pr.get_future();
          EXPECT_TRUE(bool(waitFor(f)));
        },
        [&](channel::Channel&) {});
  });
}

TPB_TEST(Channel, XthDoesNotMatchAcrossProcessesAndCmaDoes) {
  ProcessPeers::run(
      [](const ProcessPeers::Side& me) {
        auto xth = channel::xth::create();
        auto cma = channel::cma::create();
        me.send(xth->deviceDescriptors().at(Device(kCpuDeviceType, 0)));
        me.send(cma->isViable() ? cma->deviceDescriptors().at(Device(kCpuDeviceType, 0)) : std::string("n/a"));
        me.recv();
        xth->join();
        cma->join();
      },
      [](const ProcessPeers::Side& me) {
        auto xth = channel::xth::create();
        auto cma = channel::cma::create();
        std::string remoteXth = me.recv(), remoteCma = me.recv();
        const std::string& localXth = xth->deviceDescriptors().at(Device(kCpuDeviceType, 0));
        EXPECT_FALSE(xth->canCommunicateWithRemote(localXth, remoteXth));
        if (cma->isViable() && remoteCma != "n/a") {
          const std::string& localCma = cma->deviceDescriptors().at(Device(kCpuDeviceType, 0));
          EXPECT_TRUE(cma->canCommunicateWithRemote(localCma, remoteCma));
        }
        me.send("done");
        xth->join();
        cma->join();
      });
}

TPB_TEST(Channel, NonViableBackendsDegradeGracefully) {
  auto gdr = channel::cuda_gdr::create();
  EXPECT_FALSE(gdr->isViable());
  EXPECT_TRUE(gdr->deviceDescriptors().empty());
  auto ibv = transport::ibv::create();
  EXPECT_FALSE(ibv->isViable());
  // Registration silently skips them.
  Context ctx;
  ctx.registerTransport(0, "ibv", ibv);
  ctx.registerChannel(0, "cuda_gdr", gdr);
  ctx.registerTransport(1, "uv", transport::uv::create());
  EXPECT_THROWS(ctx.listen({"ibv://127.0.0.1"}));
  ctx.join();
}

TPB_TEST(Channel, CudaBasicNeverServesCpuToCpu) {
  auto cb = channel::cuda_basic::create(channel::basic::create());
  if (!cb->isViable()) return;  // no GPU here: nothing to check
  const auto& d = cb->deviceDescriptors();
  const std::string& cpu = d.at(Device(kCpuDeviceType, 0));
  EXPECT_FALSE(cb->canCommunicateWithRemote(cpu, cpu));
  cb->join();
}

// Through a full pipe: the best CPU channel wins per the priorities, and the data arrives.
TPB_TEST(Channel, PipeSelectsCmaAcrossProcessesAndXthInside) {
  auto make = [](const std::string& name) {
    auto ctx = std::make_shared<Context>(ContextOptions().name(name));
    ctx->registerTransport(0, "uv", transport::uv::create());
    ctx->registerTransport(1, "shm", transport::shm::create());
    ctx->registerChannel(0, "basic", channel::basic::create());
    ctx->registerChannel(10, "cma", channel::cma::create());
    ctx->registerChannel(20, "xth", channel::xth::create());
    return ctx;
  };
  auto data = pattern(2u << 20, 77);
  ProcessPeers::run(
      [&](const ProcessPeers::Side& me) {
        auto ctx = make("server");
        auto l = ctx->listen({"uv://127.0.0.1", "shm://"});
        me.send(l->url("uv"));
        std::promise<std::shared_ptr<Pipe>> pp;
        l->accept([&](const Error&, std::shared_ptr<Pipe> p) { pp.set_value(p); });
        auto fp = pp.get_future();
        auto pipe = waitFor(fp);
        std::promise<Descriptor> pd;
        pipe->readDescriptor([&](const Error&, Descriptor d) { pd.set_value(d); });
        auto fd = pd.get_future();
        Descriptor d = waitFor(fd);
        std::vector<uint8_t> got(d.tensors.at(0).length);
        Allocation a;
        Allocation::Tensor t;
        t.buffer = CpuBuffer{got.data()};
        a.tensors.push_back(t);
        std::promise<Error> pr;
        pipe->read(a, [&](const Error& e) { pr.set_value(e); });
        auto fr = pr.get_future();
        EXPECT_FALSE(bool(waitFor(fr)));
        EXPECT_TRUE(got == data);
        auto stats = ctx->stats();
        const bool cmaViable = channel::cma::create()->isViable();
        EXPECT_EQ(stats.bytesPerChannel[cmaViable ? "cma" : "basic"], uint64_t(data.size()));
        me.recv();
        ctx->join();
      },
      [&](const ProcessPeers::Side& me) {
        auto ctx = make("client");
        auto pipe = ctx->connect(me.recv());
        auto copy = data;
        Message m;
        Message::Tensor t;
        t.buffer = CpuBuffer{copy.data()};
        t.length = copy.size();
        m.tensors.push_back(t);
        std::promise<Error> pw;
        pipe->write(m, [&](const Error& e) { pw.set_value(e); });
        auto fw = pw.get_future();
        EXPECT_FALSE(bool(waitFor(fw)));
        me.send("done");
        ctx->join();
      });
}

// The CUDA channel's options can be overridden from the environment (no GPU needed to check).
TPB_TEST(Channel, CudaP2pOptionsFollowTheEnvironment) {
  namespace p2p = tpb::channel::cuda_p2p;
  ::setenv("TPB_CUDA_P2P_EAGER_THRESHOLD", "4096", 1);
  ::setenv("TPB_CUDA_P2P_INBOX_BYTES", "0x100000", 1);
  ::setenv("TPB_CUDA_P2P_MAX_CTAS", "37", 1);
  ::setenv("TPB_CUDA_P2P_WAIT_KERNEL", "1", 1);
  ::setenv("TPB_CUDA_P2P_WAIT_TIMEOUT_MS", "250", 1);
  ::setenv("TPB_CUDA_P2P_BULK", "0", 1);
  ::setenv("TPB_CUDA_P2P_SEND_ORDER_MIN_BYTES", "1048576", 1);
  p2p::Options o = p2p::applyEnvironment(p2p::Options());
  EXPECT_EQ(o.sendOrderMinBytes, size_t(1) << 20);
  EXPECT_EQ(o.eagerThreshold, size_t(4096));
  EXPECT_EQ(o.inboxBytes, size_t(1) << 20);
  EXPECT_EQ(o.maxCtas, 37);
  EXPECT_TRUE(o.waitWithKernel);
  EXPECT_EQ(o.waitTimeoutNs, uint64_t(250) * 1000 * 1000);
  EXPECT_FALSE(o.useBulkCopy);
  ::setenv("TPB_CUDA_P2P_MAX_CTAS", "many", 1);  // not a number: ignored with a warning
  p2p::Options keep;
  keep.maxCtas = 5;
  EXPECT_EQ(p2p::applyEnvironment(keep).maxCtas, 5);
  for (const char* n : {"TPB_CUDA_P2P_EAGER_THRESHOLD", "TPB_CUDA_P2P_INBOX_BYTES", "TPB_CUDA_P2P_MAX_CTAS",
                        "TPB_CUDA_P2P_WAIT_KERNEL", "TPB_CUDA_P2P_WAIT_TIMEOUT_MS", "TPB_CUDA_P2P_BULK",
                        "TPB_CUDA_P2P_SEND_ORDER_MIN_BYTES"})
    ::unsetenv(n);
  p2p::Options d = p2p::applyEnvironment(p2p::Options());
  EXPECT_EQ(d.eagerThreshold, size_t(64 * 1024));
  EXPECT_EQ(d.sendOrderMinBytes, size_t(8) << 20);
}

// Every channel context can be dropped without join(): its destructor closes and joins on its
// own (reference case: mpt ContextIsNotJoined, tensorpipe/test/channel/mpt/mpt_test.cc:17-109;
// here for every CPU backend, with and without a channel having existed).
TPB_TEST(Channel, ContextsCanBeDroppedWithoutJoin) {
  for (const Backend& b : kBackends) {
    {
      auto ctx = b.make();
      (void)ctx->isViable();
    }  // never used, never joined
    {
      auto ctx = b.make();
      if (!ctx->isViable()) continue;
      auto descriptors = ctx->deviceDescriptors();
      EXPECT_FALSE(descriptors.empty());
      ctx->close();
    }  // closed but not joined
  }
}
