// Integration tests of Context / Listener / Pipe over real backends on loopback. Test bodies
// mirror the cases of the reference's pipe and context suites (tensorpipe/test/core/
// pipe_test.cc:13-528, context_test.cc:303-729, listener_test.cc:21-41) re-expressed on this
// repo's harness: two peers as threads, a mailbox for the address, futures for callbacks.
#include <tpb/tpb.h>

#include <atomic>
#include <numeric>
#include <random>

#include "test_util.h"

using namespace tpb;
using namespace tpbtest;

namespace {

std::shared_ptr<Context> makeContext(const std::string& name, bool shm = false) {
  auto ctx = std::make_shared<Context>(ContextOptions().name(name));
  ctx->registerTransport(0, "uv", transport::uv::create());
  if (shm) ctx->registerTransport(1, "shm", transport::shm::create());
  ctx->registerChannel(0, "basic", channel::basic::create());
  return ctx;
}

std::vector<uint8_t> pattern(size_t n, uint32_t seed) {
  std::vector<uint8_t> v(n);
  std::mt19937 rng(seed);
  for (auto& b : v) b = static_cast<uint8_t>(rng());
  return v;
}

struct OwnedMessage {
  std::string metadata;
  std::vector<std::vector<uint8_t>> payloads;
  std::vector<std::string> payloadMeta;
  std::vector<std::vector<uint8_t>> tensors;
  std::vector<std::string> tensorMeta;
  Message view(bool withTarget) {
    Message m;
    m.metadata = metadata;
    for (size_t i = 0; i < payloads.size(); ++i)
      m.payloads.push_back({payloads[i].data(), payloads[i].size(), payloadMeta[i]});
    for (size_t i = 0; i < tensors.size(); ++i) {
      Message::Tensor t;
      t.buffer = CpuBuffer{tensors[i].data()};
      t.length = tensors[i].size();
      t.metadata = tensorMeta[i];
      if (withTarget) t.targetDevice = Device(kCpuDeviceType, 0);
      m.tensors.push_back(t);
    }
    return m;
  }
};

OwnedMessage makeMessage(uint32_t seed, std::vector<size_t> payloadSizes, std::vector<size_t> tensorSizes) {
  OwnedMessage m;
  m.metadata = "meta-" + std::to_string(seed);
  for (size_t i = 0; i < payloadSizes.size(); ++i) {
    m.payloads.push_back(pattern(payloadSizes[i], seed * 100 + i));
    m.payloadMeta.push_back("p" + std::to_string(i));
  }
  for (size_t i = 0; i < tensorSizes.size(); ++i) {
    m.tensors.push_back(pattern(tensorSizes[i], seed * 1000 + i));
    m.tensorMeta.push_back("t" + std::to_string(i));
  }
  return m;
}

// Blocking helpers over the asynchronous API.
void writeSync(Pipe& pipe, Message m) {
  std::promise<Error> p;
  pipe.write(std::move(m), [&](const Error& e) { p.set_value(e); });
  auto f = p.get_future();
  Error e = waitFor(f);
  if (e) throw TestFailure("write failed: " + e.what());
}

struct Received {
  Descriptor descriptor;
  std::vector<std::vector<uint8_t>> payloads, tensors;
};

Received readSync(Pipe& pipe) {
  std::promise<std::pair<Error, Descriptor>> pd;
  pipe.readDescriptor([&](const Error& e, Descriptor d) { pd.set_value({e, std::move(d)}); });
  auto fd = pd.get_future();
  auto [e, d] = waitFor(fd);
  if (e) throw TestFailure("readDescriptor failed: " + e.what());
  Received r;
  r.descriptor = d;
  Allocation a;
  for (auto& p : d.payloads) {
    r.payloads.emplace_back(p.length);
    a.payloads.push_back({r.payloads.back().data()});
  }
  for (auto& t : d.tensors) {
    r.tensors.emplace_back(t.length);
    Allocation::Tensor at;
    at.buffer = CpuBuffer{r.tensors.back().data()};
    a.tensors.push_back(at);
  }
  std::promise<Error> pr;
  pipe.read(std::move(a), [&](const Error& e2) { pr.set_value(e2); });
  auto fr = pr.get_future();
  Error e2 = waitFor(fr);
  if (e2) throw TestFailure("read failed: " + e2.what());
  return r;
}

void expectSame(const OwnedMessage& m, const Received& r) {
  EXPECT_EQ(r.descriptor.metadata, m.metadata);
  EXPECT_EQ(r.payloads.size(), m.payloads.size());
  EXPECT_EQ(r.tensors.size(), m.tensors.size());
  for (size_t i = 0; i < m.payloads.size(); ++i) {
    EXPECT_EQ(r.descriptor.payloads[i].metadata, m.payloadMeta[i]);
    EXPECT_TRUE(r.payloads[i] == m.payloads[i]);
  }
  for (size_t i = 0; i < m.tensors.size(); ++i) {
    EXPECT_EQ(r.descriptor.tensors[i].metadata, m.tensorMeta[i]);
    EXPECT_TRUE(r.tensors[i] == m.tensors[i]);
  }
}

std::shared_ptr<Pipe> acceptSync(Listener& l) {
  std::promise<std::pair<Error, std::shared_ptr<Pipe>>> p;
  l.accept([&](const Error& e, std::shared_ptr<Pipe> pipe) { p.set_value({e, std::move(pipe)}); });
  auto f = p.get_future();
  auto [e, pipe] = waitFor(f);
  if (e) throw TestFailure("accept failed: " + e.what());
  return pipe;
}

// Runs `server(pipe)` and `client(pipe)` on two connected contexts.
void runPair(std::function<void(Pipe&)> server, std::function<void(Pipe&)> client,
             const std::vector<std::string>& urls = {"uv://127.0.0.1"}, bool shm = false) {
  ThreadPeers peers;
  peers.run(
      [&](ThreadPeers& pg) {
        auto ctx = makeContext("server", shm);
        auto listener = ctx->listen(urls);
        pg.sendToClient(listener->url("uv"));
        auto pipe = acceptSync(*listener);
        server(*pipe);
        pg.recvFromClient();  // client is done
        pg.sendToClient("bye");
        ctx->join();
      },
      [&](ThreadPeers& pg) {
        auto ctx = makeContext("client", shm);
        auto pipe = ctx->connect(pg.recvFromServer(), PipeOptions().remoteName("server"));
        client(*pipe);
        pg.sendToServer("done");
        pg.recvFromServer();
        ctx->join();
      });
}

}  // namespace

TPB_TEST(Pipe, SimpleWriteRead) {
  auto msg = makeMessage(1, {64, 4096}, {1024, 65536});
  runPair([&](Pipe& p) { expectSame(msg, readSync(p)); },
          [&](Pipe& p) { writeSync(p, msg.view(false)); });
}

TPB_TEST(Pipe, SimpleWriteReadWithAllTargetDevices) {
  auto msg = makeMessage(2, {10}, {1000, 2000, 3000});
  runPair([&](Pipe& p) { expectSame(msg, readSync(p)); },
          [&](Pipe& p) { writeSync(p, msg.view(true)); });
}

TPB_TEST(Pipe, SimpleWriteReadWithSomeTargetDevices) {
  auto msg = makeMessage(3, {}, {100, 200, 300});
  runPair([&](Pipe& p) { expectSame(msg, readSync(p)); },
          [&](Pipe& p) {
            Message m = msg.view(false);
            m.tensors[1].targetDevice = Device(kCpuDeviceType, 0);
            writeSync(p, std::move(m));
          });
}

TPB_TEST(Pipe, PayloadsOnlyAndTensorsOnlyAndEmpty) {
  auto a = makeMessage(4, {1, 2, 3}, {});
  auto b = makeMessage(5, {}, {7, 0, 9});
  auto c = makeMessage(6, {}, {});
  runPair(
      [&](Pipe& p) {
        expectSame(a, readSync(p));
        expectSame(b, readSync(p));
        expectSame(c, readSync(p));
      },
      [&](Pipe& p) {
        writeSync(p, a.view(false));
        writeSync(p, b.view(true));
        writeSync(p, c.view(false));
      });
}

TPB_TEST(Pipe, MultipleWriteReadInOrder) {
  constexpr int kN = 50;
  std::vector<OwnedMessage> msgs;
  for (int i = 0; i < kN; ++i) msgs.push_back(makeMessage(100 + i, {size_t(8 + i)}, {size_t(1000 + 37 * i)}));
  runPair(
      [&](Pipe& p) {
        for (int i = 0; i < kN; ++i) expectSame(msgs[i], readSync(p));
      },
      [&](Pipe& p) {
        // Issue every write up front; callbacks must come back in order.
        std::vector<int> order;
        std::mutex m;
        std::promise<void> all;
        for (int i = 0; i < kN; ++i) {
          p.write(msgs[i].view(i % 2 == 0), [&, i](const Error& e) {
            std::unique_lock<std::mutex> l(m);
            if (e) order.push_back(-1);
            order.push_back(i);
            if (static_cast<int>(order.size()) == kN) all.set_value();
          });
        }
        auto f = all.get_future();
        waitFor(f);
        for (int i = 0; i < kN; ++i) EXPECT_EQ(order[i], i);
      });
}

TPB_TEST(Pipe, WriteFromBothThenRead) {
  auto a = makeMessage(7, {32}, {5000});
  auto b = makeMessage(8, {48}, {7000});
  runPair(
      [&](Pipe& p) {
        std::promise<Error> w;
        p.write(a.view(false), [&](const Error& e) { w.set_value(e); });
        expectSame(b, readSync(p));
        auto f = w.get_future();
        EXPECT_FALSE(bool(waitFor(f)));
      },
      [&](Pipe& p) {
        std::promise<Error> w;
        p.write(b.view(false), [&](const Error& e) { w.set_value(e); });
        expectSame(a, readSync(p));
        auto f = w.get_future();
        EXPECT_FALSE(bool(waitFor(f)));
      });
}

TPB_TEST(Pipe, LargeTensor) {
  auto msg = makeMessage(9, {1 << 16}, {16u << 20});
  runPair([&](Pipe& p) { expectSame(msg, readSync(p)); },
          [&](Pipe& p) { writeSync(p, msg.view(false)); });
}

TPB_TEST(Pipe, ReadWithoutDescriptorThrows) {
  runPair([&](Pipe& p) { EXPECT_THROWS(p.read(Allocation(), [](const Error&) {})); }, [&](Pipe&) {});
}

TPB_TEST(Pipe, RemoteNameIsKnown) {
  runPair([&](Pipe& p) { EXPECT_EQ(p.getRemoteName(), std::string("client")); },
          [&](Pipe& p) { EXPECT_EQ(p.getRemoteName(), std::string("server")); });
}

TPB_TEST(Pipe, CallbacksRunOneAtATime) {
  // No two callbacks of one context may run concurrently, whatever thread triggers them.
  std::atomic<int> inside{0}, maxInside{0}, count{0};
  constexpr int kN = 40;
  auto msg = makeMessage(10, {16}, {4096});
  runPair(
      [&](Pipe& p) {
        for (int i = 0; i < kN; ++i) readSync(p);
      },
      [&](Pipe& p) {
        std::promise<void> all;
        for (int i = 0; i < kN; ++i) {
          p.write(msg.view(false), [&](const Error&) {
            int now = ++inside;
            int prev = maxInside.load();
            while (now > prev && !maxInside.compare_exchange_weak(prev, now)) {}
            std::this_thread::sleep_for(std::chrono::microseconds(200));
            --inside;
            if (++count == kN) all.set_value();
          });
        }
        auto f = all.get_future();
        waitFor(f);
        EXPECT_EQ(maxInside.load(), 1);
      });
}

TPB_TEST(Pipe, ClosePipeFailsPendingOperations) {
  runPair(
      [&](Pipe& p) {
        std::promise<Error> pd;
        p.readDescriptor([&](const Error& e, Descriptor) { pd.set_value(e); });
        p.close();
        auto f = pd.get_future();
        Error e = waitFor(f);
        EXPECT_TRUE(e.isOfType<PipeClosedError>());
      },
      [&](Pipe& p) {
        // The peer closing shows up as an error on our pending read.
        std::promise<Error> pd;
        p.readDescriptor([&](const Error& e, Descriptor) { pd.set_value(e); });
        auto f = pd.get_future();
        Error e = waitFor(f);
        EXPECT_TRUE(bool(e));
      });
}

TPB_TEST(Context, JoinFailsEverythingPending) {
  auto ctx = makeContext("solo");
  auto listener = ctx->listen({"uv://127.0.0.1"});
  std::promise<Error> pa;
  listener->accept([&](const Error& e, std::shared_ptr<Pipe>) { pa.set_value(e); });
  auto pipe = ctx->connect(listener->url("uv"));
  std::promise<Error> pd;
  pipe->readDescriptor([&](const Error& e, Descriptor) { pd.set_value(e); });
  std::this_thread::sleep_for(std::chrono::milliseconds(50));
  ctx->join();
  // accept either produced a pipe or was failed; the read must have been failed.
  auto f = pd.get_future();
  Error e = waitFor(f);
  EXPECT_TRUE(bool(e));
}

TPB_TEST(Context, DuplicateRegistrationThrowsAndPriorityIsUnique) {
  Context ctx;
  ctx.registerTransport(0, "uv", transport::uv::create());
  EXPECT_THROWS(ctx.registerTransport(1, "uv", transport::uv::create()));
  EXPECT_THROWS(ctx.registerTransport(0, "uv2", transport::uv::create()));
  ctx.registerChannel(0, "basic", channel::basic::create());
  EXPECT_THROWS(ctx.registerChannel(0, "other", channel::basic::create()));
  ctx.join();
}

TPB_TEST(Listener, ClosingAbortsOperations) {
  auto ctx = makeContext("solo");
  auto listener = ctx->listen({"uv://127.0.0.1"});
  std::promise<Error> pa;
  listener->accept([&](const Error& e, std::shared_ptr<Pipe>) { pa.set_value(e); });
  listener->close();
  auto f = pa.get_future();
  Error e = waitFor(f);
  EXPECT_TRUE(e.isOfType<ListenerClosedError>());
  ctx->join();
}

TPB_TEST(Context, ServerPingPongTwice) {
  // Two pipes to the same listener, each doing a ping-pong, concurrently.
  ThreadPeers peers;
  auto ping = makeMessage(11, {8}, {256});
  peers.run(
      [&](ThreadPeers& pg) {
        auto ctx = makeContext("server");
        auto listener = ctx->listen({"uv://127.0.0.1"});
        pg.sendToClient(listener->url("uv"));
        auto p1 = acceptSync(*listener);
        auto p2 = acceptSync(*listener);
        for (auto* p : {p1.get(), p2.get()}) {
          expectSame(ping, readSync(*p));
          writeSync(*p, ping.view(false));
        }
        pg.recvFromClient();
        ctx->join();
      },
      [&](ThreadPeers& pg) {
        auto ctx = makeContext("client");
        std::string url = pg.recvFromServer();
        auto p1 = ctx->connect(url);
        auto p2 = ctx->connect(url);
        for (auto* p : {p1.get(), p2.get()}) {
          writeSync(*p, ping.view(false));
          expectSame(ping, readSync(*p));
        }
        pg.sendToServer("done");
        ctx->join();
      });
}

// The client dials the TCP address; the handshake then notices that both ends also have the
// higher-priority shm transport and moves every connection of the pipe over to it.
TPB_TEST(Pipe, UpgradesToShmTransport) {
  auto msg = makeMessage(21, {64, 70000}, {1024, 5u << 20});
  runPair([&](Pipe& p) {
            expectSame(msg, readSync(p));
            writeSync(p, msg.view(false));
          },
          [&](Pipe& p) {
            writeSync(p, msg.view(false));
            expectSame(msg, readSync(p));
          },
          {"uv://127.0.0.1", "shm://"}, true);
}

TPB_TEST(Pipe, ManyMessagesOverShm) {
  constexpr int kN = 200;
  auto msg = makeMessage(22, {256}, {4096});
  runPair([&](Pipe& p) { for (int i = 0; i < kN; ++i) { expectSame(msg, readSync(p)); writeSync(p, msg.view(true)); } },
          [&](Pipe& p) { for (int i = 0; i < kN; ++i) { writeSync(p, msg.view(true)); expectSame(msg, readSync(p)); } },
          {"uv://127.0.0.1", "shm://"}, true);
}

// Tracing: a traced ping records the pipe's write / read events, and the dump is a JSON array
// whose entries carry the sequence number of the message.
#include <tpb/trace.h>

#include <fstream>
#include <sstream>

TPB_TEST(Pipe, TraceRecordsWritesAndReadsAndDumpsJson) {
  char path[] = "/tmp/tpb_trace_test_XXXXXX";
  int fd = ::mkstemp(path);
  EXPECT_TRUE(fd >= 0);
  ::close(fd);
  const uint64_t before = traceEventCount();
  traceEnable(path);
  auto msg = makeMessage(77, {16}, {4096});
  runPair([&](Pipe& p) { expectSame(msg, readSync(p)); }, [&](Pipe& p) { writeSync(p, msg.view(false)); });
  traceDisable();
  EXPECT_TRUE(traceEventCount() >= before + 5);  // write, write.done, readDescriptor, read, read.done
  EXPECT_TRUE(traceDump());
  std::ifstream in(path);
  std::stringstream ss;
  ss << in.rdbuf();
  const std::string json = ss.str();
  ::unlink(path);
  EXPECT_TRUE(json.size() > 2 && json[0] == '[');
  for (const char* name : {"pipe.write", "pipe.write.done", "pipe.readDescriptor", "pipe.read", "pipe.read.done"})
    EXPECT_TRUE(json.find(std::string("\"name\":\"") + name + "\"") != std::string::npos);
  EXPECT_TRUE(json.find("\"ph\":\"i\"") != std::string::npos);
  // Events recorded while tracing is off are dropped.
  const uint64_t after = traceEventCount();
  runPair([&](Pipe& p) { expectSame(msg, readSync(p)); }, [&](Pipe& p) { writeSync(p, msg.view(false)); });
  EXPECT_EQ(traceEventCount(), after);
}

// Optional deadlines: a peer that never answers fails the operation with TimeoutError instead of
// hanging it; operations that finish in time are unaffected.
TPB_TEST(Pipe, DeadlinesFailASilentPeerAndSpareAPromptOne) {
  auto msg = makeMessage(91, {8}, {256});
  std::atomic<bool> timedOut{false}, laterAlsoFailed{false};
  runPair(
      [&](Pipe& p) {
        // Serve one message promptly, then go silent: never write again.
        expectSame(msg, readSync(p));
        writeSync(p, msg.view(false));
        std::this_thread::sleep_for(std::chrono::milliseconds(700));
      },
      [&](Pipe& p) {
        PipeTimeouts t;
        t.write = std::chrono::milliseconds(5000);
        t.read = std::chrono::milliseconds(5000);
        t.descriptor = std::chrono::milliseconds(300);
        p.setTimeouts(t);
        writeSync(p, msg.view(false));
        expectSame(msg, readSync(p));  // answered well inside every deadline
        std::promise<Error> first, second;
        p.readDescriptor([&](const Error& e, Descriptor) { first.set_value(e); });
        p.readDescriptor([&](const Error& e, Descriptor) { second.set_value(e); });
        auto f1 = first.get_future();
        auto f2 = second.get_future();
        Error e1 = waitFor(f1);
        Error e2 = waitFor(f2);
        timedOut = e1.isOfType<TimeoutError>();
        laterAlsoFailed = bool(e2);
      });
  EXPECT_TRUE(timedOut.load());
  EXPECT_TRUE(laterAlsoFailed.load());
}

// A tensor between devices that no registered channel connects (a CUDA buffer on contexts that
// only know CPU channels) fails the pipe on both ends with a logic error; nothing is thrown on
// the callback thread, where an exception would end the process.
TPB_TEST(Pipe, TensorWithoutASuitableChannelFailsThePipe) {
  static uint8_t fakeDeviceMemory[64];
  std::atomic<bool> writerFailed{false}, readerFailed{false};
  runPair(
      [&](Pipe& p) {
        std::promise<Error> done;
        p.readDescriptor([&](const Error& e, Descriptor d) {
          if (e) return done.set_value(e);
          Allocation a;
          Allocation::Tensor t;
          t.buffer = CpuBuffer{fakeDeviceMemory};
          a.tensors.push_back(t);
          p.read(std::move(a), [&](const Error& e2) { done.set_value(e2); });
        });
        auto f = done.get_future();
        readerFailed = bool(waitFor(f));
      },
      [&](Pipe& p) {
        Message m;
        Message::Tensor t;
        t.buffer = CudaBuffer{fakeDeviceMemory, nullptr, 0};  // never dereferenced: no CUDA channel exists here
        t.length = sizeof(fakeDeviceMemory);
        t.targetDevice = Device(kCpuDeviceType, 0);
        m.tensors.push_back(t);
        std::promise<Error> done;
        p.write(std::move(m), [&](const Error& e) { done.set_value(e); });
        auto f = done.get_future();
        Error e = waitFor(f);
        writerFailed = e.isOfType<LogicError>();
      });
  EXPECT_TRUE(writerFailed.load());
  EXPECT_TRUE(readerFailed.load());
}

// The client pings, the server answers, several times in a row on one pipe: once with the
// client waiting for each answer before the next ping, once with every step issued from inside
// the previous step's callback (nothing may run inline, or this recursion would nest).
// (Reference cases: Context.ClientPingSerial / ClientPingInline, tensorpipe/test/core/context_test.cc.)
TPB_TEST(Context, ClientPingSerialAndFromInsideCallbacks) {
  auto ping = makeMessage(21, {32}, {128, 4096});
  constexpr int kRounds = 5;
  runPair(
      [&](Pipe& p) {
        for (int i = 0; i < 2 * kRounds; ++i) {
          expectSame(ping, readSync(p));
          writeSync(p, ping.view(false));
        }
      },
      [&](Pipe& p) {
        for (int i = 0; i < kRounds; ++i) {
          writeSync(p, ping.view(false));
          expectSame(ping, readSync(p));
        }
        // Now the same conversation as a chain of callbacks.
        std::promise<Error> finished;
        std::atomic<int> depth{0}, maxDepth{0};
        std::vector<std::vector<uint8_t>> payloadIn(ping.payloads.size()), tensorIn(ping.tensors.size());
        std::function<void(int)> round = [&](int left) {
          if (left == 0) return finished.set_value(Error::kSuccess);
          p.write(ping.view(false), [&, left](const Error& e) {
            if (e) return finished.set_value(e);
            int d = ++depth;
            if (d > maxDepth) maxDepth = d;
            p.readDescriptor([&, left](const Error& e2, Descriptor desc) {
              if (e2) return finished.set_value(e2);
              Allocation a;
              for (size_t i = 0; i < desc.payloads.size(); ++i) {
                payloadIn[i].resize(desc.payloads[i].length);
                a.payloads.push_back({payloadIn[i].data()});
              }
              for (size_t i = 0; i < desc.tensors.size(); ++i) {
                tensorIn[i].resize(desc.tensors[i].length);
                Allocation::Tensor t;
                t.buffer = CpuBuffer{tensorIn[i].data()};
                a.tensors.push_back(t);
              }
              p.read(std::move(a), [&, left](const Error& e3) {
                if (e3) return finished.set_value(e3);
                round(left - 1);
              });
            });
            --depth;
          });
        };
        round(kRounds);
        auto f = finished.get_future();
        Error e = waitFor(f);
        EXPECT_FALSE(bool(e));
        EXPECT_EQ(maxDepth.load(), 1);  // callbacks never nested
        EXPECT_TRUE(tensorIn.back() == ping.tensors.back());
      });
}
