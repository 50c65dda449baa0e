// Failure handling, with every failure made on the host: a transport decorator that breaks
// connections on purpose, a peer process that is killed without saying goodbye, a context closed
// under load. What is checked is the contract "every callback is always called, in order, with an
// error" — the reference states it (README.md:78-91) and tests it only by closing objects
// (tensorpipe/test/core/listener_test.cc:21-41); no device is ever faulted here.
#include <signal.h>

#include <tpb/tpb.h>

#include <atomic>

#include "test_util.h"

using namespace tpb;
using namespace tpbtest;

namespace {
std::shared_ptr<Context> plain(const std::string& name) {
  auto ctx = std::make_shared<Context>(ContextOptions().name(name));
  ctx->registerTransport(0, "uv", transport::uv::create());
  ctx->registerChannel(0, "basic", channel::basic::create());
  return ctx;
}
std::shared_ptr<Pipe> acceptSync(Listener& l) {
  std::promise<std::pair<Error, std::shared_ptr<Pipe>>> p;
  l.accept([&](const Error& e, std::shared_ptr<Pipe> pipe) { p.set_value({e, std::move(pipe)}); });
  auto f = p.get_future();
  auto [e, pipe] = waitFor(f);
  if (e) throw TestFailure("accept failed: " + e.what());
  return pipe;
}
}  // namespace

TPB_TEST(Faults, ConnectionThatBreaksMidStreamFailsEveryPendingWriteInOrder) {
  // The client's transport fails every connection after a few frames: the handshake gets
  // through, later traffic does not.
  ThreadPeers peers;
  peers.run(
      [&](ThreadPeers& pg) {
        auto ctx = plain("server");
        auto l = ctx->listen({"uv://127.0.0.1"});
        pg.sendToClient(l->url("uv"));
        auto pipe = acceptSync(*l);
        // Keep reading until the breakage shows up on this side too.
        std::promise<Error> broke;
        std::function<void()> arm = [&]() {
          pipe->readDescriptor([&](const Error& e, Descriptor d) {
            if (e) return broke.set_value(e);
            Allocation a;
            std::vector<uint8_t>* sink = new std::vector<uint8_t>(d.tensors.empty() ? 0 : d.tensors[0].length);
            for (auto& t : d.tensors) {
              (void)t;
              Allocation::Tensor at;
              at.buffer = CpuBuffer{sink->data()};
              a.tensors.push_back(at);
            }
            pipe->read(a, [&, sink](const Error& e2) {
              delete sink;
              if (e2) return broke.set_value(e2);
              arm();
            });
          });
        };
        arm();
        auto f = broke.get_future();
        EXPECT_TRUE(bool(waitFor(f)));
        pg.recvFromClient();
        ctx->join();
      },
      [&](ThreadPeers& pg) {
        auto ctx = std::make_shared<Context>(ContextOptions().name("client"));
        transport::FaultPlan plan;
        plan.failAfterWrites = 6;  // per connection
        ctx->registerTransport(0, "uv", transport::wrapWithFaults(transport::uv::create(), plan));
        ctx->registerChannel(0, "basic", channel::basic::create());
        auto pipe = ctx->connect(pg.recvFromServer());
        constexpr int kN = 30;
        std::vector<uint8_t> data(1000, 7);
        std::mutex m;
        std::vector<std::pair<int, bool>> results;
        std::promise<void> all;
        for (int i = 0; i < kN; ++i) {
          Message msg;
          Message::Tensor t;
          t.buffer = CpuBuffer{data.data()};
          t.length = data.size();
          msg.tensors.push_back(t);
          pipe->write(msg, [&, i](const Error& e) {
            std::unique_lock<std::mutex> l(m);
            results.emplace_back(i, bool(e));
            if (static_cast<int>(results.size()) == kN) all.set_value();
          });
        }
        auto f = all.get_future();
        waitFor(f);
        // every callback fired, in order, and once errors start they never stop
        bool failing = false;
        int failures = 0;
        for (int i = 0; i < kN; ++i) {
          EXPECT_EQ(results[i].first, i);
          if (results[i].second) failing = true;
          else EXPECT_FALSE(failing);
          failures += results[i].second;
        }
        EXPECT_TRUE(failures > 0);
        // the error is sticky: a write issued now fails too
        std::promise<Error> late;
        pipe->write(Message(), [&](const Error& e) { late.set_value(e); });
        auto fl = late.get_future();
        EXPECT_TRUE(bool(waitFor(fl)));
        pg.sendToServer("done");
        ctx->join();
      });
}

TPB_TEST(Faults, KilledPeerProcessFailsPendingReadsAndWrites) {
  ProcessPeers::run(
      [](const ProcessPeers::Side& me) {
        auto ctx = std::make_shared<Context>(ContextOptions().name("survivor"));
        ctx->registerTransport(0, "uv", transport::uv::create());
        ctx->registerTransport(1, "shm", transport::shm::create());
        ctx->registerChannel(0, "basic", channel::basic::create());
        ctx->registerChannel(1, "cma", channel::cma::create());
        auto l = ctx->listen({"uv://127.0.0.1", "shm://"});
        me.send(l->url("uv"));
        auto pipe = acceptSync(*l);
        // one full exchange proves the pipe is up
        std::promise<Error> first;
        pipe->readDescriptor([&](const Error& e, Descriptor) {
          if (e) return first.set_value(e);
          pipe->read(Allocation(), [&](const Error& e2) { first.set_value(e2); });
        });
        auto ff = first.get_future();
        EXPECT_FALSE(bool(waitFor(ff)));
        // now arm a read that will never be satisfied and ask the peer to die
        std::promise<Error> pending;
        pipe->readDescriptor([&](const Error& e, Descriptor) { pending.set_value(e); });
        me.send("die");
        auto fp = pending.get_future();
        EXPECT_TRUE(bool(waitFor(fp)));
        std::promise<Error> after;
        pipe->write(Message(), [&](const Error& e) { after.set_value(e); });
        auto fa = after.get_future();
        EXPECT_TRUE(bool(waitFor(fa)));
        ctx->join();
      },
      [](const ProcessPeers::Side& me) {
        auto ctx = std::make_shared<Context>(ContextOptions().name("victim"));
        ctx->registerTransport(0, "uv", transport::uv::create());
        ctx->registerTransport(1, "shm", transport::shm::create());
        ctx->registerChannel(0, "basic", channel::basic::create());
        ctx->registerChannel(1, "cma", channel::cma::create());
        auto pipe = ctx->connect(me.recv());
        std::promise<Error> w;
        Message m;
        m.metadata = "hello";
        pipe->write(m, [&](const Error& e) { w.set_value(e); });
        auto fw = w.get_future();
        waitFor(fw);
        me.recv();
        ::kill(::getpid(), SIGKILL);
      },
      /*clientMayBeKilled=*/true);
}

TPB_TEST(Faults, ContextCloseUnderLoadCallsEverythingBack) {
  auto a = plain("a");
  auto b = plain("b");
  auto l = a->listen({"uv://127.0.0.1"});
  std::promise<std::shared_ptr<Pipe>> pp;
  l->accept([&](const Error&, std::shared_ptr<Pipe> p) { pp.set_value(p); });
  auto out = b->connect(l->url("uv"));
  auto fp = pp.get_future();
  auto in = waitFor(fp);
  constexpr int kN = 200;
  std::vector<uint8_t> data(1 << 16, 3);
  std::atomic<int> writeCallbacks{0}, readCallbacks{0};
  for (int i = 0; i < kN; ++i) {
    Message m;
    Message::Tensor t;
    t.buffer = CpuBuffer{data.data()};
    t.length = data.size();
    m.tensors.push_back(t);
    out->write(m, [&](const Error&) { ++writeCallbacks; });
    in->readDescriptor([&](const Error&, Descriptor) { ++readCallbacks; });  // never followed by read()
  }
  b->join();
  a->join();
  EXPECT_EQ(writeCallbacks.load(), kN);
  EXPECT_EQ(readCallbacks.load(), kN);
}

TPB_TEST(Faults, DroppedFramesDoNotCrashThePeer) {
  // A transport that silently swallows its first frames: the handshake never completes, and
  // closing must still call everything back.
  auto a = plain("a");
  auto b = std::make_shared<Context>(ContextOptions().name("b"));
  transport::FaultPlan plan;
  plan.dropWrites = 2;
  b->registerTransport(0, "uv", transport::wrapWithFaults(transport::uv::create(), plan));
  b->registerChannel(0, "basic", channel::basic::create());
  auto l = a->listen({"uv://127.0.0.1"});
  std::promise<Error> accepted;
  l->accept([&](const Error& e, std::shared_ptr<Pipe>) { accepted.set_value(e); });
  auto out = b->connect(l->url("uv"));
  std::promise<Error> w;
  out->write(Message(), [&](const Error& e) { w.set_value(e); });
  std::this_thread::sleep_for(std::chrono::milliseconds(50));
  b->join();
  auto fw = w.get_future();
  EXPECT_TRUE(bool(waitFor(fw)));
  a->join();
  auto fa = accepted.get_future();
  waitFor(fa);  // fired one way or the other
}

// A peer whose frames arrive scrambled (same lengths, noise for content) at every possible point
// of the conversation: during the handshake, in a descriptor, in a payload. The healthy side must
// end every operation with an error or with data, never crash or hang, and stay joinable.
TPB_TEST(Faults, ScrambledFramesAtAnyPointNeverCrashThePeer) {
  for (int from = 0; from < 10; ++from) {
    auto a = plain("a");
    auto b = std::make_shared<Context>(ContextOptions().name("b"));
    transport::FaultPlan plan;
    plan.corruptFromWrite = from;
    plan.corruptSeed = 1000 + from;
    b->registerTransport(0, "uv", transport::wrapWithFaults(transport::uv::create(), plan));
    b->registerChannel(0, "basic", channel::basic::create());
    auto l = a->listen({"uv://127.0.0.1"});
    std::atomic<int> called{0};
    std::shared_ptr<Pipe> server;
    std::vector<uint8_t> inPayload(64), inTensor(4096);
    l->accept([&](const Error& e, std::shared_ptr<Pipe> p) {
      ++called;
      if (e) return;
      server = p;
      // Try to receive whatever the scrambling peer manages to say.
      p->readDescriptor([&, p](const Error& e2, Descriptor d) {
        ++called;
        if (e2) return;
        if (d.payloads.size() != 1 || d.tensors.size() != 1 || d.payloads[0].length != inPayload.size() ||
            d.tensors[0].length != inTensor.size())
          return;  // a descriptor that decoded into something else: leave it unread, close will clean up
        Allocation al;
        al.payloads.push_back({inPayload.data()});
        Allocation::Tensor t;
        t.buffer = CpuBuffer{inTensor.data()};
        al.tensors.push_back(t);
        p->read(std::move(al), [&](const Error&) { ++called; });
      });
    });
    auto out = b->connect(l->url("uv"));
    std::vector<uint8_t> payload(64, 7), tensor(4096, 9);
    std::promise<Error> w;
    Message m;
    m.metadata = "meta";
    m.payloads.push_back({payload.data(), payload.size(), ""});
    Message::Tensor mt;
    mt.buffer = CpuBuffer{tensor.data()};
    mt.length = tensor.size();
    m.tensors.push_back(mt);
    out->write(std::move(m), [&](const Error& e) { w.set_value(e); });
    std::this_thread::sleep_for(std::chrono::milliseconds(60));
    b->join();
    auto fw = w.get_future();
    waitFor(fw);  // fired one way or the other
    a->join();
    EXPECT_TRUE(called.load() >= 1);
    server.reset();
  }
}

// A peer that speaks the wire format but answers the handshake with nonsense (here: a raw socket
// playing server and naming a transport nobody registered) fails the pipe with an error; it does
// not take the process down.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <sys/socket.h>
#include <unistd.h>

#include "common/nop.h"
#include "core/nop_types.h"

namespace {
bool readFully(int fd, void* p, size_t n) {
  auto* b = static_cast<uint8_t*>(p);
  while (n > 0) {
    ssize_t got = ::read(fd, b, n);
    if (got <= 0) return false;
    b += got;
    n -= static_cast<size_t>(got);
  }
  return true;
}
bool readFrame(int fd, std::vector<uint8_t>& out) {
  uint64_t len = 0;
  if (!readFully(fd, &len, sizeof(len)) || len > (1u << 20)) return false;
  out.resize(len);
  return len == 0 || readFully(fd, out.data(), len);
}
bool writeFrame(int fd, const std::vector<uint8_t>& bytes) {
  const uint64_t len = bytes.size();
  return ::write(fd, &len, sizeof(len)) == ssize_t(sizeof(len)) &&
      ::write(fd, bytes.data(), bytes.size()) == ssize_t(bytes.size());
}
}  // namespace

TPB_TEST(Faults, NonsenseHandshakeAnswerFailsThePipeNotTheProcess) {
  int listenFd = ::socket(AF_INET, SOCK_STREAM, 0);
  EXPECT_TRUE(listenFd >= 0);
  sockaddr_in sa{};
  sa.sin_family = AF_INET;
  sa.sin_port = 0;
  ::inet_pton(AF_INET, "127.0.0.1", &sa.sin_addr);
  EXPECT_EQ(::bind(listenFd, reinterpret_cast<sockaddr*>(&sa), sizeof(sa)), 0);
  EXPECT_EQ(::listen(listenFd, 4), 0);
  socklen_t len = sizeof(sa);
  EXPECT_EQ(::getsockname(listenFd, reinterpret_cast<sockaddr*>(&sa), &len), 0);
  const int port = ntohs(sa.sin_port);

  std::thread fakeServer([&]() {
    int fd = ::accept(listenFd, nullptr, nullptr);
    if (fd < 0) return;
    std::vector<uint8_t> hello, brochure;
    if (readFrame(fd, hello) && readFrame(fd, brochure)) {
      BrochureAnswer answer;
      answer.transport = "carrier-pigeon";  // nobody registered this
      answer.address = "127.0.0.1:1";
      answer.transportRegistrationIds[0] = 1;
      answer.transportRegistrationIds[1] = 2;
      writeFrame(fd, nop::encode(answer));
    }
    // Hold the connection until the client has reacted, then hang up.
    std::vector<uint8_t> rest;
    readFrame(fd, rest);
    ::close(fd);
  });

  auto ctx = plain("client");
  auto pipe = ctx->connect("uv://127.0.0.1:" + std::to_string(port));
  std::promise<Error> w;
  pipe->write(Message(), [&](const Error& e) { w.set_value(e); });
  auto fw = w.get_future();
  Error e = waitFor(fw);
  EXPECT_TRUE(bool(e));
  EXPECT_TRUE(e.what().find("inconsistent handshake") != std::string::npos);
  pipe->close();
  ctx->join();
  fakeServer.join();
  ::close(listenFd);
}
