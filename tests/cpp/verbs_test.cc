// The pieces under the RDMA backends, tested without InfiniBand hardware: the N-party ring with
// transactions (tensorpipe/test/common/ringbuffer_test.cc is the reference's counterpart), the
// software fabric behind the verbs interface (queue-pair states, keys and bounds, receives that
// arrive late, failure and flush), and the ibv transport on top of it beyond what the generic
// transport suite covers (work requests capped by the NIC's message size, a pipe over it).
#include <random>

#include <tpb/tpb.h>

#include "channel/cuda_gdr/cuda_gdr.h"
#include "common/role_ring.h"
#include "common/verbs.h"
#include "test_util.h"
#include "transport/ibv/ibv.h"

using namespace tpb;
using namespace tpbtest;

TPB_TEST(RoleRing, ThreePartiesChaseEachOtherAroundTheRing) {
  RoleRingHeader<3> header;
  std::vector<uint8_t> data(64);
  RoleRing<3> ring(&header, data.data(), 64, true);
  EXPECT_TRUE(ring.valid());
  EXPECT_EQ(ring.ahead(0), uint64_t(64));
  EXPECT_EQ(ring.ahead(1), uint64_t(0));
  EXPECT_EQ(ring.ahead(2), uint64_t(0));

  uint8_t in[48];
  for (int i = 0; i < 48; ++i) in[i] = static_cast<uint8_t>(i + 1);
  {
    auto tx = ring.begin(0);
    EXPECT_TRUE(tx.open());
    EXPECT_TRUE(tx.write(in, 48));
    EXPECT_FALSE(tx.write(in, 17));  // all or nothing: 16 left
    // nothing is visible to the next party before the commit
    EXPECT_EQ(ring.ahead(1), uint64_t(0));
    tx.commit();
  }
  EXPECT_EQ(ring.ahead(1), uint64_t(48));
  EXPECT_EQ(ring.ahead(0), uint64_t(16));
  {
    // the middle party looks at the bytes in place and releases only some
    auto tx = ring.begin(1);
    RoleRing<3>::Span runs[2];
    EXPECT_EQ(tx.span(48, runs), 1);
    EXPECT_TRUE(std::memcmp(runs[0].ptr, in, 48) == 0);
    tx.advance(40);
    tx.commit();
  }
  EXPECT_EQ(ring.ahead(2), uint64_t(40));
  EXPECT_EQ(ring.ahead(0), uint64_t(16));  // the last party has freed nothing yet
  {
    auto tx = ring.begin(2);
    tx.advance(40);
    tx.commit();
  }
  EXPECT_EQ(ring.ahead(0), uint64_t(56));
  {
    // 48 more bytes wrap around the end of the data area: two runs
    auto tx = ring.begin(0);
    RoleRing<3>::Span runs[2];
    EXPECT_EQ(tx.span(48, runs), 2);
    EXPECT_EQ(runs[0].length, uint64_t(16));
    EXPECT_EQ(runs[1].length, uint64_t(32));
    EXPECT_TRUE(tx.write(in, 48));
    tx.commit();
  }
  {
    auto tx = ring.begin(1);
    EXPECT_EQ(tx.available(), uint64_t(56));
    uint8_t out[56];
    EXPECT_TRUE(tx.read(out, 56));
    EXPECT_TRUE(std::memcmp(out, in + 40, 8) == 0);
    EXPECT_TRUE(std::memcmp(out + 8, in, 48) == 0);
    tx.commit();
  }
  EXPECT_EQ(ring.released(0), uint64_t(96));
  EXPECT_EQ(ring.released(1), uint64_t(96));
  EXPECT_EQ(ring.released(2), uint64_t(40));
}

TPB_TEST(RoleRing, OneTransactionPerPartyAndCancelForgets) {
  RoleRingHeader<2> header;
  std::vector<uint8_t> data(32);
  RoleRing<2> ring(&header, data.data(), 32, true);
  auto first = ring.begin(0);
  EXPECT_TRUE(first.open());
  auto second = ring.begin(0);
  EXPECT_FALSE(second.open());  // the same party twice: refused, not corrupted
  auto other = ring.begin(1);
  EXPECT_TRUE(other.open());    // another party is independent
  other.cancel();
  uint8_t bytes[8] = {1, 2, 3, 4, 5, 6, 7, 8};
  EXPECT_TRUE(first.write(bytes, 8));
  first.cancel();
  EXPECT_EQ(ring.ahead(1), uint64_t(0));  // cancelled: nothing was published
  auto again = ring.begin(0);
  EXPECT_TRUE(again.open());
  EXPECT_EQ(again.available(), uint64_t(32));
  EXPECT_TRUE(again.write(bytes, 8));
  again.commit();
  EXPECT_EQ(ring.ahead(1), uint64_t(8));
  // a transaction that goes out of scope without a commit counts as cancelled
  {
    auto dropped = ring.begin(1);
    dropped.advance(8);
  }
  EXPECT_EQ(ring.ahead(1), uint64_t(8));
  bool threw = false;
  try {
    RoleRingHeader<2> h2;
    RoleRing<2> bad(&h2, data.data(), 24, true);
  } catch (const std::exception&) {
    threw = true;
  }
  EXPECT_TRUE(threw);  // sizes that are not a power of two are refused
}

TPB_TEST(RoleRing, ProducerAndConsumerThreadsMoveAStream) {
  RoleRingHeader<2> header;
  std::vector<uint8_t> data(256);
  RoleRing<2> ring(&header, data.data(), 256, true);
  constexpr size_t kTotal = 1 << 18;
  std::thread producer([&] {
    std::mt19937 rng(3);
    size_t sent = 0;
    while (sent < kTotal) {
      auto tx = ring.begin(0);
      const uint64_t n = std::min<uint64_t>({tx.available(), kTotal - sent, 1 + rng() % 97});
      uint8_t buf[97];
      for (uint64_t i = 0; i < n; ++i) buf[i] = static_cast<uint8_t>((sent + i) * 7);
      tx.write(buf, n);
      tx.commit();
      sent += n;
    }
  });
  size_t got = 0, bad = 0;
  while (got < kTotal) {
    auto tx = ring.begin(1);
    const uint64_t n = tx.available();
    uint8_t buf[256];
    tx.read(buf, n);
    tx.commit();
    for (uint64_t i = 0; i < n; ++i) bad += buf[i] != static_cast<uint8_t>((got + i) * 7);
    got += n;
  }
  producer.join();
  EXPECT_EQ(bad, size_t(0));
}

namespace {
struct Endpoint {
  std::unique_ptr<verbs::Device> device;
  std::unique_ptr<verbs::CompletionQueue> cq;
  std::unique_ptr<verbs::SharedReceiveQueue> srq;
  std::unique_ptr<verbs::QueuePair> qp;
  std::vector<uint8_t> memory;
  std::unique_ptr<verbs::MemoryRegion> region;
  explicit Endpoint(verbs::Provider& p, size_t bytes = 4096) : memory(bytes) {
    device = p.open(p.deviceNames().front());
    cq = device->createCompletionQueue(64);
    srq = device->createSharedReceiveQueue(64);
    qp = device->createQueuePair(*cq, *srq, 64);
    region = device->registerMemory(memory.data(), memory.size());
  }
  verbs::Address address() const {
    verbs::Address a = device->portAddress();
    a.queuePair = qp->number();
    return a;
  }
  std::vector<verbs::Completion> drain() {
    std::vector<verbs::Completion> all;
    verbs::Completion batch[8];
    for (int n; (n = cq->poll(batch, 8)) > 0;) all.insert(all.end(), batch, batch + n);
    return all;
  }
};
void connect(Endpoint& a, Endpoint& b) {
  a.qp->toInit();
  b.qp->toInit();
  a.qp->toReadyToReceive(b.address());
  b.qp->toReadyToReceive(a.address());
  a.qp->toReadyToSend(0);
  b.qp->toReadyToSend(0);
}
}  // namespace

TPB_TEST(VerbsLoopback, WritesLandAndReceivesMayComeLate) {
  auto fabric = verbs::loopbackProvider();
  Endpoint a(*fabric), b(*fabric);
  connect(a, b);
  for (size_t i = 0; i < 100; ++i) a.memory[i] = static_cast<uint8_t>(i + 5);
  // No receive is posted at b yet: the write is placed, its notification waits (as the wire's
  // receiver-not-ready retries would make it).
  a.qp->postWriteWithImmediate(11, a.memory.data(), 100, a.region->localKey(),
                               reinterpret_cast<uint64_t>(b.memory.data()) + 50, b.region->remoteKey(), 100);
  auto done = a.drain();
  EXPECT_EQ(done.size(), size_t(1));
  EXPECT_TRUE(done[0].ok && done[0].work == verbs::Work::kWrite && done[0].id == 11);
  EXPECT_TRUE(b.drain().empty());
  EXPECT_TRUE(std::memcmp(b.memory.data() + 50, a.memory.data(), 100) == 0);
  // A send with a payload and a second write queue up behind it, in order.
  a.qp->postSendWithImmediate(12, a.memory.data(), 10, a.region->localKey(), 777);
  a.qp->postWriteWithImmediate(13, a.memory.data(), 4, a.region->localKey(), reinterpret_cast<uint64_t>(b.memory.data()),
                               b.region->remoteKey(), 4);
  b.srq->postReceive(1);
  verbs::ReceiveBuffer buf{b.memory.data() + 1000, 64, b.region->localKey()};
  b.srq->postReceive(2, buf);
  b.srq->postReceive(3);
  auto arrived = b.drain();
  EXPECT_EQ(arrived.size(), size_t(3));
  EXPECT_TRUE(arrived[0].work == verbs::Work::kWriteArrived && arrived[0].immediate == 100 && arrived[0].id == 1);
  EXPECT_TRUE(arrived[1].work == verbs::Work::kSendArrived && arrived[1].immediate == 777 && arrived[1].byteLength == 10);
  EXPECT_TRUE(std::memcmp(b.memory.data() + 1000, a.memory.data(), 10) == 0);
  EXPECT_TRUE(arrived[2].work == verbs::Work::kWriteArrived && arrived[2].immediate == 4 && arrived[2].id == 3);
  EXPECT_EQ(arrived[0].queuePair, b.qp->number());
}

TPB_TEST(VerbsLoopback, BadKeysAndBoundsFailTheRequestAndFlushTheQueuePair) {
  auto fabric = verbs::loopbackProvider();
  Endpoint a(*fabric), b(*fabric);
  connect(a, b);
  b.srq->postReceive(1);
  // past the end of the peer's region
  a.qp->postWriteWithImmediate(1, a.memory.data(), 200, a.region->localKey(),
                               reinterpret_cast<uint64_t>(b.memory.data()) + 4000, b.region->remoteKey(), 200);
  auto done = a.drain();
  EXPECT_EQ(done.size(), size_t(1));
  EXPECT_FALSE(done[0].ok);
  EXPECT_EQ(done[0].error, std::string("remote access error"));
  EXPECT_TRUE(b.drain().empty());  // nothing was placed, nothing announced
  // the queue pair is in the error state now: whatever is posted comes back flushed
  a.qp->postSendWithImmediate(2, nullptr, 0, 0, 5);
  done = a.drain();
  EXPECT_EQ(done.size(), size_t(1));
  EXPECT_FALSE(done[0].ok);
  EXPECT_EQ(done[0].id, uint64_t(2));

  Endpoint c(*fabric), d(*fabric);
  connect(c, d);
  // a key that was never issued, and a local buffer outside the registration
  c.qp->postWriteWithImmediate(3, c.memory.data(), 8, c.region->localKey(), reinterpret_cast<uint64_t>(d.memory.data()),
                               0xdead, 8);
  done = c.drain();
  EXPECT_FALSE(done[0].ok);
  Endpoint e(*fabric), f(*fabric);
  connect(e, f);
  std::vector<uint8_t> stray(16);
  e.qp->postWriteWithImmediate(4, stray.data(), 16, e.region->localKey(), reinterpret_cast<uint64_t>(f.memory.data()),
                               f.region->remoteKey(), 16);
  done = e.drain();
  EXPECT_EQ(done[0].error, std::string("local protection error"));
  // a peer whose queue pair is gone
  Endpoint g(*fabric);
  {
    Endpoint h(*fabric);
    connect(g, h);
  }
  g.qp->postSendWithImmediate(5, nullptr, 0, 0, 1);
  done = g.drain();
  EXPECT_EQ(done[0].error, std::string("transport retry counter exceeded"));
  // state machine misuse is a programming error
  Endpoint lone(*fabric);
  bool threw = false;
  try {
    lone.qp->toReadyToSend(0);
  } catch (const std::exception&) {
    threw = true;
  }
  EXPECT_TRUE(threw);
}

TPB_TEST(VerbsSystem, AMachineWithoutInfiniBandHasNoDevicesAndTheTransportSaysSo) {
  auto sys = verbs::systemProvider();
  auto names = sys->deviceNames();
  auto ctx = transport::ibv::create();
  EXPECT_EQ(ctx->isViable(), !names.empty());
  if (names.empty()) {
    EXPECT_FALSE(sys->whyUnavailable().empty());
    std::cout << "  no InfiniBand here: " << sys->whyUnavailable() << std::endl;
    bool threw = false;
    try {
      ctx->listen("127.0.0.1");
    } catch (const std::exception&) {
      threw = true;
    }
    EXPECT_TRUE(threw);
    // and a pipe context simply leaves the transport out
    auto pctx = std::make_shared<Context>();
    pctx->registerTransport(5, "ibv", ctx);
    pctx->registerTransport(0, "uv", transport::uv::create());
    pctx->registerChannel(0, "basic", channel::basic::create());
    auto l = pctx->listen({"uv://127.0.0.1"});
    EXPECT_FALSE(l->url("uv").empty());
    pctx->join();
  }
  ctx->join();
}

TPB_TEST(CudaGdr, GpusAreMatchedToTheNicBehindTheSameSwitch) {
  using channel::cuda_gdr::matchGpusToNics;
  // Two PCIe switches with a NIC and two GPUs each, as sysfs shows them.
  const std::vector<std::string> nics = {
      "/sys/devices/pci0000:15/0000:15:01.0/0000:16:00.0/0000:17:04.0/0000:1a:00.0",
      "/sys/devices/pci0000:97/0000:97:01.0/0000:98:00.0/0000:99:04.0/0000:9c:00.0",
  };
  const std::vector<std::string> gpus = {
      "/sys/devices/pci0000:15/0000:15:01.0/0000:16:00.0/0000:17:00.0/0000:18:00.0",
      "/sys/devices/pci0000:15/0000:15:01.0/0000:16:00.0/0000:17:08.0/0000:1b:00.0",
      "/sys/devices/pci0000:97/0000:97:01.0/0000:98:00.0/0000:99:00.0/0000:9a:00.0",
      "/sys/devices/pci0000:97/0000:97:01.0/0000:98:00.0/0000:99:08.0/0000:9d:00.0",
      "/sys/devices/pci0000:c0/0000:c0:01.0/0000:c1:00.0",  // shares no root with a NIC
      "",                                                     // unknown
  };
  auto m = matchGpusToNics(gpus, nics);
  EXPECT_EQ(m.size(), gpus.size());
  EXPECT_EQ(m[0], 0);
  EXPECT_EQ(m[1], 0);
  EXPECT_EQ(m[2], 1);
  EXPECT_EQ(m[3], 1);
  // the two without a relative are spread over the NICs
  EXPECT_EQ(m[4], 0);
  EXPECT_EQ(m[5], 1);
  // a deeper match wins over a shallower one
  const std::vector<std::string> nested = {"/sys/devices/pci0000:15/0000:15:01.0/0000:16:00.0",
                                           "/sys/devices/pci0000:15/0000:15:01.0/0000:16:00.0/0000:17:00.0/0000:19:00.0"};
  const auto deeper = matchGpusToNics({gpus[0]}, nested);
  EXPECT_EQ(deeper[0], 1);
  const auto none = matchGpusToNics(gpus, {});
  EXPECT_TRUE(none.size() == gpus.size() && none[0] == -1);
  // Without InfiniBand (or without a GPU) the channel says it is not viable instead of failing.
  auto ctx = channel::cuda_gdr::create();
  if (verbs::systemProvider()->deviceNames().empty()) EXPECT_FALSE(ctx->isViable());
  ctx->join();
}

namespace {
void expectOk(const Error& e, const char* what) {
  if (e) throw TestFailure(std::string(what) + ": " + e.what());
}
std::vector<uint8_t> noise(size_t n, uint32_t seed) {
  std::vector<uint8_t> v(n);
  std::mt19937 rng(seed);
  for (auto& b : v) b = static_cast<uint8_t>(rng());
  return v;
}
}  // namespace

TPB_TEST(TransportIbv, WorkRequestsRespectTheNicsMessageSizeAndCreditsFlow) {
  // A NIC that takes 4 KiB per work request: a 5 MiB frame (2.5 rings) needs 1280 writes, more
  // than the cap on writes in flight, and many credit messages coming back.
  auto fabric = verbs::loopbackProvider(1, nullptr, 4096);
  auto big = noise(5u << 20, 9);
  ThreadPeers peers;
  peers.run(
      [&](ThreadPeers& pg) {
        auto ctx = transport::ibv::createWithProvider(fabric);
        auto l = ctx->listen("127.0.0.1");
        pg.sendToClient(l->addr());
        std::promise<std::shared_ptr<transport::Connection>> pc;
        l->accept([&](const Error& e, std::shared_ptr<transport::Connection> c) { pc.set_value(e ? nullptr : c); });
        auto fc = pc.get_future();
        auto c = waitFor(fc);
        EXPECT_TRUE(c != nullptr);
        for (int round = 0; round < 2; ++round) {
          std::vector<uint8_t> into(big.size());
          std::promise<Error> pr;
          c->read(into.data(), into.size(), [&](const Error& e, const void*, size_t) { pr.set_value(e); });
          auto f = pr.get_future();
          expectOk(waitFor(f, 60), "read");
          EXPECT_TRUE(into == big);
        }
        pg.recvFromClient();
        ctx->join();
      },
      [&](ThreadPeers& pg) {
        auto ctx = transport::ibv::createWithProvider(fabric);
        auto c = ctx->connect(pg.recvFromServer());
        for (int round = 0; round < 2; ++round) {
          std::promise<Error> pr;
          c->write(big.data(), big.size(), [&](const Error& e) { pr.set_value(e); });
          auto f = pr.get_future();
          expectOk(waitFor(f, 60), "write");
        }
        pg.sendToServer("done");
        ctx->join();
      });
}

TPB_TEST(TransportIbv, APipeRunsOverIt) {
  auto fabric = verbs::loopbackProvider();
  auto make = [&](const char* name) {
    auto ctx = std::make_shared<Context>(ContextOptions().name(name));
    ctx->registerTransport(0, "uv", transport::uv::create());
    ctx->registerTransport(5, "ibv", transport::ibv::createWithProvider(fabric));
    ctx->registerChannel(0, "basic", channel::basic::create());
    return ctx;
  };
  auto payload = noise(70000, 1), tensor = noise(3u << 20, 2);
  ThreadPeers peers;
  peers.run(
      [&](ThreadPeers& pg) {
        auto ctx = make("server");
        auto listener = ctx->listen({"uv://127.0.0.1", "ibv://127.0.0.1"});
        pg.sendToClient(listener->url("uv"));
        std::promise<std::shared_ptr<Pipe>> pp;
        listener->accept([&](const Error& e, std::shared_ptr<Pipe> p) { pp.set_value(e ? nullptr : p); });
        auto fp = pp.get_future();
        auto pipe = waitFor(fp);
        EXPECT_TRUE(pipe != nullptr);
        for (int i = 0; i < 3; ++i) {
          std::promise<std::pair<Error, Descriptor>> pd;
          pipe->readDescriptor([&](const Error& e, Descriptor d) { pd.set_value({e, std::move(d)}); });
          auto fd = pd.get_future();
          auto [e, d] = waitFor(fd);
          EXPECT_FALSE(bool(e));
          std::vector<uint8_t> p(d.payloads[0].length), t(d.tensors[0].length);
          Allocation a;
          a.payloads.push_back({p.data()});
          Allocation::Tensor at;
          at.buffer = CpuBuffer{t.data()};
          a.tensors.push_back(at);
          std::promise<Error> pr;
          pipe->read(std::move(a), [&](const Error& e2) { pr.set_value(e2); });
          auto fr = pr.get_future();
          EXPECT_FALSE(bool(waitFor(fr)));
          EXPECT_TRUE(p == payload);
          EXPECT_TRUE(t == tensor);
        }
        EXPECT_EQ(pipe->transportName(), std::string("ibv"));
        pg.recvFromClient();
        ctx->join();
      },
      [&](ThreadPeers& pg) {
        auto ctx = make("client");
        auto pipe = ctx->connect(pg.recvFromServer());
        for (int i = 0; i < 3; ++i) {
          Message m;
          m.metadata = "over rdma";
          m.payloads.push_back({payload.data(), payload.size(), ""});
          Message::Tensor t;
          t.buffer = CpuBuffer{tensor.data()};
          t.length = tensor.size();
          m.tensors.push_back(t);
          std::promise<Error> pr;
          pipe->write(std::move(m), [&](const Error& e) { pr.set_value(e); });
          auto f = pr.get_future();
          EXPECT_FALSE(bool(waitFor(f)));
        }
        pg.sendToServer("done");
        ctx->join();
      });
}
