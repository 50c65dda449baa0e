// Channel-level GPU suite for the two CUDA channels, on raw connections without a pipe (the
// reference's generic CUDA channel cases: tensorpipe/test/channel/channel_test_cuda.cc:19-139,
// channel_test_cuda_multi_gpu.cc), plus the failure paths of cuda_p2p that only a test in control
// of the channel's connection can reach: a device-side wait that runs out, a peer that goes
// silent while it may still be writing into announced buffers, and more batches in flight than
// there are flag slots. No test here faults a GPU: failures are injected on the host.
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>

#include <tpb/tpb.h>

#include "channel/cuda_gdr/cuda_gdr.h"
#include "channel_wiring.h"
#include "common/cuda.h"
#include "kernels/push.h"
#include "test_util.h"

using namespace tpb;
using namespace tpbtest;

namespace {

#define CK(x) TPB_CUDA_CHECK(x)

using MakeContext = std::function<std::shared_ptr<channel::Context>()>;
using Body = std::function<void(channel::Channel&)>;

struct PeerSetup {
  MakeContext make;
  transport::FaultPlan faults;  // applied to this peer's connections when any field is set
  bool faulty = false;
};

// Runs the two bodies over one channel, as two threads of this process or as two processes.
void runPair(bool processes, PeerSetup serverSetup, PeerSetup clientSetup, Body server, Body client) {
  auto serverSide = [=](std::function<void(std::string)> tell, std::function<std::string()> hear) {
    auto cctx = serverSetup.make();
    if (!cctx->isViable()) throw TestFailure("the CUDA channel is not viable on a machine with a GPU");
    Wiring w;
    if (serverSetup.faulty) w.tctx = transport::wrapWithFaults(transport::uv::create(), serverSetup.faults);
    tell(w.listen());
    auto ch = cctx->createChannel(w.acceptAll(cctx->numConnectionsNeeded()), channel::Endpoint::kListen);
    server(*ch);
    hear();
    ch->close();
    ch.reset();
    cctx->join();
    w.tctx->join();
  };
  auto clientSide = [=](std::function<void(std::string)> tell, std::function<std::string()> hear) {
    std::string addr = hear();
    auto cctx = clientSetup.make();
    Wiring w;
    if (clientSetup.faulty) w.tctx = transport::wrapWithFaults(transport::uv::create(), clientSetup.faults);
    auto ch = cctx->createChannel(w.connectAll(addr, cctx->numConnectionsNeeded()), channel::Endpoint::kConnect);
    client(*ch);
    tell("done");
    ch->close();
    ch.reset();
    cctx->join();
    w.tctx->join();
  };
  if (processes) {
    ProcessPeers::run([&](const ProcessPeers::Side& me) { serverSide([&](std::string s) { me.send(s); }, [&] { return me.recv(); }); },
                      [&](const ProcessPeers::Side& me) { clientSide([&](std::string s) { me.send(s); }, [&] { return me.recv(); }); });
  } else {
    ThreadPeers peers;
    peers.run([&](ThreadPeers& pg) { serverSide([&](std::string s) { pg.sendToClient(s); }, [&] { return pg.recvFromClient(); }); },
              [&](ThreadPeers& pg) { clientSide([&](std::string s) { pg.sendToServer(s); }, [&] { return pg.recvFromServer(); }); });
  }
}

PeerSetup p2p(channel::cuda_p2p::Options o = {}) {
  return {[o] { return channel::cuda_p2p::create(o); }, {}, false};
}
// cuda_gdr over the software fabric: two "NICs" whose wire is cudaMemcpy between device pointers
// and which take at most 1 MiB per work request, so that tensors travel in several pieces. The
// fabric lives in this process: its two ends must too.
PeerSetup gdr() {
  static auto fabric = verbs::loopbackProvider(
      2,
      [](void* dst, const void* src, size_t n) {
        // A NIC reports a write done when the bytes are placed: cudaMemcpy between device pointers
        // may return earlier, so wait for the copy.
        cudaMemcpyAsync(dst, src, n, cudaMemcpyDefault, cudaStreamPerThread);
        cudaStreamSynchronize(cudaStreamPerThread);
      },
      1u << 20);
  channel::cuda_gdr::Options o;
  o.requirePeerMemoryModule = false;
  o.maxPostedBytes = 2u << 20;
  return {[o] { return channel::cuda_gdr::createWithProvider(fabric, o); }, {}, false};
}
PeerSetup cudaBasic() {
  return {[] { return channel::cuda_basic::create(channel::basic::create()); }, {}, false};
}

struct DeviceTensor {
  int device;
  size_t bytes;
  uint8_t* p = nullptr;
  cudaStream_t stream = nullptr;
  DeviceTensor(int device, size_t bytes) : device(device), bytes(bytes) {
    CK(cudaSetDevice(device));
    CK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    CK(cudaMalloc(&p, bytes + 512));
    CK(cudaMemset(p, 0xCD, bytes + 512));
    // The fill runs on the default stream, which the tensor's own (non-blocking) stream is not
    // ordered with, and a peer may start writing the moment it learns the address.
    CK(cudaDeviceSynchronize());
  }
  ~DeviceTensor() {
    cudaSetDevice(device);
    cudaStreamSynchronize(stream);
    cudaFree(p);
    cudaStreamDestroy(stream);
  }
  uint8_t* data() const { return p + 256; }  // off the allocation's base, like a caching allocator's blocks
  CudaBuffer buffer() const { return CudaBuffer{data(), stream, device}; }
  void fill(uint64_t seed) {
    CK(cudaSetDevice(device));
    kernels::launchFill(stream, data(), bytes, seed);
  }
  uint64_t mismatches(uint64_t seed) {
    CK(cudaSetDevice(device));
    unsigned long long* bad;
    CK(cudaMalloc(&bad, 8));
    CK(cudaMemsetAsync(bad, 0, 8, stream));
    kernels::launchVerify(stream, data(), bytes, seed, bad);
    CK(cudaStreamSynchronize(stream));
    unsigned long long h = 1;
    CK(cudaMemcpy(&h, bad, 8, cudaMemcpyDeviceToHost));
    uint8_t guard[2];
    CK(cudaMemcpy(&guard[0], data() - 1, 1, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(&guard[1], data() + bytes, 1, cudaMemcpyDeviceToHost));
    cudaFree(bad);
    return h + (guard[0] != 0xCD) + (guard[1] != 0xCD);
  }
};

Error sendOne(channel::Channel& ch, const DeviceTensor& t, int targetDevice, int seconds = 30) {
  std::promise<Error> pr;
  channel::SendItem it;
  it.buffer = t.buffer();
  it.length = t.bytes;
  it.targetDevice = Device(kCudaDeviceType, targetDevice);
  it.callback = [&](const Error& e) { pr.set_value(e); };
  std::vector<channel::SendItem> v;
  v.push_back(std::move(it));
  ch.sendBatch(std::move(v));
  auto f = pr.get_future();
  return waitFor(f, seconds);
}

Error recvOne(channel::Channel& ch, const DeviceTensor& t, int sourceDevice, int seconds = 30) {
  std::promise<Error> pr;
  channel::RecvItem it;
  it.buffer = t.buffer();
  it.length = t.bytes;
  it.sourceDevice = Device(kCudaDeviceType, sourceDevice);
  it.callback = [&](const Error& e) { pr.set_value(e); };
  std::vector<channel::RecvItem> v;
  v.push_back(std::move(it));
  ch.recvBatch(std::move(v));
  auto f = pr.get_future();
  return waitFor(f, seconds);
}

void expectOk(const Error& e, const char* what) {
  if (e) throw TestFailure(std::string(what) + ": " + e.what());
}

// The reference's ClientToServer / ServerToClient / SendMultipleTensors / EmptyTensor cases, with
// both the per-tensor calls (send / recv) and the batch calls.
void basicCases(bool processes, PeerSetup setup, int serverDevice, int clientDevice) {
  const std::vector<size_t> sizes = {4096, 1u << 20, (4u << 20) + 12, 100, (24u << 20) + 4};
  runPair(
      processes, setup, setup,
      [=](channel::Channel& ch) {
        for (size_t i = 0; i < sizes.size(); ++i) {
          DeviceTensor t(serverDevice, sizes[i]);
          // first two through the per-tensor API, the rest through the batch API
          if (i < 2) {
            std::promise<Error> pr;
            ch.recv(t.buffer(), t.bytes, [&](const Error& e) { pr.set_value(e); });
            auto f = pr.get_future();
            expectOk(waitFor(f), "recv");
          } else {
            expectOk(recvOne(ch, t, clientDevice), "recvBatch");
          }
          EXPECT_EQ(t.mismatches(500 + i), uint64_t(0));
        }
        // and back, including an empty tensor (nothing may touch the wire for it)
        DeviceTensor back(serverDevice, 3u << 20);
        back.fill(900);
        expectOk(sendOne(ch, back, clientDevice), "sendBatch");
        std::promise<Error> pe;
        ch.send(CudaBuffer{nullptr, back.stream, serverDevice}, 0, [&](const Error& e) { pe.set_value(e); });
        auto fe = pe.get_future();
        expectOk(waitFor(fe), "empty send");
        CK(cudaStreamSynchronize(back.stream));
      },
      [=](channel::Channel& ch) {
        std::vector<std::unique_ptr<DeviceTensor>> sent;
        for (size_t i = 0; i < sizes.size(); ++i) {
          sent.push_back(std::make_unique<DeviceTensor>(clientDevice, sizes[i]));
          DeviceTensor& t = *sent.back();
          t.fill(500 + i);
          if (i < 2) {
            std::promise<Error> pr;
            ch.send(t.buffer(), t.bytes, [&](const Error& e) { pr.set_value(e); });
            auto f = pr.get_future();
            expectOk(waitFor(f), "send");
          } else {
            expectOk(sendOne(ch, t, serverDevice), "sendBatch");
          }
        }
        DeviceTensor back(clientDevice, 3u << 20);
        expectOk(recvOne(ch, back, serverDevice), "recvBatch");
        EXPECT_EQ(back.mismatches(900), uint64_t(0));
        std::promise<Error> pe;
        ch.recv(CudaBuffer{nullptr, back.stream, clientDevice}, 0, [&](const Error& e) { pe.set_value(e); });
        auto fe = pe.get_future();
        expectOk(waitFor(fe), "empty recv");
        for (auto& t : sent) CK(cudaStreamSynchronize(t->stream));
      });
}

}  // namespace

TPB_GPU_TEST(CudaChannel, P2pSameProcess, 1) { basicCases(false, p2p(), 0, 0); }
TPB_GPU_TEST(CudaChannel, P2pTwoProcesses, 1) { basicCases(true, p2p(), 0, 0); }
TPB_GPU_TEST(CudaChannel, P2pAcrossDevices, 2) { basicCases(true, p2p(), 0, 1); }
TPB_GPU_TEST(CudaChannel, P2pReverseAcrossDevices, 2) { basicCases(true, p2p(), 1, 0); }
TPB_GPU_TEST(CudaChannel, P2pSameProcessAcrossDevices, 2) { basicCases(false, p2p(), 0, 1); }
// Batches that take their place in the sender's stream at send() time and leave from the channel's
// own stream (Options::sendOrderMinBytes): from 1 MiB on, and never (every push on the sender's
// stream). The default, 8 MiB, is what the cases above ran with.
static PeerSetup p2pSendOrder(size_t minBytes) {
  channel::cuda_p2p::Options o;
  o.sendOrderMinBytes = minBytes;
  return p2p(o);
}
TPB_GPU_TEST(CudaChannel, P2pSendOrderSameProcess, 1) { basicCases(false, p2pSendOrder(1u << 20), 0, 0); }
TPB_GPU_TEST(CudaChannel, P2pSendOrderTwoProcesses, 1) { basicCases(true, p2pSendOrder(1u << 20), 0, 0); }
TPB_GPU_TEST(CudaChannel, P2pSendOrderAcrossDevices, 2) { basicCases(true, p2pSendOrder(1u << 20), 0, 1); }
TPB_GPU_TEST(CudaChannel, P2pLaunchOrderTwoProcesses, 1) { basicCases(true, p2pSendOrder(0), 0, 0); }
TPB_GPU_TEST(CudaChannel, P2pLaunchOrderAcrossDevices, 2) { basicCases(true, p2pSendOrder(0), 0, 1); }
// A large batch keeps the place in the sender's stream that it had when sendBatch() was called:
// 600 ms of other work queued on that stream right after the call, and long before the receiver
// names its buffers, does not stand between the receiver and its data.
static void laterWorkDoesNotDelayALargeSend(bool processes, int serverDevice, int clientDevice) {
  constexpr size_t kBytes = 16u << 20;
  constexpr uint32_t kBusyUs = 600000;
  runPair(
      processes, p2p(), p2p(),
      [=](channel::Channel& ch) {
        DeviceTensor t(serverDevice, kBytes);
        // Once without anything in the way: kernels are loaded, streams made and mappings opened
        // on first use, and some of that waits for the device to fall idle.
        expectOk(recvOne(ch, t, clientDevice), "first recv");
        CK(cudaStreamSynchronize(t.stream));
        EXPECT_EQ(t.mismatches(5149), uint64_t(0));
        std::this_thread::sleep_for(std::chrono::milliseconds(60));  // the sender has queued its busy kernel by now
        const auto t0 = std::chrono::steady_clock::now();
        expectOk(recvOne(ch, t, clientDevice), "recv");
        CK(cudaStreamSynchronize(t.stream));
        const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        EXPECT_EQ(t.mismatches(5150), uint64_t(0));
        if (ms > kBusyUs / 1000.0 / 2) throw TestFailure("the data took " + std::to_string(ms) + " ms: it waited for work queued after the send");
      },
      [=](channel::Channel& ch) {
        DeviceTensor t(clientDevice, kBytes);
        DeviceTensor scratch(clientDevice, 4096);
        CK(cudaSetDevice(clientDevice));
        kernels::launchDelay(t.stream, scratch.data(), scratch.bytes, 10);
        t.fill(5149);
        expectOk(sendOne(ch, t, serverDevice), "first send");
        CK(cudaStreamSynchronize(t.stream));
        t.fill(5150);
        std::promise<Error> sent;
        channel::SendItem it;
        it.buffer = t.buffer();
        it.length = t.bytes;
        it.targetDevice = Device(kCudaDeviceType, serverDevice);
        it.callback = [&](const Error& e) { sent.set_value(e); };
        std::vector<channel::SendItem> v;
        v.push_back(std::move(it));
        ch.sendBatch(std::move(v));
        CK(cudaSetDevice(clientDevice));
        kernels::launchDelay(t.stream, scratch.data(), scratch.bytes, kBusyUs);
        auto f = sent.get_future();
        expectOk(waitFor(f, 30), "send");
        CK(cudaStreamSynchronize(t.stream));
      });
}
// (Within one process and one GPU a batch is launched on the sender's stream whatever its size.)
TPB_GPU_TEST(CudaChannel, P2pLaterWorkDoesNotDelayALargeSendTwoProcesses, 1) { laterWorkDoesNotDelayALargeSend(true, 0, 0); }
TPB_GPU_TEST(CudaChannel, P2pLaterWorkDoesNotDelayALargeSendAcrossDevices, 2) { laterWorkDoesNotDelayALargeSend(true, 0, 1); }

TPB_GPU_TEST(CudaChannel, GdrOverASoftwareFabric, 1) { basicCases(false, gdr(), 0, 0); }
TPB_GPU_TEST(CudaChannel, GdrOverASoftwareFabricAcrossDevices, 2) { basicCases(false, gdr(), 0, 1); }
TPB_GPU_TEST(CudaChannel, BasicSameProcess, 1) { basicCases(false, cudaBasic(), 0, 0); }
TPB_GPU_TEST(CudaChannel, BasicTwoProcesses, 1) { basicCases(true, cudaBasic(), 0, 0); }
TPB_GPU_TEST(CudaChannel, BasicAcrossDevices, 2) { basicCases(true, cudaBasic(), 0, 1); }

// Many more small batches in flight than there are flag slots (256) or than the inbox could hold
// without credits coming back: the sender must pace itself and every batch must arrive intact.
static void manyInFlight(int serverDevice, int clientDevice) {
  constexpr int kBatches = 700;
  constexpr size_t kBytes = 48 * 1024;
  channel::cuda_p2p::Options o;
  o.inboxBytes = 4u << 20;  // 85 batches' worth: credits must flow
  runPair(
      true, p2p(o), p2p(o),
      [=](channel::Channel& ch) {
        // the first batch is a rendezvous that announces the arena; the rest arrive eagerly
        DeviceTensor first(serverDevice, kBytes);
        expectOk(recvOne(ch, first, clientDevice), "first recv");
        EXPECT_EQ(first.mismatches(7000), uint64_t(0));
        CK(cudaSetDevice(serverDevice));
        DeviceTensor all(serverDevice, kBytes * kBatches);
        std::atomic<int> done{0}, failed{0};
        std::promise<void> finished;
        for (int i = 0; i < kBatches; ++i) {
          channel::RecvItem it;
          it.buffer = CudaBuffer{all.data() + static_cast<size_t>(i) * kBytes, all.stream, serverDevice};
          it.length = kBytes;
          it.sourceDevice = Device(kCudaDeviceType, clientDevice);
          it.callback = [&](const Error& e) {
            if (e) ++failed;
            if (++done == kBatches) finished.set_value();
          };
          std::vector<channel::RecvItem> v;
          v.push_back(std::move(it));
          ch.recvBatch(std::move(v));
        }
        auto f = finished.get_future();
        waitFor(f, 60);
        EXPECT_EQ(failed.load(), 0);
        // every batch was filled with the same seeded pattern
        CK(cudaStreamSynchronize(all.stream));
        unsigned long long* bad;
        CK(cudaMalloc(&bad, 8));
        CK(cudaMemset(bad, 0, 8));
        for (int i = 0; i < kBatches; ++i)
          kernels::launchVerify(all.stream, all.data() + static_cast<size_t>(i) * kBytes, kBytes, 7001, bad);
        CK(cudaStreamSynchronize(all.stream));
        unsigned long long h = 1;
        CK(cudaMemcpy(&h, bad, 8, cudaMemcpyDeviceToHost));
        cudaFree(bad);
        EXPECT_EQ(h, 0ull);
      },
      [=](channel::Channel& ch) {
        DeviceTensor first(clientDevice, kBytes);
        first.fill(7000);
        expectOk(sendOne(ch, first, serverDevice), "first send");
        DeviceTensor src(clientDevice, kBytes);
        src.fill(7001);
        std::atomic<int> done{0}, failed{0};
        std::promise<void> finished;
        for (int i = 0; i < kBatches; ++i) {
          channel::SendItem it;
          it.buffer = src.buffer();
          it.length = kBytes;
          it.targetDevice = Device(kCudaDeviceType, serverDevice);
          it.callback = [&](const Error& e) {
            if (e) ++failed;
            if (++done == kBatches) finished.set_value();
          };
          std::vector<channel::SendItem> v;
          v.push_back(std::move(it));
          ch.sendBatch(std::move(v));
        }
        auto f = finished.get_future();
        waitFor(f, 60);
        EXPECT_EQ(failed.load(), 0);
        CK(cudaStreamSynchronize(src.stream));
      });
}
TPB_GPU_TEST(CudaChannel, P2pManyBatchesInFlightOneDevice, 1) { manyInFlight(0, 0); }
TPB_GPU_TEST(CudaChannel, P2pManyBatchesInFlightTwoDevices, 2) { manyInFlight(0, 1); }

// A large tensor in pinned host memory, handed over as a tensor of the sending GPU, comes in
// through the copy engine (straight into a receiver on the same GPU, in pieces forwarded by the
// kernel to another GPU) except for a short tail, which travels with the kernel launch that also
// carries the device tensor of the same batch. A ragged size, twice in a row, with pieces small
// enough that both slots are reused.
static void hostFed(bool processes, int serverDevice, int clientDevice) {
  constexpr size_t kHostBytes = (21u << 20) + 40;
  constexpr size_t kDeviceBytes = (1u << 20) + 8;
  channel::cuda_p2p::Options o;
  o.hostPieceBytes = 4u << 20;
  runPair(
      processes, p2p(o), p2p(o),
      [=](channel::Channel& ch) {
        for (int round = 0; round < 2; ++round) {
          DeviceTensor big(serverDevice, kHostBytes), small(serverDevice, kDeviceBytes);
          std::promise<Error> pr;
          std::atomic<int> left{2}, failed{0};
          std::vector<channel::RecvItem> v;
          for (DeviceTensor* t : {&big, &small}) {
            channel::RecvItem it;
            it.buffer = CudaBuffer{t->data(), big.stream, serverDevice};
            it.length = t->bytes;
            it.sourceDevice = Device(kCudaDeviceType, clientDevice);
            it.callback = [&](const Error& e) {
              if (e) ++failed;
              if (--left == 0) pr.set_value(e);
            };
            v.push_back(std::move(it));
          }
          ch.recvBatch(std::move(v));
          auto f = pr.get_future();
          expectOk(waitFor(f), "recvBatch");
          EXPECT_EQ(failed.load(), 0);
          CK(cudaStreamSynchronize(big.stream));
          EXPECT_EQ(big.mismatches(8100 + round), uint64_t(0));
          EXPECT_EQ(small.mismatches(8200 + round), uint64_t(0));
        }
      },
      [=](channel::Channel& ch) {
        CK(cudaSetDevice(clientDevice));
        uint8_t* host = nullptr;
        CK(cudaHostAlloc(reinterpret_cast<void**>(&host), kHostBytes, cudaHostAllocPortable));
        DeviceTensor small(clientDevice, kDeviceBytes);
        for (int round = 0; round < 2; ++round) {
          kernels::launchFill(small.stream, host, kHostBytes, 8100 + round);
          small.fill(8200 + round);
          std::promise<Error> pr;
          std::atomic<int> left{2}, failed{0};
          std::vector<channel::SendItem> v;
          for (int i = 0; i < 2; ++i) {
            channel::SendItem it;
            it.buffer = i == 0 ? CudaBuffer{host, small.stream, clientDevice} : small.buffer();
            it.length = i == 0 ? kHostBytes : kDeviceBytes;
            it.targetDevice = Device(kCudaDeviceType, serverDevice);
            it.callback = [&](const Error& e) {
              if (e) ++failed;
              if (--left == 0) pr.set_value(e);
            };
            v.push_back(std::move(it));
          }
          ch.sendBatch(std::move(v));
          auto f = pr.get_future();
          expectOk(waitFor(f), "sendBatch");
          EXPECT_EQ(failed.load(), 0);
          // the next fill of the host buffer is ordered behind the copies by the stream
        }
        CK(cudaStreamSynchronize(small.stream));
        CK(cudaFreeHost(host));
      });
}
TPB_GPU_TEST(CudaChannel, P2pPinnedHostTensorSameProcess, 1) { hostFed(false, 0, 0); }
TPB_GPU_TEST(CudaChannel, P2pPinnedHostTensorTwoProcesses, 1) { hostFed(true, 0, 0); }
TPB_GPU_TEST(CudaChannel, P2pPinnedHostTensorAcrossDevices, 2) { hostFed(true, 0, 1); }

// The sender announces a push that it never launches (host-side fault injection). The receiver's
// bounded wait runs out: its stream drains instead of hanging, the kernel reports the time-out,
// and the channel fails, so that whatever is received next says so instead of delivering data
// that never arrived.
static void waitRunsOut(int serverDevice, int clientDevice, bool waitKernel) {
  channel::cuda_p2p::Options receiver;
  receiver.waitWithKernel = waitKernel;
  receiver.waitTimeoutNs = 100'000'000ull;  // 100 ms
  channel::cuda_p2p::Options sender;
  sender.faultSkipLaunch = waitKernel ? 0 : 1;
  if (waitKernel) {
    // a large message by rendezvous: the separate wait kernel is what runs out
    receiver.eagerThreshold = 0;
    sender.eagerThreshold = 0;
  }
  const size_t bytes = 64 * 1024;
  runPair(
      true, p2p(receiver), p2p(sender),
      [=](channel::Channel& ch) {
        DeviceTensor a(serverDevice, bytes), b(serverDevice, bytes), c(serverDevice, bytes);
        if (!waitKernel) {
          // the unpack kernel itself waits only for eager batches, which come after the first
          expectOk(recvOne(ch, a, clientDevice), "first recv");
          EXPECT_EQ(a.mismatches(31), uint64_t(0));
        }
        // The callback of the receive whose data never comes still reports success: it fires when
        // the wait is enqueued. The stream then drains by itself, within the limit.
        auto t0 = std::chrono::steady_clock::now();
        expectOk(recvOne(ch, b, clientDevice), "recv of the batch that is never pushed");
        CK(cudaStreamSynchronize(b.stream));
        const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        EXPECT_TRUE(ms >= 80 && ms < 10000);
        // From here on the channel is broken and says so.
        Error e;
        for (int attempt = 0; attempt < 50 && !e; ++attempt) {
          e = recvOne(ch, c, clientDevice, 10);
          if (!e) std::this_thread::sleep_for(std::chrono::milliseconds(20));
        }
        EXPECT_TRUE(bool(e));
        EXPECT_TRUE(e.isOfType<CudaError>());
        // and the GPU still works
        DeviceTensor again(serverDevice, 4096);
        again.fill(77);
        EXPECT_EQ(again.mismatches(77), uint64_t(0));
      },
      [=](channel::Channel& ch) {
        DeviceTensor t(clientDevice, bytes);
        t.fill(31);
        if (!waitKernel) expectOk(sendOne(ch, t, serverDevice), "first send");
        // skipped launch, then sends that may or may not get through before the peer gives up
        (void)sendOne(ch, t, serverDevice);
        for (int i = 0; i < 50; ++i) {
          if (sendOne(ch, t, serverDevice, 10)) break;
          std::this_thread::sleep_for(std::chrono::milliseconds(20));
        }
        CK(cudaStreamSynchronize(t.stream));
      });
}
TPB_GPU_TEST(CudaChannel, P2pAWaitKernelThatRunsOutFailsTheChannel, 1) { waitRunsOut(0, 0, true); }
TPB_GPU_TEST(CudaChannel, P2pAnUnpackThatWaitsInVainFailsTheChannel, 2) { waitRunsOut(0, 1, false); }

// A receiver that closes while the sender may be writing into buffers it has announced gets
// those buffers back only once the sender has said goodbye (or its connection has ended). In the
// silent variant both ends lose every frame after their first exchange (host-side fault
// injection): the sender's "launched" and the receiver's goodbye vanish, nobody answers, and the
// receiver waits out its time limit; with healthy peers the same close completes at once.
static void closeWhileAnnounced(bool silentSender) {
  channel::cuda_p2p::Options o;
  o.eagerThreshold = 0;
  o.closeTimeoutMs = silentSender ? 400 : 5000;
  PeerSetup receiver = p2p(o), sender = p2p(o);
  if (silentSender) {
    sender.faulty = true;
    sender.faults.swallowFromWrite = 2;    // connection tag, hello, then silence
    receiver.faulty = true;
    receiver.faults.swallowFromWrite = 2;  // hello, the announcement of the buffer, then silence
  }
  const size_t bytes = 1u << 20;
  runPair(
      true, receiver, sender,
      [=](channel::Channel& ch) {
        DeviceTensor t(0, bytes);
        std::promise<Error> pr;
        channel::RecvItem it;
        it.buffer = t.buffer();
        it.length = bytes;
        it.sourceDevice = Device(kCudaDeviceType, 0);
        it.callback = [&](const Error& e) { pr.set_value(e); };
        std::vector<channel::RecvItem> v;
        v.push_back(std::move(it));
        ch.recvBatch(std::move(v));
        // give the announcement time to reach the sender (and, when it is silent, its push time to run)
        std::this_thread::sleep_for(std::chrono::milliseconds(200));
        auto t0 = std::chrono::steady_clock::now();
        ch.close();
        auto f = pr.get_future();
        Error e = waitFor(f, 20);
        const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        EXPECT_TRUE(bool(e));
        if (silentSender) EXPECT_TRUE(ms >= 300 && ms < 5000);
        else EXPECT_TRUE(ms < 3000);
        CK(cudaStreamSynchronize(t.stream));
      },
      [=](channel::Channel& ch) {
        DeviceTensor t(0, bytes);
        t.fill(5);
        if (silentSender) {
          // pushes into the announced buffer; the Launched frame (and later the goodbye) vanish
          (void)sendOne(ch, t, 0);
          CK(cudaStreamSynchronize(t.stream));
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(silentSender ? 1000 : 400));
      });
}
TPB_GPU_TEST(CudaChannel, P2pClosingWithAnnouncedBuffersWaitsForTheSendersGoodbye, 1) { closeWhileAnnounced(false); }
TPB_GPU_TEST(CudaChannel, P2pClosingWithAnnouncedBuffersAndASilentSenderWaitsOutItsLimit, 1) {
  closeWhileAnnounced(true);
}
