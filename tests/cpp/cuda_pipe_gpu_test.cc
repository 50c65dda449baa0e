// GPU tests of the device-to-device channel through full pipes: same process (raw pointers and
// events), two processes sharing one GPU (IPC mappings, flags, the eager inbox), and two
// processes on two GPUs. They follow the reference's CUDA channel cases
// (tensorpipe/test/channel/channel_test_cuda.cc:19-139: the receiver must wait for work already
// on the sender's stream; tensors at an offset inside an allocation) and add what the reference
// cannot do: many tensors in one launch, strided views, receiver-requested casts.
#include <cuda_runtime.h>

#include <cstring>
#include <random>

#include <tpb/tpb.h>

#include "common/cuda.h"
#include "kernels/push.h"
#include "test_util.h"

using namespace tpb;
using namespace tpbtest;

namespace {

#define CK(x) TPB_CUDA_CHECK(x)

std::shared_ptr<Context> makeContext(const std::string& name, channel::cuda_p2p::Options o = {}) {
  auto ctx = std::make_shared<Context>(ContextOptions().name(name));
  ctx->registerTransport(0, "uv", transport::uv::create());
  ctx->registerTransport(1, "shm", transport::shm::create());
  ctx->registerChannel(0, "basic", channel::basic::create());
  ctx->registerChannel(10, "cuda_p2p", channel::cuda_p2p::create(o));
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

void writeSync(Pipe& pipe, Message m) {
  std::promise<Error> p;
  pipe.write(std::move(m), [&](const Error& e) { p.set_value(e); });
  auto f = p.get_future();
  Error e = waitFor(f);
  if (e) throw TestFailure("write failed: " + e.what());
}

Descriptor readDescriptorSync(Pipe& pipe) {
  std::promise<std::pair<Error, Descriptor>> pd;
  pipe.readDescriptor([&](const Error& e, Descriptor d) { pd.set_value({e, std::move(d)}); });
  auto fd = pd.get_future();
  auto [e, d] = waitFor(fd);
  if (e) throw TestFailure("readDescriptor failed: " + e.what());
  return d;
}

void readSync(Pipe& pipe, Allocation a) {
  std::promise<Error> pr;
  pipe.read(std::move(a), [&](const Error& e) { pr.set_value(e); });
  auto fr = pr.get_future();
  Error e = waitFor(fr);
  if (e) throw TestFailure("read failed: " + e.what());
}

uint16_t f32ToBf16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  uint32_t lsb = (x >> 16) & 1;
  x += 0x7fffu + lsb;
  return static_cast<uint16_t>(x >> 16);
}

// The message both sides agree on: sizes chosen to hit empty, tiny, ragged, tile-edge and large.
const std::vector<size_t> kDefaultSizes = {0, 1, 17, 4096, 70001, (1u << 20) + 3, 8u << 20};

void senderSide(Pipe& pipe, int device, int targetDevice, uint64_t seedBase, int rounds,
                const std::vector<size_t>& kSizes = kDefaultSizes) {
  CK(cudaSetDevice(device));
  cudaStream_t stream;
  CK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  for (int round = 0; round < rounds; ++round) {
    std::vector<uint8_t*> bufs;
    Message m;
    m.metadata = "round" + std::to_string(round);
    for (size_t i = 0; i < kSizes.size(); ++i) {
      uint8_t* p = nullptr;
      CK(cudaMalloc(&p, kSizes[i] + 32));
      bufs.push_back(p);
      // tensors start at an odd offset inside their allocation
      kernels::launchFill(stream, p + 16, kSizes[i], seedBase + round * 100 + i);
      Message::Tensor t;
      t.buffer = CudaBuffer{p + 16, stream, device};
      t.length = kSizes[i];
      if (i % 2 == 0) t.targetDevice = Device(kCudaDeviceType, targetDevice);
      m.tensors.push_back(t);
    }
    writeSync(pipe, std::move(m));
    CK(cudaStreamSynchronize(stream));
    for (auto* p : bufs) cudaFree(p);
  }
  cudaStreamDestroy(stream);
}

void receiverSide(Pipe& pipe, int device, uint64_t seedBase, int rounds,
                  const std::vector<size_t>& kSizes = kDefaultSizes, bool poolMemory = false) {
  CK(cudaSetDevice(device));
  cudaStream_t stream;
  CK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  unsigned long long* bad;
  CK(cudaMalloc(&bad, 8));
  CK(cudaMemset(bad, 0, 8));
  for (int round = 0; round < rounds; ++round) {
    Descriptor d = readDescriptorSync(pipe);
    EXPECT_EQ(d.metadata, "round" + std::to_string(round));
    EXPECT_EQ(d.tensors.size(), kSizes.size());
    std::vector<uint8_t*> bufs;
    Allocation a;
    for (size_t i = 0; i < kSizes.size(); ++i) {
      EXPECT_EQ(d.tensors[i].length, kSizes[i]);
      uint8_t* p = nullptr;
      // Stream-ordered pool memory has no legacy IPC handle: the channel must stage such buffers.
      if (poolMemory) CK(cudaMallocAsync(reinterpret_cast<void**>(&p), kSizes[i] + 512, stream));
      else CK(cudaMalloc(&p, kSizes[i] + 512));
      CK(cudaMemsetAsync(p, 0xCD, kSizes[i] + 512, stream));
      bufs.push_back(p);
      Allocation::Tensor t;
      t.buffer = CudaBuffer{p + 256, stream, device};
      a.tensors.push_back(t);
    }
    readSync(pipe, std::move(a));
    for (size_t i = 0; i < kSizes.size(); ++i)
      kernels::launchVerify(stream, bufs[i] + 256, kSizes[i], seedBase + round * 100 + i, bad);
    CK(cudaStreamSynchronize(stream));
    unsigned long long h = 1;
    CK(cudaMemcpy(&h, bad, 8, cudaMemcpyDeviceToHost));
    if (h != 0) throw TestFailure("received data differs in " + std::to_string(h) + " bytes (round " + std::to_string(round) + ")");
    for (size_t i = 0; i < kSizes.size(); ++i) {
      uint8_t guard[2];
      CK(cudaMemcpy(&guard[0], bufs[i] + 255, 1, cudaMemcpyDeviceToHost));
      CK(cudaMemcpy(&guard[1], bufs[i] + 256 + kSizes[i], 1, cudaMemcpyDeviceToHost));
      EXPECT_EQ(int(guard[0]), 0xCD);
      EXPECT_EQ(int(guard[1]), 0xCD);
      if (poolMemory) cudaFreeAsync(bufs[i], stream);
      else cudaFree(bufs[i]);
    }
  }
  cudaFree(bad);
  cudaStreamDestroy(stream);
}

void crossProcess(int serverDevice, int clientDevice, channel::cuda_p2p::Options opts) {
  ProcessPeers::run(
      [=](const ProcessPeers::Side& me) {
        auto ctx = makeContext("server", opts);
        auto listener = ctx->listen({"uv://127.0.0.1", "shm://"});
        me.send(listener->url("uv"));
        auto pipe = acceptSync(*listener);
        receiverSide(*pipe, serverDevice, 1000, 3);
        senderSide(*pipe, serverDevice, clientDevice, 2000, 2);
        me.recv();
        me.send("bye");
        ctx->join();
      },
      [=](const ProcessPeers::Side& me) {
        auto ctx = makeContext("client", opts);
        auto pipe = ctx->connect(me.recv());
        senderSide(*pipe, clientDevice, serverDevice, 1000, 3);
        receiverSide(*pipe, clientDevice, 2000, 2);
        me.send("done");
        me.recv();
        ctx->join();
      });
}

}  // namespace

TPB_GPU_TEST(CudaPipe, SameProcessSameDevice, 1) {
  ThreadPeers peers;
  peers.run(
      [&](ThreadPeers& pg) {
        auto ctx = makeContext("server");
        auto listener = ctx->listen({"uv://127.0.0.1"});
        pg.sendToClient(listener->url("uv"));
        auto pipe = acceptSync(*listener);
        receiverSide(*pipe, 0, 1000, 3);
        senderSide(*pipe, 0, 0, 2000, 2);
        pg.recvFromClient();
        ctx->join();
      },
      [&](ThreadPeers& pg) {
        auto ctx = makeContext("client");
        auto pipe = ctx->connect(pg.recvFromServer());
        senderSide(*pipe, 0, 0, 1000, 3);
        receiverSide(*pipe, 0, 2000, 2);
        pg.sendToServer("done");
        ctx->join();
      });
}

// Moving tensors that live on the second GPU must not create a context on the first one (the
// reference checks the same through NVML's process list, tensorpipe/test/channel/cuda_helpers.h:50-95;
// the driver's primary-context state is exact and also works inside a pid namespace).
TPB_GPU_TEST(CudaPipe, NoContextOnADeviceTheUserNeverTouched, 2) {
  EXPECT_EQ(cudaPrimaryContextActive(0), 0);
  ThreadPeers peers;
  peers.run(
      [&](ThreadPeers& pg) {
        auto ctx = makeContext("server");
        auto listener = ctx->listen({"uv://127.0.0.1"});
        pg.sendToClient(listener->url("uv"));
        auto pipe = acceptSync(*listener);
        receiverSide(*pipe, 1, 1000, 3);
        pg.recvFromClient();
        ctx->join();
      },
      [&](ThreadPeers& pg) {
        auto ctx = makeContext("client");
        auto pipe = ctx->connect(pg.recvFromServer());
        senderSide(*pipe, 1, 1, 1000, 3);
        pg.sendToServer("done");
        ctx->join();
      });
  EXPECT_EQ(cudaPrimaryContextActive(1), 1);
  EXPECT_EQ(cudaPrimaryContextActive(0), 0);
}

TPB_GPU_TEST(CudaPipe, ReceiverWaitsForWorkOnTheSendersStream, 1) {
  // The sender's stream first spends ~30 ms scribbling garbage over the tensor and only then
  // writes the real data; the pipe write is issued while all of that is still queued.
  ThreadPeers peers;
  constexpr size_t kBytes = 1 << 20;
  peers.run(
      [&](ThreadPeers& pg) {
        auto ctx = makeContext("server");
        auto listener = ctx->listen({"uv://127.0.0.1"});
        pg.sendToClient(listener->url("uv"));
        auto pipe = acceptSync(*listener);
        CK(cudaSetDevice(0));
        cudaStream_t stream;
        CK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
        uint8_t* p;
        CK(cudaMalloc(&p, kBytes));
        Descriptor d = readDescriptorSync(*pipe);
        Allocation a;
        Allocation::Tensor t;
        t.buffer = CudaBuffer{p, stream, 0};
        a.tensors.push_back(t);
        readSync(*pipe, std::move(a));
        unsigned long long* bad;
        CK(cudaMalloc(&bad, 8));
        CK(cudaMemsetAsync(bad, 0, 8, stream));
        kernels::launchVerify(stream, p, kBytes, 4242, bad);
        CK(cudaStreamSynchronize(stream));
        unsigned long long h = 1;
        CK(cudaMemcpy(&h, bad, 8, cudaMemcpyDeviceToHost));
        EXPECT_EQ(h, 0ull);
        pg.recvFromClient();
        ctx->join();
      },
      [&](ThreadPeers& pg) {
        auto ctx = makeContext("client");
        auto pipe = ctx->connect(pg.recvFromServer());
        CK(cudaSetDevice(0));
        cudaStream_t stream;
        CK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
        uint8_t* p;
        CK(cudaMalloc(&p, kBytes));
        kernels::launchDelay(stream, p, kBytes, 30000);
        kernels::launchFill(stream, p, kBytes, 4242);
        Message m;
        Message::Tensor t;
        t.buffer = CudaBuffer{p, stream, 0};
        t.length = kBytes;
        m.tensors.push_back(t);
        writeSync(*pipe, std::move(m));
        CK(cudaStreamSynchronize(stream));
        pg.sendToServer("done");
        ctx->join();
      });
}

TPB_GPU_TEST(CudaPipe, TwoProcessesOneDevice, 1) { crossProcess(0, 0, {}); }

TPB_GPU_TEST(CudaPipe, TwoProcessesOneDeviceWithoutBulkCopiesOrEager, 1) {
  channel::cuda_p2p::Options o;
  o.useBulkCopy = false;
  o.eagerThreshold = 0;
  crossProcess(0, 0, o);
}

TPB_GPU_TEST(CudaPipe, TwoProcessesTwoDevices, 2) { crossProcess(0, 1, {}); }

// The receiver's buffers come from a stream-ordered memory pool, which CUDA IPC cannot export:
// the channel lets the sender write into exportable staging buffers of its own and copies out on
// the receiver's stream. (The reference never exports user memory for this reason,
// tensorpipe/channel/cuda_ipc/context_impl.h:101-115, and always pays the staging copy.)
TPB_GPU_TEST(CudaPipe, ReceiveIntoMemoryThatCannotBeExported, 1) {
  channel::cuda_p2p::Options o;
  o.eagerThreshold = 0;  // everything by rendezvous, so every tensor needs a destination handle
  const std::vector<size_t> sizes = {4096, 70001, (1u << 20) + 3, 8u << 20};
  ProcessPeers::run(
      [=](const ProcessPeers::Side& me) {
        auto ctx = makeContext("server", o);
        auto listener = ctx->listen({"uv://127.0.0.1", "shm://"});
        me.send(listener->url("uv"));
        auto pipe = acceptSync(*listener);
        // Does this driver refuse a legacy IPC handle for pool memory? (It should.)
        CK(cudaSetDevice(0));
        void* probe = nullptr;
        CK(cudaMallocAsync(&probe, 4096, nullptr));
        CK(cudaStreamSynchronize(nullptr));
        cudaIpcMemHandle_t h;
        const bool exportable = cudaIpcGetMemHandle(&h, probe) == cudaSuccess;
        cudaGetLastError();
        CK(cudaFreeAsync(probe, nullptr));
        std::cout << "  a legacy IPC handle for pool memory: " << (exportable ? "granted" : "refused") << std::endl;
        const uint64_t before = channel::cuda_p2p::stagedReceives();
        receiverSide(*pipe, 0, 1000, 3, sizes, true);
        if (!exportable) EXPECT_EQ(channel::cuda_p2p::stagedReceives() - before, uint64_t(3 * sizes.size()));
        me.recv();
        me.send("bye");
        ctx->join();
      },
      [=](const ProcessPeers::Side& me) {
        auto ctx = makeContext("client", o);
        auto pipe = ctx->connect(me.recv());
        senderSide(*pipe, 0, 0, 1000, 3, sizes);
        me.send("done");
        me.recv();
        ctx->join();
      });
}

TPB_GPU_TEST(CudaPipe, EagerInboxWrapsAndRunsOutOfCredits, 1) {
  // Small messages go through the peer's inbox ring without waiting for the receiver; a tiny
  // ring makes it wrap many times and run out of credits (falling back to rendezvous).
  channel::cuda_p2p::Options o;
  o.inboxBytes = 64 * 1024;
  o.eagerThreshold = 16 * 1024;
  const std::vector<size_t> sizes = {1024, 5000, 17, 0, 256};
  ProcessPeers::run(
      [=](const ProcessPeers::Side& me) {
        auto ctx = makeContext("server", o);
        auto listener = ctx->listen({"uv://127.0.0.1", "shm://"});
        me.send(listener->url("uv"));
        auto pipe = acceptSync(*listener);
        receiverSide(*pipe, 0, 1000, 60, sizes);
        me.recv();
        ctx->join();
      },
      [=](const ProcessPeers::Side& me) {
        auto ctx = makeContext("client", o);
        auto pipe = ctx->connect(me.recv());
        senderSide(*pipe, 0, 0, 1000, 60, sizes);
        me.send("done");
        ctx->join();
      });
}

TPB_GPU_TEST(CudaPipe, TwoProcessesTwoDevicesWaitKernel, 2) {
  channel::cuda_p2p::Options o;
  o.waitWithKernel = true;
  crossProcess(0, 1, o);
}

TPB_GPU_TEST(CudaPipe, SameProcessTwoDevices, 2) {
  ThreadPeers peers;
  peers.run(
      [&](ThreadPeers& pg) {
        auto ctx = makeContext("server");
        auto listener = ctx->listen({"uv://127.0.0.1"});
        pg.sendToClient(listener->url("uv"));
        auto pipe = acceptSync(*listener);
        receiverSide(*pipe, 1, 1000, 2);
        senderSide(*pipe, 1, 0, 2000, 2);
        pg.recvFromClient();
        ctx->join();
      },
      [&](ThreadPeers& pg) {
        auto ctx = makeContext("client");
        auto pipe = ctx->connect(pg.recvFromServer());
        senderSide(*pipe, 0, 1, 1000, 2);
        receiverSide(*pipe, 0, 2000, 2);
        pg.sendToServer("done");
        ctx->join();
      });
}

namespace {
// Strided view + cast, checked element by element against a host gather and host rounding.
// With `staged` the contexts have no device-to-device channel: the same message goes through
// pinned host memory (cuda_basic), which packs views on the sender and converts on the receiver.
void layoutsCase(bool crossProc, int recvDevice, int sendDevice, bool staged = false) {
  constexpr int64_t kRows = 300, kCols = 129;
  auto makeContext = [staged](const std::string& name) {
    if (!staged) return ::makeContext(name);
    auto ctx = std::make_shared<Context>(ContextOptions().name(name));
    ctx->registerTransport(0, "uv", transport::uv::create());
    ctx->registerTransport(1, "shm", transport::shm::create());
    ctx->registerChannel(0, "basic", channel::basic::create());
    ctx->registerChannel(5, "cuda_basic", channel::cuda_basic::create(channel::basic::create()));
    return ctx;
  };
  auto server = [=](std::function<void(std::string)> tell, std::function<std::string()> hear) {
    auto ctx = makeContext("server");
    auto listener = ctx->listen({"uv://127.0.0.1", "shm://"});
    tell(listener->url("uv"));
    auto pipe = acceptSync(*listener);
    CK(cudaSetDevice(recvDevice));
    cudaStream_t stream;
    CK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    for (int round = 0; round < 2; ++round) {  // round 0 rendezvous, round 1 may go through the inbox
      Descriptor d = readDescriptorSync(*pipe);
      EXPECT_EQ(d.tensors.size(), size_t(3));
      EXPECT_EQ(d.tensors[0].length, size_t(kRows * kCols * 4));
      uint16_t* bf;
      float* plain;
      uint16_t* flat;  // contiguous source, converted on the way
      CK(cudaMalloc(&bf, kRows * kCols * 2));
      CK(cudaMalloc(&plain, kRows * kCols * 4));
      CK(cudaMalloc(&flat, kRows * kCols * 2));
      Allocation a;
      Allocation::Tensor t0;
      t0.buffer = CudaBuffer{bf, stream, recvDevice};
      t0.castTo = DType::kBF16;
      t0.sourceDtype = DType::kF32;
      Allocation::Tensor t1;
      t1.buffer = CudaBuffer{plain, stream, recvDevice};
      Allocation::Tensor t2;
      t2.buffer = CudaBuffer{flat, stream, recvDevice};
      t2.castTo = DType::kBF16;
      t2.sourceDtype = DType::kF32;
      a.tensors = {t0, t1, t2};
      readSync(*pipe, std::move(a));
      CK(cudaStreamSynchronize(stream));
      std::vector<uint16_t> gotFlat(kRows * kCols);
      CK(cudaMemcpy(gotFlat.data(), flat, gotFlat.size() * 2, cudaMemcpyDeviceToHost));
      for (int64_t c = 0; c < kCols; ++c)
        for (int64_t r = 0; r < kRows; ++r)
          EXPECT_EQ(gotFlat[c * kRows + r], f32ToBf16(static_cast<float>(c * 1000 + r) * 0.37f + round));
      cudaFree(flat);
      std::vector<uint16_t> gotBf(kRows * kCols);
      std::vector<float> gotPlain(kRows * kCols);
      CK(cudaMemcpy(gotBf.data(), bf, gotBf.size() * 2, cudaMemcpyDeviceToHost));
      CK(cudaMemcpy(gotPlain.data(), plain, gotPlain.size() * 4, cudaMemcpyDeviceToHost));
      // The sender's storage is a [kCols, kRows] matrix with value f(c, r); we get its transpose.
      for (int64_t r = 0; r < kRows; ++r)
        for (int64_t c = 0; c < kCols; ++c) {
          float want = static_cast<float>(c * 1000 + r) * 0.37f + round;
          EXPECT_EQ(gotBf[r * kCols + c], f32ToBf16(want));
          EXPECT_TRUE(gotPlain[r * kCols + c] == want);
        }
      cudaFree(bf);
      cudaFree(plain);
    }
    hear();
    ctx->join();
  };
  auto client = [=](std::function<void(std::string)> tell, std::function<std::string()> hear) {
    auto ctx = makeContext("client");
    auto pipe = ctx->connect(hear());
    CK(cudaSetDevice(sendDevice));
    cudaStream_t stream;
    CK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    for (int round = 0; round < 2; ++round) {
      std::vector<float> host(kRows * kCols);
      for (int64_t c = 0; c < kCols; ++c)
        for (int64_t r = 0; r < kRows; ++r) host[c * kRows + r] = static_cast<float>(c * 1000 + r) * 0.37f + round;
      float* dev;
      CK(cudaMalloc(&dev, host.size() * 4));
      CK(cudaMemcpyAsync(dev, host.data(), host.size() * 4, cudaMemcpyHostToDevice, stream));
      Message m;
      for (int i = 0; i < 2; ++i) {
        Message::Tensor t;
        t.buffer = CudaBuffer{dev, stream, sendDevice};
        t.length = host.size() * 4;
        t.dtype = DType::kF32;
        t.view = StridedView{DType::kF32, kRows, kCols, 1, kRows};
        t.targetDevice = Device(kCudaDeviceType, recvDevice);
        m.tensors.push_back(t);
      }
      {
        Message::Tensor t;  // the same storage, sent as it lies in memory
        t.buffer = CudaBuffer{dev, stream, sendDevice};
        t.length = host.size() * 4;
        t.dtype = DType::kF32;
        t.targetDevice = Device(kCudaDeviceType, recvDevice);
        m.tensors.push_back(t);
      }
      writeSync(*pipe, std::move(m));
      CK(cudaStreamSynchronize(stream));
      cudaFree(dev);
    }
    tell("done");
    ctx->join();
  };
  if (crossProc) {
    ProcessPeers::run([=](const ProcessPeers::Side& me) { server([&](std::string s) { me.send(s); }, [&] { return me.recv(); }); },
                      [=](const ProcessPeers::Side& me) { client([&](std::string s) { me.send(s); }, [&] { return me.recv(); }); });
  } else {
    ThreadPeers peers;
    peers.run([&](ThreadPeers& pg) { server([&](std::string s) { pg.sendToClient(s); }, [&] { return pg.recvFromClient(); }); },
              [&](ThreadPeers& pg) { client([&](std::string s) { pg.sendToServer(s); }, [&] { return pg.recvFromServer(); }); });
  }
}
}  // namespace

TPB_GPU_TEST(CudaPipe, StridedViewAndCastSameProcess, 1) { layoutsCase(false, 0, 0); }
TPB_GPU_TEST(CudaPipe, StridedViewAndCastTwoProcesses, 1) { layoutsCase(true, 0, 0); }
TPB_GPU_TEST(CudaPipe, StridedViewAndCastTwoDevices, 2) { layoutsCase(true, 0, 1); }
TPB_GPU_TEST(CudaBasic, StridedViewAndCastSameProcess, 1) { layoutsCase(false, 0, 0, true); }
TPB_GPU_TEST(CudaBasic, StridedViewAndCastTwoProcesses, 1) { layoutsCase(true, 0, 0, true); }
TPB_GPU_TEST(CudaBasic, StridedViewAndCastTwoDevices, 2) { layoutsCase(true, 0, 1, true); }
