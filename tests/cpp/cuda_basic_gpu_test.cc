// GPU tests of cuda_basic, the staging channel: CUDA<->CUDA through pinned host memory, and the
// cross-device-type cases CPU->CUDA and CUDA->CPU (the reference's XDTT suite,
// tensorpipe/test/channel/channel_test_cuda_xdtt.cc:19-195), with tensors larger than one staging
// slot so that chunks pipeline through the pool and the pool runs dry.
#include <cuda_runtime.h>

#include <cstring>

#include <tpb/tpb.h>

#include "common/cuda.h"
#include "kernels/push.h"
#include "test_util.h"

using namespace tpb;
using namespace tpbtest;

namespace {

#define CK(x) TPB_CUDA_CHECK(x)

std::shared_ptr<Context> makeContext(const std::string& name) {
  auto ctx = std::make_shared<Context>(ContextOptions().name(name));
  ctx->registerTransport(0, "uv", transport::uv::create());
  ctx->registerTransport(1, "shm", transport::shm::create());
  ctx->registerChannel(0, "basic", channel::basic::create());
  ctx->registerChannel(5, "cuda_basic", channel::cuda_basic::create(channel::basic::create()));
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

const std::vector<size_t> kSizes = {0, 5, 4096, (4u << 20) + 17, 40u << 20};  // the last needs 11 slots of 4 MiB

// kind[i]: 'g' = tensor i lives on the GPU on this side, 'c' = on the CPU.
void sender(Pipe& pipe, const std::string& kinds, const std::string& peerKinds, uint64_t seed) {
  CK(cudaSetDevice(0));
  cudaStream_t stream;
  CK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  std::vector<uint8_t*> dev;
  std::vector<std::vector<uint8_t>> host(kSizes.size());
  Message m;
  for (size_t i = 0; i < kSizes.size(); ++i) {
    Message::Tensor t;
    t.length = kSizes[i];
    if (kinds[i] == 'g') {
      uint8_t* p;
      CK(cudaMalloc(&p, kSizes[i] + 16));
      dev.push_back(p);
      kernels::launchFill(stream, p, kSizes[i], seed + i);
      t.buffer = CudaBuffer{p, stream, 0};
    } else {
      host[i].resize(kSizes[i]);
      for (size_t b = 0; b < kSizes[i]; ++b) host[i][b] = kernels::patternByte(seed + i, b);
      t.buffer = CpuBuffer{host[i].data()};
    }
    t.targetDevice = peerKinds[i] == 'g' ? Device(kCudaDeviceType, 0) : Device(kCpuDeviceType, 0);
    m.tensors.push_back(t);
  }
  std::promise<Error> pw;
  pipe.write(std::move(m), [&](const Error& e) { pw.set_value(e); });
  auto fw = pw.get_future();
  Error e = waitFor(fw, 60);
  if (e) throw TestFailure("write failed: " + e.what());
  CK(cudaStreamSynchronize(stream));
  for (auto* p : dev) cudaFree(p);
  cudaStreamDestroy(stream);
}

void receiver(Pipe& pipe, const std::string& kinds, uint64_t seed) {
  CK(cudaSetDevice(0));
  cudaStream_t stream;
  CK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  std::promise<std::pair<Error, Descriptor>> pd;
  pipe.readDescriptor([&](const Error& e, Descriptor d) { pd.set_value({e, std::move(d)}); });
  auto fd = pd.get_future();
  auto [e, d] = waitFor(fd, 60);
  if (e) throw TestFailure("readDescriptor failed: " + e.what());
  EXPECT_EQ(d.tensors.size(), kSizes.size());
  std::vector<uint8_t*> dev(kSizes.size(), nullptr);
  std::vector<std::vector<uint8_t>> host(kSizes.size());
  Allocation a;
  for (size_t i = 0; i < kSizes.size(); ++i) {
    Allocation::Tensor t;
    if (kinds[i] == 'g') {
      CK(cudaMalloc(&dev[i], kSizes[i] + 16));
      t.buffer = CudaBuffer{dev[i], stream, 0};
    } else {
      host[i].resize(kSizes[i]);
      t.buffer = CpuBuffer{host[i].data()};
    }
    a.tensors.push_back(t);
  }
  std::promise<Error> pr;
  pipe.read(std::move(a), [&](const Error& e2) { pr.set_value(e2); });
  auto fr = pr.get_future();
  Error e2 = waitFor(fr, 60);
  if (e2) throw TestFailure("read failed: " + e2.what());
  unsigned long long* bad;
  CK(cudaMalloc(&bad, 8));
  CK(cudaMemsetAsync(bad, 0, 8, stream));
  for (size_t i = 0; i < kSizes.size(); ++i) {
    if (kinds[i] == 'g') {
      kernels::launchVerify(stream, dev[i], kSizes[i], seed + i, bad);
    } else {
      for (size_t b = 0; b < kSizes[i]; ++b)
        if (host[i][b] != kernels::patternByte(seed + i, b))
          throw TestFailure("CPU tensor " + std::to_string(i) + " differs at byte " + std::to_string(b));
    }
  }
  CK(cudaStreamSynchronize(stream));
  unsigned long long h = 1;
  CK(cudaMemcpy(&h, bad, 8, cudaMemcpyDeviceToHost));
  if (h) throw TestFailure("GPU tensors differ in " + std::to_string(h) + " bytes");
  for (auto* p : dev)
    if (p) cudaFree(p);
  cudaFree(bad);
  cudaStreamDestroy(stream);
}

void runCase(bool processes, const std::string& senderKinds, const std::string& receiverKinds) {
  auto server = [=](std::function<void(std::string)> tell, std::function<std::string()> hear) {
    auto ctx = makeContext("server");
    auto l = ctx->listen({"uv://127.0.0.1", "shm://"});
    tell(l->url("uv"));
    auto pipe = acceptSync(*l);
    receiver(*pipe, receiverKinds, 500);
    sender(*pipe, receiverKinds, senderKinds, 900);  // and back, roles swapped
    hear();
    EXPECT_TRUE(ctx->stats().bytesPerChannel.count("cuda_basic") == 1);
    ctx->join();
  };
  auto client = [=](std::function<void(std::string)> tell, std::function<std::string()> hear) {
    auto ctx = makeContext("client");
    auto pipe = ctx->connect(hear());
    sender(*pipe, senderKinds, receiverKinds, 500);
    receiver(*pipe, senderKinds, 900);
    tell("done");
    ctx->join();
  };
  if (processes) {
    ProcessPeers::run([=](const ProcessPeers::Side& me) { server([&](std::string s) { me.send(s); }, [&] { return me.recv(); }); },
                      [=](const ProcessPeers::Side& me) { client([&](std::string s) { me.send(s); }, [&] { return me.recv(); }); });
  } else {
    ThreadPeers peers;
    peers.run([&](ThreadPeers& pg) { server([&](std::string s) { pg.sendToClient(s); }, [&] { return pg.recvFromClient(); }); },
              [&](ThreadPeers& pg) { client([&](std::string s) { pg.sendToServer(s); }, [&] { return pg.recvFromServer(); }); });
  }
}

}  // namespace

TPB_GPU_TEST(CudaBasic, GpuToGpuSameProcess, 1) { runCase(false, "ggggg", "ggggg"); }
TPB_GPU_TEST(CudaBasic, GpuToGpuTwoProcesses, 1) { runCase(true, "ggggg", "ggggg"); }
TPB_GPU_TEST(CudaBasic, CpuToGpuAndGpuToCpu, 1) { runCase(true, "ccccc", "ggggg"); }
TPB_GPU_TEST(CudaBasic, MixedDeviceTypesInOneMessage, 1) { runCase(false, "gcgcg", "cggcc"); }
