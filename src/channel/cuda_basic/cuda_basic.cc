// cuda_basic: the universal fallback for tensors that touch a GPU (cuda<->cuda without peer
// access, cpu<->cuda), staged through pinned host memory and carried by any CPU channel.
//
// Same role and negotiation as the reference's channel (tensorpipe/channel/cuda_basic/
// context_impl.cc:27-128: wraps a CPU channel, never serves cpu->cpu, descriptor = {device type,
// inner descriptor}) with a different data path: instead of cudaMemcpyAsync plus
// cudaStreamAddCallback per 1 MiB chunk (channel_impl.cc:58-71), a pack kernel on the user's
// stream writes each chunk into a mapped pinned slot and publishes a host-visible flag with a
// system-scope release store; a poller thread notices the flag and hands the slot to the CPU
// channel. On the receiving side the CPU channel fills a pinned slot and an unpack kernel on the
// user's stream moves it into the tensor; the slot returns to the pool when an event recorded
// after the kernel has fired.
//
// Ordering: both ends cut every tensor into the same chunks and feed the inner channel strictly
// in chunk order (one ordered queue per direction), because the inner channel matches its k-th
// send with the peer's k-th recv.
#include <atomic>
#include <condition_variable>
#include <deque>
#include <list>
#include <map>
#include <set>
#include <thread>

#include <tpb/channel.h>

#include "channel/nonviable.h"
#include "common/cuda.h"
#include "common/defs.h"
#include "common/loop.h"
#include "common/nop.h"
#include "kernels/push.h"

namespace tpb {
namespace channel {
namespace cuda_basic {

namespace {

constexpr size_t kChunkBytes = 4u << 20;
constexpr int kSlotsPerDirection = 8;

struct DeviceDescriptor {
  std::string deviceType;
  std::string cpuDescriptor;
  TPB_NOP_STRUCTURE(DeviceDescriptor, deviceType, cpuDescriptor)
};

// Polls conditions (host flags written by kernels, CUDA events) off the loop thread and fires a
// one-shot callback when one turns true. Sleeps when there is nothing to watch.
class Poller {
 public:
  Poller() {
    thread_ = std::thread([this]() {
      setThreadName("TP_CUDA_poller");
      run();
    });
  }
  ~Poller() { stop(); }
  void watch(std::function<bool()> ready, std::function<void()> fire) {
    {
      std::unique_lock<std::mutex> l(mu_);
      items_.push_back({std::move(ready), std::move(fire)});
    }
    cv_.notify_one();
  }
  void stop() {
    {
      std::unique_lock<std::mutex> l(mu_);
      if (stop_) return;
      stop_ = true;
    }
    cv_.notify_all();
    if (thread_.joinable()) thread_.join();
  }

 private:
  struct Item {
    std::function<bool()> ready;
    std::function<void()> fire;
  };
  void run() {
    std::unique_lock<std::mutex> l(mu_);
    for (;;) {
      cv_.wait(l, [&] { return stop_ || !items_.empty(); });
      if (stop_) {
        // Fire what is left so that nobody waits forever; the channels are closing anyway.
        auto rest = std::move(items_);
        items_.clear();
        l.unlock();
        for (auto& it : rest) it.fire();
        return;
      }
      std::vector<std::function<void()>> fired;
      for (auto it = items_.begin(); it != items_.end();) {
        bool ok = false;
        try {
          ok = it->ready();
        } catch (...) {
          ok = true;  // a failing query must not wedge the queue; the fire path re-checks
        }
        if (ok) {
          fired.push_back(std::move(it->fire));
          it = items_.erase(it);
        } else {
          ++it;
        }
      }
      l.unlock();
      for (auto& f : fired) f();
      if (fired.empty()) std::this_thread::yield();
      l.lock();
    }
  }
  std::mutex mu_;
  std::condition_variable cv_;
  std::list<Item> items_;
  bool stop_ = false;
  std::thread thread_;
};

// Pinned, mapped staging slots of one direction, allocated on first use.
struct SlotPool {
  uint8_t* base = nullptr;
  volatile uint32_t* flags = nullptr;  // one host-visible word per slot
  std::deque<int> free;
  bool ensure() {
    if (base) return true;
    void* p = nullptr;
    if (cudaHostAlloc(&p, kChunkBytes * kSlotsPerDirection + 4096, cudaHostAllocPortable | cudaHostAllocMapped) !=
        cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    base = static_cast<uint8_t*>(p);
    flags = reinterpret_cast<volatile uint32_t*>(base + kChunkBytes * kSlotsPerDirection);
    for (int i = 0; i < kSlotsPerDirection; ++i) {
      flags[i] = 0;
      free.push_back(i);
    }
    return true;
  }
  uint8_t* slot(int i) const { return base + static_cast<size_t>(i) * kChunkBytes; }
  ~SlotPool() {
    if (base) cudaFreeHost(base);
  }
};

class ContextImpl;

class ChannelImpl final : public Channel, public std::enable_shared_from_this<ChannelImpl> {
 public:
  ChannelImpl(std::shared_ptr<ContextImpl> ctx, std::shared_ptr<Channel> inner) : ctx_(std::move(ctx)), inner_(std::move(inner)) {}
  void init();
  void send(Buffer buffer, size_t length, TSendCallback cb) override;
  void recv(Buffer buffer, size_t length, TRecvCallback cb) override;
  void setId(std::string id) override { inner_->setId(id + ".cpu"); }
  void close() override;
  void closeFromLoop(const Error& e);

 private:
  struct Op {
    size_t remaining = 0;   // chunks not yet accounted for
    Error error;
    std::function<void(const Error&)> cb;
  };
  struct Chunk {
    std::shared_ptr<Op> op;
    bool cuda = false;
    uint8_t* ptr = nullptr;  // CPU pointer, or device pointer
    size_t len = 0;
    int device = -1;
    cudaStream_t stream = nullptr;
    int slot = -1;
    uint32_t flagValue = 0;
    bool staged = false;    // send: pack kernel launched / recv: inner recv issued
    bool ready = false;     // send: pack finished
  };
  void pumpSend();
  void pumpRecv();
  void chunkDone(const std::shared_ptr<Op>& op, const Error& e);
  uint32_t* counterFor(int device, cudaStream_t stream);

  std::shared_ptr<ContextImpl> ctx_;
  std::shared_ptr<Channel> inner_;
  Error error_;
  std::deque<Chunk> sendQueue_;  // in chunk order; front = next to hand to the inner channel
  std::deque<Chunk> recvQueue_;  // chunks whose inner recv has not been issued yet
  SlotPool sendSlots_, recvSlots_;
  uint32_t nextFlagValue_ = 1;
  std::map<std::pair<int, cudaStream_t>, uint32_t*> counters_;  // one arrive counter per launching stream

 public:
  ~ChannelImpl() override {
    for (auto& c : counters_) {
      try {
        CudaDeviceGuard g(c.first.first);
        cudaFree(c.second);
      } catch (...) {
      }
    }
  }
};

class ContextImpl final : public Context, public std::enable_shared_from_this<ContextImpl> {
 public:
  explicit ContextImpl(std::shared_ptr<Context> cpu) : cpu_(std::move(cpu)) {
    const auto& inner = cpu_->deviceDescriptors();
    auto it = inner.find(Device(kCpuDeviceType, 0));
    if (it == inner.end()) return;
    const int n = cudaDeviceCountNoThrow();
    if (n == 0) return;
    auto add = [&](const Device& d) {
      // Same structure as the reference's descriptor (tensorpipe/channel/cuda_basic/context_impl.cc:
      // 27-31,64-80) but with a prefixed inner descriptor, so that a reference peer's cuda_basic
      // never matches: the chunking and the control traffic of the two differ.
      DeviceDescriptor dd;
      dd.deviceType = d.type;
      dd.cpuDescriptor = "tpbcb1:" + it->second;
      auto bytes = nop::encode(dd);
      descriptors_[d] = std::string(bytes.begin(), bytes.end());
    };
    add(Device(kCpuDeviceType, 0));
    for (int i = 0; i < n; ++i) add(Device(kCudaDeviceType, i));
    viable_ = true;
  }
  bool isViable() const override { return viable_ && cpu_->isViable(); }
  size_t numConnectionsNeeded() const override { return cpu_->numConnectionsNeeded(); }
  const std::unordered_map<Device, std::string>& deviceDescriptors() const override { return descriptors_; }
  bool canCommunicateWithRemote(const std::string& local, const std::string& remote) const override {
    DeviceDescriptor l, r;
    if (!nop::decode(local.data(), local.size(), l) || !nop::decode(remote.data(), remote.size(), r)) return false;
    if (l.deviceType == kCpuDeviceType && r.deviceType == kCpuDeviceType) return false;  // not our job
    const std::string prefix = "tpbcb1:";
    if (l.cpuDescriptor.compare(0, prefix.size(), prefix) != 0 || r.cpuDescriptor.compare(0, prefix.size(), prefix) != 0)
      return false;
    return cpu_->canCommunicateWithRemote(l.cpuDescriptor.substr(prefix.size()), r.cpuDescriptor.substr(prefix.size()));
  }
  std::shared_ptr<Channel> createChannel(std::vector<std::shared_ptr<transport::Connection>> conns, Endpoint ep) override {
    auto inner = cpu_->createChannel(std::move(conns), ep);
    auto ch = std::make_shared<ChannelImpl>(shared_from_this(), std::move(inner));
    ch->init();
    return ch;
  }
  void setId(std::string id) override { cpu_->setId(id + ".cpu"); }
  void close() override {
    loop_.deferToLoop([this, self = shared_from_this()]() {
      if (closed_) return;
      closed_ = true;
      auto chans = channels_;
      for (auto& w : chans)
        if (auto c = w.lock()) c->closeFromLoop(TPB_CREATE_ERROR(ContextClosedError));
      channels_.clear();
      cpu_->close();
    });
  }
  void join() override {
    close();
    loop_.runInLoop([]() {});
    poller_.stop();
    cpu_->join();
    loop_.runInLoop([]() {});
  }
  OnDemandLoop loop_;
  Poller poller_;
  bool closed_ = false;
  std::set<std::weak_ptr<ChannelImpl>, std::owner_less<std::weak_ptr<ChannelImpl>>> channels_;

 private:
  std::shared_ptr<Context> cpu_;
  bool viable_ = false;
  std::unordered_map<Device, std::string> descriptors_;
};

void ChannelImpl::init() {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self]() {
    if (self->ctx_->closed_) return self->closeFromLoop(TPB_CREATE_ERROR(ContextClosedError));
    self->ctx_->channels_.insert(self);
  });
}

uint32_t* ChannelImpl::counterFor(int device, cudaStream_t stream) {
  auto key = std::make_pair(device, stream);
  auto it = counters_.find(key);
  if (it != counters_.end()) return it->second;
  void* p = nullptr;
  TPB_CUDA_CHECK(cudaMalloc(&p, 256));
  // Zero it for certain before the first kernel that counts on it can run (that kernel goes to
  // the user's stream, which a memset on the default stream would not be ordered with).
  if (!cudaZeroNow(p, 256, device)) throw std::runtime_error("cannot clear the arrive counter");
  counters_[key] = static_cast<uint32_t*>(p);
  return static_cast<uint32_t*>(p);
}

void ChannelImpl::chunkDone(const std::shared_ptr<Op>& op, const Error& e) {
  if (e && !op->error) op->error = e;
  if (--op->remaining == 0) {
    auto cb = std::move(op->cb);
    cb(op->error ? op->error : error_);
  }
}

void ChannelImpl::send(Buffer buffer, size_t length, TSendCallback cb) {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self, buffer, length, cb = std::move(cb)]() mutable {
    if (self->error_) return cb(self->error_);
    if (length == 0) return cb(Error::kSuccess);
    auto op = std::make_shared<Op>();
    op->cb = std::move(cb);
    op->remaining = (length + kChunkBytes - 1) / kChunkBytes;
    for (size_t off = 0; off < length; off += kChunkBytes) {
      Chunk c;
      c.op = op;
      c.len = std::min(kChunkBytes, length - off);
      if (buffer.isCuda()) {
        const CudaBuffer& b = buffer.unwrap<CudaBuffer>();
        c.cuda = true;
        c.ptr = static_cast<uint8_t*>(b.ptr) + off;
        c.device = cudaDeviceForPointerOrHint(b);
        c.stream = static_cast<cudaStream_t>(b.stream);
      } else {
        c.ptr = static_cast<uint8_t*>(buffer.unwrap<CpuBuffer>().ptr) + off;
      }
      self->sendQueue_.push_back(std::move(c));
    }
    self->pumpSend();
  });
}

void ChannelImpl::pumpSend() {
  if (error_) return;
  auto self = shared_from_this();
  try {
    // Stage: start the pack kernel of every CUDA chunk for which a slot is free, in order.
    for (auto& c : sendQueue_) {
      if (c.staged) continue;
      if (!c.cuda) {
        c.staged = c.ready = true;
        continue;
      }
      if (!sendSlots_.ensure()) throw std::runtime_error("cannot allocate pinned staging memory");
      if (sendSlots_.free.empty()) break;
      c.slot = sendSlots_.free.front();
      sendSlots_.free.pop_front();
      c.flagValue = nextFlagValue_++;
      CudaDeviceGuard g(c.device);
      kernels::PushPlan plan;
      kernels::CopyItem item;
      item.src = c.ptr;
      item.dst = sendSlots_.slot(c.slot);
      item.srcBytes = c.len;
      kernels::appendToPlan(plan, item, false);
      uint32_t* flag = const_cast<uint32_t*>(sendSlots_.flags + c.slot);
      kernels::launchPush(plan, c.stream, cudaSmCount(c.device), flag, c.flagValue, counterFor(c.device, c.stream), nullptr);
      c.staged = true;
      volatile uint32_t* hostFlag = sendSlots_.flags + c.slot;
      const uint32_t want = c.flagValue;
      ctx_->poller_.watch([hostFlag, want]() { return static_cast<int32_t>(*hostFlag - want) >= 0; },
                          [self]() { self->ctx_->loop_.deferToLoop([self]() { self->pumpSend(); }); });
    }
    // Hand over: the front chunk goes to the CPU channel once its bytes are in the slot.
    while (!sendQueue_.empty()) {
      Chunk& c = sendQueue_.front();
      if (!c.staged) break;
      if (c.cuda && !c.ready) {
        if (static_cast<int32_t>(sendSlots_.flags[c.slot] - c.flagValue) < 0) break;
        std::atomic_thread_fence(std::memory_order_acquire);
        c.ready = true;
      }
      Chunk chunk = std::move(c);
      sendQueue_.pop_front();
      if (chunk.cuda) {
        // The source is reusable once packed; the op completes when all its chunks are packed
        // (stream order) — the slot lives on until the CPU channel is done with it.
        const int slot = chunk.slot;
        inner_->send(CpuBuffer{sendSlots_.slot(slot)}, chunk.len, [self, slot](const Error& e) {
          self->ctx_->loop_.deferToLoop([self, slot, e]() {
            self->sendSlots_.free.push_back(slot);
            if (e) return self->closeFromLoop(e);
            self->pumpSend();
          });
        });
        chunkDone(chunk.op, Error::kSuccess);
      } else {
        auto op = chunk.op;
        inner_->send(CpuBuffer{chunk.ptr}, chunk.len, [self, op](const Error& e) {
          self->ctx_->loop_.deferToLoop([self, op, e]() {
            self->chunkDone(op, e);
            if (e) self->closeFromLoop(e);
          });
        });
      }
    }
  } catch (const std::exception& ex) {
    closeFromLoop(TPB_CREATE_ERROR(CudaError, ex.what()));
  }
}

void ChannelImpl::recv(Buffer buffer, size_t length, TRecvCallback cb) {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self, buffer, length, cb = std::move(cb)]() mutable {
    if (self->error_) return cb(self->error_);
    if (length == 0) return cb(Error::kSuccess);
    auto op = std::make_shared<Op>();
    op->cb = std::move(cb);
    op->remaining = (length + kChunkBytes - 1) / kChunkBytes;
    for (size_t off = 0; off < length; off += kChunkBytes) {
      Chunk c;
      c.op = op;
      c.len = std::min(kChunkBytes, length - off);
      if (buffer.isCuda()) {
        const CudaBuffer& b = buffer.unwrap<CudaBuffer>();
        c.cuda = true;
        c.ptr = static_cast<uint8_t*>(b.ptr) + off;
        c.device = cudaDeviceForPointerOrHint(b);
        c.stream = static_cast<cudaStream_t>(b.stream);
      } else {
        c.ptr = static_cast<uint8_t*>(buffer.unwrap<CpuBuffer>().ptr) + off;
      }
      self->recvQueue_.push_back(std::move(c));
    }
    self->pumpRecv();
  });
}

void ChannelImpl::pumpRecv() {
  if (error_) return;
  auto self = shared_from_this();
  try {
    while (!recvQueue_.empty()) {
      Chunk& front = recvQueue_.front();
      if (front.cuda) {
        if (!recvSlots_.ensure()) throw std::runtime_error("cannot allocate pinned staging memory");
        if (recvSlots_.free.empty()) break;
        front.slot = recvSlots_.free.front();
        recvSlots_.free.pop_front();
      }
      Chunk c = std::move(front);
      recvQueue_.pop_front();
      if (!c.cuda) {
        auto op = c.op;
        inner_->recv(CpuBuffer{c.ptr}, c.len, [self, op](const Error& e) {
          self->ctx_->loop_.deferToLoop([self, op, e]() {
            self->chunkDone(op, e);
            if (e) self->closeFromLoop(e);
          });
        });
        continue;
      }
      inner_->recv(CpuBuffer{recvSlots_.slot(c.slot)}, c.len, [self, c](const Error& e) {
        self->ctx_->loop_.deferToLoop([self, c, e]() {
          if (e || self->error_) {
            self->recvSlots_.free.push_back(c.slot);
            self->chunkDone(c.op, e ? e : self->error_);
            if (e) self->closeFromLoop(e);
            return;
          }
          try {
            // Unpack on the user's stream; the slot is reusable once the kernel has run.
            CudaDeviceGuard g(c.device);
            kernels::PushPlan plan;
            kernels::CopyItem item;
            item.src = self->recvSlots_.slot(c.slot);
            item.dst = c.ptr;
            item.srcBytes = c.len;
            kernels::appendToPlan(plan, item, false);
            kernels::launchPush(plan, c.stream, cudaSmCount(c.device), nullptr, 0, nullptr, nullptr);
            auto ev = std::make_shared<CudaEvent>(c.device);
            ev->record(c.stream);
            const int slot = c.slot;
            self->ctx_->poller_.watch([ev]() { return ev->query(); },
                                      [self, slot, ev]() {
                                        self->ctx_->loop_.deferToLoop([self, slot]() {
                                          self->recvSlots_.free.push_back(slot);
                                          self->pumpRecv();
                                        });
                                      });
            self->chunkDone(c.op, Error::kSuccess);  // enqueued on the stream = received
          } catch (const std::exception& ex) {
            self->chunkDone(c.op, TPB_CREATE_ERROR(CudaError, ex.what()));
            self->closeFromLoop(TPB_CREATE_ERROR(CudaError, ex.what()));
          }
        });
      });
    }
  } catch (const std::exception& ex) {
    closeFromLoop(TPB_CREATE_ERROR(CudaError, ex.what()));
  }
}

void ChannelImpl::close() {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self]() { self->closeFromLoop(TPB_CREATE_ERROR(ChannelClosedError)); });
}

void ChannelImpl::closeFromLoop(const Error& e) {
  if (error_) return;
  error_ = e;
  inner_->close();
  ctx_->channels_.erase(weak_from_this());
  auto sends = std::move(sendQueue_);
  auto recvs = std::move(recvQueue_);
  sendQueue_.clear();
  recvQueue_.clear();
  for (auto& c : sends) chunkDone(c.op, error_);
  for (auto& c : recvs) chunkDone(c.op, error_);
}

}  // namespace

std::shared_ptr<Context> create(std::shared_ptr<Context> cpuContext) {
  if (!cpuContext || !cpuContext->isViable()) return std::make_shared<NonViableContext>();
  auto ctx = std::make_shared<ContextImpl>(std::move(cpuContext));
  if (!ctx->isViable()) return std::make_shared<NonViableContext>();
  return ctx;
}

}  // namespace cuda_basic
}  // namespace channel
}  // namespace tpb
