// Shared machinery of the two "receiver pulls" CPU channels:
//   xth — both endpoints are in one process; the receiver memcpy's from the sender's pointer
//         (tensorpipe/channel/xth/channel_impl.cc:30-33,101-126,260-272, context_impl.cc:84-123);
//   cma — endpoints are different processes on one host; the receiver reads the sender's memory
//         with process_vm_readv (tensorpipe/channel/cma/channel_impl.cc:30-34,
//         context_impl.cc:39-68,109-127).
// Protocol on the channel's connection (both directions share it): the sender writes
// Descriptor{pid, ptr}; the receiver, once its matching recv() exists, queues the copy on the
// context's copy thread, fires its callback and writes Done{}; the sender's callback fires when
// Done arrives. Sends and receives are matched in order, so no sequence numbers travel; the
// copies themselves may finish in any order (several worker threads, large tensors cut into
// slices that run side by side: one core copies 10-13 GB/s, the memory system several times
// that), so a receiver holds each Done back until the copies before it are through.
#pragma once

#include <atomic>
#include <cstdlib>
#include <deque>
#include <mutex>
#include <optional>
#include <set>
#include <thread>
#include <variant>

#include <tpb/channel.h>

#include "common/defs.h"
#include "common/loop.h"
#include "common/queue.h"
#include "common/nop.h"
#include "transport/nop_io.h"

namespace tpb {
namespace channel {
namespace copy {

struct DescriptorMsg {
  uint64_t pid = 0;
  uint64_t ptr = 0;
  TPB_NOP_STRUCTURE(DescriptorMsg, pid, ptr)
};
struct DoneMsg {
  uint8_t ok = 1;
  TPB_NOP_STRUCTURE(DoneMsg, ok)
};
using Packet = std::variant<DescriptorMsg, DoneMsg>;

// Does the copy; returns an error or success. Runs on the copy thread.
using CopyFn = Error (*)(uint64_t remotePid, const void* remotePtr, void* localPtr, size_t length);

class ContextImpl;

class ChannelImpl final : public Channel, public std::enable_shared_from_this<ChannelImpl> {
 public:
  ChannelImpl(std::shared_ptr<ContextImpl> ctx, std::shared_ptr<transport::Connection> conn)
      : ctx_(std::move(ctx)), conn_(std::move(conn)) {}
  ~ChannelImpl() override { conn_->close(); }
  void init();
  void send(Buffer buffer, size_t length, TSendCallback cb) override;
  void recv(Buffer buffer, size_t length, TRecvCallback cb) override;
  void setId(std::string id) override { (void)id; }
  void close() override;
  void closeFromLoop(const Error& e);

 private:
  void armRead();
  void matchRecvs();
  void onCopyDone(uint64_t seq, const Error& e);
  struct RunningCopy {
    TRecvCallback cb;
    std::optional<Error> result;  // set when the copy is through
  };
  struct PendingRecv {
    void* ptr;
    size_t length;
    TRecvCallback cb;
  };
  std::shared_ptr<ContextImpl> ctx_;
  std::shared_ptr<transport::Connection> conn_;
  Error error_;
  std::deque<TSendCallback> sendsAwaitingDone_;
  std::deque<PendingRecv> recvs_;
  std::deque<DescriptorMsg> descriptors_;
  // Copies handed to the workers, oldest first; firstCopySeq_ is the sequence number of the front.
  std::deque<RunningCopy> copies_;
  uint64_t firstCopySeq_ = 0;
};

class ContextImpl final : public Context, public std::enable_shared_from_this<ContextImpl> {
 public:
  ContextImpl(std::string descriptor, CopyFn fn, const char* threadName)
      : copyFn_(fn), threadName_(threadName) {
    descriptors_[Device(kCpuDeviceType, 0)] = std::move(descriptor);
    // TPB_COPY_THREADS: how many threads copy at once (default: half of the cores, at most 4).
    // One starts now; the others when the first tensor large enough to be sliced comes by.
    const char* env = std::getenv("TPB_COPY_THREADS");
    const unsigned cores = std::max(1u, std::thread::hardware_concurrency());
    maxThreads_ = env ? std::max<long>(1, std::strtol(env, nullptr, 10)) : std::min<size_t>(4, std::max(1u, cores / 2));
    startWorker();
  }
  ~ContextImpl() override { stopThread(); }
  bool isViable() const override { return true; }
  const std::unordered_map<Device, std::string>& deviceDescriptors() const override { return descriptors_; }
  std::shared_ptr<Channel> createChannel(std::vector<std::shared_ptr<transport::Connection>> conns, Endpoint) override {
    TPB_THROW_ASSERT_IF(conns.size() != 1, "this channel needs exactly one connection");
    auto ch = std::make_shared<ChannelImpl>(shared_from_this(), std::move(conns[0]));
    ch->init();
    return ch;
  }
  void setId(std::string id) override { (void)id; }
  void close() override {
    loop_.deferToLoop([this, self = shared_from_this()]() {
      if (closed_) return;
      closed_ = true;
      auto chans = channels_;
      for (auto& w : chans)
        if (auto c = w.lock()) c->closeFromLoop(TPB_CREATE_ERROR(ContextClosedError));
      channels_.clear();
    });
  }
  void join() override {
    if (joined_.exchange(true)) return;
    close();
    loop_.runInLoop([]() {});
    stopThread();
    loop_.runInLoop([]() {});
  }
  void stopThread() {
    std::vector<std::thread> threads;
    {
      std::lock_guard<std::mutex> lock(threadsMutex_);
      if (stopRequested_.exchange(true)) return;
      threads = std::move(threads_);
      threads_.clear();
    }
    // An empty function is the request to stop, one per worker, queued behind whatever copies
    // were requested before.
    for (size_t i = 0; i < threads.size(); ++i) jobs_->push(nullptr);
    for (auto& t : threads) {
      // The last reference to the context may die inside a job, on a worker: that worker cannot
      // wait for itself and is left to run out on its own (it only touches the job queue, which
      // it shares ownership of, and finds its request to stop there).
      if (t.get_id() == std::this_thread::get_id()) t.detach();
      else t.join();
    }
  }
  // The copy runs on the worker threads, cut into slices when it is large; `done` is deferred to
  // the loop when the last slice is through and gets the first error, if there was one.
  void requestCopy(uint64_t pid, const void* remote, void* local, size_t len, std::function<void(const Error&)> done) {
    auto self = shared_from_this();
    size_t slices = std::min<size_t>(maxThreads_, len / kSliceMinBytes);
    if (slices < 2) slices = 1;
    for (size_t i = 1; i < slices; ++i) startWorker();
    struct Whole {
      std::atomic<size_t> left;
      std::mutex mutex;
      Error firstError;
      std::function<void(const Error&)> done;
    };
    auto whole = std::make_shared<Whole>();
    whole->left = slices;
    whole->done = std::move(done);
    const size_t per = ((len + slices - 1) / slices + 4095) & ~size_t(4095);
    for (size_t i = 0; i < slices; ++i) {
      const size_t begin = std::min(len, i * per), end = std::min(len, begin + per);
      jobs_->push([self, whole, pid, remote, local, begin, end]() {
        Error e = begin < end ? self->copyFn_(pid, static_cast<const uint8_t*>(remote) + begin,
                                              static_cast<uint8_t*>(local) + begin, end - begin)
                              : Error::kSuccess;
        if (e) {
          std::lock_guard<std::mutex> lock(whole->mutex);
          if (!whole->firstError) whole->firstError = e;
        }
        if (whole->left.fetch_sub(1) == 1) {
          Error result;
          {
            std::lock_guard<std::mutex> lock(whole->mutex);
            result = whole->firstError;
          }
          self->loop_.deferToLoop([whole, result]() { whole->done(result); });
        }
      });
    }
  }
  OnDemandLoop loop_;
  bool closed_ = false;
  std::set<std::weak_ptr<ChannelImpl>, std::owner_less<std::weak_ptr<ChannelImpl>>> channels_;

 private:
  static constexpr size_t kSliceMinBytes = 512u << 10;
  void startWorker() {
    std::lock_guard<std::mutex> lock(threadsMutex_);
    if (stopRequested_ || threads_.size() >= maxThreads_) return;
    threads_.emplace_back([jobs = jobs_, name = threadName_]() {
      setThreadName(name);
      // A worker sleeps in pop(); an empty function tells it to stop.
      for (;;) {
        std::function<void()> job = jobs->pop();
        if (!job) return;
        job();
      }
    });
  }
  CopyFn copyFn_;
  const char* threadName_;
  size_t maxThreads_ = 1;
  std::unordered_map<Device, std::string> descriptors_;
  std::mutex threadsMutex_;
  std::vector<std::thread> threads_;
  // Copies wait here for the workers. The bound only matters to a caller that queues thousands
  // of tensors without waiting for any: it then blocks until the workers catch up.
  std::shared_ptr<Queue<std::function<void()>>> jobs_ = std::make_shared<Queue<std::function<void()>>>(4096);
  std::atomic<bool> stopRequested_{false};
  std::atomic<bool> joined_{false};
};

inline void ChannelImpl::init() {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self]() {
    if (self->ctx_->closed_) return self->closeFromLoop(TPB_CREATE_ERROR(ContextClosedError));
    self->ctx_->channels_.insert(self);
    self->armRead();
  });
}

inline void ChannelImpl::armRead() {
  auto self = shared_from_this();
  transport::readNop<Packet>(*conn_, [self](const Error& e, Packet p) {
    self->ctx_->loop_.deferToLoop([self, e, p]() {
      if (self->error_) return;
      if (e) return self->closeFromLoop(e);
      if (std::holds_alternative<DescriptorMsg>(p)) {
        self->descriptors_.push_back(std::get<DescriptorMsg>(p));
        self->matchRecvs();
      } else {
        if (self->sendsAwaitingDone_.empty())
          return self->closeFromLoop(TPB_CREATE_ERROR(LogicError, "unexpected completion from the peer"));
        auto cb = std::move(self->sendsAwaitingDone_.front());
        self->sendsAwaitingDone_.pop_front();
        cb(Error::kSuccess);
      }
      if (!self->error_) self->armRead();
    });
  });
}

inline void ChannelImpl::matchRecvs() {
  auto self = shared_from_this();
  while (!recvs_.empty() && !descriptors_.empty()) {
    PendingRecv r = std::move(recvs_.front());
    recvs_.pop_front();
    DescriptorMsg d = descriptors_.front();
    descriptors_.pop_front();
    const uint64_t seq = firstCopySeq_ + copies_.size();
    copies_.push_back({std::move(r.cb), std::nullopt});
    ctx_->requestCopy(d.pid, reinterpret_cast<const void*>(d.ptr), r.ptr, r.length,
                      [self, seq](const Error& e) { self->onCopyDone(seq, e); });
  }
}

// Copies may finish out of order; the peer matches Done frames to its sends by counting, so they
// (and the callbacks) go out in the order of the receives.
inline void ChannelImpl::onCopyDone(uint64_t seq, const Error& e) {
  if (seq < firstCopySeq_ || seq - firstCopySeq_ >= copies_.size()) return;
  copies_[seq - firstCopySeq_].result = e;
  auto self = shared_from_this();
  while (!copies_.empty() && copies_.front().result) {
    RunningCopy c = std::move(copies_.front());
    copies_.pop_front();
    ++firstCopySeq_;
    if (*c.result) {
      c.cb(*c.result);
      closeFromLoop(*c.result);
      continue;
    }
    if (error_) {
      c.cb(error_);
      continue;
    }
    c.cb(Error::kSuccess);
    Packet done = DoneMsg{};
    transport::writeNop(*conn_, done, [self](const Error& we) {
      if (we) self->ctx_->loop_.deferToLoop([self, we]() { self->closeFromLoop(we); });
    });
  }
}

inline void ChannelImpl::send(Buffer buffer, size_t length, TSendCallback cb) {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self, buffer, length, cb = std::move(cb)]() mutable {
    if (self->error_) return cb(self->error_);
    if (length == 0) return cb(Error::kSuccess);
    Packet p = DescriptorMsg{static_cast<uint64_t>(::getpid()),
                             reinterpret_cast<uint64_t>(buffer.unwrap<CpuBuffer>().ptr)};
    self->sendsAwaitingDone_.push_back(std::move(cb));
    transport::writeNop(*self->conn_, p, [self](const Error& we) {
      if (we) self->ctx_->loop_.deferToLoop([self, we]() { self->closeFromLoop(we); });
    });
  });
}

inline void ChannelImpl::recv(Buffer buffer, size_t length, TRecvCallback cb) {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self, buffer, length, cb = std::move(cb)]() mutable {
    if (self->error_) return cb(self->error_);
    if (length == 0) return cb(Error::kSuccess);
    self->recvs_.push_back({buffer.unwrap<CpuBuffer>().ptr, length, std::move(cb)});
    self->matchRecvs();
  });
}

inline void ChannelImpl::close() {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self]() { self->closeFromLoop(TPB_CREATE_ERROR(ChannelClosedError)); });
}

inline void ChannelImpl::closeFromLoop(const Error& e) {
  if (error_) return;
  error_ = e;
  conn_->close();
  ctx_->channels_.erase(weak_from_this());
  auto sends = std::move(sendsAwaitingDone_);
  auto recvs = std::move(recvs_);
  sendsAwaitingDone_.clear();
  recvs_.clear();
  for (auto& cb : sends) cb(error_);
  for (auto& r : recvs) r.cb(error_);
}

}  // namespace copy
}  // namespace channel
}  // namespace tpb
