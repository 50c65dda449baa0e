// cuda_gdr: GPU memory to GPU memory across hosts, moved by the NICs (GPUDirect RDMA). No byte of
// a tensor touches host memory or an SM on either side.
//
//  * Each GPU works with the NIC nearest to it in the PCIe tree (matchGpusToNics).
//  * Rendezvous: the receiver waits until its stream has reached the point of the recv (its buffer
//    is free to be overwritten), registers the buffer's allocation with its NIC (once: the
//    registration is cached by the driver's buffer id) and tells the sender address, key and NIC
//    in a RecvReady. The sender waits for its own stream likewise, then posts RDMA writes from the
//    registered source straight into the receiver's buffer, in pieces of at most the NIC's
//    message size, a bounded number of bytes at a time. Every write carries an immediate: the
//    batch's sequence number and whether it is the last piece.
//  * Completion: the sender's callback fires when the NIC has reported every piece done; the
//    receiver's when the last piece's immediate arrives (a reliable connection delivers in order)
//    and the GPU has been told to make the NIC's writes visible.
//  * Lanes: a queue pair per (sending NIC, receiving NIC) pair in use, opened on first use with an
//    OpenLane / LaneOpened exchange on the channel's control connection. Control frames are
//    ordered, so a RecvReady never overtakes the opening of the lane it will be served on.
//  * One polling thread per context watches the NICs' completion queues and the CUDA events.
//
// Same job as tensorpipe/channel/cuda_gdr/* (channel_impl.cc:50-170,506-556, context_impl.cc:
// 112-208,412-442,609-640: NIC matching by sysfs path, registration cache keyed by buffer id,
// event polling before posting). That design posts sends into posted receives over a full
// NIC x NIC matrix of queue pairs made at channel creation; this one writes into the announced
// buffer over lanes made on demand. The descriptor differs accordingly ("tpbgdr1:*").
#include "channel/cuda_gdr/cuda_gdr.h"

#include <unistd.h>

#include <deque>
#include <list>
#include <map>
#include <unordered_map>
#include <unordered_set>
#include <variant>

#include "common/busy_polling_loop.h"
#include "common/cuda.h"
#include "common/defs.h"
#include "common/nop.h"
#include "transport/nop_io.h"

namespace tpb {
namespace channel {
namespace cuda_gdr {

std::vector<int> matchGpusToNics(const std::vector<std::string>& gpus, const std::vector<std::string>& nics) {
  auto components = [](const std::string& path) {
    std::vector<std::string> parts;
    size_t i = 0;
    while (i < path.size()) {
      size_t j = path.find('/', i);
      if (j == std::string::npos) j = path.size();
      if (j > i) parts.push_back(path.substr(i, j - i));
      i = j + 1;
    }
    return parts;
  };
  std::vector<std::vector<std::string>> nicParts;
  for (auto& n : nics) nicParts.push_back(components(n));
  std::vector<int> out(gpus.size(), -1);
  if (nics.empty()) return out;
  size_t orphans = 0;
  for (size_t g = 0; g < gpus.size(); ++g) {
    const auto gp = components(gpus[g]);
    size_t best = 0;
    int pick = -1;
    for (size_t n = 0; n < nicParts.size(); ++n) {
      size_t common = 0;
      while (common < gp.size() && common < nicParts[n].size() && gp[common] == nicParts[n][common]) ++common;
      // "/sys/devices" is common to everything; a PCI root or deeper is a real relation.
      if (common > best && common > 2) {
        best = common;
        pick = static_cast<int>(n);
      }
    }
    out[g] = pick >= 0 ? pick : static_cast<int>(orphans++ % nics.size());
  }
  return out;
}

namespace {

const std::string kDescriptor = "tpbgdr1:*";
constexpr int kReceiveDepth = 1024;
constexpr int kSendDepth = 1024;
constexpr int kCompletionDepth = 4096;
constexpr int kPollBatch = 32;

struct AddressWire {
  uint32_t localId = 0;
  std::string gid;
  uint32_t queuePair = 0;
  uint32_t mtu = 0;
  TPB_NOP_STRUCTURE(AddressWire, localId, gid, queuePair, mtu)
  static AddressWire from(const verbs::Address& a) {
    AddressWire w;
    w.localId = a.localId;
    w.gid.assign(reinterpret_cast<const char*>(a.gid.data()), a.gid.size());
    w.queuePair = a.queuePair;
    w.mtu = a.mtu;
    return w;
  }
  bool to(verbs::Address& a) const {
    if (gid.size() != a.gid.size()) return false;
    a.localId = localId;
    std::memcpy(a.gid.data(), gid.data(), gid.size());
    a.queuePair = queuePair;
    a.mtu = static_cast<uint8_t>(mtu);
    return true;
  }
};
// The sender of data opens the lane (fromNic is its NIC, toNic the receiver's).
struct OpenLane {
  uint32_t fromNic = 0, toNic = 0;
  AddressWire address;
  TPB_NOP_STRUCTURE(OpenLane, fromNic, toNic, address)
};
struct LaneOpened {
  uint32_t fromNic = 0, toNic = 0;
  AddressWire address;
  std::string error;
  TPB_NOP_STRUCTURE(LaneOpened, fromNic, toNic, address, error)
};
struct RecvReady {
  uint64_t seq = 0;
  uint32_t nic = 0;
  uint64_t address = 0;
  uint32_t key = 0;
  uint64_t length = 0;
  TPB_NOP_STRUCTURE(RecvReady, seq, nic, address, key, length)
};
using Packet = std::variant<OpenLane, LaneOpened, RecvReady>;

// Immediates: the low bit says "last piece", the rest is the batch's sequence number.
uint32_t makeImmediate(uint64_t seq, bool last) { return static_cast<uint32_t>((seq << 1) | (last ? 1 : 0)); }

class ContextImpl;
class ChannelImpl;

// One NIC as the context uses it.
struct Nic {
  std::unique_ptr<verbs::Device> device;
  std::unique_ptr<verbs::CompletionQueue> cq;
  std::unique_ptr<verbs::SharedReceiveQueue> srq;
  // Registrations by the driver's id of the allocation (a freed and reallocated address gets a
  // new id, so a stale registration is never used for new memory).
  struct Registration {
    std::unique_ptr<verbs::MemoryRegion> region;
    uint8_t* base = nullptr;
    size_t size = 0;
  };
  std::map<unsigned long long, Registration> registrations;
  std::unordered_map<uint32_t, ChannelImpl*> byQueuePair;
};

struct Lane {
  std::unique_ptr<verbs::QueuePair> qp;
  int myNic = -1;
  bool open = false;      // both ends ready to send
  bool requested = false;
  uint64_t postedBytes = 0;
};

struct SendOp {
  uint64_t seq = 0;
  const uint8_t* ptr = nullptr;
  size_t length = 0;
  int device = -1;
  TSendCallback callback;
  bool streamReached = false;
  std::optional<RecvReady> ready;
  uint64_t posted = 0, completed = 0;
  uint32_t localKey = 0;
  bool keyed = false;
};

struct RecvOp {
  uint64_t seq = 0;
  uint8_t* ptr = nullptr;
  size_t length = 0;
  int device = -1;
  TRecvCallback callback;
};

class ChannelImpl final : public Channel, public std::enable_shared_from_this<ChannelImpl> {
 public:
  ChannelImpl(std::shared_ptr<ContextImpl> ctx, std::shared_ptr<transport::Connection> conn)
      : ctx_(std::move(ctx)), conn_(std::move(conn)) {}
  void init();
  void send(Buffer buffer, size_t length, TSendCallback cb) override;
  void recv(Buffer buffer, size_t length, TRecvCallback cb) override;
  void setId(std::string id) override { conn_->setId(id + ".ctl"); }
  void close() override;
  void closeFromLoop(const Error& e);
  void onCompletion(int nic, const verbs::Completion& c);

 private:
  void armRead();
  void onPacket(Packet p);
  void pumpSends();
  Lane* laneFor(int myNic, uint32_t peerNic, bool asSender);
  bool registered(int nic, int device, const void* ptr, size_t length, uint32_t* localKey, uint32_t* remoteKey,
                  std::string* why);
  void write(const Packet& p);

  std::shared_ptr<ContextImpl> ctx_;
  std::shared_ptr<transport::Connection> conn_;
  Error error_;
  uint64_t nextSendSeq_ = 0, nextRecvSeq_ = 0;
  std::deque<SendOp> sends_;
  std::map<uint64_t, RecvOp> recvs_;             // announced, waiting for the last piece
  std::map<uint64_t, RecvReady> earlyReady_;     // RecvReady that came before its send()
  // (my NIC, peer's NIC) -> lane; separate maps for the two directions of data.
  std::map<std::pair<int, uint32_t>, Lane> sendLanes_, recvLanes_;
};

class ContextImpl final : public Context, public BusyPollingLoop, public std::enable_shared_from_this<ContextImpl> {
 public:
  ContextImpl(std::shared_ptr<verbs::Provider> provider, Options options) : options_(options), provider_(std::move(provider)) {
    const int gpus = cudaDeviceCountNoThrow();
    if (gpus == 0) {
      why_ = "no CUDA device";
      return;
    }
    if (options_.requirePeerMemoryModule &&
        ::access("/sys/kernel/mm/memory_peers/nv_mem/version", F_OK) != 0 &&
        ::access("/sys/module/nvidia_peermem/version", F_OK) != 0 && ::access("/sys/module/nv_peer_mem/version", F_OK) != 0) {
      why_ = "the GPU peer-memory kernel module (nvidia-peermem) is not loaded";
      return;
    }
    auto names = provider_->deviceNames();
    if (names.empty()) {
      why_ = provider_->whyUnavailable();
      return;
    }
    std::vector<std::string> nicPaths;
    try {
      for (auto& name : names) {
        auto nic = std::make_unique<Nic>();
        nic->device = provider_->open(name);
        nic->cq = nic->device->createCompletionQueue(kCompletionDepth);
        nic->srq = nic->device->createSharedReceiveQueue(kReceiveDepth);
        for (int i = 0; i < kReceiveDepth; ++i) nic->srq->postReceive(0);
        nicPaths.push_back(nic->device->pciPath());
        nics_.push_back(std::move(nic));
      }
    } catch (const std::exception& ex) {
      why_ = ex.what();
      nics_.clear();
      return;
    }
    std::vector<std::string> gpuPaths;
    for (int g = 0; g < gpus; ++g) {
      char busId[32] = {};
      std::string path;
      if (cudaDeviceGetPCIBusId(busId, sizeof(busId), g) == cudaSuccess) {
        std::string id(busId);
        for (auto& ch : id) ch = static_cast<char>(::tolower(ch));
        char* real = ::realpath(("/sys/bus/pci/devices/" + id).c_str(), nullptr);
        if (real) {
          path = real;
          ::free(real);
        }
      } else {
        cudaGetLastError();
      }
      gpuPaths.push_back(path);
      descriptors_[Device(kCudaDeviceType, g)] = kDescriptor;
    }
    nicOfGpu_ = matchGpusToNics(gpuPaths, nicPaths);
    for (int g = 0; g < gpus; ++g)
      TPB_VLOG(5) << "cuda_gdr: GPU " << g << " works with NIC " << nics_[nicOfGpu_[g]]->device->name();
    viable_ = true;
    startThread("TPB_CUDA_GDR_loop");
  }
  ~ContextImpl() override { BusyPollingLoop::join(); }

  bool isViable() const override { return viable_; }
  const std::string& why() const { return why_; }
  const std::unordered_map<Device, std::string>& deviceDescriptors() const override { return descriptors_; }
  std::shared_ptr<Channel> createChannel(std::vector<std::shared_ptr<transport::Connection>> conns, Endpoint) override {
    TPB_THROW_ASSERT_IF(!viable_, "cuda_gdr is not viable here");
    TPB_THROW_ASSERT_IF(conns.size() != 1, "cuda_gdr takes one connection");
    auto ch = std::make_shared<ChannelImpl>(shared_from_this(), std::move(conns[0]));
    ch->init();
    return ch;
  }
  void setId(std::string) override {}
  void close() override {
    if (!viable_) return;
    auto self = shared_from_this();
    deferToLoop([self]() {
      if (self->closed_) return;
      self->closed_ = true;
      auto chans = self->channels_;
      for (auto& c : chans) c->closeFromLoop(TPB_CREATE_ERROR(ContextClosedError));
      self->BusyPollingLoop::close();
    });
  }
  void join() override {
    close();
    if (viable_) BusyPollingLoop::join();
  }

  const Options& options() const { return options_; }
  bool closed() const { return closed_; }
  Nic& nic(int i) { return *nics_[i]; }
  int numNics() const { return static_cast<int>(nics_.size()); }
  int nicOfGpu(int gpu) const { return gpu >= 0 && gpu < static_cast<int>(nicOfGpu_.size()) ? nicOfGpu_[gpu] : 0; }
  void enroll(std::shared_ptr<ChannelImpl> c) { channels_.insert(std::move(c)); }
  void unenroll(const std::shared_ptr<ChannelImpl>& c) { channels_.erase(c); }

  // Runs `fn` on the loop once `stream` has got past everything queued on it so far.
  void whenStreamReaches(int device, cudaStream_t stream, std::function<void(const Error&)> fn) {
    try {
      auto ev = std::make_unique<CudaEvent>(device);
      ev->record(stream);
      events_.push_back({std::move(ev), std::move(fn)});
    } catch (const std::exception& ex) {
      fn(TPB_CREATE_ERROR(CudaError, ex.what()));
    }
  }

 protected:
  bool pollOnce() override {
    bool worked = false;
    for (size_t n = 0; n < nics_.size(); ++n) {
      verbs::Completion batch[kPollBatch];
      int got = 0;
      try {
        got = nics_[n]->cq->poll(batch, kPollBatch);
      } catch (const std::exception& ex) {
        TPB_LOG_ERROR << "cuda_gdr: " << ex.what();
        continue;
      }
      for (int i = 0; i < got; ++i) {
        const verbs::Completion& c = batch[i];
        if (c.work == verbs::Work::kWriteArrived || c.work == verbs::Work::kSendArrived) {
          try {
            nics_[n]->srq->postReceive(0);
          } catch (const std::exception& ex) {
            TPB_LOG_ERROR << "cuda_gdr: " << ex.what();
          }
        }
        auto it = nics_[n]->byQueuePair.find(c.queuePair);
        if (it != nics_[n]->byQueuePair.end()) it->second->onCompletion(static_cast<int>(n), c);
      }
      worked = worked || got > 0;
    }
    for (auto it = events_.begin(); it != events_.end();) {
      cudaError_t rc = cudaEventQuery(it->event->raw());
      if (rc == cudaErrorNotReady) {
        ++it;
        continue;
      }
      auto fn = std::move(it->fn);
      it = events_.erase(it);
      worked = true;
      if (rc != cudaSuccess) {
        cudaGetLastError();
        fn(TPB_CREATE_ERROR(CudaError, cudaGetErrorString(rc)));
      } else {
        fn(Error::kSuccess);
      }
    }
    return worked;
  }
  bool readyToClose() override { return channels_.empty() && events_.empty(); }

 private:
  struct Watched {
    std::unique_ptr<CudaEvent> event;
    std::function<void(const Error&)> fn;
  };
  Options options_;
  std::shared_ptr<verbs::Provider> provider_;
  std::vector<std::unique_ptr<Nic>> nics_;
  std::vector<int> nicOfGpu_;
  std::unordered_map<Device, std::string> descriptors_;
  std::unordered_set<std::shared_ptr<ChannelImpl>> channels_;
  std::list<Watched> events_;
  bool viable_ = false;
  bool closed_ = false;
  std::string why_;
};

// ---- channel ----------------------------------------------------------------------------------
void ChannelImpl::init() {
  auto self = shared_from_this();
  ctx_->deferToLoop([self]() {
    self->ctx_->enroll(self);
    if (self->ctx_->closed()) return self->closeFromLoop(TPB_CREATE_ERROR(ContextClosedError));
    self->armRead();
  });
}

void ChannelImpl::armRead() {
  auto self = shared_from_this();
  transport::readNop<Packet>(*conn_, [self](const Error& e, Packet p) {
    self->ctx_->deferToLoop([self, e, p = std::move(p)]() mutable {
      if (self->error_) return;
      if (e) return self->closeFromLoop(e);
      self->onPacket(std::move(p));
      if (!self->error_) self->armRead();
    });
  });
}

void ChannelImpl::write(const Packet& p) {
  auto self = shared_from_this();
  transport::writeNop(*conn_, p, [self](const Error& e) {
    if (e) self->ctx_->deferToLoop([self, e]() { self->closeFromLoop(e); });
  });
}

void ChannelImpl::send(Buffer buffer, size_t length, TSendCallback cb) {
  auto self = shared_from_this();
  const CudaBuffer cb_ = buffer.unwrap<CudaBuffer>();
  ctx_->deferToLoop([self, cb_, length, cb = std::move(cb)]() mutable {
    if (self->error_) return cb(self->error_);
    const uint64_t seq = self->nextSendSeq_++;
    if (length == 0) return cb(Error::kSuccess);  // nothing travels; the peer skips it as well
    SendOp op;
    op.seq = seq;
    op.ptr = static_cast<const uint8_t*>(cb_.ptr);
    op.length = length;
    op.device = cudaDeviceForPointerOrHint(cb_);
    op.callback = std::move(cb);
    auto early = self->earlyReady_.find(seq);
    if (early != self->earlyReady_.end()) {
      op.ready = std::move(early->second);
      self->earlyReady_.erase(early);
    }
    self->sends_.push_back(std::move(op));
    // The NIC reads the source once the stream has produced it.
    self->ctx_->whenStreamReaches(self->sends_.back().device, static_cast<cudaStream_t>(cb_.stream), [self, seq](const Error& e) {
      if (self->error_) return;
      if (e) return self->closeFromLoop(e);
      for (auto& s : self->sends_)
        if (s.seq == seq) s.streamReached = true;
      self->pumpSends();
    });
  });
}

void ChannelImpl::recv(Buffer buffer, size_t length, TRecvCallback cb) {
  auto self = shared_from_this();
  const CudaBuffer cb_ = buffer.unwrap<CudaBuffer>();
  ctx_->deferToLoop([self, cb_, length, cb = std::move(cb)]() mutable {
    if (self->error_) return cb(self->error_);
    const uint64_t seq = self->nextRecvSeq_++;
    if (length == 0) return cb(Error::kSuccess);
    RecvOp op;
    op.seq = seq;
    op.ptr = static_cast<uint8_t*>(cb_.ptr);
    op.length = length;
    op.device = cudaDeviceForPointerOrHint(cb_);
    op.callback = std::move(cb);
    const int device = op.device;
    self->recvs_.emplace(seq, std::move(op));
    // The NIC may overwrite the buffer once the stream is done with what it held before.
    self->ctx_->whenStreamReaches(device, static_cast<cudaStream_t>(cb_.stream), [self, seq](const Error& e) {
      if (self->error_) return;
      if (e) return self->closeFromLoop(e);
      auto it = self->recvs_.find(seq);
      if (it == self->recvs_.end()) return;
      RecvOp& op = it->second;
      const int nic = self->ctx_->nicOfGpu(op.device);
      uint32_t localKey = 0, remoteKey = 0;
      std::string why;
      if (!self->registered(nic, op.device, op.ptr, op.length, &localKey, &remoteKey, &why))
        return self->closeFromLoop(TPB_CREATE_ERROR(IbvError, why));
      RecvReady r;
      r.seq = seq;
      r.nic = static_cast<uint32_t>(nic);
      r.address = reinterpret_cast<uint64_t>(op.ptr);
      r.key = remoteKey;
      r.length = op.length;
      self->write(r);
    });
  });
}

// Makes sure the allocation around [ptr, ptr + length) is registered with `nic`; gives its keys.
bool ChannelImpl::registered(int nicIndex, int device, const void* ptr, size_t length, uint32_t* localKey,
                             uint32_t* remoteKey, std::string* why) {
  Nic& nic = ctx_->nic(nicIndex);
  CudaDeviceGuard onDevice(device);  // the driver answers questions about memory of the current context
  void* base = nullptr;
  size_t size = 0;
  unsigned long long id = 0;
  if (!cudaAllocationInfo(ptr, &base, &size, &id)) {
    *why = "cannot find the allocation behind a tensor";
    return false;
  }
  auto it = nic.registrations.find(id);
  if (it == nic.registrations.end()) {
    try {
      Nic::Registration r;
      r.region = nic.device->registerMemory(base, size);
      r.base = static_cast<uint8_t*>(base);
      r.size = size;
      it = nic.registrations.emplace(id, std::move(r)).first;
      TPB_VLOG(6) << "cuda_gdr: registered " << size << " bytes of GPU memory with " << nic.device->name();
    } catch (const std::exception& ex) {
      *why = ex.what();
      return false;
    }
  }
  const uint8_t* p = static_cast<const uint8_t*>(ptr);
  if (p < it->second.base || length > it->second.size || static_cast<size_t>(p - it->second.base) > it->second.size - length) {
    *why = "a tensor reaches outside its allocation";
    return false;
  }
  *localKey = it->second.region->localKey();
  *remoteKey = it->second.region->remoteKey();
  return true;
}

Lane* ChannelImpl::laneFor(int myNic, uint32_t peerNic, bool asSender) {
  auto& lanes = asSender ? sendLanes_ : recvLanes_;
  auto key = std::make_pair(myNic, peerNic);
  auto it = lanes.find(key);
  if (it != lanes.end()) return &it->second;
  Nic& nic = ctx_->nic(myNic);
  Lane lane;
  lane.myNic = myNic;
  lane.qp = nic.device->createQueuePair(*nic.cq, *nic.srq, kSendDepth);
  lane.qp->toInit();
  nic.byQueuePair[lane.qp->number()] = this;
  return &lanes.emplace(key, std::move(lane)).first->second;
}

void ChannelImpl::onPacket(Packet p) {
  try {
    if (std::holds_alternative<RecvReady>(p)) {
      RecvReady& r = std::get<RecvReady>(p);
      bool matched = false;
      for (auto& s : sends_)
        if (s.seq == r.seq) {
          s.ready = std::move(r);
          matched = true;
          break;
        }
      if (!matched) {
        if (r.seq < nextSendSeq_) return closeFromLoop(TPB_CREATE_ERROR(LogicError, "the peer announced a buffer for a batch that is over"));
        earlyReady_.emplace(r.seq, std::move(r));
      }
      pumpSends();
    } else if (std::holds_alternative<OpenLane>(p)) {
      // The peer will send over (its NIC fromNic -> my NIC toNic): make my end and answer.
      const OpenLane& o = std::get<OpenLane>(p);
      LaneOpened answer;
      answer.fromNic = o.fromNic;
      answer.toNic = o.toNic;
      verbs::Address remote;
      if (o.toNic >= static_cast<uint32_t>(ctx_->numNics()) || !o.address.to(remote))
        return closeFromLoop(TPB_CREATE_ERROR(LogicError, "the peer asked for a lane to a NIC this end does not have"));
      Lane* lane = laneFor(static_cast<int>(o.toNic), o.fromNic, false);
      lane->qp->toReadyToReceive(remote);
      lane->qp->toReadyToSend(0);
      lane->open = true;
      verbs::Address mine = ctx_->nic(static_cast<int>(o.toNic)).device->portAddress();
      mine.queuePair = lane->qp->number();
      answer.address = AddressWire::from(mine);
      write(answer);
    } else {
      const LaneOpened& o = std::get<LaneOpened>(p);
      if (!o.error.empty()) return closeFromLoop(TPB_CREATE_ERROR(IbvError, o.error));
      auto it = sendLanes_.find({static_cast<int>(o.fromNic), o.toNic});
      verbs::Address remote;
      if (it == sendLanes_.end() || it->second.open || !o.address.to(remote))
        return closeFromLoop(TPB_CREATE_ERROR(LogicError, "the peer opened a lane nobody asked for"));
      it->second.qp->toReadyToReceive(remote);
      it->second.qp->toReadyToSend(0);
      it->second.open = true;
      pumpSends();
    }
  } catch (const std::exception& ex) {
    closeFromLoop(TPB_CREATE_ERROR(IbvError, ex.what()));
  }
}

// Posts what can be posted: batches in order per lane, a bounded number of bytes per lane.
void ChannelImpl::pumpSends() {
  if (error_) return;
  try {
    for (auto& op : sends_) {
      if (!op.streamReached || !op.ready) continue;
      if (op.posted == op.length) continue;
      const RecvReady& r = *op.ready;
      if (r.length != op.length) return closeFromLoop(TPB_CREATE_ERROR(LogicError, "the receiver's buffer size does not match the tensor"));
      const int myNic = ctx_->nicOfGpu(op.device);
      Lane* lane = laneFor(myNic, r.nic, true);
      if (!lane->open) {
        if (!lane->requested) {
          lane->requested = true;
          OpenLane o;
          o.fromNic = static_cast<uint32_t>(myNic);
          o.toNic = r.nic;
          verbs::Address mine = ctx_->nic(myNic).device->portAddress();
          mine.queuePair = lane->qp->number();
          o.address = AddressWire::from(mine);
          write(o);
        }
        continue;
      }
      if (!op.keyed) {
        uint32_t remoteKey = 0;
        std::string why;
        if (!registered(myNic, op.device, op.ptr, op.length, &op.localKey, &remoteKey, &why))
          return closeFromLoop(TPB_CREATE_ERROR(IbvError, why));
        op.keyed = true;
      }
      const uint64_t piece = ctx_->nic(myNic).device->maxMessageBytes();
      while (op.posted < op.length && lane->postedBytes < ctx_->options().maxPostedBytes) {
        const uint64_t n = std::min<uint64_t>(piece, op.length - op.posted);
        const bool last = op.posted + n == op.length;
        // The id carries the sequence number (its low half) and the piece's length: a send-side
        // completion reports no byte count of its own.
        lane->qp->postWriteWithImmediate((op.seq << 32) | n, op.ptr + op.posted, static_cast<uint32_t>(n), op.localKey,
                                         r.address + op.posted, r.key, makeImmediate(op.seq, last));
        op.posted += n;
        lane->postedBytes += n;
      }
    }
  } catch (const std::exception& ex) {
    closeFromLoop(TPB_CREATE_ERROR(IbvError, ex.what()));
  }
}

void ChannelImpl::onCompletion(int nicIndex, const verbs::Completion& c) {
  if (error_) return;
  if (!c.ok) return closeFromLoop(TPB_CREATE_ERROR(IbvError, c.error));
  if (c.work == verbs::Work::kWrite) {
    const uint64_t bytes = c.id & 0xffffffffull, seqLow = c.id >> 32;
    for (auto& kv : sendLanes_)
      if (kv.second.qp && kv.second.qp->number() == c.queuePair) kv.second.postedBytes -= std::min<uint64_t>(kv.second.postedBytes, bytes);
    for (auto it = sends_.begin(); it != sends_.end(); ++it) {
      if ((it->seq & 0xffffffffull) != seqLow) continue;
      it->completed += bytes;
      if (it->completed == it->length) {
        auto cb = std::move(it->callback);
        sends_.erase(it);
        cb(Error::kSuccess);
      }
      break;
    }
    if (!error_) pumpSends();
    return;
  }
  if (c.work == verbs::Work::kWriteArrived) {
    if ((c.immediate & 1) == 0) return;  // not the last piece of its batch
    // Sequence numbers travel modulo 2^31; the oldest announced batch with those low bits is meant.
    const uint32_t low = c.immediate >> 1;
    for (auto it = recvs_.begin(); it != recvs_.end(); ++it) {
      if ((static_cast<uint32_t>(it->first) & 0x7fffffffu) != low) continue;
      RecvOp op = std::move(it->second);
      recvs_.erase(it);
      {
        // What the NIC wrote must be visible to work queued on the GPU from now on.
        CudaDeviceGuard g(op.device);
        if (cudaDeviceFlushGPUDirectRDMAWrites(cudaFlushGPUDirectRDMAWritesTargetCurrentDevice,
                                               cudaFlushGPUDirectRDMAWritesToOwner) != cudaSuccess)
          cudaGetLastError();  // not supported where such writes are ordered anyway
      }
      op.callback(Error::kSuccess);
      return;
    }
    closeFromLoop(TPB_CREATE_ERROR(LogicError, "data arrived for a batch nobody is receiving"));
  }
}

void ChannelImpl::close() {
  auto self = shared_from_this();
  ctx_->deferToLoop([self]() { self->closeFromLoop(TPB_CREATE_ERROR(ChannelClosedError)); });
}

void ChannelImpl::closeFromLoop(const Error& e) {
  if (error_) return;
  error_ = e;
  TPB_VLOG(5) << "cuda_gdr channel closes: " << e.what();
  // The queue pairs go first: once they are in the error state no NIC reads a source or writes a
  // destination of this channel any more, and only then are the users told (and free to release
  // the memory).
  for (auto* lanes : {&sendLanes_, &recvLanes_})
    for (auto& kv : *lanes) {
      if (!kv.second.qp) continue;
      try {
        kv.second.qp->toError();
      } catch (...) {
      }
      ctx_->nic(kv.second.myNic).byQueuePair.erase(kv.second.qp->number());
      kv.second.qp.reset();
    }
  conn_->close();
  auto sends = std::move(sends_);
  auto recvs = std::move(recvs_);
  sends_.clear();
  recvs_.clear();
  for (auto& s : sends) s.callback(e);
  for (auto& r : recvs) r.second.callback(e);
  ctx_->unenroll(shared_from_this());
}

}  // namespace

std::shared_ptr<Context> createWithProvider(std::shared_ptr<verbs::Provider> provider, Options options) {
  auto ctx = std::make_shared<ContextImpl>(std::move(provider), options);
  if (!ctx->isViable()) TPB_VLOG(4) << "cuda_gdr is not viable: " << ctx->why();
  return ctx;
}

std::shared_ptr<Context> create() { return createWithProvider(verbs::systemProvider()); }

}  // namespace cuda_gdr
}  // namespace channel
}  // namespace tpb
