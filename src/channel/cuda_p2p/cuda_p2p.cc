// The CUDA device-to-device channel.
//
// One channel covers what the reference needs two for: cuda_xth (same process,
// tensorpipe/channel/cuda_xth/channel_impl.cc:40-77,147-168) and cuda_ipc (other process on the
// same host, tensorpipe/channel/cuda_ipc/channel_impl.cc:107-317,319-492). Instead of copy-engine
// memcpys through staging slots with a control round trip per 8 MiB chunk, the SENDER runs one
// persistent kernel (kernels/push.cu) that reads its own tensors and stores straight into the
// receiver's memory, for all tensors of the message at once, then publishes a flag in the
// receiver's memory.
//
// Control protocol on the channel's single connection (one nop-encoded Packet per frame); both
// endpoints number their non-empty batches independently per direction, and the k-th batch sent
// matches the k-th batch received:
//
//   rendezvous   R -> S  RecvReady{seq, where each tensor goes (raw pointer if same process, else
//                        IPC handle of the allocation + offset), requested dtypes}
//                S       launches the push on the sender's stream, fires send callbacks
//                S -> R  Launched{seq}
//                R       makes its stream wait for the flag (stream memory op, or the bounded
//                        wait kernel), fires recv callbacks
//   eager        S       (small batch, peer inbox already mapped, credits left) pushes into the
//                        peer's inbox ring at send time without waiting for the receiver
//                S -> R  Launched{seq, eager, inbox offset}
//                R       waits for the flag, unpacks inbox -> tensors (applying casts), later
//                        returns the ring space with Credit{}
//
// Which batches go eager is a rule both ends evaluate identically, so the receiver never sends a
// RecvReady for them: a batch is eager iff it is no larger than the receiver's eager threshold
// and comes after the batch whose RecvReady announced the receiver's arena for that device.
// Sends launch strictly in order, which is what makes "after" well defined on the sender. A sender
// without inbox credits waits for a Credit, which the receiver returns as soon as its unpack
// kernel has finished (a poller thread watches the event).
//
// Why the receiver only enqueues a wait after Launched arrived: a wait placed on a stream before
// the matching push exists could end up ahead of a push that the peer is itself waiting for (both
// sides using one stream for sends and receives) and dead-lock the two GPUs. With this rule every
// wait refers to a push that is already enqueued, so stream dependencies cannot form a cycle.
//
// Same process: completion is a CUDA event instead of a flag; nothing is mapped.
#include <unistd.h>

#include <array>
#include <deque>
#include <map>
#include <set>

#include <tpb/channel.h>

#include "common/cuda.h"
#include "common/trace.h"
#include "common/defs.h"
#include "common/loop.h"
#include "common/nop.h"
#include "common/poller.h"
#include "common/system.h"
#include "kernels/push.h"
#include "transport/nop_io.h"

namespace tpb {
namespace channel {
namespace cuda_p2p {

namespace {

using Handle = std::array<uint8_t, 64>;
static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");

constexpr uint32_t kFlagSlots = 256;
constexpr size_t kFlagsBytes = 4096;      // flags, then counter/status words, then the inbox
constexpr size_t kCounterOffset = 2048;   // within the first 4 KiB
constexpr size_t kStatusOffset = 2304;
constexpr size_t kInboxAlign = 256;

struct DeviceDescriptor {
  std::string bootId;
  int64_t pid = 0;
  std::string uuid;
  TPB_NOP_STRUCTURE(DeviceDescriptor, bootId, pid, uuid)
};

struct TargetWire {
  uint64_t ptr = 0;       // same process: the address; else: offset inside the allocation
  uint64_t bytes = 0;     // bytes the destination holds
  uint8_t dtype = 0;      // requested destination dtype (DType), 0 = as sent
  uint8_t srcDtype = 0;   // what the receiver believes the source dtype is (with a cast)
  uint8_t hasHandle = 0;
  Handle handle{};
  uint64_t bufferId = 0;
  TPB_NOP_STRUCTURE(TargetWire, ptr, bytes, dtype, srcDtype, hasHandle, handle, bufferId)
};

struct ArenaWire {
  Handle handle{};
  uint64_t inboxBytes = 0;
  uint64_t eagerThreshold = 0;  // the receiver owns the inbox, so it sets the limit
  TPB_NOP_STRUCTURE(ArenaWire, handle, inboxBytes, eagerThreshold)
};

struct RecvReady {
  uint64_t seq = 0;
  int32_t deviceIdx = 0;  // receiver-side device of this batch
  std::optional<ArenaWire> arena;
  std::vector<TargetWire> targets;
  TPB_NOP_STRUCTURE(RecvReady, seq, deviceIdx, arena, targets)
};

struct Launched {
  uint64_t seq = 0;
  uint8_t eager = 0;
  uint64_t inboxOffset = 0;
  uint64_t creditValue = 0;
  uint64_t event = 0;  // same process: cudaEvent_t recorded after the push
  std::string error;
  TPB_NOP_STRUCTURE(Launched, seq, eager, inboxOffset, creditValue, event, error)
};

struct Credit {
  int32_t deviceIdx = 0;
  uint64_t value = 0;
  TPB_NOP_STRUCTURE(Credit, deviceIdx, value)
};

// A sender that ran out of inbox space asks for credits; until then the receiver returns them
// opportunistically (whenever it handles something else) and keeps its poller thread idle.
struct CreditRequest {
  int32_t deviceIdx = 0;
  TPB_NOP_STRUCTURE(CreditRequest, deviceIdx)
};

using Packet = std::variant<RecvReady, Launched, Credit, CreditRequest>;

std::string processIdentity() {
  auto boot = getBootID();
  return (boot ? *boot : std::string("?")) + "_" + std::to_string(::getpid());
}

// ---- process-wide cache of opened IPC mappings ----------------------------------------------
class MappingCache {
 public:
  static MappingCache& get() {
    static MappingCache c;
    return c;
  }
  // Returns the local address of the peer allocation's base, opening it on first use. The
  // current device must be the one that will access it.
  void* open(const Handle& h, std::string* err) {
    std::unique_lock<std::mutex> lock(m_);
    auto it = map_.find(h);
    if (it != map_.end()) return it->second;
    cudaIpcMemHandle_t ch;
    std::memcpy(&ch, h.data(), sizeof(ch));
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, ch, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      cudaGetLastError();
      if (err) *err = std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e);
      return nullptr;
    }
    map_.emplace(h, p);
    return p;
  }

 private:
  std::mutex m_;
  std::map<Handle, void*> map_;
};

// ---- process-wide cache of exported IPC handles ---------------------------------------------
// Exporting a handle is a driver round trip per call; a message of many tensors carved out of a
// few allocations (a caching allocator's blocks) would pay it per tensor per message. Entries are
// keyed by allocation range and checked against the driver's buffer id, which is unique for the
// life of the process, so a freed and re-used address range is noticed and re-exported.
class ExportCache {
 public:
  struct Entry {
    uintptr_t base = 0;
    size_t size = 0;
    unsigned long long id = 0;
    Handle handle{};
  };
  static ExportCache& get() {
    static ExportCache c;
    return c;
  }
  // The device that owns `ptr` must be current. False if the pointer cannot be exported.
  bool lookup(const void* ptr, Entry* out) {
    const CudaLib& lib = CudaLib::get();
    if (!lib.ok) return false;
    unsigned long long id = 0;
    if (lib.cuPointerGetAttribute(&id, CudaLib::kAttrBufferId, reinterpret_cast<CUdeviceptr_t>(ptr)) != 0) return false;
    const uintptr_t a = reinterpret_cast<uintptr_t>(ptr);
    std::unique_lock<std::mutex> lock(m_);
    auto it = byBase_.upper_bound(a);
    if (it != byBase_.begin()) {
      --it;
      if (a - it->second.base < it->second.size && it->second.id == id) {
        *out = it->second;
        return true;
      }
    }
    void* base = nullptr;
    size_t size = 0;
    unsigned long long id2 = 0;
    if (!cudaAllocationInfo(ptr, &base, &size, &id2)) return false;
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, base) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    Entry e;
    e.base = reinterpret_cast<uintptr_t>(base);
    e.size = size;
    e.id = id2;
    std::memcpy(e.handle.data(), &h, sizeof(h));
    // Drop whatever used to live in this address range.
    auto first = byBase_.lower_bound(e.base);
    if (first != byBase_.begin()) {
      auto prev = std::prev(first);
      if (prev->second.base + prev->second.size > e.base) first = prev;
    }
    auto last = first;
    while (last != byBase_.end() && last->second.base < e.base + e.size) ++last;
    byBase_.erase(first, last);
    if (byBase_.size() > 8192) byBase_.clear();
    byBase_[e.base] = e;
    *out = e;
    return true;
  }

 private:
  std::mutex m_;
  std::map<uintptr_t, Entry> byBase_;
};

class ContextImpl;

struct Arena {
  int device = -1;
  uint8_t* base = nullptr;  // cudaMalloc'ed: [4 KiB flags/counter/status][inbox]
  size_t inboxBytes = 0;
  Handle handle{};
  int64_t announcedSeq = -1;  // receive batch whose RecvReady told the peer about this arena
  uint32_t* flag(uint64_t seq) const { return reinterpret_cast<uint32_t*>(base) + (seq % kFlagSlots); }
  // One arrive counter per launching stream: launches on different streams may overlap.
  uint32_t* counter(cudaStream_t s) {
    auto it = counterOf.find(s);
    if (it == counterOf.end()) {
      if (counterOf.size() >= (kStatusOffset - kCounterOffset) / 4)
        throw std::runtime_error("cuda_p2p: too many distinct streams used with one channel");
      it = counterOf.emplace(s, static_cast<uint32_t>(counterOf.size())).first;
    }
    return reinterpret_cast<uint32_t*>(base + kCounterOffset) + it->second;
  }
  std::map<cudaStream_t, uint32_t> counterOf;
  uint32_t* status() const { return reinterpret_cast<uint32_t*>(base + kStatusOffset); }
  uint8_t* inbox() const { return base + kFlagsBytes; }
};

struct PeerArena {  // the peer's arena for one of ITS devices, mapped here
  uint8_t* base = nullptr;
  size_t inboxBytes = 0;
  uint64_t head = 0, tail = 0;  // inbox ring cursors (bytes, free-running)
  int64_t announcedSeq = -1;
  uint64_t eagerThreshold = 0;
  bool creditRequested = false;
  uint32_t* flag(uint64_t seq) const { return reinterpret_cast<uint32_t*>(base) + (seq % kFlagSlots); }
  uint8_t* inbox() const { return base + kFlagsBytes; }
};

inline uint32_t flagValueFor(uint64_t seq) { return static_cast<uint32_t>(seq / kFlagSlots + 1); }

struct SendOp {
  uint64_t seq = 0;
  int srcDevice = -1;
  Device targetDevice;
  std::vector<SendItem> items;
  bool launched = false;
  std::optional<RecvReady> ready;
};

// A receive buffer that CUDA IPC cannot export (memory from a stream-ordered pool, a virtual-memory
// allocation, ...) is replaced, for the sender's eyes, by an exportable buffer of this channel; the
// receiver copies from it to the user's buffer on the user's stream once the data has landed.
struct StagingBuffer {
  uint8_t* ptr = nullptr;
  size_t bytes = 0;
  bool busy = false;                 // handed to a receive that has not been completed yet
  std::unique_ptr<CudaEvent> drained;  // recorded after the copy out of it; reusable once it has fired
};
std::atomic<uint64_t> gStagedReceives{0};

struct RecvOp {
  uint64_t seq = 0;
  int device = -1;
  std::vector<RecvItem> items;
  std::vector<std::pair<size_t, size_t>> staged;  // (item index, staging buffer index on `device`)
  bool readySent = false;
  bool expectEager = false;
  std::optional<Launched> notice;
};

class ChannelImpl final : public Channel, public std::enable_shared_from_this<ChannelImpl> {
 public:
  ChannelImpl(std::shared_ptr<ContextImpl> ctx, std::shared_ptr<transport::Connection> conn, Options opts)
      : ctx_(std::move(ctx)), conn_(std::move(conn)), opts_(opts) {}
  ~ChannelImpl() override;

  void init();
  void send(Buffer buffer, size_t length, TSendCallback cb) override {
    SendItem it;
    it.buffer = buffer;
    it.length = length;
    it.targetDevice = Device(kCudaDeviceType, -1);
    it.callback = std::move(cb);
    std::vector<SendItem> v;
    v.push_back(std::move(it));
    sendBatch(std::move(v));
  }
  void recv(Buffer buffer, size_t length, TRecvCallback cb) override {
    RecvItem it;
    it.buffer = buffer;
    it.length = length;
    it.sourceDevice = Device(kCudaDeviceType, -1);
    it.callback = std::move(cb);
    std::vector<RecvItem> v;
    v.push_back(std::move(it));
    recvBatch(std::move(v));
  }
  void sendBatch(std::vector<SendItem> items) override;
  void recvBatch(std::vector<RecvItem> items) override;
  bool supportsLayouts() const override { return true; }
  void setId(std::string id) override { id_ = std::move(id); }
  void close() override;
  void closeFromLoop(const Error& e);

 private:
  void initFromLoop();
  void armRead();
  void onPacket(Packet p);
  void onHello(const std::string& peerIdentity);
  void sendBatchFromLoop(std::vector<SendItem> items);
  void recvBatchFromLoop(std::vector<RecvItem> items);
  void pumpSends();
  bool tryLaunch(SendOp& op);
  enum class Eager { kNotEligible, kLaunched, kNoCredits };
  Eager tryEager(SendOp& op);
  uint64_t alignedTotal(const std::vector<SendItem>& items) const;
  std::unique_ptr<CudaEvent> takeEvent(int device);
  uint8_t* takeStaging(int device, size_t bytes, size_t* index);
  void watchLastCredit();
  bool creditWanted_ = false;
  void launchRendezvous(SendOp& op);
  void finishSend(SendOp& op, const Error& e);
  void sendReady(RecvOp& op);
  void completeRecv(RecvOp& op);
  void finishRecv(RecvOp& op, const Error& e);
  void returnCredits();
  void writePacket(const Packet& p);
  Arena* arenaFor(int device, Error& err);
  template <typename It>
  static std::vector<std::vector<It>> splitByDevicePair(std::vector<It>& items, bool send);

  std::shared_ptr<ContextImpl> ctx_;
  std::shared_ptr<transport::Connection> conn_;
  Options opts_;
  std::string id_ = "N/A";
  Error error_;
  bool helloDone_ = false;
  bool sameProcess_ = false;
  std::string peerIdentity_;
  uint64_t nextSendSeq_ = 0, nextRecvSeq_ = 0;
  std::deque<SendOp> sendOps_;
  std::deque<RecvOp> recvOps_;
  std::map<uint64_t, RecvReady> earlyReady_;     // RecvReady that arrived before its sendBatch
  std::map<uint64_t, Launched> earlyLaunched_;   // Launched that arrived before its recvBatch
  std::map<int, Arena> arenas_;                  // my devices
  std::map<int, PeerArena> peerArenas_;          // peer's devices
  struct PendingCredit {
    std::unique_ptr<CudaEvent> done;
    int device;
    uint64_t value;
  };
  std::deque<PendingCredit> pendingCredits_;
  // Events handed to the peer (same process) must outlive their use.
  std::deque<std::unique_ptr<CudaEvent>> eventPool_;
  std::map<int, std::vector<std::unique_ptr<CudaEvent>>> freeEvents_;  // recycled credit events
  std::map<int, std::vector<StagingBuffer>> staging_;                  // per device, kept until the channel dies
  std::vector<std::pair<uint32_t*, uint32_t>> enqueuedWaits_;  // for cancellation on error
};

class ContextImpl final : public Context, public std::enable_shared_from_this<ContextImpl> {
 public:
  explicit ContextImpl(Options opts) : opts_(opts) {
    const int n = cudaDeviceCountNoThrow();
    if (n == 0) return;
    auto boot = getBootID();
    if (!boot) return;
    for (int i = 0; i < n; ++i) {
      cudaDeviceProp prop;
      if (cudaGetDeviceProperties(&prop, i) != cudaSuccess) {
        cudaGetLastError();
        return;
      }
      if (!prop.unifiedAddressing) return;
      DeviceDescriptor d;
      d.bootId = *boot;
      d.pid = ::getpid();
      d.uuid = cudaDeviceUuid(i);
      uuids_.push_back(d.uuid);
      auto bytes = nop::encode(d);
      descriptors_[Device(kCudaDeviceType, i)] = std::string(bytes.begin(), bytes.end());
    }
    viable_ = true;
  }
  bool isViable() const override { return viable_; }
  const std::unordered_map<Device, std::string>& deviceDescriptors() const override { return descriptors_; }
  bool canCommunicateWithRemote(const std::string& local, const std::string& remote) const override {
    DeviceDescriptor l, r;
    if (!nop::decode(local.data(), local.size(), l) || !nop::decode(remote.data(), remote.size(), r)) return false;
    if (l.bootId != r.bootId) return false;
    int li = indexOf(l.uuid), ri = indexOf(r.uuid);
    if (li < 0) return false;
    if (l.uuid == r.uuid) return true;  // same GPU (two pipes, or two processes sharing it)
    if (ri >= 0) {
      int ab = 0, ba = 0;
      if (cudaDeviceCanAccessPeer(&ab, li, ri) != cudaSuccess || cudaDeviceCanAccessPeer(&ba, ri, li) != cudaSuccess) {
        cudaGetLastError();
        return false;
      }
      return ab && ba;
    }
    // The peer's GPU is hidden from this process (CUDA_VISIBLE_DEVICES): ask NVML.
    const NvmlLib& nvml = NvmlLib::get();
    return nvml.p2pOk(l.uuid, r.uuid) && nvml.p2pOk(r.uuid, l.uuid);
  }
  std::shared_ptr<Channel> createChannel(std::vector<std::shared_ptr<transport::Connection>> conns,
                                         Endpoint) override {
    TPB_THROW_ASSERT_IF(conns.size() != 1, "cuda_p2p needs exactly one connection");
    auto ch = std::make_shared<ChannelImpl>(shared_from_this(), std::move(conns[0]), opts_);
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
    close();
    loop_.runInLoop([]() {});
    poller_.stop();
    loop_.runInLoop([]() {});
  }
  Poller poller_;
  void enroll(std::weak_ptr<ChannelImpl> c) { channels_.insert(std::move(c)); }
  void unenroll(const std::weak_ptr<ChannelImpl>& c) { channels_.erase(c); }
  bool closed() const { return closed_; }
  OnDemandLoop loop_;

 private:
  int indexOf(const std::string& uuid) const {
    for (size_t i = 0; i < uuids_.size(); ++i)
      if (uuids_[i] == uuid) return static_cast<int>(i);
    return -1;
  }
  Options opts_;
  bool viable_ = false;
  bool closed_ = false;
  std::vector<std::string> uuids_;
  std::unordered_map<Device, std::string> descriptors_;
  std::set<std::weak_ptr<ChannelImpl>, std::owner_less<std::weak_ptr<ChannelImpl>>> channels_;
};

// ---- channel --------------------------------------------------------------------------------
ChannelImpl::~ChannelImpl() {
  conn_->close();
  for (auto& perDevice : staging_) {
    try {
      CudaDeviceGuard g(perDevice.first);
      for (auto& b : perDevice.second) {
        b.drained.reset();
        if (b.ptr) cudaFree(b.ptr);
      }
    } catch (...) {
    }
  }
  for (auto& a : arenas_) {
    if (a.second.base) {
      // Freeing synchronises the device; this only happens when a pipe goes away.
      try {
        CudaDeviceGuard g(a.second.device);
        cudaFree(a.second.base);
      } catch (...) {
      }
    }
  }
}

void ChannelImpl::init() {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self]() { self->initFromLoop(); });
}

void ChannelImpl::initFromLoop() {
  if (ctx_->closed()) return closeFromLoop(TPB_CREATE_ERROR(ContextClosedError));
  ctx_->enroll(weak_from_this());
  // Hello: who am I (decides between raw pointers and IPC mappings).
  auto self = shared_from_this();
  transport::writeNop(*conn_, processIdentity(), [self](const Error& e) {
    if (e) self->ctx_->loop_.deferToLoop([self, e]() { self->closeFromLoop(e); });
  });
  transport::readNop<std::string>(*conn_, [self](const Error& e, std::string peer) {
    self->ctx_->loop_.deferToLoop([self, e, peer]() {
      if (e) return self->closeFromLoop(e);
      self->onHello(peer);
    });
  });
}

void ChannelImpl::onHello(const std::string& peer) {
  if (error_) return;
  peerIdentity_ = peer;
  sameProcess_ = peer == processIdentity();
  helloDone_ = true;
  TPB_VLOG(4) << "Channel " << id_ << " peer " << peer << (sameProcess_ ? " (same process)" : " (other process)");
  armRead();
  for (size_t i = 0; i < recvOps_.size() && !error_; ++i)
    if (!recvOps_[i].readySent && !recvOps_[i].notice && !recvOps_[i].expectEager) sendReady(recvOps_[i]);
  pumpSends();
}

void ChannelImpl::armRead() {
  auto self = shared_from_this();
  transport::readNop<Packet>(*conn_, [self](const Error& e, Packet p) {
    self->ctx_->loop_.deferToLoop([self, e, p = std::move(p)]() mutable {
      if (self->error_) return;
      if (e) return self->closeFromLoop(e);
      self->onPacket(std::move(p));
      if (!self->error_) self->armRead();
    });
  });
}

void ChannelImpl::writePacket(const Packet& p) {
  auto self = shared_from_this();
  transport::writeNop(*conn_, p, [self](const Error& e) {
    if (e) self->ctx_->loop_.deferToLoop([self, e]() { self->closeFromLoop(e); });
  });
}

Arena* ChannelImpl::arenaFor(int device, Error& err) {
  auto it = arenas_.find(device);
  if (it != arenas_.end()) return &it->second;
  Arena a;
  a.device = device;
  a.inboxBytes = opts_.inboxBytes;
  CudaDeviceGuard g(device);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, kFlagsBytes + a.inboxBytes);
  // The flags and counters must read zero BEFORE the peer learns this address: a memset queued
  // on the default stream could run after the peer's first push has already set a flag.
  if (e == cudaSuccess && !cudaZeroNow(p, kFlagsBytes, device)) e = cudaErrorUnknown;
  if (e == cudaSuccess && !sameProcess_) {
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, p);
    if (e == cudaSuccess) std::memcpy(a.handle.data(), &h, sizeof(h));
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    if (p) cudaFree(p);
    err = cudaErrorToError(e, "allocating the channel arena");
    return nullptr;
  }
  a.base = static_cast<uint8_t*>(p);
  return &arenas_.emplace(device, a).first->second;
}

template <typename It>
std::vector<std::vector<It>> ChannelImpl::splitByDevicePair(std::vector<It>& items, bool send) {
  // Both ends split a batch by (source device, target device) in order of first appearance, so
  // that every sub-batch has one launching GPU and one flag.
  std::vector<std::pair<std::pair<int, int>, std::vector<It>>> groups;
  for (auto& it : items) {
    int mine = it.buffer.device().index;
    int theirs;
    if constexpr (std::is_same_v<It, SendItem>) theirs = it.targetDevice.index;
    else theirs = it.sourceDevice.index;
    std::pair<int, int> key = send ? std::make_pair(mine, theirs) : std::make_pair(theirs, mine);
    auto g = std::find_if(groups.begin(), groups.end(), [&](const auto& p) { return p.first == key; });
    if (g == groups.end()) {
      groups.emplace_back(key, std::vector<It>());
      g = groups.end() - 1;
    }
    g->second.push_back(std::move(it));
  }
  std::vector<std::vector<It>> out;
  for (auto& g : groups) out.push_back(std::move(g.second));
  return out;
}

void ChannelImpl::sendBatch(std::vector<SendItem> items) {
  auto self = shared_from_this();
  auto shared = std::make_shared<std::vector<SendItem>>(std::move(items));
  ctx_->loop_.deferToLoop([self, shared]() { self->sendBatchFromLoop(std::move(*shared)); });
}

void ChannelImpl::recvBatch(std::vector<RecvItem> items) {
  auto self = shared_from_this();
  auto shared = std::make_shared<std::vector<RecvItem>>(std::move(items));
  ctx_->loop_.deferToLoop([self, shared]() { self->recvBatchFromLoop(std::move(*shared)); });
}

void ChannelImpl::sendBatchFromLoop(std::vector<SendItem> items) {
  std::vector<SendItem> live;
  for (auto& it : items) {
    if (error_) it.callback(error_);
    else if (it.length == 0) it.callback(Error::kSuccess);  // nothing travels for an empty tensor
    else live.push_back(std::move(it));
  }
  if (live.empty()) return;
  returnCredits();
  for (auto& group : splitByDevicePair(live, true)) {
    if (error_) {
      for (auto& it : group) it.callback(error_);
      continue;
    }
    SendOp op;
    op.seq = nextSendSeq_++;
    op.srcDevice = group[0].buffer.device().index;
    op.targetDevice = group[0].targetDevice;
    op.items = std::move(group);
    auto early = earlyReady_.find(op.seq);
    if (early != earlyReady_.end()) {
      op.ready = std::move(early->second);
      earlyReady_.erase(early);
    }
    TPB_VLOG(6) << "Channel " << id_ << " send batch #" << op.seq << " (" << op.items.size() << " tensors)"
                << (op.ready ? ", receiver already announced its buffers" : "");
    sendOps_.push_back(std::move(op));
  }
  pumpSends();
}

// Sends launch strictly in order: the first batch that cannot go yet (no RecvReady, or no inbox
// credits) holds back the ones behind it.
void ChannelImpl::pumpSends() {
  while (!error_ && helloDone_ && !sendOps_.empty()) {
    SendOp& op = sendOps_.front();
    if (!op.launched && !tryLaunch(op)) break;
    if (error_ || sendOps_.empty()) break;
    sendOps_.pop_front();
  }
}

bool ChannelImpl::tryLaunch(SendOp& op) {
  try {
    if (!sameProcess_) {
      Eager e = tryEager(op);
      if (e == Eager::kLaunched) return true;
      if (e == Eager::kNoCredits) return false;
    }
    if (!op.ready) return false;
    launchRendezvous(op);
    return !error_;
  } catch (const std::exception& ex) {
    closeFromLoop(TPB_CREATE_ERROR(CudaError, ex.what()));
    return false;
  }
}

uint64_t ChannelImpl::alignedTotal(const std::vector<SendItem>& items) const {
  uint64_t total = 0;
  for (auto& it : items) total += (it.length + kInboxAlign - 1) / kInboxAlign * kInboxAlign;
  return total;
}

ChannelImpl::Eager ChannelImpl::tryEager(SendOp& op) {
  auto pa = peerArenas_.find(op.targetDevice.index);
  if (pa == peerArenas_.end()) return Eager::kNotEligible;
  PeerArena& peer = pa->second;
  const uint64_t total = alignedTotal(op.items);
  // The rule the receiver evaluates too (see the top of this file).
  if (static_cast<int64_t>(op.seq) <= peer.announcedSeq || total > peer.eagerThreshold) return Eager::kNotEligible;
  const uint64_t cap = peer.inboxBytes;
  const uint64_t pos = peer.head % cap;
  const uint64_t skip = pos + total > cap ? cap - pos : 0;
  if (peer.head + skip + total - peer.tail > cap) {
    if (!peer.creditRequested) {
      peer.creditRequested = true;
      CreditRequest req;
      req.deviceIdx = op.targetDevice.index;
      writePacket(req);
    }
    return Eager::kNoCredits;  // wait for a Credit
  }
  const uint64_t offset = (peer.head + skip) % cap;
  peer.head += skip + total;

  Error err;
  Arena* mine = arenaFor(op.srcDevice, err);
  if (!mine) {
    closeFromLoop(err);
    return Eager::kLaunched;
  }
  CudaDeviceGuard g(op.srcDevice);
  kernels::PushPlan plan;
  uint64_t cursor = offset;
  for (auto& it : op.items) {
    kernels::CopyItem c;
    c.src = it.buffer.unwrap<CudaBuffer>().ptr;
    c.dst = peer.inbox() + cursor;
    c.srcBytes = it.length;
    c.srcDtype = it.dtype;
    c.dstDtype = it.dtype;  // a requested cast is applied by the receiver's unpack
    if (it.view) {
      c.strided = true;
      c.view = *it.view;
      c.srcDtype = c.dstDtype = it.view->dtype;
    }
    kernels::appendToPlan(plan, c, opts_.useBulkCopy);
    cursor += (it.length + kInboxAlign - 1) / kInboxAlign * kInboxAlign;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(op.items[0].buffer.unwrap<CudaBuffer>().stream);
  const int ctas = opts_.maxCtas > 0 ? opts_.maxCtas : cudaSmCount(op.srcDevice);
  kernels::launchPush(plan, stream, ctas, peer.flag(op.seq), flagValueFor(op.seq), mine->counter(stream), mine->status());
  Launched l;
  l.seq = op.seq;
  l.eager = 1;
  l.inboxOffset = offset;
  l.creditValue = peer.head;
  TPB_VLOG(6) << "Channel " << id_ << " pushed batch #" << op.seq << " eagerly into the peer's inbox at " << offset;
  writePacket(l);
  finishSend(op, Error::kSuccess);
  return Eager::kLaunched;
}

void ChannelImpl::launchRendezvous(SendOp& op) {
  trace::Scope traced("cuda_p2p.launchRendezvous", op.seq);
  const RecvReady& ready = *op.ready;
  if (ready.targets.size() != op.items.size()) {
    return closeFromLoop(TPB_CREATE_ERROR(LogicError, "peer announced a different number of tensors"));
  }
  CudaDeviceGuard g(op.srcDevice);
  uint8_t* peerArenaBase = nullptr;
  if (!sameProcess_) {
    if (ready.arena) {
      std::string why;
      void* base = MappingCache::get().open(ready.arena->handle, &why);
      if (!base) return closeFromLoop(TPB_CREATE_ERROR(CudaError, why));
      PeerArena pa;
      pa.base = static_cast<uint8_t*>(base);
      pa.inboxBytes = ready.arena->inboxBytes;
      pa.eagerThreshold = std::min<uint64_t>(ready.arena->eagerThreshold, ready.arena->inboxBytes / 2);
      pa.announcedSeq = static_cast<int64_t>(ready.seq);
      peerArenas_[ready.deviceIdx] = pa;
    }
    auto it = peerArenas_.find(ready.deviceIdx);
    if (it == peerArenas_.end())
      return closeFromLoop(TPB_CREATE_ERROR(LogicError, "peer never announced its arena for that device"));
    peerArenaBase = it->second.base;
  } else if (ready.deviceIdx != op.srcDevice) {
    if (!cudaEnablePeerAccessOnce(op.srcDevice, ready.deviceIdx))
      return closeFromLoop(TPB_CREATE_ERROR(CudaError, "peer access between the two GPUs cannot be enabled"));
  }

  kernels::PushPlan plan;
  for (size_t i = 0; i < op.items.size(); ++i) {
    SendItem& it = op.items[i];
    const TargetWire& t = ready.targets[i];
    kernels::CopyItem c;
    c.src = it.buffer.unwrap<CudaBuffer>().ptr;
    if (sameProcess_) {
      c.dst = reinterpret_cast<void*>(t.ptr);
    } else {
      if (!t.hasHandle)
        return closeFromLoop(TPB_CREATE_ERROR(CudaError, "the receiver could not export its buffer over CUDA IPC"));
      std::string why;
      void* base = MappingCache::get().open(t.handle, &why);
      if (!base) return closeFromLoop(TPB_CREATE_ERROR(CudaError, why));
      c.dst = static_cast<uint8_t*>(base) + t.ptr;
    }
    c.srcBytes = it.length;
    c.srcDtype = it.view ? it.view->dtype : it.dtype;
    if (c.srcDtype == DType::kBytes && t.dtype) c.srcDtype = static_cast<DType>(t.srcDtype);
    c.dstDtype = t.dtype ? static_cast<DType>(t.dtype) : c.srcDtype;
    if (it.view) {
      c.strided = true;
      c.view = *it.view;
    }
    c.remote = ready.deviceIdx != op.srcDevice;
    if (c.dstDtype != c.srcDtype && !kernels::castSupported(c.srcDtype, c.dstDtype))
      return closeFromLoop(TPB_CREATE_ERROR(LogicError, "unsupported dtype conversion requested by the receiver"));
    if (kernels::convertedBytes(it.length, c.srcDtype, c.dstDtype) != t.bytes)
      return closeFromLoop(TPB_CREATE_ERROR(LogicError, "receiver's buffer size does not match the tensor"));
    kernels::appendToPlan(plan, c, opts_.useBulkCopy);
  }

  // Launch on the first tensor's stream; tensors on other streams are fenced in and out with events.
  cudaStream_t stream = static_cast<cudaStream_t>(op.items[0].buffer.unwrap<CudaBuffer>().stream);
  std::vector<cudaStream_t> others;
  for (auto& it : op.items) {
    cudaStream_t s = static_cast<cudaStream_t>(it.buffer.unwrap<CudaBuffer>().stream);
    if (s != stream && std::find(others.begin(), others.end(), s) == others.end()) others.push_back(s);
  }
  for (cudaStream_t s : others) {
    CudaEvent ev(op.srcDevice);
    ev.record(s);
    ev.wait(stream, op.srcDevice);
  }
  const int ctas = opts_.maxCtas > 0 ? opts_.maxCtas : cudaSmCount(op.srcDevice);
  Launched l;
  l.seq = op.seq;
  if (sameProcess_) {
    kernels::launchPush(plan, stream, ctas, nullptr, 0, nullptr, nullptr);
    auto ev = std::make_unique<CudaEvent>(op.srcDevice);
    ev->record(stream);
    l.event = reinterpret_cast<uint64_t>(ev->raw());
    for (cudaStream_t s : others) ev->wait(s, op.srcDevice);
    eventPool_.push_back(std::move(ev));
    if (eventPool_.size() > 1024) eventPool_.pop_front();  // long since consumed by the receiver
  } else {
    Error err;
    Arena* mine = arenaFor(op.srcDevice, err);
    if (!mine) return closeFromLoop(err);
    uint32_t* flag = reinterpret_cast<uint32_t*>(peerArenaBase) + (op.seq % kFlagSlots);
    kernels::launchPush(plan, stream, ctas, flag, flagValueFor(op.seq), mine->counter(stream), mine->status());
    if (!others.empty()) {
      CudaEvent ev(op.srcDevice);
      ev.record(stream);
      for (cudaStream_t s : others) ev.wait(s, op.srcDevice);
    }
  }
  TPB_VLOG(6) << "Channel " << id_ << " launched the push of batch #" << op.seq << " (" << plan.entries.size()
              << " entries, " << plan.totalBytesOut << " bytes)";
  writePacket(l);
  finishSend(op, Error::kSuccess);
}

void ChannelImpl::finishSend(SendOp& op, const Error& e) {
  op.launched = true;
  auto items = std::move(op.items);
  for (auto& it : items) it.callback(e);
}

void ChannelImpl::recvBatchFromLoop(std::vector<RecvItem> items) {
  std::vector<RecvItem> live;
  for (auto& it : items) {
    if (error_) it.callback(error_);
    else if (it.length == 0) it.callback(Error::kSuccess);
    else live.push_back(std::move(it));
  }
  if (live.empty()) return;
  returnCredits();
  for (auto& group : splitByDevicePair(live, false)) {
    if (error_) {
      for (auto& it : group) it.callback(error_);
      continue;
    }
    RecvOp op;
    op.seq = nextRecvSeq_++;
    op.device = group[0].buffer.device().index;
    op.items = std::move(group);
    auto early = earlyLaunched_.find(op.seq);
    if (early != earlyLaunched_.end()) {
      op.notice = std::move(early->second);
      earlyLaunched_.erase(early);
    }
    // Same rule as the sender's: small batches after the arena announcement arrive eagerly.
    if (!sameProcess_) {
      auto a = arenas_.find(op.device);
      uint64_t total = 0;
      for (auto& it : op.items) total += (it.length + kInboxAlign - 1) / kInboxAlign * kInboxAlign;
      const uint64_t threshold = std::min<uint64_t>(opts_.eagerThreshold, opts_.inboxBytes / 2);
      op.expectEager = a != arenas_.end() && a->second.announcedSeq >= 0 &&
          static_cast<int64_t>(op.seq) > a->second.announcedSeq && total <= threshold;
    }
    recvOps_.push_back(std::move(op));
    RecvOp& ref = recvOps_.back();
    if (ref.notice) completeRecv(ref);
    else if (helloDone_ && !ref.expectEager) sendReady(ref);
  }
  while (!recvOps_.empty() && recvOps_.front().items.empty()) recvOps_.pop_front();
}

void ChannelImpl::sendReady(RecvOp& op) {
  if (error_) return;
  trace::Scope traced("cuda_p2p.sendReady", op.seq);
  RecvReady r;
  r.seq = op.seq;
  r.deviceIdx = op.device;
  try {
    if (!sameProcess_) {
      Error err;
      Arena* a = arenaFor(op.device, err);
      if (!a) return closeFromLoop(err);
      if (a->announcedSeq < 0) {
        ArenaWire w;
        w.handle = a->handle;
        w.inboxBytes = a->inboxBytes;
        w.eagerThreshold = opts_.eagerThreshold;
        r.arena = w;
        a->announcedSeq = static_cast<int64_t>(op.seq);
      }
    }
    // The driver queries below need this device's context current on the calling thread, which
    // may be a transport thread that never touched CUDA.
    CudaDeviceGuard g(op.device);
    for (auto& it : op.items) {
      TargetWire t;
      void* ptr = it.buffer.unwrap<CudaBuffer>().ptr;
      t.dtype = it.castTo ? static_cast<uint8_t>(*it.castTo) : 0;
      t.srcDtype = static_cast<uint8_t>(it.srcDtype);
      // Bytes the destination holds; the sender checks them against what it is about to write.
      t.bytes = it.castTo ? kernels::convertedBytes(it.length, it.srcDtype, *it.castTo) : it.length;
      if (sameProcess_) {
        t.ptr = reinterpret_cast<uint64_t>(ptr);
      } else {
        ExportCache::Entry exported;
        if (ExportCache::get().lookup(ptr, &exported)) {
          t.handle = exported.handle;
          t.hasHandle = 1;
          t.bufferId = exported.id;
          t.ptr = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(ptr) - exported.base);
        } else {
          // Not exportable: let the sender write into a staging buffer of ours instead.
          size_t index = 0;
          uint8_t* stage = takeStaging(op.device, t.bytes, &index);
          if (stage && ExportCache::get().lookup(stage, &exported)) {
            t.handle = exported.handle;
            t.hasHandle = 1;
            t.bufferId = exported.id;
            t.ptr = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(stage) - exported.base);
            op.staged.emplace_back(static_cast<size_t>(&it - op.items.data()), index);
            ++gStagedReceives;
            TPB_VLOG(5) << "Channel " << id_ << " stages a tensor of batch #" << op.seq
                        << " whose buffer CUDA IPC cannot export";
          } else if (stage) {
            staging_[op.device][index].busy = false;
          }
        }
      }
      r.targets.push_back(t);
    }
  } catch (const std::exception& ex) {
    return closeFromLoop(TPB_CREATE_ERROR(CudaError, ex.what()));
  }
  op.readySent = true;
  TPB_VLOG(6) << "Channel " << id_ << " announces its buffers for receive batch #" << op.seq;
  writePacket(r);
}

void ChannelImpl::completeRecv(RecvOp& op) {
  trace::Scope traced("cuda_p2p.completeRecv", op.seq);
  const Launched& n = *op.notice;
  TPB_VLOG(6) << "Channel " << id_ << " learnt that batch #" << op.seq << " is on its way"
              << (n.eager ? " (eager)" : "") << "; making the stream wait";
  if (!n.error.empty()) return closeFromLoop(TPB_CREATE_ERROR(CudaError, n.error));
  try {
    CudaDeviceGuard g(op.device);
    cudaStream_t stream = static_cast<cudaStream_t>(op.items[0].buffer.unwrap<CudaBuffer>().stream);
    std::vector<cudaStream_t> others;
    for (auto& it : op.items) {
      cudaStream_t s = static_cast<cudaStream_t>(it.buffer.unwrap<CudaBuffer>().stream);
      if (s != stream && std::find(others.begin(), others.end(), s) == others.end()) others.push_back(s);
    }
    if (sameProcess_) {
      cudaEvent_t ev = reinterpret_cast<cudaEvent_t>(n.event);
      TPB_CUDA_CHECK(cudaStreamWaitEvent(stream, ev, 0));
      for (cudaStream_t s : others) TPB_CUDA_CHECK(cudaStreamWaitEvent(s, ev, 0));
    } else {
      Error err;
      Arena* a = arenaFor(op.device, err);
      if (!a) return closeFromLoop(err);
      uint32_t* flag = a->flag(op.seq);
      const uint32_t value = flagValueFor(op.seq);
      const CudaLib& lib = CudaLib::get();
      if (!opts_.waitWithKernel && lib.cuStreamWaitValue32) {
        int rc = lib.cuStreamWaitValue32(stream, reinterpret_cast<CUdeviceptr_t>(flag), value, CudaLib::kWaitGeq);
        if (rc != 0) return closeFromLoop(TPB_CREATE_ERROR(CudaError, "cuStreamWaitValue32: " + lib.errorString(rc)));
      } else {
        kernels::launchWaitFlag(stream, flag, value, opts_.waitTimeoutNs, a->status());
      }
      enqueuedWaits_.emplace_back(flag, value);
      if (enqueuedWaits_.size() > 64) enqueuedWaits_.erase(enqueuedWaits_.begin());
      if (n.eager) {
        // Unpack inbox -> tensors on the receiver's stream, applying the requested casts.
        kernels::PushPlan plan;
        uint64_t cursor = n.inboxOffset;
        for (auto& it : op.items) {
          kernels::CopyItem c;
          c.src = a->inbox() + cursor;
          c.dst = it.buffer.unwrap<CudaBuffer>().ptr;
          c.srcBytes = it.length;
          if (it.castTo) {
            c.srcDtype = it.srcDtype;
            c.dstDtype = *it.castTo;
          }
          kernels::appendToPlan(plan, c, opts_.useBulkCopy);
          cursor += (it.length + kInboxAlign - 1) / kInboxAlign * kInboxAlign;
        }
        const int ctas = opts_.maxCtas > 0 ? opts_.maxCtas : cudaSmCount(op.device);
        kernels::launchPush(plan, stream, ctas, nullptr, 0, nullptr, nullptr);
        PendingCredit pc;
        pc.done = takeEvent(op.device);
        pc.done->record(stream);
        pc.device = op.device;
        pc.value = n.creditValue;
        pendingCredits_.push_back(std::move(pc));
        if (creditWanted_) watchLastCredit();
      }
      if (!op.staged.empty()) {
        // The sender wrote (and converted) into our staging buffers: move the bytes to where the
        // user wants them, behind the wait that was just enqueued.
        kernels::PushPlan plan;
        auto& pool = staging_[op.device];
        for (auto& [item, index] : op.staged) {
          RecvItem& it = op.items[item];
          kernels::CopyItem c;
          c.src = pool[index].ptr;
          c.dst = it.buffer.unwrap<CudaBuffer>().ptr;
          c.srcBytes = it.castTo ? kernels::convertedBytes(it.length, it.srcDtype, *it.castTo) : it.length;
          kernels::appendToPlan(plan, c, opts_.useBulkCopy);
        }
        const int ctas = opts_.maxCtas > 0 ? opts_.maxCtas : cudaSmCount(op.device);
        kernels::launchPush(plan, stream, ctas, nullptr, 0, nullptr, nullptr);
        for (auto& [item, index] : op.staged) {
          (void)item;
          if (!pool[index].drained) pool[index].drained = std::make_unique<CudaEvent>(op.device);
          pool[index].drained->record(stream);
          pool[index].busy = false;
        }
        op.staged.clear();
      }
      if (!others.empty()) {
        CudaEvent ev(op.device);
        ev.record(stream);
        for (cudaStream_t s : others) ev.wait(s, op.device);
      }
    }
  } catch (const std::exception& ex) {
    return closeFromLoop(TPB_CREATE_ERROR(CudaError, ex.what()));
  }
  finishRecv(op, Error::kSuccess);
}

uint8_t* ChannelImpl::takeStaging(int device, size_t bytes, size_t* index) {
  constexpr size_t kGranule = 2u << 20;
  const size_t want = (std::max<size_t>(bytes, 1) + kGranule - 1) / kGranule * kGranule;
  auto& pool = staging_[device];
  for (size_t i = 0; i < pool.size(); ++i) {
    StagingBuffer& b = pool[i];
    if (b.busy || b.bytes < bytes || b.bytes > 2 * want) continue;
    if (b.drained && !b.drained->query()) continue;  // the copy out of it is still queued
    b.busy = true;
    *index = i;
    return b.ptr;
  }
  CudaDeviceGuard g(device);
  void* p = nullptr;
  if (cudaMalloc(&p, want) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  StagingBuffer b;
  b.ptr = static_cast<uint8_t*>(p);
  b.bytes = want;
  b.busy = true;
  pool.push_back(std::move(b));
  *index = pool.size() - 1;
  return pool.back().ptr;
}

void ChannelImpl::finishRecv(RecvOp& op, const Error& e) {
  auto items = std::move(op.items);
  op.items.clear();
  for (auto& it : items) it.callback(e);
}

// The sender is starved: have the poller tell us the moment the newest unpack has finished.
void ChannelImpl::watchLastCredit() {
  if (pendingCredits_.empty()) return;
  cudaEvent_t raw = pendingCredits_.back().done->raw();
  auto self = shared_from_this();
  ctx_->poller_.watch([raw]() { return cudaEventQuery(raw) != cudaErrorNotReady; },
                      [self]() { self->ctx_->loop_.deferToLoop([self]() { self->returnCredits(); }); });
}

std::unique_ptr<CudaEvent> ChannelImpl::takeEvent(int device) {
  auto& pool = freeEvents_[device];
  if (pool.empty()) return std::make_unique<CudaEvent>(device);
  auto ev = std::move(pool.back());
  pool.pop_back();
  return ev;
}

void ChannelImpl::returnCredits() {
  // Inbox space is handed back once the unpack kernel that read it has finished; this is
  // checked opportunistically whenever the channel does anything (a sender that runs out of
  // credits falls back to rendezvous, whose traffic makes us come through here again).
  uint64_t value = 0;
  int device = -1;
  while (!pendingCredits_.empty() && pendingCredits_.front().done->query()) {
    value = pendingCredits_.front().value;
    device = pendingCredits_.front().device;
    freeEvents_[device].push_back(std::move(pendingCredits_.front().done));
    pendingCredits_.pop_front();
  }
  if (device >= 0 && !error_) {
    Credit c;
    c.deviceIdx = device;
    c.value = value;
    writePacket(c);
    if (pendingCredits_.empty()) creditWanted_ = false;
  }
}

void ChannelImpl::onPacket(Packet p) {
  if (std::holds_alternative<RecvReady>(p)) {
    RecvReady& r = std::get<RecvReady>(p);
    bool matched = false;
    for (auto& op : sendOps_) {
      if (op.seq == r.seq) {
        op.ready = std::move(r);
        matched = true;
        break;
      }
    }
    if (!matched && r.seq >= nextSendSeq_) earlyReady_.emplace(r.seq, std::move(r));
    pumpSends();
  } else if (std::holds_alternative<Launched>(p)) {
    Launched& l = std::get<Launched>(p);
    for (auto& op : recvOps_) {
      if (op.seq == l.seq && !op.items.empty()) {
        op.notice = std::move(l);
        completeRecv(op);
        while (!recvOps_.empty() && recvOps_.front().items.empty()) recvOps_.pop_front();
        returnCredits();
        return;
      }
    }
    earlyLaunched_.emplace(l.seq, std::move(l));
  } else if (std::holds_alternative<Credit>(p)) {
    const Credit& c = std::get<Credit>(p);
    auto it = peerArenas_.find(c.deviceIdx);
    if (it != peerArenas_.end()) {
      if (c.value > it->second.tail) it->second.tail = c.value;
      it->second.creditRequested = false;
    }
    pumpSends();
  } else if (std::holds_alternative<CreditRequest>(p)) {
    creditWanted_ = true;
    returnCredits();
    watchLastCredit();
  }
}

void ChannelImpl::close() {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self]() { self->closeFromLoop(TPB_CREATE_ERROR(ChannelClosedError)); });
}

void ChannelImpl::closeFromLoop(const Error& e) {
  if (error_) return;
  error_ = e;
  TPB_VLOG(4) << "Channel " << id_ << " is closing: " << e.what();
  conn_->close();
  ctx_->unenroll(weak_from_this());
  // Release any stream still parked on a flag that will now never be written: write the awaited
  // value from the host so the stream drains (the error reaches the user through callbacks).
  if (!enqueuedWaits_.empty()) {
    // On a private non-blocking stream: the user's stream (possibly the legacy default stream,
    // which blocking calls would queue behind) is exactly what is stuck.
    cudaStream_t s = nullptr;
    if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) == cudaSuccess) {
      for (auto& w : enqueuedWaits_)
        cudaMemcpyAsync(w.first, &w.second, sizeof(uint32_t), cudaMemcpyHostToDevice, s);
      cudaStreamSynchronize(s);
      cudaStreamDestroy(s);
    }
    cudaGetLastError();
    enqueuedWaits_.clear();
  }
  auto sends = std::move(sendOps_);
  auto recvs = std::move(recvOps_);
  sendOps_.clear();
  recvOps_.clear();
  for (auto& op : sends)
    for (auto& it : op.items) it.callback(error_);
  for (auto& op : recvs)
    for (auto& it : op.items) it.callback(error_);
}

}  // namespace

uint64_t stagedReceives() { return gStagedReceives.load(); }

Options applyEnvironment(Options o) {
  auto num = [](const char* name, auto& field) {
    const char* s = std::getenv(name);
    if (!s || !*s) return;
    char* end = nullptr;
    const unsigned long long v = std::strtoull(s, &end, 0);
    if (end && *end == 0) field = static_cast<std::decay_t<decltype(field)>>(v);
    else TPB_LOG_WARNING << name << "=" << s << " is not a number; ignored";
  };
  num("TPB_CUDA_P2P_EAGER_THRESHOLD", o.eagerThreshold);
  num("TPB_CUDA_P2P_INBOX_BYTES", o.inboxBytes);
  num("TPB_CUDA_P2P_MAX_CTAS", o.maxCtas);
  num("TPB_CUDA_P2P_WAIT_KERNEL", o.waitWithKernel);
  num("TPB_CUDA_P2P_BULK", o.useBulkCopy);
  unsigned long long ms = o.waitTimeoutNs / 1'000'000ull;
  num("TPB_CUDA_P2P_WAIT_TIMEOUT_MS", ms);
  o.waitTimeoutNs = ms * 1'000'000ull;
  return o;
}

std::shared_ptr<Context> create(Options options) { return std::make_shared<ContextImpl>(applyEnvironment(options)); }

}  // namespace cuda_p2p
}  // namespace channel
}  // namespace tpb
