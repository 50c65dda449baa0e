// The CUDA device-to-device channel.
//
// One channel covers what the reference needs two for: cuda_xth (same process,
// tensorpipe/channel/cuda_xth/channel_impl.cc:40-77,147-168) and cuda_ipc (other process on the
// same host, tensorpipe/channel/cuda_ipc/channel_impl.cc:107-317,319-492). Instead of copy-engine
// memcpys through staging slots with a control round trip per 8 MiB chunk, the SENDER runs one
// persistent kernel (kernels/push.cu) that reads its own tensors and stores straight into the
// receiver's memory, for all tensors of the message at once, then publishes a flag in the
// receiver's memory. When both ends live in one process the targets are raw pointers, completion
// is a CUDA event the receiver's stream waits for (no flag, no fence at the end of the kernel) and
// everything goes by rendezvous; between processes the targets are CUDA IPC mappings, completion is
// a flag, and small batches go eagerly.
//
// Control protocol on the channel's single connection (one nop-encoded Packet per frame). Both
// endpoints number their non-empty batches independently per direction; the k-th batch sent
// meets the k-th batch received.
//
//   eager        S       (batch no larger than the receiver's eager threshold, receiver's arena
//                        for the target device known, ring space left) pushes into the receiver's
//                        inbox ring at send time, without waiting for the receiver
//                S -> R  Launched{seq, eager, inbox offset}
//                R       after the user's read(): makes its stream wait for the flag and unpacks
//                        inbox -> tensors (applying casts); across GPUs the wait is the first
//                        step of the unpack kernel itself
//   rendezvous   R -> S  RecvReady{seq, where each tensor goes, requested dtypes}. Memory is named
//                        by region: an allocation of the receiver, exported once per channel
//                        (IPC handle + size) and referred to by a small number afterwards.
//                S       launches the push on the sender's stream, fires send callbacks
//                S -> R  Launched{seq}
//                R       makes its stream wait for the flag (stream memory operation, or the
//                        bounded wait kernel), fires recv callbacks
//   credits      S -> R  CreditRequest when the inbox ring is half used; R answers with Credit once
//                        the unpack kernels that read the ring have finished. Nothing per message.
//                        Neither end uses CUDA events for this book-keeping: the last CTA of
//                        every push and of every unpack writes the launch's number into a word of
//                        mapped host memory, which the channel simply reads.
//   closing      either  Bye = "I launch nothing more and everything I launched has finished".
//                        An end that closes fails what it can at once, but keeps the receives
//                        whose buffers it has announced until the peer's Bye (or the connection's
//                        end, or a time limit): until then a peer kernel may still be writing
//                        into them and the user must not get them back. The end that RECEIVES a
//                        Bye while it is still open can go on receiving what the peer pushed
//                        eagerly before it left (the data sits in this end's inbox); everything
//                        that would need the peer fails.
//
// Which batches go eager is a rule both ends evaluate identically, so the receiver never sends a
// RecvReady for them: a batch is eager iff it is no larger than the receiver's eager threshold
// and comes after the batch whose RecvReady announced the receiver's arena for that device.
// Sends launch strictly in order, which is what makes "after" well defined on the sender.
//
// Why the receiver only enqueues a wait after Launched arrived: a wait placed on a stream before
// the matching push exists could end up ahead of a push that the peer is itself waiting for (both
// sides using one stream for sends and receives) and dead-lock the two GPUs. With this rule every
// wait refers to a push that is already enqueued, so stream dependencies cannot form a cycle.
//
// Flags live in 256 slots per receiving device (slot = seq mod 256, value = seq / 256 + 1,
// "greater or equal" waits). A sender therefore never has more than 254 pushes unfinished, and
// never more than 254 eager batches whose unpack the receiver has not reported finished; it holds
// further launches back until the completion words say otherwise. The same bounds let arrive
// counters and completion words be handed out round-robin.
#include <unistd.h>

#include <array>
#include <chrono>
#include <deque>
#include <map>
#include <set>

#include <tpb/channel.h>

#include "common/cuda.h"
#include "common/defs.h"
#include "common/loop.h"
#include "common/nop.h"
#include "common/poller.h"
#include "common/system.h"
#include "common/timer.h"
#include "channel/cuda_p2p/mapping_cache.h"
#include "common/trace.h"
#include "kernels/push.h"
#include "transport/nop_io.h"

namespace tpb {
namespace channel {
namespace cuda_p2p {

namespace {

using Handle = std::array<uint8_t, 64>;
static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");

constexpr uint32_t kFlagSlots = 256;
constexpr uint32_t kMaxUnfinished = kFlagSlots - 2;  // pushes (and unfinished unpacks) a sender may have in flight
constexpr uint32_t kCounters = 512;                   // arrive counters per device: [0,256) pushes, [256,512) unpacks
constexpr size_t kHeaderBytes = 4096;     // [flags 1 KiB][counters 2 KiB][spare], then the inbox
constexpr size_t kCounterOffset = 1024;
constexpr size_t kHostWords = 1024;       // mapped host block of a channel: [0] status, [256,512) push completion words
constexpr size_t kInboxAlign = 256;
constexpr uint32_t kNoRegion = UINT32_MAX;  // same process: the target is a plain address
static_assert(kCounterOffset + kCounters * 4 <= kHeaderBytes, "arena header layout");
static_assert(kCounters == 2 * kFlagSlots, "one counter per unfinished push and per unfinished unpack");

struct DeviceDescriptor {
  std::string bootId;
  int64_t pid = 0;
  std::string uuid;
  TPB_NOP_STRUCTURE(DeviceDescriptor, bootId, pid, uuid)
};

struct Hello {
  std::string identity;             // boot id + pid: equal identities share an address space
  std::vector<std::string> uuids;   // UUID of each CUDA device the sender of this hello sees, by index
  TPB_NOP_STRUCTURE(Hello, identity, uuids)
};

struct RegionWire {
  uint32_t id = 0;
  Handle handle{};
  uint64_t size = 0;
  TPB_NOP_STRUCTURE(RegionWire, id, handle, size)
};

struct TargetWire {
  uint32_t region = kNoRegion;
  uint64_t offset = 0;    // inside the region; the address itself when region == kNoRegion
  uint64_t bytes = 0;     // bytes the destination holds
  uint8_t dtype = 0;      // requested destination dtype (DType), 0 = as sent
  uint8_t srcDtype = 0;   // what the receiver believes the source dtype is (with a cast)
  TPB_NOP_STRUCTURE(TargetWire, region, offset, bytes, dtype, srcDtype)
};

struct ArenaWire {
  uint64_t address = 0;  // same process
  Handle handle{};       // other process
  uint64_t inboxBytes = 0;
  uint64_t eagerThreshold = 0;  // the receiver owns the inbox, so it sets the limit
  TPB_NOP_STRUCTURE(ArenaWire, address, handle, inboxBytes, eagerThreshold)
};

struct RecvReady {
  uint64_t seq = 0;
  int32_t deviceIdx = 0;  // receiver-side device of this batch
  std::optional<ArenaWire> arena;
  std::vector<RegionWire> newRegions;
  std::vector<TargetWire> targets;
  TPB_NOP_STRUCTURE(RecvReady, seq, deviceIdx, arena, newRegions, targets)
};

struct Launched {
  uint64_t seq = 0;
  uint8_t eager = 0;
  uint64_t inboxOffset = 0;
  uint64_t creditValue = 0;
  uint64_t event = 0;  // same process: the cudaEvent_t recorded behind the push
  std::string error;
  TPB_NOP_STRUCTURE(Launched, seq, eager, inboxOffset, creditValue, event, error)
};

struct Credit {
  int32_t deviceIdx = 0;
  uint64_t value = 0;   // inbox ring cursor up to which space is free again
  uint64_t count = 0;   // eager batches of this device whose unpack has finished
  TPB_NOP_STRUCTURE(Credit, deviceIdx, value, count)
};

struct CreditRequest {
  int32_t deviceIdx = 0;
  TPB_NOP_STRUCTURE(CreditRequest, deviceIdx)
};

struct Bye {
  uint8_t reserved = 0;
  TPB_NOP_STRUCTURE(Bye, reserved)
};

using Packet = std::variant<RecvReady, Launched, Credit, CreditRequest, Bye>;

std::string processIdentity() {
  auto boot = getBootID();
  return (boot ? *boot : std::string("?")) + "_" + std::to_string(::getpid());
}

uint64_t nowNs() {
  return static_cast<uint64_t>(
      std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count());
}

size_t envNumber(const char* name, size_t fallback) {
  const char* s = std::getenv(name);
  if (!s || !*s) return fallback;
  char* end = nullptr;
  const unsigned long long v = std::strtoull(s, &end, 0);
  return end && *end == 0 ? static_cast<size_t>(v) : fallback;
}

}  // namespace

// ---- process-wide cache of opened IPC mappings ----------------------------------------------
// A mapping is opened for the device that will access it: cudaIpcOpenMemHandle with the lazy
// peer-access flag enables access only for the device that is current at the time, so the key is
// (handle, accessing device) — as the reference keys by (process, remote device, local device),
// tensorpipe/channel/cuda_ipc/context_impl.cc:388-418. An open mapping pins the exporter's memory
// (even after the exporter freed it), so the cache is bounded: beyond the limit, mappings that
// nobody used for a while are closed, oldest first.
MappingCache& MappingCache::get() {
  static MappingCache* c = new MappingCache();  // outlives every static that might still use it
  return *c;
}

MappingCache::MappingCache() : limit_(envNumber("TPB_CUDA_P2P_MAX_MAPPINGS", 512)) {}

void MappingCache::setBackendForTesting(Opener opener, Closer closer) {
  std::unique_lock<std::mutex> lock(m_);
  opener_ = std::move(opener);
  closer_ = std::move(closer);
}
void MappingCache::setLimits(size_t maxMappings, uint64_t idleNs) {
  std::unique_lock<std::mutex> lock(m_);
  limit_ = maxMappings;
  idleNs_ = idleNs;
}
size_t MappingCache::size() {
  std::unique_lock<std::mutex> lock(m_);
  return map_.size();
}
uint64_t MappingCache::closedCount() {
  std::unique_lock<std::mutex> lock(m_);
  return closed_;
}

void* MappingCache::open(const Handle& handle, int device, size_t* size, std::string* err, bool pin) {
  std::unique_lock<std::mutex> lock(m_);
  const Key key{handle, device};
  auto it = map_.find(key);
  if (it != map_.end()) {
    it->second.lastUseNs = nowNs();
    it->second.pinned = it->second.pinned || pin;
    if (size) *size = it->second.size;
    return it->second.base;
  }
  if (map_.size() >= limit_) evictIdle();
  void* p = nullptr;
  if (opener_) {
    size_t bytes = 0;
    p = opener_(handle, device, &bytes);  // tests count opens and closes without a GPU
    if (!p) {
      if (err) *err = "the mapping could not be opened";
      return nullptr;
    }
    map_.emplace(key, Entry{p, bytes, nowNs(), pin});
    if (size) *size = bytes;
    return p;
  }
  cudaIpcMemHandle_t ch;
  std::memcpy(&ch, handle.data(), sizeof(ch));
  cudaError_t e = cudaIpcOpenMemHandle(&p, ch, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    if (err) *err = std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e);
    return nullptr;
  }
  size_t bytes = 0;
  const CudaLib& lib = CudaLib::get();
  CUdeviceptr_t base = 0;
  if (lib.ok && lib.cuMemGetAddressRange(&base, &bytes, reinterpret_cast<CUdeviceptr_t>(p)) != 0) bytes = 0;
  map_.emplace(key, Entry{p, bytes, nowNs(), pin});
  if (size) *size = bytes;
  return p;
}

void MappingCache::evictIdle() {
  // Oldest first, and only what has rested for a while: a kernel launched with the mapping a
  // moment ago may still be running.
  const uint64_t now = nowNs();
  std::vector<std::pair<uint64_t, Key>> idle;
  for (auto& e : map_)
    if (!e.second.pinned && now - e.second.lastUseNs > idleNs_) idle.emplace_back(e.second.lastUseNs, e.first);
  std::sort(idle.begin(), idle.end(), [](const auto& a, const auto& b) { return a.first < b.first; });
  const size_t want = map_.size() - limit_ / 2;
  for (size_t i = 0; i < idle.size() && i < want; ++i) {
    auto it = map_.find(idle[i].second);
    if (closer_) {
      closer_(it->second.base, it->first.second);
    } else {
      try {
        CudaDeviceGuard g(it->first.second);
        cudaIpcCloseMemHandle(it->second.base);
        cudaGetLastError();
      } catch (...) {
      }
    }
    map_.erase(it);
    generation_.fetch_add(1, std::memory_order_release);
    ++closed_;
  }
}

// ---- process-wide cache of exported IPC handles ---------------------------------------------
// Exporting a handle is a driver round trip per call; a message of many tensors carved out of a
// few allocations (a caching allocator's blocks) would pay it per tensor per message. Entries are
// keyed by allocation range and checked against the driver's buffer id, which is unique for the
// life of the process, so a freed and re-used address range is noticed and re-exported.
namespace {

class ExportCache {
 public:
  struct Entry {
    uintptr_t base = 0;
    size_t size = 0;
    unsigned long long id = 0;
    Handle handle{};
    uint64_t lastUseNs = 0;
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
        it->second.lastUseNs = nowNs();
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
    e.lastUseNs = nowNs();
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
    if (byBase_.size() >= kLimit) trim();
    byBase_[e.base] = e;
    *out = e;
    return true;
  }

 private:
  static constexpr size_t kLimit = 8192;
  // Forget the half that has gone unused the longest (a forgotten entry is simply exported again).
  void trim() {
    std::vector<uint64_t> ages;
    for (auto& e : byBase_) ages.push_back(e.second.lastUseNs);
    std::nth_element(ages.begin(), ages.begin() + ages.size() / 2, ages.end());
    const uint64_t cut = ages[ages.size() / 2];
    for (auto it = byBase_.begin(); it != byBase_.end();)
      it = it->second.lastUseNs < cut ? byBase_.erase(it) : std::next(it);
  }
  std::mutex m_;
  std::map<uintptr_t, Entry> byBase_;
};

// A large tensor in pinned host memory never goes through the kernel's own loads (SM-issued reads
// over PCIe reach 40 GB/s, the copy engine 55). Bound for this GPU's memory, the copy engine puts
// it straight into the receiver's buffer. Bound for another GPU, it travels in pieces: the copy
// engine brings a piece into a slot of device memory while the push kernel sends the piece before
// it over NVLink, so the NVLink hop hides behind the PCIe copy. (One copy-engine copy from host
// memory into the peer GPU also runs at 55 GB/s alone, but measured well below the pieces when
// both GPUs of a pair do it at once.) In both cases a short tail travels with the launch that
// publishes the batch. One feed per context and sending device, shared by its channels (all of
// them work from the context's one loop thread; the slots pass from use to use by events).
constexpr uint64_t kHostTailBytes = 64u << 10;      // read by the kernel from host memory in place
constexpr uint64_t kHostLastPieceBytes = 2u << 20;  // nothing hides the push of the last piece: it is short
struct HostFeed {
  static constexpr size_t kSlots = 2;
  int device = -1;
  size_t pieceBytes = 0;
  cudaStream_t copyStream = nullptr;
  uint8_t* slots = nullptr;
  std::unique_ptr<CudaEvent> begin;
  std::unique_ptr<CudaEvent> copied[kSlots], sent[kSlots];
  bool everSent[kSlots] = {};
  uint64_t next = 0;
  // A third slot for the head start: the first piece of a host tensor is copied in as soon as the
  // batch is handed over, while the descriptor and the receiver's answer are still travelling, so
  // the PCIe copy does not wait for the handshake. One batch owns it at a time (host-side flag:
  // taken at the head start, given back when the push that reads the slot has been launched).
  uint8_t* early = nullptr;
  std::unique_ptr<CudaEvent> earlyCopied, earlySent;
  bool earlyTaken = false, earlyEverSent = false;
  ~HostFeed() {
    if (device < 0) return;
    try {
      CudaDeviceGuard g(device);
      if (copyStream) cudaStreamSynchronize(copyStream), cudaStreamDestroy(copyStream);
      if (slots) cudaFree(slots);  // the early slot is part of the same allocation
    } catch (...) {
    }
  }
};

class ContextImpl;

// This end's arena on one of its devices: flags and arrive counters, then the inbox ring.
struct Arena {
  int device = -1;
  uint8_t* base = nullptr;
  size_t inboxBytes = 0;
  Handle handle{};
  int64_t announcedSeq = -1;  // receive batch whose RecvReady told the peer about this arena
  uint32_t awaited[kFlagSlots] = {};  // per slot, the newest value a stream of ours was told to wait for
  bool anyWait = false;
  // Inbox bookkeeping (receiving side). Eager batches of this device are numbered as their
  // unpack kernels are enqueued; the last CTA of unpack k writes k + 1 into unpackDone[k mod 256].
  uint32_t* unpackDone = nullptr;       // mapped host memory, kFlagSlots words
  uint64_t unpacksQueued = 0;
  uint64_t unpacksDone = 0;
  std::deque<uint64_t> creditValues;    // ring cursor freed by each unpack in [unpacksDone, unpacksQueued)
  uint64_t freedUpTo = 0;               // ring cursor freed by the unpacks known to have finished
  uint64_t creditSent = 0;              // unpacksDone at the time of the last Credit
  bool creditWanted = false;
  bool creditWatching = false;
  uint32_t* flag(uint64_t seq) const { return reinterpret_cast<uint32_t*>(base) + (seq % kFlagSlots); }
  uint32_t* pushCounter(uint64_t seq) const {
    return reinterpret_cast<uint32_t*>(base + kCounterOffset) + (seq % kFlagSlots);
  }
  uint32_t* unpackCounter(uint64_t ordinal) const {
    return reinterpret_cast<uint32_t*>(base + kCounterOffset) + kFlagSlots + (ordinal % kFlagSlots);
  }
  uint8_t* inbox() const { return base + kHeaderBytes; }
};

// The peer's arena for one of ITS devices, as this end can address it.
struct PeerArena {
  uint8_t* base = nullptr;
  Handle handle{};
  uint64_t address = 0;
  std::map<int, uint8_t*> mappedFor;  // other process: local address per accessing device
  size_t inboxBytes = 0;
  uint64_t head = 0, tail = 0;  // inbox ring cursors (bytes, free-running)
  uint64_t eagerSent = 0, eagerAcked = 0;  // eager batches pushed / reported unpacked
  int64_t announcedSeq = -1;
  uint64_t eagerThreshold = 0;
  bool creditRequested = false;
};

// A peer allocation this end may write into.
struct PeerRegion {
  Handle handle{};
  uint64_t size = 0;
  struct Mapped {
    uint8_t* base = nullptr;
    uint64_t generation = 0;
    uint64_t refreshedNs = 0;
  };
  std::map<int, Mapped> mappedFor;  // per accessing device
};

inline uint32_t flagValueFor(uint64_t seq) { return static_cast<uint32_t>(seq / kFlagSlots + 1); }
inline uint64_t alignUp(uint64_t v) { return (v + kInboxAlign - 1) / kInboxAlign * kInboxAlign; }

struct SendOp {
  uint64_t seq = 0;
  int srcDevice = -1;
  Device targetDevice;
  std::vector<SendItem> items;
  bool launched = false;
  std::optional<RecvReady> ready;
  // The head of one large host tensor of this batch that the copy engine started on when the
  // batch was handed over, before the receiver answered (see HostFeed::early).
  int earlyItem = -1;
  uint64_t earlyBytes = 0;
  // Recorded on the sender's stream when the batch was handed over (Options::sendOrderMinBytes);
  // empty for a batch that is launched on the sender's stream itself.
  std::shared_ptr<CudaEvent> sent;
};

// A receive buffer that CUDA IPC cannot export (memory from a stream-ordered pool, a virtual-memory
// allocation, ...) is replaced, for the sender's eyes, by an exportable buffer of this channel; the
// receiver copies from it to the user's buffer on the user's stream once the data has landed.
struct StagingBuffer {
  uint8_t* ptr = nullptr;
  size_t bytes = 0;
  bool busy = false;                   // handed to a receive that has not been completed yet
  std::unique_ptr<CudaEvent> drained;  // recorded after the copy out of it; reusable once it has fired
};
std::atomic<uint64_t> gStagedReceives{0};

struct RecvOp {
  uint64_t seq = 0;
  int device = -1;
  int sourceDevice = -1;  // the peer's index of the device the data comes from (-1 unknown)
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
    it.targetDevice = Device(kCudaDeviceType, -1);  // unknown: such sends always meet the receiver first
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
  // connectionBroken: the control connection itself reported the failure, so nothing more will
  // come from the peer and nothing can be sent to it.
  void closeFromLoop(const Error& e, bool connectionBroken = false);
  void finishClose();

 private:
  void initFromLoop();
  void armRead();
  void onPacket(Packet p);
  void onHello(const Hello& peer);
  void sendBatchFromLoop(std::vector<SendItem> items, std::shared_ptr<CudaEvent> sent);
  void recvBatchFromLoop(std::vector<RecvItem> items);
  void pumpSends();
  bool tryLaunch(SendOp& op);
  enum class Eager { kNotEligible, kLaunched, kNoCredits };
  Eager tryEager(SendOp& op);
  void launchRendezvous(SendOp& op);
  void finishSend(SendOp& op, const Error& e);
  void sendReady(RecvOp& op);
  void completeRecv(RecvOp& op);
  void finishRecv(RecvOp& op, const Error& e);
  void answerCreditRequest(Arena& arena);
  void advanceUnpacks(Arena& arena);
  void writePacket(const Packet& p);
  Arena* arenaFor(int device, Error& err);
  uint32_t* statusWord();
  bool deviceFailed();
  uint8_t* peerArenaBase(PeerArena& peer, int fromDevice, std::string* why);
  uint8_t* takeStaging(int device, size_t bytes, size_t* index);
  std::unique_ptr<CudaEvent> takeEvent(int device);
  void recycleEvent(std::unique_ptr<CudaEvent> ev);
  // Sender-side bound on unfinished pushes.
  kernels::DoneSlot doneSlotFor(uint64_t seq);
  void noteLaunch(uint64_t seq, bool launched);
  void advanceConfirmed();
  bool roomFor(uint64_t seq);
  void whenPushFinishes(uint64_t seq, std::function<void()> then);
  void sendBye();
  void sendByeWhenIdle();
  int allCtas(int device) const { return opts_.maxCtas > 0 ? opts_.maxCtas : cudaSmCount(device); }
  int ctasFor(int device);
  // Whether a source may go through the bulk-copy (TMA) pipeline: memory of the launching GPU
  // does, and so does pinned host memory that a user hands over as a tensor of this GPU (the
  // deep queue of bulk loads is what keeps PCIe busy); memory of another GPU is read with
  // ordinary loads. (Asked only for tensors large enough to take the bulk path at all.)
  bool bulkFor(const void* src, size_t bytes, int device) const {
    if (!opts_.useBulkCopy) return false;
    if (bytes < kernels::getPushTuning().bulkMinBytes) return true;
    return cudaIsLocalMemory(src, device);
  }
  bool sourceIsOtherGpu(const RecvOp& op) const;
  template <typename It>
  static std::vector<std::vector<It>> splitByDevicePair(std::vector<It>& items, bool send);

  std::shared_ptr<ContextImpl> ctx_;
  std::shared_ptr<transport::Connection> conn_;
  Options opts_;
  std::string id_ = "N/A";
  Error error_;
  bool helloDone_ = false;
  bool sameProcess_ = false;
  std::atomic<bool> sameProcessForCallers_{false};  // the same, readable from the threads that call sendBatch()
  std::vector<std::string> peerUuids_, myUuids_;
  uint64_t nextSendSeq_ = 0, nextRecvSeq_ = 0;
  std::deque<SendOp> sendOps_;
  std::deque<RecvOp> recvOps_;
  std::map<uint64_t, RecvReady> earlyReady_;     // RecvReady that arrived before its sendBatch
  std::map<uint64_t, Launched> earlyLaunched_;   // Launched that arrived before its recvBatch
  std::map<int, Arena> arenas_;                  // my devices
  std::map<int, PeerArena> peerArenas_;          // peer's devices
  std::vector<PeerRegion> peerRegions_;          // what the peer has exported to me, by id
  std::map<unsigned long long, uint32_t> regionIds_;  // my allocations already exported to the peer (by buffer id)
  uint32_t nextRegionId_ = 0;
  std::map<int, std::vector<std::unique_ptr<CudaEvent>>> freeEvents_;
  std::map<int, std::vector<StagingBuffer>> staging_;  // per device, kept until the channel dies
  // Mapped host memory that kernels of this channel report to: word 0 takes failure codes, words
  // [256, 512) take the sequence number (+1) of every push when its last CTA is through.
  uint32_t* hostWords_ = nullptr;
  // Unfinished pushes (sending side).
  uint64_t confirmed_ = 0;      // every push with a smaller sequence number has finished
  uint64_t launchedUpTo_ = 0;   // one past the newest launched sequence number
  bool waitingForRoom_ = false;
  int launchesMade_ = 0;
  // Same process: events recorded behind the pushes, reused round-robin. The receiver makes its
  // stream wait for an event as soon as the Launched frame naming it arrives, long before the
  // sender comes round to that event again.
  static constexpr size_t kEventRing = 512;
  std::map<int, std::vector<std::unique_ptr<CudaEvent>>> eventRings_;
  CudaEvent* lastPushEvent_ = nullptr;
  CudaEvent& eventFor(int device, uint64_t seq);
  // Large batches (Options::sendOrderMinBytes) leave from a stream of the channel's own, one per
  // sending device, behind an event that sendBatch() recorded on the sender's stream from the
  // calling thread. The events come from a pool that both threads reach.
  std::map<int, cudaStream_t> asideStreams_;
  std::map<int, std::unique_ptr<CudaEvent>> asideDone_;  // "the push on the aside stream is over", per device
  cudaStream_t asideStreamFor(int device);
  std::mutex sentEventsMutex_;
  std::map<int, std::vector<std::unique_ptr<CudaEvent>>> sentEvents_;
  std::shared_ptr<CudaEvent> markSendTime(const std::vector<SendItem>& items);
  struct HostItem {
    const uint8_t* src;
    uint8_t* dst;
    uint64_t bytes;  // without the tail
  };
  void feedFromHost(HostFeed& feed, const HostItem& item, cudaStream_t stream, int ctas);
  void startEarly(SendOp& op);
  void releaseEarly(SendOp& op);
  // Closing.
  bool byeSent_ = false, byeReceived_ = false, finished_ = false;
  bool peerLeft_ = false;  // the peer said goodbye while this end was open: only early arrivals can still be received
  void onPeerLeft();
  std::vector<RecvOp> held_;  // receives whose buffers the peer may still be writing
};

class ContextImpl final : public Context, public std::enable_shared_from_this<ContextImpl> {
 public:
  HostFeed* hostFeedFor(int device);
  std::map<int, std::unique_ptr<HostFeed>> hostFeeds_;
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
      // The prefix keeps a reference peer's cuda_ipc (whose descriptor is the bare structure,
      // tensorpipe/channel/cuda_ipc/context_impl.cc:108-113) from ever matching this channel:
      // the two speak different protocols on their connections.
      auto bytes = nop::encode(d);
      descriptors_[Device(kCudaDeviceType, i)] = kDescriptorPrefix + std::string(bytes.begin(), bytes.end());
    }
    viable_ = true;
  }
  bool isViable() const override { return viable_; }
  const std::unordered_map<Device, std::string>& deviceDescriptors() const override { return descriptors_; }
  bool canCommunicateWithRemote(const std::string& local, const std::string& remote) const override {
    DeviceDescriptor l, r;
    if (!parse(local, l) || !parse(remote, r)) return false;
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
      for (auto& c : chans) c->closeFromLoop(TPB_CREATE_ERROR(ContextClosedError));
    });
  }
  void join() override {
    close();
    loop_.runInLoop([]() {});
    // Nobody waits for a peer's goodbye beyond this point: every callback fires before join returns.
    loop_.runInLoop([this]() {
      auto chans = channels_;
      for (auto& c : chans) c->finishClose();
    });
    poller_.stop();
    loop_.runInLoop([]() {});
  }
  Poller poller_;
  // A channel stays enrolled (and thereby alive) until it has fired its last callback.
  void enroll(std::shared_ptr<ChannelImpl> c) { channels_.insert(std::move(c)); }
  void unenroll(const std::shared_ptr<ChannelImpl>& c) { channels_.erase(c); }
  bool closed() const { return closed_; }
  const std::vector<std::string>& uuids() const { return uuids_; }
  OnDemandLoop loop_;

  // How many CTAs a push from `device` should take: the whole GPU when this is the only channel
  // sending from it at the moment, a share when several are (all-pairs traffic), so that pushes
  // to different destinations run side by side instead of one after the other.
  int ctaShare(const void* channel, int device, int sms) {
    const uint64_t now = nowNs();
    auto& recent = recentSenders_[device];
    recent[channel] = now;
    int active = 0;
    for (auto it = recent.begin(); it != recent.end();) {
      if (now - it->second > 2'000'000ull) it = recent.erase(it);
      else {
        ++active;
        ++it;
      }
    }
    if (active <= 1) return sms;
    const int share = sms / active;
    return share < 16 ? 16 : share;
  }

 private:
  static constexpr const char* kDescriptorPrefix = "tpbp2p1:";
  static bool parse(const std::string& s, DeviceDescriptor& d) {
    const size_t n = std::strlen(kDescriptorPrefix);
    if (s.compare(0, n, kDescriptorPrefix) != 0) return false;
    return nop::decode(s.data() + n, s.size() - n, d);
  }
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
  std::set<std::shared_ptr<ChannelImpl>> channels_;
  std::map<int, std::map<const void*, uint64_t>> recentSenders_;
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
  for (auto& a : arenas_)
    if (a.second.unpackDone) cudaFreeHost(a.second.unpackDone);
  if (hostWords_) cudaFreeHost(hostWords_);
  cudaGetLastError();
}

void ChannelImpl::init() {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self]() { self->initFromLoop(); });
}

void ChannelImpl::initFromLoop() {
  auto self = shared_from_this();
  ctx_->enroll(self);
  if (ctx_->closed()) return closeFromLoop(TPB_CREATE_ERROR(ContextClosedError));
  // Hello: who am I (decides between raw pointers and IPC mappings) and which GPUs do I see.
  Hello hello;
  hello.identity = processIdentity();
  hello.uuids = ctx_->uuids();
  myUuids_ = hello.uuids;
  transport::writeNop(*conn_, hello, [self](const Error& e) {
    if (e) self->ctx_->loop_.deferToLoop([self, e]() { self->closeFromLoop(e, true); });
  });
  transport::readNop<Hello>(*conn_, [self](const Error& e, Hello peer) {
    self->ctx_->loop_.deferToLoop([self, e, peer = std::move(peer)]() {
      if (self->finished_) return;
      if (e) return self->error_ ? self->finishClose() : self->closeFromLoop(e, true);
      self->onHello(peer);
    });
  });
}

void ChannelImpl::onHello(const Hello& peer) {
  sameProcess_ = peer.identity == processIdentity();
  sameProcessForCallers_.store(sameProcess_, std::memory_order_relaxed);
  peerUuids_ = peer.uuids;
  helloDone_ = true;
  TPB_VLOG(4) << "Channel " << id_ << " peer " << peer.identity << (sameProcess_ ? " (same process)" : " (other process)");
  armRead();
  if (error_) {
    // Closed before the peer was known: say goodbye now (nothing was ever launched).
    sendByeWhenIdle();
    return;
  }
  for (size_t i = 0; i < recvOps_.size() && !error_; ++i)
    if (!recvOps_[i].readySent && !recvOps_[i].notice && !recvOps_[i].expectEager) sendReady(recvOps_[i]);
  pumpSends();
}

void ChannelImpl::armRead() {
  auto self = shared_from_this();
  transport::readNop<Packet>(*conn_, [self](const Error& e, Packet p) {
    self->ctx_->loop_.deferToLoop([self, e, p = std::move(p)]() mutable {
      if (self->finished_) return;
      if (e) {
        if (self->error_) return self->finishClose();
        if (self->peerLeft_) return;  // expected: the peer closed after its goodbye
        return self->closeFromLoop(e, true);
      }
      self->onPacket(std::move(p));
      if (!self->finished_) self->armRead();
    });
  });
}

void ChannelImpl::writePacket(const Packet& p) {
  auto self = shared_from_this();
  transport::writeNop(*conn_, p, [self](const Error& e) {
    if (!e) return;
    self->ctx_->loop_.deferToLoop([self, e]() {
      if (self->finished_) return;
      if (self->error_) self->finishClose();
      else if (!self->peerLeft_) self->closeFromLoop(e, true);
    });
  });
}

uint32_t* ChannelImpl::statusWord() {
  if (hostWords_) return hostWords_;
  void* p = nullptr;
  if (cudaHostAlloc(&p, kHostWords * sizeof(uint32_t), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
    cudaGetLastError();
    throw std::runtime_error("cuda_p2p: cannot allocate the channel's mapped host words");
  }
  std::memset(p, 0, kHostWords * sizeof(uint32_t));
  hostWords_ = static_cast<uint32_t*>(p);
  return hostWords_;
}

// A kernel of this channel gave up (a wait that ran out, a bulk copy that never completed): the
// data of some receive is not what the sender sent, although its callback may already have
// reported success. The channel cannot be trusted any further and fails.
bool ChannelImpl::deviceFailed() {
  if (!hostWords_) return false;
  const uint32_t code = *reinterpret_cast<volatile uint32_t*>(hostWords_);
  if (code == kernels::kStatusOk) return false;
  if (!error_) {
    const char* what = code == kernels::kStatusWaitTimeout ? "a device-side wait for the peer's data ran out of time"
                                                           : "a bulk copy on the device never completed";
    closeFromLoop(TPB_CREATE_ERROR(CudaError, std::string("cuda_p2p: ") + what + " (kernel status " +
                                                  std::to_string(code) + "); data received on this channel may be incomplete"));
  }
  return true;
}

Arena* ChannelImpl::arenaFor(int device, Error& err) {
  auto it = arenas_.find(device);
  if (it != arenas_.end()) return &it->second;
  Arena a;
  a.device = device;
  a.inboxBytes = opts_.inboxBytes;
  CudaDeviceGuard g(device);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, kHeaderBytes + a.inboxBytes);
  // The flags and counters must read zero BEFORE the peer learns this address: a memset queued
  // on the default stream could run after the peer's first push has already set a flag.
  if (e == cudaSuccess && !cudaZeroNow(p, kHeaderBytes, device)) e = cudaErrorUnknown;
  if (e == cudaSuccess && !sameProcess_) {
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, p);
    if (e == cudaSuccess) std::memcpy(a.handle.data(), &h, sizeof(h));
  }
  void* words = nullptr;
  if (e == cudaSuccess) e = cudaHostAlloc(&words, kFlagSlots * sizeof(uint32_t), cudaHostAllocMapped | cudaHostAllocPortable);
  if (e != cudaSuccess) {
    cudaGetLastError();
    if (p) cudaFree(p);
    err = cudaErrorToError(e, "allocating the channel arena");
    return nullptr;
  }
  std::memset(words, 0, kFlagSlots * sizeof(uint32_t));
  a.unpackDone = static_cast<uint32_t*>(words);
  a.base = static_cast<uint8_t*>(p);
  return &arenas_.emplace(device, a).first->second;
}

uint8_t* ChannelImpl::peerArenaBase(PeerArena& peer, int fromDevice, std::string* why) {
  if (sameProcess_) return reinterpret_cast<uint8_t*>(peer.address);
  auto it = peer.mappedFor.find(fromDevice);
  if (it != peer.mappedFor.end()) return it->second;
  // Arena mappings stay open for as long as the process lives: their addresses are kept here.
  void* base = MappingCache::get().open(peer.handle, fromDevice, nullptr, why, /*pin=*/true);
  if (!base) return nullptr;
  peer.mappedFor[fromDevice] = static_cast<uint8_t*>(base);
  return static_cast<uint8_t*>(base);
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
  std::shared_ptr<CudaEvent> sent = markSendTime(items);
  auto shared = std::make_shared<std::vector<SendItem>>(std::move(items));
  ctx_->loop_.deferToLoop([self, shared, sent]() { self->sendBatchFromLoop(std::move(*shared), sent); });
}

// Runs on the thread that called sendBatch(), so that the event lands in the sender's stream ahead
// of whatever that thread queues next. The push is launched much later, by the loop thread, when
// the receiver has named its buffers: launched on the sender's stream then, it would sit behind
// all that the user queued in between (and a pipeline stage queues the next micro-batch's compute
// there, which the stage downstream then waits out).
std::shared_ptr<CudaEvent> ChannelImpl::markSendTime(const std::vector<SendItem>& items) {
  if (opts_.sendOrderMinBytes == 0 || items.empty()) return nullptr;
  uint64_t bytes = 0;
  for (const SendItem& it : items) bytes += it.length;
  if (bytes < opts_.sendOrderMinBytes) return nullptr;
  try {
    // (Looking a pointer's device up may fail for memory the driver does not know: such a batch
    // goes the ordinary way, where the failure is reported through its callback.)
    const void* stream = items[0].buffer.unwrap<CudaBuffer>().stream;
    const int device = items[0].buffer.device().index;
    bool leavesTheGpu = !sameProcessForCallers_.load(std::memory_order_relaxed);
    for (const SendItem& it : items) {
      if (it.buffer.unwrap<CudaBuffer>().stream != stream || it.buffer.device().index != device) return nullptr;
      leavesTheGpu = leavesTheGpu || it.targetDevice.type != kCudaDeviceType || it.targetDevice.index != device;
    }
    // A batch that stays on its GPU within this process is a local copy at memory speed: the two
    // hand-offs between streams would cost it 3 % at 256 MiB, and it is launched on the sender's
    // stream like a small one.
    if (!leavesTheGpu) return nullptr;
    std::unique_ptr<CudaEvent> ev;
    {
      std::lock_guard<std::mutex> lock(sentEventsMutex_);
      auto& pool = sentEvents_[device];
      if (!pool.empty()) {
        ev = std::move(pool.back());
        pool.pop_back();
      }
    }
    if (!ev) ev = std::make_unique<CudaEvent>(device);
    ev->record(static_cast<cudaStream_t>(const_cast<void*>(stream)));
    std::weak_ptr<ChannelImpl> weak = weak_from_this();
    return std::shared_ptr<CudaEvent>(ev.release(), [weak, device](CudaEvent* e) {
      std::unique_ptr<CudaEvent> owned(e);
      if (auto self = weak.lock()) {
        std::lock_guard<std::mutex> lock(self->sentEventsMutex_);
        auto& pool = self->sentEvents_[device];
        if (pool.size() < 64) pool.push_back(std::move(owned));
      }
    });
  } catch (const std::exception&) {
    return nullptr;  // the batch then goes the ordinary way, where a dead device is reported
  }
}

void ChannelImpl::recvBatch(std::vector<RecvItem> items) {
  auto self = shared_from_this();
  auto shared = std::make_shared<std::vector<RecvItem>>(std::move(items));
  ctx_->loop_.deferToLoop([self, shared]() { self->recvBatchFromLoop(std::move(*shared)); });
}

void ChannelImpl::sendBatchFromLoop(std::vector<SendItem> items, std::shared_ptr<CudaEvent> sent) {
  deviceFailed();
  if (peerLeft_ && !error_) closeFromLoop(TPB_CREATE_ERROR(ChannelClosedError));
  std::vector<SendItem> live;
  for (auto& it : items) {
    if (error_) it.callback(error_);
    else if (it.length == 0) it.callback(Error::kSuccess);  // nothing travels for an empty tensor
    else live.push_back(std::move(it));
  }
  if (live.empty()) return;
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
    op.sent = sent;
    auto early = earlyReady_.find(op.seq);
    if (early != earlyReady_.end()) {
      op.ready = std::move(early->second);
      earlyReady_.erase(early);
    }
    TPB_VLOG(6) << "Channel " << id_ << " send batch #" << op.seq << " (" << op.items.size() << " tensors)"
                << (op.ready ? ", receiver already announced its buffers" : "");
    if (!op.ready) startEarly(op);
    sendOps_.push_back(std::move(op));
  }
  pumpSends();
}

// Sends launch strictly in order: the first batch that cannot go yet (no RecvReady, no inbox
// space, too many pushes unfinished) holds back the ones behind it.
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
    if (!roomFor(op.seq)) return false;
    Eager e = tryEager(op);
    if (e == Eager::kLaunched) return true;
    if (e == Eager::kNoCredits) return false;
    if (!op.ready) return false;
    launchRendezvous(op);
    return !error_;
  } catch (const std::exception& ex) {
    closeFromLoop(TPB_CREATE_ERROR(CudaError, ex.what()));
    return false;
  }
}

// ---- the bound on unfinished pushes -----------------------------------------------------------
kernels::DoneSlot ChannelImpl::doneSlotFor(uint64_t seq) {
  kernels::DoneSlot d;
  d.slot = statusWord() + kFlagSlots + (seq % kFlagSlots);
  d.value = static_cast<uint32_t>(seq + 1);
  return d;
}

void ChannelImpl::noteLaunch(uint64_t seq, bool launched) {
  // A push that was skipped on purpose (fault injection) is "finished" at once.
  if (!launched) *reinterpret_cast<volatile uint32_t*>(doneSlotFor(seq).slot) = static_cast<uint32_t>(seq + 1);
  launchedUpTo_ = seq + 1;
}

void ChannelImpl::advanceConfirmed() {
  if (!hostWords_) return;
  const volatile uint32_t* done = hostWords_ + kFlagSlots;
  while (confirmed_ < launchedUpTo_ && done[confirmed_ % kFlagSlots] == static_cast<uint32_t>(confirmed_ + 1)) ++confirmed_;
}

CudaEvent& ChannelImpl::eventFor(int device, uint64_t seq) {
  auto& ring = eventRings_[device];
  if (ring.empty()) ring.resize(kEventRing);
  auto& slot = ring[seq % kEventRing];
  if (!slot) slot = std::make_unique<CudaEvent>(device);
  return *slot;
}

bool ChannelImpl::roomFor(uint64_t seq) {
  if (sameProcess_) return true;  // no flag slots, no counters: nothing to run out of
  if (seq - confirmed_ < kMaxUnfinished) return true;
  advanceConfirmed();
  if (seq - confirmed_ < kMaxUnfinished) return true;
  if (!waitingForRoom_) {
    waitingForRoom_ = true;
    auto self = shared_from_this();
    whenPushFinishes(confirmed_, [self]() {
      self->waitingForRoom_ = false;
      self->pumpSends();
    });
  }
  return false;
}

// Runs `then` on the loop once push number `seq` (which has been launched) has finished.
void ChannelImpl::whenPushFinishes(uint64_t seq, std::function<void()> then) {
  auto self = shared_from_this();
  const volatile uint32_t* word = hostWords_ + kFlagSlots + (seq % kFlagSlots);
  const uint32_t want = static_cast<uint32_t>(seq + 1);
  ctx_->poller_.watch([self, word, want]() { return *word == want; },
                      [self, then = std::move(then)]() mutable {
                        self->ctx_->loop_.deferToLoop([self, then = std::move(then)]() {
                          self->advanceConfirmed();
                          then();
                        });
                      });
}

int ChannelImpl::ctasFor(int device) {
  if (opts_.maxCtas > 0) return opts_.maxCtas;
  return ctx_->ctaShare(this, device, cudaSmCount(device));
}

ChannelImpl::Eager ChannelImpl::tryEager(SendOp& op) {
  if (sameProcess_) return Eager::kNotEligible;
  auto pa = peerArenas_.find(op.targetDevice.index);
  if (pa == peerArenas_.end()) return Eager::kNotEligible;
  PeerArena& peer = pa->second;
  uint64_t total = 0;
  for (auto& it : op.items) total += alignUp(it.length);
  // The rule the receiver evaluates too (see the top of this file).
  if (static_cast<int64_t>(op.seq) <= peer.announcedSeq || total > peer.eagerThreshold) return Eager::kNotEligible;
  const uint64_t cap = peer.inboxBytes;
  const uint64_t pos = peer.head % cap;
  const uint64_t skip = pos + total > cap ? cap - pos : 0;
  const uint64_t used = peer.head + skip + total - peer.tail;
  const uint64_t unacked = peer.eagerSent - peer.eagerAcked;
  if ((used > cap / 2 || unacked >= kMaxUnfinished / 2) && !peer.creditRequested) {
    // Ask early, so that the answer is here before the ring is full.
    peer.creditRequested = true;
    CreditRequest req;
    req.deviceIdx = op.targetDevice.index;
    writePacket(req);
  }
  if (used > cap || unacked >= kMaxUnfinished) return Eager::kNoCredits;  // wait for a Credit
  const uint64_t offset = (peer.head + skip) % cap;
  peer.head += skip + total;
  ++peer.eagerSent;

  trace::Scope traced("p2p.send.eager", op.seq);
  std::string why;
  uint8_t* base = peerArenaBase(peer, op.srcDevice, &why);
  if (!base) {
    closeFromLoop(TPB_CREATE_ERROR(CudaError, why));
    return Eager::kLaunched;
  }
  if (sameProcess_ && op.targetDevice.index != op.srcDevice &&
      !cudaEnablePeerAccessOnce(op.srcDevice, op.targetDevice.index)) {
    closeFromLoop(TPB_CREATE_ERROR(CudaError, "peer access between the two GPUs cannot be enabled"));
    return Eager::kLaunched;
  }
  Error err;
  Arena* mine = arenaFor(op.srcDevice, err);
  if (!mine) {
    closeFromLoop(err);
    return Eager::kLaunched;
  }
  CudaDeviceGuard g(op.srcDevice);
  kernels::PushPlan plan;
  const int ctas = ctasFor(op.srcDevice);
  {
    uint64_t bulkBytes = 0;
    const uint64_t bulkMin = kernels::getPushTuning().bulkMinBytes;
    for (auto& it : op.items)
      if (!it.view && it.length >= bulkMin) bulkBytes += it.length;
    kernels::chooseBulkTile(plan, bulkBytes, ctas);
  }
  uint64_t cursor = offset;
  for (auto& it : op.items) {
    kernels::CopyItem c;
    c.src = it.buffer.unwrap<CudaBuffer>().ptr;
    c.dst = base + kHeaderBytes + cursor;
    c.srcBytes = it.length;
    c.srcDtype = it.dtype;
    c.dstDtype = it.dtype;  // a requested cast is applied by the receiver's unpack
    if (it.view) {
      c.strided = true;
      c.view = *it.view;
      c.srcDtype = c.dstDtype = it.view->dtype;
    }
    kernels::appendToPlan(plan, c, bulkFor(c.src, it.length, op.srcDevice));
    cursor += alignUp(it.length);
  }
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
  uint32_t* flag = reinterpret_cast<uint32_t*>(base) + (op.seq % kFlagSlots);
  const bool launch = launchesMade_++ != opts_.faultSkipLaunch;
  if (launch)
    kernels::launchPush(plan, stream, ctas, flag, flagValueFor(op.seq), mine->pushCounter(op.seq), statusWord(),
                        kernels::WaitBefore(), doneSlotFor(op.seq));
  if (!others.empty()) {
    CudaEvent ev(op.srcDevice);
    ev.record(stream);
    for (cudaStream_t s : others) ev.wait(s, op.srcDevice);
  }
  noteLaunch(op.seq, launch);
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

HostFeed* ContextImpl::hostFeedFor(int device) {
  auto& feed = hostFeeds_[device];
  if (feed) return feed.get();
  auto f = std::make_unique<HostFeed>();
  f->pieceBytes = (std::max<size_t>(opts_.hostPieceBytes, 1u << 20) + 255) / 256 * 256;
  CudaDeviceGuard g(device);
  if (cudaStreamCreateWithFlags(&f->copyStream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaMalloc(reinterpret_cast<void**>(&f->slots), (HostFeed::kSlots + 1) * f->pieceBytes) != cudaSuccess) {
    cudaGetLastError();
    if (f->copyStream) cudaStreamDestroy(f->copyStream);
    return nullptr;
  }
  f->device = device;
  f->early = f->slots + HostFeed::kSlots * f->pieceBytes;
  f->earlyCopied = std::make_unique<CudaEvent>(device);
  f->earlySent = std::make_unique<CudaEvent>(device);
  f->begin = std::make_unique<CudaEvent>(device);
  for (size_t i = 0; i < HostFeed::kSlots; ++i) {
    f->copied[i] = std::make_unique<CudaEvent>(device);
    f->sent[i] = std::make_unique<CudaEvent>(device);
  }
  feed = std::move(f);
  return feed.get();
}

// Head start for a batch whose receiver has not answered yet: the first piece of its first large
// pinned host tensor goes into the feed's early slot now.
void ChannelImpl::startEarly(SendOp& op) {
  if (opts_.hostCopyMinBytes == 0 || op.srcDevice < 0) return;
  for (size_t i = 0; i < op.items.size(); ++i) {
    SendItem& it = op.items[i];
    const void* src = it.buffer.unwrap<CudaBuffer>().ptr;
    if (it.view || it.length < opts_.hostCopyMinBytes || it.length <= 2 * kHostTailBytes || !cudaIsPinnedHostMemory(src)) continue;
    try {
      CudaDeviceGuard g(op.srcDevice);
      HostFeed* feed = ctx_->hostFeedFor(op.srcDevice);
      if (!feed || feed->earlyTaken) return;
      const uint64_t head = (it.length - kHostTailBytes) & ~uint64_t(255);
      const uint64_t n = std::min<uint64_t>(feed->pieceBytes, head);
      cudaStream_t stream = static_cast<cudaStream_t>(it.buffer.unwrap<CudaBuffer>().stream);
      trace::Scope traced("p2p.send.hostearly", op.seq);
      feed->begin->record(stream);
      feed->begin->wait(feed->copyStream, feed->device);
      if (feed->earlyEverSent) feed->earlySent->wait(feed->copyStream, feed->device);
      TPB_CUDA_CHECK(cudaMemcpyAsync(feed->early, src, n, cudaMemcpyHostToDevice, feed->copyStream));
      feed->earlyCopied->record(feed->copyStream);
      feed->earlyTaken = true;
      op.earlyItem = static_cast<int>(i);
      op.earlyBytes = n;
    } catch (const std::exception& ex) {
      TPB_VLOG(4) << "Channel " << id_ << " gives the head start of batch #" << op.seq << " a miss: " << ex.what();
    }
    return;
  }
}

// The early slot goes back to the feed: either the push that reads it has been launched (and
// earlySent recorded behind it) or the batch will not use it after all.
void ChannelImpl::releaseEarly(SendOp& op) {
  if (op.earlyItem < 0) return;
  op.earlyItem = -1;
  auto it = ctx_->hostFeeds_.find(op.srcDevice);
  if (it != ctx_->hostFeeds_.end() && it->second) it->second->earlyTaken = false;
}

// Queues the pieces of one host tensor bound for another GPU: copies on the feed's stream, pushes
// on the user's. May throw (CUDA errors).
void ChannelImpl::feedFromHost(HostFeed& feed, const HostItem& item, cudaStream_t stream, int ctas) {
  // The host memory is read after whatever the user queued on the stream before the send.
  feed.begin->record(stream);
  feed.begin->wait(feed.copyStream, feed.device);
  for (uint64_t off = 0; off < item.bytes;) {
    uint64_t len = std::min<uint64_t>(feed.pieceBytes, item.bytes - off);
    if (off + len >= item.bytes && len > 2 * kHostLastPieceBytes) len = (len - kHostLastPieceBytes) & ~uint64_t(255);
    const size_t slot = feed.next++ % HostFeed::kSlots;
    uint8_t* piece = feed.slots + slot * feed.pieceBytes;
    if (feed.everSent[slot]) feed.sent[slot]->wait(feed.copyStream, feed.device);
    TPB_CUDA_CHECK(cudaMemcpyAsync(piece, item.src + off, len, cudaMemcpyHostToDevice, feed.copyStream));
    feed.copied[slot]->record(feed.copyStream);
    feed.copied[slot]->wait(stream, feed.device);
    kernels::CopyItem c;
    c.src = piece;
    c.dst = item.dst + off;
    c.srcBytes = len;
    c.remote = true;
    kernels::PushPlan piecePlan;
    kernels::chooseBulkTile(piecePlan, len, ctas);
    kernels::appendToPlan(piecePlan, c, opts_.useBulkCopy);
    kernels::launchPush(piecePlan, stream, ctas, nullptr, 0, nullptr, statusWord());
    feed.sent[slot]->record(stream);
    feed.everSent[slot] = true;
    off += len;
  }
}

void ChannelImpl::launchRendezvous(SendOp& op) {
  trace::Scope traced("p2p.send.rendezvous", op.seq);
  const RecvReady& ready = *op.ready;
  if (ready.targets.size() != op.items.size())
    return closeFromLoop(TPB_CREATE_ERROR(LogicError, "peer announced a different number of tensors"));
  CudaDeviceGuard g(op.srcDevice);
  if (ready.arena && !sameProcess_) {
    PeerArena pa;
    pa.handle = ready.arena->handle;
    pa.address = ready.arena->address;
    pa.inboxBytes = ready.arena->inboxBytes;
    pa.eagerThreshold = std::min<uint64_t>(ready.arena->eagerThreshold, ready.arena->inboxBytes / 2);
    pa.announcedSeq = static_cast<int64_t>(ready.seq);
    peerArenas_[ready.deviceIdx] = pa;
  }
  std::string why;
  uint8_t* arenaBase = nullptr;
  if (!sameProcess_) {
    auto arena = peerArenas_.find(ready.deviceIdx);
    if (arena == peerArenas_.end())
      return closeFromLoop(TPB_CREATE_ERROR(LogicError, "peer never announced its arena for that device"));
    arenaBase = peerArenaBase(arena->second, op.srcDevice, &why);
    if (!arenaBase) return closeFromLoop(TPB_CREATE_ERROR(CudaError, why));
  }
  if (sameProcess_ && ready.deviceIdx != op.srcDevice && !cudaEnablePeerAccessOnce(op.srcDevice, ready.deviceIdx))
    return closeFromLoop(TPB_CREATE_ERROR(CudaError, "peer access between the two GPUs cannot be enabled"));
  for (const RegionWire& r : ready.newRegions) {
    if (r.id != peerRegions_.size())
      return closeFromLoop(TPB_CREATE_ERROR(LogicError, "peer numbered its memory regions out of order"));
    PeerRegion region;
    region.handle = r.handle;
    region.size = r.size;
    peerRegions_.push_back(std::move(region));
  }

  kernels::PushPlan plan;
  const int ctas = ctasFor(op.srcDevice);
  {
    uint64_t bulkBytes = 0;
    const uint64_t bulkMin = kernels::getPushTuning().bulkMinBytes;
    for (auto& it : op.items) {
      if (it.view || it.length < bulkMin) continue;
      // Host memory never takes the bulk path (and of a large host tensor only the tail is here).
      if (cudaIsPinnedHostMemory(it.buffer.unwrap<CudaBuffer>().ptr)) continue;
      bulkBytes += it.length;
    }
    kernels::chooseBulkTile(plan, bulkBytes, ctas);
  }
  const uint64_t generation = MappingCache::get().generation();
  const uint64_t now = nowNs();
  std::vector<HostItem> hostLocal, hostRemote;
  std::optional<HostItem> early;
  bool earlyRemote = false;
  for (size_t i = 0; i < op.items.size(); ++i) {
    SendItem& it = op.items[i];
    const TargetWire& t = ready.targets[i];
    kernels::CopyItem c;
    c.src = it.buffer.unwrap<CudaBuffer>().ptr;
    if (t.region == kNoRegion) {
      if (!sameProcess_)
        return closeFromLoop(TPB_CREATE_ERROR(CudaError, "the receiver could not export its buffer over CUDA IPC"));
      c.dst = reinterpret_cast<void*>(t.offset);
    } else {
      if (t.region >= peerRegions_.size())
        return closeFromLoop(TPB_CREATE_ERROR(LogicError, "peer named a memory region it never announced"));
      PeerRegion& region = peerRegions_[t.region];
      // The peer chose offset and length: they must stay inside what it exported.
      if (t.offset > region.size || t.bytes > region.size - t.offset)
        return closeFromLoop(TPB_CREATE_ERROR(LogicError, "peer's target lies outside the memory region it announced"));
      PeerRegion::Mapped& m = region.mappedFor[op.srcDevice];
      if (m.base == nullptr || m.generation != generation || now - m.refreshedNs > MappingCache::kRefreshNs) {
        size_t mappedSize = 0;
        void* base = MappingCache::get().open(region.handle, op.srcDevice, &mappedSize, &why);
        if (!base) return closeFromLoop(TPB_CREATE_ERROR(CudaError, why));
        if (mappedSize != 0 && mappedSize < region.size)
          return closeFromLoop(TPB_CREATE_ERROR(LogicError, "peer announced a memory region larger than the allocation behind its handle"));
        m.base = static_cast<uint8_t*>(base);
        m.generation = generation;
        m.refreshedNs = now;
      }
      c.dst = m.base + t.offset;
    }
    c.srcBytes = it.length;
    c.srcDtype = it.view ? it.view->dtype : it.dtype;
    if (c.srcDtype == DType::kBytes && t.dtype) c.srcDtype = static_cast<DType>(t.srcDtype);
    c.dstDtype = t.dtype ? static_cast<DType>(t.dtype) : c.srcDtype;
    if (it.view) {
      c.strided = true;
      c.view = *it.view;
    }
    c.remote = ready.deviceIdx != op.srcDevice || !sameProcess_;
    if (c.dstDtype != c.srcDtype && !kernels::castSupported(c.srcDtype, c.dstDtype))
      return closeFromLoop(TPB_CREATE_ERROR(LogicError, "unsupported dtype conversion requested by the receiver"));
    if (kernels::convertedBytes(it.length, c.srcDtype, c.dstDtype) != t.bytes)
      return closeFromLoop(TPB_CREATE_ERROR(LogicError, "receiver's buffer size does not match the tensor"));
    if (opts_.hostCopyMinBytes != 0 && !c.strided && c.dstDtype == c.srcDtype && it.length >= opts_.hostCopyMinBytes &&
        it.length > 2 * kHostTailBytes && cudaIsPinnedHostMemory(c.src)) {
      const uint64_t head = (it.length - kHostTailBytes) & ~uint64_t(255);
      const bool otherGpu = ready.deviceIdx >= 0 && static_cast<size_t>(ready.deviceIdx) < peerUuids_.size() &&
          peerUuids_[ready.deviceIdx] != myUuids_[op.srcDevice];
      // What the head start already brought into the early slot is pushed from there.
      uint64_t skip = 0;
      if (op.earlyItem == static_cast<int>(i) && op.earlyBytes <= head) {
        skip = op.earlyBytes;
        early = HostItem{nullptr, static_cast<uint8_t*>(c.dst), skip};
        earlyRemote = c.remote;
      }
      if (head > skip)
        (otherGpu ? hostRemote : hostLocal)
            .push_back({static_cast<const uint8_t*>(c.src) + skip, static_cast<uint8_t*>(c.dst) + skip, head - skip});
      c.src = static_cast<const uint8_t*>(c.src) + head;
      c.dst = static_cast<uint8_t*>(c.dst) + head;
      c.srcBytes = it.length - head;
      kernels::appendToPlan(plan, c, false);
      continue;
    }
    kernels::appendToPlan(plan, c, bulkFor(c.src, it.length, op.srcDevice));
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
  // A batch that was marked in the sender's stream when it was handed over leaves from the
  // channel's own stream, behind that mark.
  cudaStream_t senderStream = stream;
  const bool aside = op.sent != nullptr && others.empty();
  if (aside) {
    try {
      cudaStream_t own = asideStreamFor(op.srcDevice);
      op.sent->wait(own, op.srcDevice);
      stream = own;
    } catch (const std::exception& ex) {
      return closeFromLoop(TPB_CREATE_ERROR(CudaError, ex.what()));
    }
  }
  try {
    for (const HostItem& h : hostLocal) {
      trace::Scope copyTraced("p2p.send.hostcopy", op.seq);
      TPB_CUDA_CHECK(cudaMemcpyAsync(h.dst, h.src, h.bytes, cudaMemcpyDefault, stream));
    }
    if (early) {
      HostFeed* feed = ctx_->hostFeedFor(op.srcDevice);
      feed->earlyCopied->wait(stream, feed->device);
      kernels::CopyItem c;
      c.src = feed->early;
      c.dst = early->dst;
      c.srcBytes = early->bytes;
      c.remote = earlyRemote;
      kernels::PushPlan piecePlan;
      kernels::chooseBulkTile(piecePlan, early->bytes, ctas);
      kernels::appendToPlan(piecePlan, c, opts_.useBulkCopy);
      kernels::launchPush(piecePlan, stream, ctas, nullptr, 0, nullptr, statusWord());
      feed->earlySent->record(stream);
      feed->earlyEverSent = true;
    }
    releaseEarly(op);  // used or not: the slot is free for the next batch from here on
    if (!hostRemote.empty()) {
      trace::Scope feedTraced("p2p.send.hostfeed", op.seq);
      HostFeed* feed = ctx_->hostFeedFor(op.srcDevice);
      if (!feed) return closeFromLoop(TPB_CREATE_ERROR(CudaError, "no device memory for the pieces of a host tensor"));
      for (const HostItem& h : hostRemote) feedFromHost(*feed, h, stream, ctas);
    }
  } catch (const std::exception& ex) {
    return closeFromLoop(TPB_CREATE_ERROR(CudaError, ex.what()));
  }
  Launched l;
  l.seq = op.seq;
  const bool launch = launchesMade_++ != opts_.faultSkipLaunch;
  try {
    if (sameProcess_) {
      // Nothing to publish: the receiver's stream waits for an event recorded behind the kernel.
      if (launch) kernels::launchPush(plan, stream, ctas, nullptr, 0, nullptr, statusWord());
      CudaEvent& done = eventFor(op.srcDevice, op.seq);
      done.record(stream);
      l.event = reinterpret_cast<uint64_t>(done.raw());
      lastPushEvent_ = &done;
      for (cudaStream_t s : others) done.wait(s, op.srcDevice);
      if (aside) done.wait(senderStream, op.srcDevice);
      launchedUpTo_ = op.seq + 1;
    } else {
      Error err;
      Arena* mine = arenaFor(op.srcDevice, err);
      if (!mine) return closeFromLoop(err);
      uint32_t* flag = reinterpret_cast<uint32_t*>(arenaBase) + (op.seq % kFlagSlots);
      if (launch)
        kernels::launchPush(plan, stream, ctas, flag, flagValueFor(op.seq), mine->pushCounter(op.seq), statusWord(),
                            kernels::WaitBefore(), doneSlotFor(op.seq));
      if (!others.empty()) {
        CudaEvent ev(op.srcDevice);
        ev.record(stream);
        for (cudaStream_t s : others) ev.wait(s, op.srcDevice);
      }
      if (aside) {
        // The sender's stream takes the push in at the point it has reached by now: what the user
        // queues from here on (a write into the source among it) runs after the push, which is what
        // the send callback promises.
        auto& done = asideDone_[op.srcDevice];
        if (!done) done = std::make_unique<CudaEvent>(op.srcDevice);
        done->record(stream);  // waited for on the next line: re-recording it for the next batch is safe
        done->wait(senderStream, op.srcDevice);
      }
      noteLaunch(op.seq, launch);
    }
  } catch (const std::exception& ex) {
    return closeFromLoop(TPB_CREATE_ERROR(CudaError, ex.what()));
  }
  op.sent.reset();
  TPB_VLOG(6) << "Channel " << id_ << " launched the push of batch #" << op.seq << " (" << plan.entries.size()
              << " entries, " << plan.totalBytesOut << " bytes" << (aside ? ", from the channel's own stream" : "") << ")";
  writePacket(l);
  finishSend(op, Error::kSuccess);
}

cudaStream_t ChannelImpl::asideStreamFor(int device) {
  auto it = asideStreams_.find(device);
  if (it != asideStreams_.end()) return it->second;
  CudaDeviceGuard g(device);
  int least = 0, greatest = 0;
  TPB_CUDA_CHECK(cudaDeviceGetStreamPriorityRange(&least, &greatest));
  cudaStream_t s = nullptr;
  TPB_CUDA_CHECK(cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, greatest));
  asideStreams_[device] = s;
  return s;
}

void ChannelImpl::finishSend(SendOp& op, const Error& e) {
  op.launched = true;
  auto items = std::move(op.items);
  for (auto& it : items) it.callback(e);
}

void ChannelImpl::recvBatchFromLoop(std::vector<RecvItem> items) {
  deviceFailed();
  std::vector<RecvItem> live;
  for (auto& it : items) {
    if (error_) it.callback(error_);
    else if (it.length == 0) it.callback(Error::kSuccess);
    else live.push_back(std::move(it));
  }
  if (live.empty()) return;
  for (auto& group : splitByDevicePair(live, false)) {
    if (error_) {
      for (auto& it : group) it.callback(error_);
      continue;
    }
    RecvOp op;
    op.seq = nextRecvSeq_++;
    op.device = group[0].buffer.device().index;
    op.sourceDevice = group[0].sourceDevice.index;
    op.items = std::move(group);
    auto early = earlyLaunched_.find(op.seq);
    if (early != earlyLaunched_.end()) {
      op.notice = std::move(early->second);
      earlyLaunched_.erase(early);
    }
    // Same rule as the sender's: small batches after the arena announcement arrive eagerly.
    auto a = arenas_.find(op.device);
    uint64_t total = 0;
    for (auto& it : op.items) total += alignUp(it.length);
    const uint64_t threshold = std::min<uint64_t>(opts_.eagerThreshold, opts_.inboxBytes / 2);
    op.expectEager = !sameProcess_ && op.sourceDevice >= 0 && a != arenas_.end() && a->second.announcedSeq >= 0 &&
        static_cast<int64_t>(op.seq) > a->second.announcedSeq && total <= threshold;
    if (peerLeft_ && !op.notice) {
      // Nothing announces this batch any more.
      closeFromLoop(TPB_CREATE_ERROR(ChannelClosedError));
      for (auto& it : op.items) it.callback(error_);
      continue;
    }
    recvOps_.push_back(std::move(op));
    RecvOp& ref = recvOps_.back();
    if (ref.notice) completeRecv(ref);
    else if (helloDone_ && !ref.expectEager) sendReady(ref);
  }
  while (!recvOps_.empty() && recvOps_.front().items.empty()) recvOps_.pop_front();
  if (peerLeft_ && !error_ && earlyLaunched_.empty()) closeFromLoop(TPB_CREATE_ERROR(ChannelClosedError));
}

void ChannelImpl::sendReady(RecvOp& op) {
  if (error_) return;
  trace::Scope traced("p2p.recv.ready", op.seq);
  RecvReady r;
  r.seq = op.seq;
  r.deviceIdx = op.device;
  try {
    Error err;
    Arena* a = sameProcess_ ? nullptr : arenaFor(op.device, err);
    if (!sameProcess_ && !a) return closeFromLoop(err);
    if (a && a->announcedSeq < 0) {
      ArenaWire w;
      w.handle = a->handle;
      w.address = reinterpret_cast<uint64_t>(a->base);
      w.inboxBytes = a->inboxBytes;
      w.eagerThreshold = opts_.eagerThreshold;
      r.arena = w;
      a->announcedSeq = static_cast<int64_t>(op.seq);
    }
    // The driver queries below need this device's context current on the calling thread, which
    // may be a transport thread that never touched CUDA.
    CudaDeviceGuard g(op.device);
    auto regionOf = [&](const ExportCache::Entry& exported) {
      auto known = regionIds_.find(exported.id);
      if (known != regionIds_.end()) return known->second;
      RegionWire w;
      w.id = nextRegionId_++;
      w.handle = exported.handle;
      w.size = exported.size;
      r.newRegions.push_back(w);
      regionIds_.emplace(exported.id, w.id);
      return w.id;
    };
    for (auto& it : op.items) {
      TargetWire t;
      void* ptr = it.buffer.unwrap<CudaBuffer>().ptr;
      t.dtype = it.castTo ? static_cast<uint8_t>(*it.castTo) : 0;
      t.srcDtype = static_cast<uint8_t>(it.srcDtype);
      // Bytes the destination holds; the sender checks them against what it is about to write.
      t.bytes = it.castTo ? kernels::convertedBytes(it.length, it.srcDtype, *it.castTo) : it.length;
      if (sameProcess_) {
        t.offset = reinterpret_cast<uint64_t>(ptr);
      } else {
        ExportCache::Entry exported;
        if (ExportCache::get().lookup(ptr, &exported)) {
          t.region = regionOf(exported);
          t.offset = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(ptr) - exported.base);
        } else {
          // Not exportable: let the sender write into a staging buffer of ours instead.
          size_t index = 0;
          uint8_t* stage = takeStaging(op.device, t.bytes, &index);
          if (stage && ExportCache::get().lookup(stage, &exported)) {
            t.region = regionOf(exported);
            t.offset = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(stage) - exported.base);
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

// Whether the data of this batch comes from a GPU other than the one receiving it. Only then may
// the unpack kernel itself wait for the sender: a kernel never spins on what another launch on
// its own GPU produces.
bool ChannelImpl::sourceIsOtherGpu(const RecvOp& op) const {
  if (op.sourceDevice < 0 || op.device < 0) return false;
  if (static_cast<size_t>(op.sourceDevice) >= peerUuids_.size() || static_cast<size_t>(op.device) >= myUuids_.size())
    return false;
  return peerUuids_[op.sourceDevice] != myUuids_[op.device];
}

void ChannelImpl::completeRecv(RecvOp& op) {
  trace::Scope traced("p2p.recv.complete", op.seq);
  const Launched& n = *op.notice;
  TPB_VLOG(6) << "Channel " << id_ << " learnt that batch #" << op.seq << " is on its way"
              << (n.eager ? " (eager)" : "") << "; making the stream wait";
  if (!n.error.empty()) return closeFromLoop(TPB_CREATE_ERROR(CudaError, n.error));
  if (bool(n.eager) != op.expectEager)
    return closeFromLoop(TPB_CREATE_ERROR(LogicError, "the two ends disagree on how a batch travels"));
  try {
    CudaDeviceGuard g(op.device);
    cudaStream_t stream = static_cast<cudaStream_t>(op.items[0].buffer.unwrap<CudaBuffer>().stream);
    std::vector<cudaStream_t> others;
    for (auto& it : op.items) {
      cudaStream_t s = static_cast<cudaStream_t>(it.buffer.unwrap<CudaBuffer>().stream);
      if (s != stream && std::find(others.begin(), others.end(), s) == others.end()) others.push_back(s);
    }
    Error err;
    Arena* a = sameProcess_ ? nullptr : arenaFor(op.device, err);
    if (!sameProcess_ && !a) return closeFromLoop(err);
    if (sameProcess_) {
      if (n.eager || !n.event)
        return closeFromLoop(TPB_CREATE_ERROR(LogicError, "a push within one process must come with its event"));
      TPB_CUDA_CHECK(cudaStreamWaitEvent(stream, reinterpret_cast<cudaEvent_t>(n.event), 0));
    }
    uint32_t* flag = a ? a->flag(op.seq) : nullptr;
    const uint32_t value = flagValueFor(op.seq);
    if (a) {
      a->awaited[op.seq % kFlagSlots] = value;
      a->anyWait = true;
    }
    const CudaLib& lib = CudaLib::get();
    const bool fuse = n.eager && opts_.fuseWaitIntoUnpack && op.staged.empty() && sourceIsOtherGpu(op);
    bool watchStatus = false;
    if (!fuse && !sameProcess_) {
      if (!opts_.waitWithKernel && lib.cuStreamWaitValue32) {
        trace::Scope w("p2p.recv.waitvalue", op.seq);
        int rc = lib.cuStreamWaitValue32(stream, reinterpret_cast<CUdeviceptr_t>(flag), value, CudaLib::kWaitGeq);
        if (rc != 0) return closeFromLoop(TPB_CREATE_ERROR(CudaError, "cuStreamWaitValue32: " + lib.errorString(rc)));
      } else {
        kernels::launchWaitFlag(stream, flag, value, opts_.waitTimeoutNs, statusWord());
        watchStatus = true;
      }
    }
    if (n.eager) {
      // Unpack inbox -> tensors on the receiver's stream, applying the requested casts.
      trace::Scope u("p2p.recv.unpack", op.seq);
      kernels::PushPlan plan;
      {
        uint64_t bulkBytes = 0;
        const uint64_t bulkMin = kernels::getPushTuning().bulkMinBytes;
        for (auto& it : op.items)
          if (!it.castTo && it.length >= bulkMin) bulkBytes += it.length;
        kernels::chooseBulkTile(plan, bulkBytes, allCtas(op.device));
      }
      uint64_t cursor = n.inboxOffset;
      for (auto& it : op.items) {
        if (cursor + it.length > a->inboxBytes)
          return closeFromLoop(TPB_CREATE_ERROR(LogicError, "peer placed an eager batch outside the inbox"));
        kernels::CopyItem c;
        c.src = a->inbox() + cursor;
        c.dst = it.buffer.unwrap<CudaBuffer>().ptr;
        c.srcBytes = it.length;
        if (it.castTo) {
          c.srcDtype = it.srcDtype;
          c.dstDtype = *it.castTo;
        }
        kernels::appendToPlan(plan, c, opts_.useBulkCopy);
        cursor += alignUp(it.length);
      }
      kernels::WaitBefore wait;
      if (fuse) {
        wait.flag = flag;
        wait.value = value;
        wait.timeoutNs = opts_.waitTimeoutNs;
      }
      // The sender keeps at most 254 eager batches unacknowledged, so neither the counter nor the
      // completion word of this unpack can still belong to an earlier one.
      kernels::DoneSlot done;
      done.slot = a->unpackDone + (a->unpacksQueued % kFlagSlots);
      done.value = static_cast<uint32_t>(a->unpacksQueued + 1);
      kernels::launchPush(plan, stream, allCtas(op.device), nullptr, 0, a->unpackCounter(a->unpacksQueued), statusWord(),
                          wait, done);
      ++a->unpacksQueued;
      a->creditValues.push_back(n.creditValue);
      if (a->creditWanted) answerCreditRequest(*a);
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
      kernels::launchPush(plan, stream, allCtas(op.device), nullptr, 0, nullptr, nullptr);
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
    if (watchStatus) {
      // With the wait kernel (not the default) every wait is followed up: should it run out, the
      // channel fails as soon as the stream gets there.
      auto ev = std::shared_ptr<CudaEvent>(takeEvent(op.device).release());
      ev->record(stream);
      auto self = shared_from_this();
      cudaEvent_t raw = ev->raw();
      ctx_->poller_.watch([raw]() { return cudaEventQuery(raw) != cudaErrorNotReady; },
                          [self, ev]() { self->ctx_->loop_.deferToLoop([self, ev]() { self->deviceFailed(); }); });
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

std::unique_ptr<CudaEvent> ChannelImpl::takeEvent(int device) {
  auto& pool = freeEvents_[device];
  if (pool.empty()) return std::make_unique<CudaEvent>(device);
  auto ev = std::move(pool.back());
  pool.pop_back();
  return ev;
}

void ChannelImpl::recycleEvent(std::unique_ptr<CudaEvent> ev) {
  auto& pool = freeEvents_[ev->device()];
  if (pool.size() < 64) pool.push_back(std::move(ev));
}

void ChannelImpl::advanceUnpacks(Arena& arena) {
  const volatile uint32_t* done = arena.unpackDone;
  while (arena.unpacksDone < arena.unpacksQueued &&
         done[arena.unpacksDone % kFlagSlots] == static_cast<uint32_t>(arena.unpacksDone + 1)) {
    arena.freedUpTo = arena.creditValues.front();
    arena.creditValues.pop_front();
    ++arena.unpacksDone;
  }
}

// The sender wants inbox space back. Space is free once the unpack kernels that read it have
// finished, which their completion words tell. If nothing new has finished since the last answer,
// the request stays open: while unpacks are in flight a poller entry watches the next completion
// word, otherwise the next unpack to be enqueued picks the request up.
void ChannelImpl::answerCreditRequest(Arena& arena) {
  arena.creditWanted = true;
  if (error_) return;
  advanceUnpacks(arena);
  if (arena.unpacksDone > arena.creditSent) {
    arena.creditWanted = false;
    arena.creditSent = arena.unpacksDone;
    Credit c;
    c.deviceIdx = arena.device;
    c.value = arena.freedUpTo;
    c.count = arena.unpacksDone;
    writePacket(c);
    return;
  }
  if (arena.creditWatching || arena.unpacksDone == arena.unpacksQueued) return;
  arena.creditWatching = true;
  auto self = shared_from_this();
  const int device = arena.device;
  const volatile uint32_t* word = arena.unpackDone + (arena.unpacksDone % kFlagSlots);
  const uint32_t want = static_cast<uint32_t>(arena.unpacksDone + 1);
  ctx_->poller_.watch([self, word, want]() { return *word == want; },
                      [self, device]() {
                        self->ctx_->loop_.deferToLoop([self, device]() {
                          auto a = self->arenas_.find(device);
                          if (a == self->arenas_.end()) return;
                          a->second.creditWatching = false;
                          if (self->deviceFailed()) return;
                          if (a->second.creditWanted) self->answerCreditRequest(a->second);
                        });
                      });
}

void ChannelImpl::onPacket(Packet p) {
  if (std::holds_alternative<Bye>(p)) {
    byeReceived_ = true;
    if (!error_) onPeerLeft();
    else if (byeSent_) finishClose();
    return;
  }
  if (error_ || deviceFailed()) return;
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
        return;
      }
    }
    earlyLaunched_.emplace(l.seq, std::move(l));
  } else if (std::holds_alternative<Credit>(p)) {
    const Credit& c = std::get<Credit>(p);
    auto it = peerArenas_.find(c.deviceIdx);
    if (it != peerArenas_.end()) {
      if (c.value > it->second.tail) it->second.tail = c.value;
      if (c.count > it->second.eagerAcked) it->second.eagerAcked = c.count;
      it->second.creditRequested = false;
    }
    pumpSends();
  } else if (std::holds_alternative<CreditRequest>(p)) {
    auto a = arenas_.find(std::get<CreditRequest>(p).deviceIdx);
    if (a != arenas_.end()) answerCreditRequest(a->second);
  }
}

// The peer closed its end in good order: everything it launched has finished, nothing more will
// come. Batches that it pushed into the inbox and announced before leaving can still be received
// (their data is already here); anything else is over.
void ChannelImpl::onPeerLeft() {
  peerLeft_ = true;
  const Error gone = TPB_CREATE_ERROR(ChannelClosedError);
  auto sends = std::move(sendOps_);
  sendOps_.clear();
  for (auto& op : sends)
    for (auto& it : op.items) it.callback(gone);
  auto recvs = std::move(recvOps_);
  recvOps_.clear();
  for (auto& op : recvs)
    for (auto& it : op.items) it.callback(gone);  // no push was announced for these, so none happened
  if (earlyLaunched_.empty()) closeFromLoop(gone);
}

void ChannelImpl::close() {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self]() { self->closeFromLoop(TPB_CREATE_ERROR(ChannelClosedError)); });
}

void ChannelImpl::closeFromLoop(const Error& e, bool connectionBroken) {
  if (error_) return;
  error_ = e;
  auto self = shared_from_this();
  TPB_VLOG(4) << "Channel " << id_ << " is closing: " << e.what();
  // Release every stream still parked on a flag that may now never be written: put the awaited
  // values there from the host so the streams drain (the error reaches the user through
  // callbacks). Every slot a wait was ever enqueued for is covered, however long ago.
  for (auto& entry : arenas_) {
    Arena& a = entry.second;
    if (!a.anyWait) continue;
    try {
      CudaDeviceGuard g(a.device);
      // On a private non-blocking stream: the user's stream (possibly the legacy default stream,
      // which blocking calls would queue behind) is exactly what is stuck.
      cudaStream_t s = nullptr;
      if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) == cudaSuccess) {
        for (uint32_t slot = 0; slot < kFlagSlots; ++slot)
          if (a.awaited[slot] != 0)
            cudaMemcpyAsync(reinterpret_cast<uint32_t*>(a.base) + slot, &a.awaited[slot], sizeof(uint32_t),
                            cudaMemcpyHostToDevice, s);
        cudaStreamSynchronize(s);
        cudaStreamDestroy(s);
      }
      cudaGetLastError();
    } catch (...) {
    }
    a.anyWait = false;
  }
  auto sends = std::move(sendOps_);
  auto recvs = std::move(recvOps_);
  sendOps_.clear();
  recvOps_.clear();
  for (auto& op : sends) {
    releaseEarly(op);
    for (auto& it : op.items) it.callback(error_);
  }
  for (auto& op : recvs) {
    if (op.items.empty()) continue;
    // Buffers the peer has been told about and whose push has not been announced: a kernel of
    // the peer may be writing them right now, or may start to. They go back to the user only
    // once the peer has said goodbye (or cannot say anything any more).
    if (op.readySent && !op.notice && !connectionBroken && helloDone_) {
      held_.push_back(std::move(op));
      continue;
    }
    for (auto& it : op.items) it.callback(error_);
  }
  if (connectionBroken) return finishClose();
  if (!helloDone_) {
    // The goodbye is owed once the peer's hello has been read; without a usable connection
    // that never happens and the read fails instead. Nothing is held at this point.
    std::weak_ptr<ChannelImpl> weak = self;
    TimerThread::get().schedule(std::chrono::milliseconds(opts_.closeTimeoutMs), [weak]() {
      if (auto self = weak.lock()) self->ctx_->loop_.deferToLoop([self]() { self->finishClose(); });
    });
    return;
  }
  // Goodbye goes out once everything this end launched has finished.
  sendByeWhenIdle();
  std::weak_ptr<ChannelImpl> weak = self;
  TimerThread::get().schedule(std::chrono::milliseconds(opts_.closeTimeoutMs), [weak]() {
    if (auto self = weak.lock()) self->ctx_->loop_.deferToLoop([self]() { self->finishClose(); });
  });
}

void ChannelImpl::sendByeWhenIdle() {
  if (byeSent_ || finished_) return;
  auto self = shared_from_this();
  if (sameProcess_) {
    // The newest event stands for every push before it: they ran on streams the user ordered.
    if (!lastPushEvent_ || cudaEventQuery(lastPushEvent_->raw()) != cudaErrorNotReady) return sendBye();
    cudaEvent_t raw = lastPushEvent_->raw();
    ctx_->poller_.watch([raw]() { return cudaEventQuery(raw) != cudaErrorNotReady; },
                        [self]() { self->ctx_->loop_.deferToLoop([self]() { self->sendBye(); }); });
    return;
  }
  advanceConfirmed();
  if (confirmed_ == launchedUpTo_) return sendBye();
  whenPushFinishes(confirmed_, [self]() { self->sendByeWhenIdle(); });
}

void ChannelImpl::sendBye() {
  if (byeSent_ || finished_) return;
  byeSent_ = true;
  writePacket(Bye{});
  if (byeReceived_) finishClose();
}

// Last step of closing: the receives that were kept back report the error, the connection goes.
void ChannelImpl::finishClose() {
  if (finished_) return;
  if (!error_) error_ = TPB_CREATE_ERROR(ChannelClosedError);
  finished_ = true;
  auto self = shared_from_this();
  auto held = std::move(held_);
  held_.clear();
  for (auto& op : held)
    for (auto& it : op.items) it.callback(error_);
  for (auto& entry : asideStreams_) {
    try {
      CudaDeviceGuard g(entry.first);
      cudaStreamDestroy(entry.second);  // what is queued on it still runs to the end
    } catch (...) {
    }
  }
  asideStreams_.clear();
  conn_->close();
  ctx_->unenroll(self);
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
  num("TPB_CUDA_P2P_FUSED_WAIT", o.fuseWaitIntoUnpack);
  num("TPB_CUDA_P2P_BULK", o.useBulkCopy);
  num("TPB_CUDA_P2P_CLOSE_TIMEOUT_MS", o.closeTimeoutMs);
  num("TPB_CUDA_P2P_HOST_COPY_MIN_BYTES", o.hostCopyMinBytes);
  num("TPB_CUDA_P2P_HOST_PIECE_BYTES", o.hostPieceBytes);
  num("TPB_CUDA_P2P_SEND_ORDER_MIN_BYTES", o.sendOrderMinBytes);
  unsigned long long ms = o.waitTimeoutNs / 1'000'000ull;
  num("TPB_CUDA_P2P_WAIT_TIMEOUT_MS", ms);
  o.waitTimeoutNs = ms * 1'000'000ull;
  return o;
}

std::shared_ptr<Context> create(Options options) { return std::make_shared<ContextImpl>(applyEnvironment(options)); }

}  // namespace cuda_p2p
}  // namespace channel
}  // namespace tpb
