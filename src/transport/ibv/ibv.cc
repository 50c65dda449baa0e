// ibv: framed connections over RDMA. What travels and how:
//
//  * Bootstrap. A connection starts life as a connection of this library's TCP transport, over
//    which the two ends swap one Hello (queue-pair address, where the inbox ring lives and the key
//    to write it) and, once their queue pairs are ready to send, one Ready. Nobody posts RDMA work
//    before it has the peer's Ready. The TCP connection then stays open for one purpose: its end
//    of file is how a vanished peer is noticed.
//  * Data. Each end owns an inbox ring (registered memory the peer writes with RDMA writes) and an
//    outbox ring of the same size (registered memory the bytes are staged in, because the NIC reads
//    from registered memory only). The stream position is the same in both, so a byte staged at
//    outbox offset p lands at inbox offset p. The outbox is a three-party ring: the producer
//    copies frames in (4-byte length, then the bytes), the poster hands staged bytes to the NIC
//    as RDMA writes whose immediate says how many bytes they carry, the reclaimer frees them when
//    the NIC reports the write done. The inbox is a two-party ring: write-arrived completions
//    extend it, the reader consumes it.
//  * Credit. A poster never has more bytes on the wire or unconsumed at the peer than the inbox
//    holds. The reader returns consumed bytes with an empty send whose immediate is their count,
//    a quarter ring at a time or when the inbox runs empty.
//  * Closing. A write reports success once its bytes are staged, so an end that closes first
//    hands what is staged to the NIC (for a few seconds at most, should the peer not read) and
//    only then lets go of the queue pair and the TCP connection. The end that sees the TCP end of
//    file lets the completions that are already there come in, then serves reads from what its
//    inbox holds and fails the first read that it cannot serve.
//  * One completion queue, one shared receive queue and one polling thread per context; caps on
//    the writes and credit messages in flight over all its connections.
//
// Same job as tensorpipe/transport/ibv/* (connection_impl.cc:264-419, reactor.cc:80-220,
// constants.h:18-69: 2 MiB rings, 1024-deep queues, 32 completions per poll); the protocol is this
// library's own, so the domain descriptor is "tpbibv1:*" and a reference peer never pairs with it.
// Hardware comes through common/verbs.h: libibverbs when the machine has it, a software fabric in
// tests.
#include "transport/ibv/ibv.h"

#include <deque>
#include <map>
#include <unordered_map>
#include <unordered_set>

#include "common/busy_polling_loop.h"
#include "common/defs.h"
#include "common/memory.h"
#include "common/role_ring.h"
#include "common/timer.h"
#include "transport/nop_io.h"

namespace tpb {
namespace transport {
namespace ibv {

namespace {

constexpr uint64_t kRingBytes = 2u << 20;
constexpr int kReceiveDepth = 1024;
constexpr int kSendDepth = 1024;
constexpr int kCompletionDepth = 4096;
constexpr int kMaxWritesInFlight = 1000;
constexpr int kMaxCreditsInFlight = 1000;
constexpr int kPollBatch = 32;
constexpr int kDrainMs = 3000;  // how long a closing end keeps trying to deliver what is staged
const std::string kDomainDescriptor = "tpbibv1:*";

// Work-request ids: the kind in the top byte, a length below it.
enum : uint64_t { kIdWrite = 1, kIdCredit = 2, kIdReceive = 3 };
constexpr uint64_t makeId(uint64_t kind, uint64_t value) { return (kind << 56) | value; }
constexpr uint64_t idKind(uint64_t id) { return id >> 56; }
constexpr uint64_t idValue(uint64_t id) { return id & ((1ull << 56) - 1); }

struct Hello {
  uint32_t localId = 0;
  std::string gid;
  uint32_t queuePair = 0;
  uint32_t packetSequence = 0;
  uint32_t mtu = 0;
  uint64_t inboxAddress = 0;
  uint32_t inboxKey = 0;
  uint64_t ringBytes = 0;
  TPB_NOP_STRUCTURE(Hello, localId, gid, queuePair, packetSequence, mtu, inboxAddress, inboxKey, ringBytes)
};
struct Ready {
  uint32_t queuePair = 0;
  TPB_NOP_STRUCTURE(Ready, queuePair)
};

enum { kProducer = 0, kPoster = 1, kReclaimer = 2 };  // outbox parties
enum { kArrived = 0, kReader = 1 };                   // inbox parties

struct ReadOp {
  bool userBuffer = false;
  void* ptr = nullptr;
  size_t length = 0;
  Connection::read_callback_fn fn;
  bool haveHeader = false;
  uint32_t frameBytes = 0;
  size_t got = 0;
  std::vector<uint8_t> owned;
};

struct WriteOp {
  const uint8_t* ptr = nullptr;
  size_t length = 0;
  Connection::write_callback_fn fn;
  bool headerStaged = false;
  size_t staged = 0;
};

class ContextImpl;

class ConnectionImpl final : public std::enable_shared_from_this<ConnectionImpl> {
 public:
  ConnectionImpl(std::shared_ptr<ContextImpl> ctx, std::shared_ptr<Connection> boot) : ctx_(std::move(ctx)), boot_(std::move(boot)) {}
  void init();
  void read(ReadOp op);
  void write(WriteOp op);
  void close();
  // From the reactor.
  void onCompletion(const verbs::Completion& c);
  void retryPosting() { postWrites(); sendCredit(false); }
  // Ends the connection now: pending operations fail with `e`, staged bytes are dropped.
  void closeFromLoop(const Error& e);
  // Ends it once the staged bytes are out (or the drain time is up).
  void closeGracefully(const Error& e);

 private:
  void initFromLoop();
  void onHello(const Hello& h);
  void onReady();
  void watchBootstrap();
  void onPeerGone(const Error& e);
  bool outboxEmpty() const { return outbox_.released(kProducer) == outbox_.released(kReclaimer); }
  void processReads();
  void processWrites();
  void postWrites();
  void sendCredit(bool force);

  enum State { kNew, kWaitingForHello, kWaitingForReady, kEstablished, kDraining, kClosed };
  std::shared_ptr<ContextImpl> ctx_;
  std::shared_ptr<Connection> boot_;
  State state_ = kNew;
  Error error_;
  bool peerGone_ = false;   // the peer closed: reads are served from what the inbox holds
  bool peerLeaving_ = false;
  Error peerGoneError_;
  std::unique_ptr<verbs::QueuePair> qp_;
  uint32_t qpNumber_ = 0;
  bool registered_ = false;
  MmappedPtr inboxMem_, outboxMem_;
  std::unique_ptr<verbs::MemoryRegion> inboxRegion_, outboxRegion_;
  RoleRingHeader<2> inboxHeader_;
  RoleRingHeader<3> outboxHeader_;
  RoleRing<2> inbox_;
  RoleRing<3> outbox_;
  uint64_t peerInboxAddress_ = 0;
  uint32_t peerInboxKey_ = 0;
  uint64_t peerFree_ = 0;    // bytes the peer's inbox can still take
  uint64_t unreturned_ = 0;  // bytes consumed here whose credit has not gone back yet
  int writesInFlight_ = 0, creditsInFlight_ = 0;
  std::deque<ReadOp> reads_;
  std::deque<WriteOp> writes_;
};

class ListenerImpl;

class ContextImpl final : public BusyPollingLoop, public std::enable_shared_from_this<ContextImpl> {
 public:
  explicit ContextImpl(std::shared_ptr<verbs::Provider> provider) : provider_(std::move(provider)) {
    inner_ = tcp::create();
    if (!inner_->isViable()) {
      why_ = "the TCP transport it bootstraps over is not viable";
      return;
    }
    auto names = provider_->deviceNames();
    if (names.empty()) {
      why_ = provider_->whyUnavailable();
      return;
    }
    std::string pick = names.front();
    if (const char* env = std::getenv("TPB_IBV_DEVICE")) {
      for (auto& n : names)
        if (n == env) pick = n;
    }
    try {
      device_ = provider_->open(pick);
      cq_ = device_->createCompletionQueue(kCompletionDepth);
      srq_ = device_->createSharedReceiveQueue(kReceiveDepth);
      for (int i = 0; i < kReceiveDepth; ++i) srq_->postReceive(makeId(kIdReceive, 0));
    } catch (const std::exception& ex) {
      why_ = ex.what();
      cq_.reset();
      srq_.reset();
      device_.reset();
      return;
    }
    viable_ = true;
    startThread("TPB_IBV_reactor");
  }
  ~ContextImpl() override { join(); }

  bool viable() const { return viable_; }
  const std::string& why() const { return why_; }
  verbs::Device& device() { return *device_; }
  verbs::CompletionQueue& cq() { return *cq_; }
  verbs::SharedReceiveQueue& srq() { return *srq_; }
  Context& inner() { return *inner_; }
  bool closed() const { return closed_; }

  void enroll(std::shared_ptr<ConnectionImpl> c) { conns_.insert(std::move(c)); }
  void unenroll(const std::shared_ptr<ConnectionImpl>& c) { conns_.erase(c); }
  void enroll(std::shared_ptr<ListenerImpl> l) { listeners_.insert(std::move(l)); }
  void unenroll(const std::shared_ptr<ListenerImpl>& l) { listeners_.erase(l); }
  void bind(uint32_t qp, ConnectionImpl* c) { byQueuePair_[qp] = c; }
  void unbind(uint32_t qp) { byQueuePair_.erase(qp); }

  // The caps over all connections. A connection that could not post waits for wakeStalled().
  bool mayPostWrite() const { return writesInFlight_ < kMaxWritesInFlight; }
  bool mayPostCredit() const { return creditsInFlight_ < kMaxCreditsInFlight; }
  void countWrite(int d) { writesInFlight_ += d; }
  void countCredit(int d) { creditsInFlight_ += d; }
  void stalled(std::shared_ptr<ConnectionImpl> c) { stalled_.insert(std::move(c)); }
  // Runs `fn` on the loop once a poll of the completion queue has come back empty.
  void whenCompletionsRunDry(std::function<void()> fn) { runDry_.push_back(std::move(fn)); }

  void closeContext();
  void joinContext() {
    closeContext();
    if (viable_) BusyPollingLoop::join();  // returns once every connection has closed
    inner_->close();
    inner_->join();
  }

 protected:
  bool pollOnce() override {
    verbs::Completion batch[kPollBatch];
    int n = 0;
    try {
      n = cq_->poll(batch, kPollBatch);
    } catch (const std::exception& ex) {
      TPB_LOG_ERROR << "ibv: " << ex.what();
      return false;
    }
    for (int i = 0; i < n; ++i) {
      const verbs::Completion& c = batch[i];
      // Every arrival used up a receive of the shared queue, whoever it was for.
      if (c.work == verbs::Work::kWriteArrived || c.work == verbs::Work::kSendArrived || idKind(c.id) == kIdReceive) {
        try {
          srq_->postReceive(makeId(kIdReceive, 0));
        } catch (const std::exception& ex) {
          TPB_LOG_ERROR << "ibv: " << ex.what();
        }
      }
      auto it = byQueuePair_.find(c.queuePair);
      if (it == byQueuePair_.end()) continue;  // flushed work of a connection that is gone
      it->second->onCompletion(c);
    }
    if (n == 0 && !runDry_.empty()) {
      auto fns = std::move(runDry_);
      runDry_.clear();
      for (auto& f : fns) f();
      return true;
    }
    if (n > 0 && !stalled_.empty()) {
      auto again = std::move(stalled_);
      stalled_.clear();
      for (auto& c : again) c->retryPosting();
    }
    return n > 0;
  }
  bool readyToClose() override { return conns_.empty() && listeners_.empty(); }

 private:
  std::shared_ptr<verbs::Provider> provider_;
  std::shared_ptr<Context> inner_;
  std::unique_ptr<verbs::Device> device_;
  std::unique_ptr<verbs::CompletionQueue> cq_;
  std::unique_ptr<verbs::SharedReceiveQueue> srq_;
  bool viable_ = false;
  bool closed_ = false;
  std::string why_;
  std::unordered_set<std::shared_ptr<ConnectionImpl>> conns_;
  std::unordered_set<std::shared_ptr<ListenerImpl>> listeners_;
  std::unordered_set<std::shared_ptr<ConnectionImpl>> stalled_;
  std::vector<std::function<void()>> runDry_;
  std::unordered_map<uint32_t, ConnectionImpl*> byQueuePair_;
  int writesInFlight_ = 0, creditsInFlight_ = 0;
};

// ---- connection -----------------------------------------------------------------------------
void ConnectionImpl::init() {
  auto self = shared_from_this();
  ctx_->deferToLoop([self]() { self->initFromLoop(); });
}

void ConnectionImpl::initFromLoop() {
  ctx_->enroll(shared_from_this());
  if (ctx_->closed()) return closeFromLoop(TPB_CREATE_ERROR(ContextClosedError));
  try {
    Error e;
    std::tie(e, inboxMem_) = MmappedPtr::map(kRingBytes, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1);
    if (e) return closeFromLoop(e);
    std::tie(e, outboxMem_) = MmappedPtr::map(kRingBytes, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1);
    if (e) return closeFromLoop(e);
    inbox_ = RoleRing<2>(&inboxHeader_, static_cast<uint8_t*>(inboxMem_.ptr()), kRingBytes, true);
    outbox_ = RoleRing<3>(&outboxHeader_, static_cast<uint8_t*>(outboxMem_.ptr()), kRingBytes, true);
    inboxRegion_ = ctx_->device().registerMemory(inboxMem_.ptr(), kRingBytes);
    outboxRegion_ = ctx_->device().registerMemory(outboxMem_.ptr(), kRingBytes);
    qp_ = ctx_->device().createQueuePair(ctx_->cq(), ctx_->srq(), kSendDepth);
    qp_->toInit();
    qpNumber_ = qp_->number();
    ctx_->bind(qpNumber_, this);
    registered_ = true;
  } catch (const std::exception& ex) {
    return closeFromLoop(TPB_CREATE_ERROR(IbvError, ex.what()));
  }
  const verbs::Address port = ctx_->device().portAddress();
  Hello h;
  h.localId = port.localId;
  h.gid.assign(reinterpret_cast<const char*>(port.gid.data()), port.gid.size());
  h.queuePair = qpNumber_;
  h.packetSequence = 0;
  h.mtu = port.mtu;
  h.inboxAddress = reinterpret_cast<uint64_t>(inboxMem_.ptr());
  h.inboxKey = inboxRegion_->remoteKey();
  h.ringBytes = kRingBytes;
  state_ = kWaitingForHello;
  auto self = shared_from_this();
  writeNop(*boot_, h, [self](const Error& e) {
    if (e) self->ctx_->deferToLoop([self, e]() { self->closeFromLoop(e); });
  });
  readNop<Hello>(*boot_, [self](const Error& e, Hello peer) {
    self->ctx_->deferToLoop([self, e, peer = std::move(peer)]() {
      if (self->state_ != kWaitingForHello) return;
      if (e) return self->closeFromLoop(e);
      self->onHello(peer);
    });
  });
}

void ConnectionImpl::onHello(const Hello& h) {
  if (h.ringBytes != kRingBytes || h.gid.size() != 16)
    return closeFromLoop(TPB_CREATE_ERROR(IbvError, "the peer's greeting does not fit this transport"));
  verbs::Address remote;
  remote.localId = h.localId;
  std::memcpy(remote.gid.data(), h.gid.data(), 16);
  remote.queuePair = h.queuePair;
  remote.packetSequence = h.packetSequence;
  remote.mtu = static_cast<uint8_t>(h.mtu);
  try {
    qp_->toReadyToReceive(remote);
    qp_->toReadyToSend(0);
  } catch (const std::exception& ex) {
    return closeFromLoop(TPB_CREATE_ERROR(IbvError, ex.what()));
  }
  peerInboxAddress_ = h.inboxAddress;
  peerInboxKey_ = h.inboxKey;
  peerFree_ = kRingBytes;
  state_ = kWaitingForReady;
  auto self = shared_from_this();
  Ready r;
  r.queuePair = qpNumber_;
  writeNop(*boot_, r, [self](const Error& e) {
    if (e) self->ctx_->deferToLoop([self, e]() { self->closeFromLoop(e); });
  });
  readNop<Ready>(*boot_, [self](const Error& e, Ready) {
    self->ctx_->deferToLoop([self, e]() {
      if (self->state_ != kWaitingForReady) return;
      if (e) return self->closeFromLoop(e);
      self->onReady();
    });
  });
}

void ConnectionImpl::onReady() {
  state_ = kEstablished;
  watchBootstrap();
  processWrites();
  processReads();
}

// Nothing more is expected on the bootstrap connection: whatever comes (end of file when the peer
// goes away, an error) ends this connection.
void ConnectionImpl::watchBootstrap() {
  auto self = shared_from_this();
  boot_->read([self](const Error& e, const void*, size_t) {
    self->ctx_->deferToLoop([self, e]() {
      if (self->state_ == kClosed) return;
      const Error why = e ? e : TPB_CREATE_ERROR(EOFError);
      if (self->state_ == kDraining) return self->closeFromLoop(self->error_);
      self->onPeerGone(why);
    });
  });
}

// The peer has closed (or is unreachable). What it wrote before that has been placed in the inbox
// already; its completions may still sit in the queue, so wait until a poll comes back empty.
void ConnectionImpl::onPeerGone(const Error& e) {
  if (peerLeaving_ || state_ == kClosed) return;
  peerLeaving_ = true;
  peerGoneError_ = e;
  auto self = shared_from_this();
  ctx_->whenCompletionsRunDry([self]() {
    if (self->state_ != kEstablished) return;
    self->peerGone_ = true;
    auto writes = std::move(self->writes_);
    self->writes_.clear();
    for (auto& w : writes) w.fn(self->peerGoneError_);
    self->processReads();
  });
}

void ConnectionImpl::read(ReadOp op) {
  auto self = shared_from_this();
  ctx_->deferToLoop([self, op = std::move(op)]() mutable {
    if (self->state_ == kClosed || self->state_ == kDraining) {
      op.fn(self->error_, nullptr, 0);
      return;
    }
    self->reads_.push_back(std::move(op));
    if (self->state_ == kEstablished) self->processReads();
  });
}

void ConnectionImpl::write(WriteOp op) {
  auto self = shared_from_this();
  ctx_->deferToLoop([self, op = std::move(op)]() mutable {
    if (self->state_ == kClosed || self->state_ == kDraining || self->peerGone_) {
      op.fn(self->peerGone_ && self->state_ == kEstablished ? self->peerGoneError_ : self->error_);
      return;
    }
    self->writes_.push_back(std::move(op));
    if (self->state_ == kEstablished) self->processWrites();
  });
}

void ConnectionImpl::close() {
  auto self = shared_from_this();
  ctx_->deferToLoop([self]() { self->closeGracefully(TPB_CREATE_ERROR(ConnectionClosedError)); });
}

void ConnectionImpl::closeGracefully(const Error& e) {
  if (state_ == kClosed || state_ == kDraining) return;
  TPB_VLOG(7) << "ibv connection (queue pair " << qpNumber_ << ") is asked to close; staged " << outbox_.released(kProducer)
              << ", posted " << outbox_.released(kPoster) << ", done " << outbox_.released(kReclaimer);
  if (state_ != kEstablished || peerLeaving_ || outboxEmpty()) return closeFromLoop(e);
  state_ = kDraining;
  error_ = e;
  auto reads = std::move(reads_);
  auto writes = std::move(writes_);
  reads_.clear();
  writes_.clear();
  for (auto& r : reads) r.fn(e, nullptr, 0);
  for (auto& w : writes) w.fn(e);  // not (fully) staged: the peer will see the stream end inside that frame
  std::weak_ptr<ConnectionImpl> weak = shared_from_this();
  auto ctx = ctx_;
  TimerThread::get().schedule(std::chrono::milliseconds(kDrainMs), [weak, ctx]() {
    if (auto self = weak.lock()) ctx->deferToLoop([self]() { self->closeFromLoop(self->error_); });
  });
  postWrites();
}

void ConnectionImpl::processWrites() {
  bool stagedAny = false;
  {
    auto tx = outbox_.begin(kProducer);
    TPB_DCHECK(tx.open());
    while (!writes_.empty()) {
      WriteOp& op = writes_.front();
      if (!op.headerStaged) {
        const uint32_t len = static_cast<uint32_t>(op.length);
        if (!tx.write(&len, sizeof(len))) break;
        op.headerStaged = true;
        stagedAny = true;
      }
      const uint64_t n = std::min<uint64_t>(tx.available(), op.length - op.staged);
      if (n > 0) {
        tx.write(op.ptr + op.staged, n);
        op.staged += n;
        stagedAny = true;
      }
      if (op.staged < op.length) break;  // the ring is full; more when the NIC frees some
      // The bytes are staged: the caller's buffer is free again, which is what the callback says.
      auto fn = std::move(op.fn);
      writes_.pop_front();
      tx.commit();
      fn(Error::kSuccess);
      if (state_ != kEstablished) return;
      tx = outbox_.begin(kProducer);
    }
    tx.commit();
  }
  if (stagedAny) postWrites();
}

void ConnectionImpl::postWrites() {
  if (state_ != kEstablished && state_ != kDraining) return;
  if (peerGone_) return;
  auto tx = outbox_.begin(kPoster);
  TPB_DCHECK(tx.open());
  const uint32_t maxMessage = ctx_->device().maxMessageBytes();
  bool capped = false;
  try {
    while (tx.available() > 0 && peerFree_ > 0) {
      if (!ctx_->mayPostWrite()) {
        capped = true;
        break;
      }
      uint64_t n = std::min<uint64_t>(tx.available(), peerFree_);
      RoleRing<3>::Span runs[2];
      tx.span(n, runs);
      // One contiguous run per work request, no longer than the NIC takes.
      n = std::min<uint64_t>(runs[0].length, maxMessage);
      const uint64_t offset = tx.position() & (kRingBytes - 1);
      qp_->postWriteWithImmediate(makeId(kIdWrite, n), runs[0].ptr, static_cast<uint32_t>(n), outboxRegion_->localKey(),
                                  peerInboxAddress_ + offset, peerInboxKey_, static_cast<uint32_t>(n));
      tx.advance(n);
      peerFree_ -= n;
      ++writesInFlight_;
      ctx_->countWrite(+1);
    }
  } catch (const std::exception& ex) {
    tx.commit();
    return closeFromLoop(TPB_CREATE_ERROR(IbvError, ex.what()));
  }
  tx.commit();
  if (capped) ctx_->stalled(shared_from_this());
}

void ConnectionImpl::processReads() {
  uint64_t consumed = 0;
  {
    auto tx = inbox_.begin(kReader);
    TPB_DCHECK(tx.open());
    while (state_ == kEstablished && !reads_.empty()) {
      ReadOp& op = reads_.front();
      if (!op.haveHeader) {
        uint32_t len = 0;
        if (!tx.read(&len, sizeof(len))) break;
        consumed += sizeof(len);
        op.haveHeader = true;
        op.frameBytes = len;
        if (op.userBuffer) {
          if (len != op.length) {
            tx.commit();
            return closeFromLoop(TPB_CREATE_ERROR(IbvError, "a frame of " + std::to_string(len) + " bytes arrived where " +
                                                               std::to_string(op.length) + " were expected"));
          }
        } else {
          if (len > kMaxAllocatedFrame) {
            tx.commit();
            return closeFromLoop(TPB_CREATE_ERROR(IbvError, "the peer announced a frame larger than this side allocates"));
          }
          op.owned.resize(len);
          op.ptr = op.owned.data();
          op.length = len;
        }
      }
      const uint64_t n = std::min<uint64_t>(tx.available(), op.length - op.got);
      if (n > 0) {
        tx.read(static_cast<uint8_t*>(op.ptr) + op.got, n);
        op.got += n;
        consumed += n;
      }
      if (op.got < op.length) break;
      ReadOp done = std::move(op);
      reads_.pop_front();
      tx.commit();
      unreturned_ += consumed;
      consumed = 0;
      done.fn(Error::kSuccess, done.ptr, done.length);
      if (state_ != kEstablished) return;
      tx = inbox_.begin(kReader);
    }
    tx.commit();
  }
  unreturned_ += consumed;
  // With the peer gone, the first read that what is left cannot serve ends the connection.
  if (peerGone_ && state_ == kEstablished && !reads_.empty()) {
    TPB_VLOG(7) << "ibv connection (queue pair " << qpNumber_ << "): the peer left with " << reads_.size()
                << " reads unserved; the first has " << reads_.front().got << " of " << reads_.front().length
                << " bytes, the inbox holds " << inbox_.ahead(kReader) << ", arrived " << inbox_.released(kArrived);
    return closeFromLoop(peerGoneError_);
  }
  sendCredit(false);
}

// Tell the peer how much of its view of our inbox is free again. Small amounts wait until they
// add up to a quarter ring, unless the inbox has run empty (the peer may be waiting for exactly
// these bytes) or `force`.
void ConnectionImpl::sendCredit(bool force) {
  if (state_ != kEstablished || unreturned_ == 0 || peerLeaving_) return;
  if (!force && unreturned_ < kRingBytes / 4 && inbox_.ahead(kReader) != 0) return;
  if (!ctx_->mayPostCredit()) {
    ctx_->stalled(shared_from_this());
    return;
  }
  try {
    qp_->postSendWithImmediate(makeId(kIdCredit, unreturned_), nullptr, 0, 0, static_cast<uint32_t>(unreturned_));
  } catch (const std::exception& ex) {
    return closeFromLoop(TPB_CREATE_ERROR(IbvError, ex.what()));
  }
  unreturned_ = 0;
  ++creditsInFlight_;
  ctx_->countCredit(+1);
}

void ConnectionImpl::onCompletion(const verbs::Completion& c) {
  if (state_ == kClosed) return;
  // Own work first (told apart by id, which a failed completion still carries).
  if (idKind(c.id) == kIdWrite) {
    --writesInFlight_;
    ctx_->countWrite(-1);
    if (!c.ok) return closeFromLoop(TPB_CREATE_ERROR(IbvError, c.error));
    auto tx = outbox_.begin(kReclaimer);
    tx.advance(idValue(c.id));
    tx.commit();
    if (state_ == kDraining) {
      if (outboxEmpty()) return closeFromLoop(error_);
      return postWrites();
    }
    processWrites();
    return;
  }
  if (idKind(c.id) == kIdCredit) {
    --creditsInFlight_;
    ctx_->countCredit(-1);
    // A credit that found nobody: the peer has left; what it sent before is still ours to read.
    if (!c.ok && state_ == kEstablished) return onPeerGone(TPB_CREATE_ERROR(EOFError));
    if (!c.ok) return closeFromLoop(TPB_CREATE_ERROR(IbvError, c.error));
    return;
  }
  if (!c.ok) return closeFromLoop(TPB_CREATE_ERROR(IbvError, c.error));
  if (state_ == kDraining && c.work == verbs::Work::kWriteArrived) return;  // nobody reads any more
  if (c.work == verbs::Work::kWriteArrived) {
    auto tx = inbox_.begin(kArrived);
    if (c.immediate > tx.available()) {
      tx.cancel();
      return closeFromLoop(TPB_CREATE_ERROR(IbvError, "the peer wrote more than the inbox had room for"));
    }
    tx.advance(c.immediate);
    tx.commit();
    processReads();
  } else if (c.work == verbs::Work::kSendArrived) {
    peerFree_ += c.immediate;
    if (peerFree_ > kRingBytes) return closeFromLoop(TPB_CREATE_ERROR(IbvError, "the peer returned more credit than it was given"));
    postWrites();
  }
}

void ConnectionImpl::closeFromLoop(const Error& e) {
  if (state_ == kClosed) return;
  state_ = kClosed;
  error_ = e;
  TPB_VLOG(7) << "ibv connection (queue pair " << qpNumber_ << ") closes: " << e.what();
  if (qp_) {
    try {
      qp_->toError();
    } catch (...) {
    }
  }
  if (registered_) ctx_->unbind(qpNumber_);
  ctx_->countWrite(-writesInFlight_);
  ctx_->countCredit(-creditsInFlight_);
  writesInFlight_ = creditsInFlight_ = 0;
  boot_->close();
  auto reads = std::move(reads_);
  auto writes = std::move(writes_);
  reads_.clear();
  writes_.clear();
  for (auto& r : reads) r.fn(e, nullptr, 0);
  for (auto& w : writes) w.fn(e);
  qp_.reset();
  inboxRegion_.reset();
  outboxRegion_.reset();
  ctx_->unenroll(shared_from_this());
}

class ConnectionShell final : public Connection {
 public:
  ConnectionShell(std::shared_ptr<ContextImpl> ctx, std::shared_ptr<Connection> boot)
      : impl_(std::make_shared<ConnectionImpl>(std::move(ctx), std::move(boot))) {
    impl_->init();
  }
  ~ConnectionShell() override { impl_->close(); }
  void read(read_callback_fn fn) override {
    ReadOp op;
    op.fn = std::move(fn);
    impl_->read(std::move(op));
  }
  void read(void* ptr, size_t length, read_callback_fn fn) override {
    ReadOp op;
    op.userBuffer = true;
    op.ptr = ptr;
    op.length = length;
    op.fn = std::move(fn);
    impl_->read(std::move(op));
  }
  void write(const void* ptr, size_t length, write_callback_fn fn) override {
    if (length > UINT32_MAX) {
      // The frame header is 32 bits wide.
      fn(TPB_CREATE_ERROR(IbvError, "a frame must be shorter than 4 GiB"));
      return;
    }
    WriteOp op;
    op.ptr = static_cast<const uint8_t*>(ptr);
    op.length = length;
    op.fn = std::move(fn);
    impl_->write(std::move(op));
  }
  void setId(std::string) override {}
  void close() override { impl_->close(); }

 private:
  std::shared_ptr<ConnectionImpl> impl_;
};

// ---- listener -------------------------------------------------------------------------------
// The TCP listener does the accepting; every accepted bootstrap connection becomes a connection of
// this transport.
class ListenerImpl final : public std::enable_shared_from_this<ListenerImpl> {
 public:
  ListenerImpl(std::shared_ptr<ContextImpl> ctx, std::shared_ptr<Listener> inner) : ctx_(std::move(ctx)), inner_(std::move(inner)) {}
  void init() {
    auto self = shared_from_this();
    ctx_->deferToLoop([self]() {
      self->ctx_->enroll(self);
      if (self->ctx_->closed()) self->closeFromLoop();
    });
  }
  void accept(Listener::accept_callback_fn fn) {
    auto self = shared_from_this();
    inner_->accept([self, fn = std::move(fn)](const Error& e, std::shared_ptr<Connection> boot) {
      self->ctx_->deferToLoop([self, fn, e, boot]() {
        if (e) return fn(e, nullptr);
        if (self->closed_) {
          boot->close();
          return fn(TPB_CREATE_ERROR(ListenerClosedError), nullptr);
        }
        fn(Error::kSuccess, std::make_shared<ConnectionShell>(self->ctx_, boot));
      });
    });
  }
  std::string addr() const { return inner_->addr(); }
  void close() {
    auto self = shared_from_this();
    ctx_->deferToLoop([self]() { self->closeFromLoop(); });
  }
  void closeFromLoop() {
    if (closed_) return;
    closed_ = true;
    inner_->close();
    ctx_->unenroll(shared_from_this());
  }

 private:
  std::shared_ptr<ContextImpl> ctx_;
  std::shared_ptr<Listener> inner_;
  bool closed_ = false;
};

class ListenerShell final : public Listener {
 public:
  ListenerShell(std::shared_ptr<ContextImpl> ctx, std::shared_ptr<Listener> inner)
      : impl_(std::make_shared<ListenerImpl>(std::move(ctx), std::move(inner))) {
    impl_->init();
  }
  ~ListenerShell() override { impl_->close(); }
  void accept(accept_callback_fn fn) override { impl_->accept(std::move(fn)); }
  std::string addr() const override { return impl_->addr(); }
  void setId(std::string) override {}
  void close() override { impl_->close(); }

 private:
  std::shared_ptr<ListenerImpl> impl_;
};

void ContextImpl::closeContext() {
  if (!viable_) {
    inner_->close();
    return;
  }
  auto self = shared_from_this();
  deferToLoop([self]() {
    if (self->closed_) return;
    self->closed_ = true;
    auto conns = self->conns_;
    for (auto& c : conns) c->closeGracefully(TPB_CREATE_ERROR(ContextClosedError));
    auto listeners = self->listeners_;
    for (auto& l : listeners) l->closeFromLoop();
    // The TCP context under the bootstrap connections goes last (joinContext): a connection that
    // is still handing staged bytes to the NIC must not see its bootstrap connection fail.
    self->BusyPollingLoop::close();
  });
}

class ContextShell final : public Context {
 public:
  explicit ContextShell(std::shared_ptr<verbs::Provider> provider) : impl_(std::make_shared<ContextImpl>(std::move(provider))) {
    if (!impl_->viable()) TPB_VLOG(7) << "ibv transport is not viable: " << impl_->why();
  }
  ~ContextShell() override { join(); }
  std::shared_ptr<Connection> connect(std::string addr) override {
    if (!impl_->viable()) throw std::runtime_error("ibv transport is not viable");
    return std::make_shared<ConnectionShell>(impl_, impl_->inner().connect(std::move(addr)));
  }
  std::shared_ptr<Listener> listen(std::string addr) override {
    if (!impl_->viable()) throw std::runtime_error("ibv transport is not viable");
    return std::make_shared<ListenerShell>(impl_, impl_->inner().listen(std::move(addr)));
  }
  bool isViable() const override { return impl_->viable(); }
  const std::string& domainDescriptor() const override { return kDomainDescriptor; }
  void setId(std::string) override {}
  void close() override { impl_->closeContext(); }
  void join() override {
    if (joined_.exchange(true)) return;
    impl_->joinContext();
  }

 private:
  std::shared_ptr<ContextImpl> impl_;
  std::atomic<bool> joined_{false};
};

}  // namespace

std::shared_ptr<Context> createWithProvider(std::shared_ptr<verbs::Provider> provider) {
  return std::make_shared<ContextShell>(std::move(provider));
}

std::shared_ptr<Context> create() { return createWithProvider(verbs::systemProvider()); }

}  // namespace ibv
}  // namespace transport
}  // namespace tpb
