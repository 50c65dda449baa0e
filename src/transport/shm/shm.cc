// The shared-memory transport for two processes (or threads) on one host.
//
// What it keeps from the reference's design (tensorpipe/transport/shm/*, docs/shm.md): an
// abstract-namespace UNIX socket used only for bootstrap and for noticing that the peer died;
// one inbox ring per connection end, created by its reader and passed to the writer as a file
// descriptor (SCM_RIGHTS); frames are a 4-byte length followed by the payload and may be
// written/read in pieces when larger than the ring; and a per-context *reactor* that peers poke
// by pushing a small token into a shared token queue — the reader finds out about new data by
// polling memory, not through a system call.
//
// What is different: the reactor, the epoll set and the deferred-function queue are served by
// ONE thread, which spins while there is traffic and, after a short idle period, publishes a
// "sleeping" flag and blocks in epoll_wait on an eventfd that pokers write to only when they
// see the flag. Traffic keeps the microsecond latency of busy polling; an idle context costs
// no CPU. The segment layouts are this library's own, so the domain descriptor carries its own
// prefix and never matches a reference peer's "shm:" descriptor.
#include <sys/epoll.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <chrono>
#include <deque>
#include <set>
#include <vector>

#include <tpb/transport.h>

#include "common/busy_polling_loop.h"
#include "common/defs.h"
#include "common/loop.h"
#include "common/ringbuffer.h"
#include "common/shm_segment.h"
#include "common/socket.h"
#include "common/system.h"

namespace tpb {
namespace transport {
namespace shm {

namespace {

constexpr uint64_t kRingBytes = 2u << 20;        // per connection and direction
// A frame larger than this moves through the ring in pieces of this size: the writer publishes
// (and pokes the reader) after every piece and the reader frees after every piece, so that the
// two memcpys of a large frame overlap instead of taking turns with a whole ring at a time.
constexpr uint64_t kDefaultPieceBytes = 256u << 10;
// TPB_SHM_PIECE_BYTES overrides it (4 KiB to the whole ring), for tuning on a given CPU.
uint64_t pieceBytes() {
  static const uint64_t value = [] {
    const char* s = std::getenv("TPB_SHM_PIECE_BYTES");
    const uint64_t v = s ? std::strtoull(s, nullptr, 10) : 0;
    return v == 0 ? kDefaultPieceBytes : std::min<uint64_t>(std::max<uint64_t>(v, 4096), kRingBytes);
  }();
  return value;
}
// TPB_SHM_DIRECT_WRITE_MAX_BYTES: the largest frame that write() copies on the caller's thread.
uint64_t directWriteMaxBytes() {
  static const uint64_t value = [] {
    const char* s = std::getenv("TPB_SHM_DIRECT_WRITE_MAX_BYTES");
    return s ? std::strtoull(s, nullptr, 10) : uint64_t(64u << 10);
  }();
  return value;
}
constexpr uint32_t kReactorSlots = 1u << 16;     // tokens that can be queued at once
constexpr uint64_t kReactorMagic = 0x7470625f72656163ull;

// ---- the token queue: many producers (peers), one consumer (the owner's reactor thread) -----
struct alignas(64) ReactorHeader {
  uint64_t magic;
  uint32_t numSlots;
  alignas(64) std::atomic<uint32_t> sleeping;
  alignas(64) std::atomic<uint64_t> tail;  // next ticket for producers
  alignas(64) std::atomic<uint64_t> slots[1];  // really numSlots; value = ((ticket+1)<<32)|token
};

class ReactorQueue {
 public:
  ReactorQueue() = default;
  ReactorQueue(void* mem, bool init) : h_(static_cast<ReactorHeader*>(mem)) {
    if (init) {
      h_->magic = kReactorMagic;
      h_->numSlots = kReactorSlots;
      h_->sleeping.store(0);
      h_->tail.store(0);
      for (uint32_t i = 0; i < kReactorSlots; ++i) h_->slots[i].store(0, std::memory_order_relaxed);
      std::atomic_thread_fence(std::memory_order_seq_cst);
    }
  }
  static size_t bytesNeeded() { return sizeof(ReactorHeader) + sizeof(std::atomic<uint64_t>) * kReactorSlots; }
  bool valid(size_t bytes) const {
    return h_ && h_->magic == kReactorMagic && h_->numSlots == kReactorSlots && bytes >= bytesNeeded();
  }
  // Producer. Returns true if the consumer announced that it sleeps (caller writes its eventfd).
  bool push(uint32_t token) {
    uint64_t ticket = h_->tail.fetch_add(1, std::memory_order_relaxed);
    std::atomic<uint64_t>& slot = h_->slots[ticket & (kReactorSlots - 1)];
    // The slot is free once the consumer cleared the entry from the previous lap. With 64K
    // slots and at most two outstanding tokens per connection this never waits in practice.
    int spins = 0;
    while (slot.load(std::memory_order_acquire) != 0) {
      if (++spins > 1000000) return true;  // consumer is gone; drop the token
    }
    slot.store((((ticket + 1) & 0xffffffffull) << 32) | token, std::memory_order_seq_cst);
    return h_->sleeping.load(std::memory_order_seq_cst) != 0;
  }
  // Consumer.
  bool pop(uint32_t& token) {
    std::atomic<uint64_t>& slot = h_->slots[head_ & (kReactorSlots - 1)];
    uint64_t v = slot.load(std::memory_order_acquire);
    if ((v >> 32) != ((head_ + 1) & 0xffffffffull)) return false;
    token = static_cast<uint32_t>(v);
    slot.store(0, std::memory_order_release);
    ++head_;
    return true;
  }
  void setSleeping(bool s) { h_->sleeping.store(s ? 1 : 0, std::memory_order_seq_cst); }

 private:
  ReactorHeader* h_ = nullptr;
  uint64_t head_ = 0;  // consumer-private
};

// What the two ends tell each other over the bootstrap socket, next to three descriptors
// (reactor segment, reactor eventfd, inbox segment) carried as SCM_RIGHTS.
struct Bootstrap {
  uint32_t inboxToken = 0;
  uint32_t outboxToken = 0;
};

class ContextImpl;

struct ReadOp {
  bool userBuffer = false;
  uint8_t* ptr = nullptr;
  size_t expected = 0;
  Connection::read_callback_fn fn;
  uint32_t frameLen = 0;
  bool haveHeader = false;
  size_t bodyRead = 0;
  std::vector<uint8_t> owned;
};
struct WriteOp {
  const uint8_t* ptr = nullptr;
  uint32_t length = 0;
  Connection::write_callback_fn fn;
  bool headerWritten = false;
  size_t bodyWritten = 0;
};

class FdHandler {
 public:
  virtual void handleFdEvents(int events) = 0;
  virtual ~FdHandler() = default;
};

// ---- the reactor thread ---------------------------------------------------------------------
class Reactor final : public BusyPollingLoop {
 public:
  Reactor() {
    auto [e, seg] = ShmSegment::create(ReactorQueue::bytesNeeded());
    TPB_THROW_ASSERT_IF(bool(e), "cannot allocate the reactor segment: " + e.what());
    segment_ = std::move(seg);
    queue_ = ReactorQueue(segment_.ptr(), true);
    eventFd_ = ::eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
    TPB_THROW_SYSTEM_IF(eventFd_ < 0, errno, "eventfd");
    epollFd_ = ::epoll_create1(EPOLL_CLOEXEC);
    TPB_THROW_SYSTEM_IF(epollFd_ < 0, errno, "epoll_create1");
    epoll_event ev{};
    ev.events = EPOLLIN;
    ev.data.u64 = 0;
    ::epoll_ctl(epollFd_, EPOLL_CTL_ADD, eventFd_, &ev);
    const char* s = std::getenv("TPB_SHM_SPIN_US");
    spinUs_ = s ? std::strtol(s, nullptr, 10) : 2000;
    startThread("TP_SHM_reactor");
  }
  ~Reactor() override {
    join();
    ::close(epollFd_);
    ::close(eventFd_);
  }

  int segmentFd() const { return segment_.fd(); }
  int eventFd() const { return eventFd_; }

  // From the loop only.
  uint32_t addToken(std::function<void()> fn) {
    uint32_t t;
    if (!freeTokens_.empty()) {
      t = freeTokens_.back();
      freeTokens_.pop_back();
      functions_[t] = std::move(fn);
    } else {
      t = static_cast<uint32_t>(functions_.size());
      functions_.push_back(std::move(fn));
    }
    return t;
  }
  void removeToken(uint32_t t) {
    functions_[t] = nullptr;
    freeTokens_.push_back(t);
  }
  void watchFd(int fd, int events, std::shared_ptr<FdHandler> h) {
    uint64_t rec = nextRecord_++;
    epoll_event ev{};
    ev.events = events;
    ev.data.u64 = rec;
    TPB_THROW_SYSTEM_IF(::epoll_ctl(epollFd_, EPOLL_CTL_ADD, fd, &ev) < 0, errno, "epoll_ctl");
    fdRecords_[fd] = rec;
    handlers_[rec] = std::move(h);
  }
  void unwatchFd(int fd) {
    auto it = fdRecords_.find(fd);
    if (it == fdRecords_.end()) return;
    ::epoll_ctl(epollFd_, EPOLL_CTL_DEL, fd, nullptr);
    handlers_.erase(it->second);
    fdRecords_.erase(it);
  }

 protected:
  // Tokens that peers pushed into the shared queue since the last pass.
  bool pollOnce() override {
    bool worked = false;
    uint32_t token;
    int budget = 256;
    while (budget-- > 0 && queue_.pop(token)) {
      worked = true;
      runToken(token);
    }
    return worked;
  }
  bool readyToClose() override { return handlers_.empty(); }
  void onWork() override { lastWork_ = Clock::now(); }
  // Spin for a while after the last piece of work (looking at the descriptors now and then),
  // then sleep until a peer or a deferred function pokes the eventfd.
  void onIdle(uint64_t idlePasses) override {
    if ((idlePasses & 0x3f) != 0) return pause();
    pollFds(0);
    if (std::chrono::duration_cast<std::chrono::microseconds>(Clock::now() - lastWork_).count() <= spinUs_) return;
    // Go to sleep: announce it, look once more, then block until poked.
    queue_.setSleeping(true);
    sleeping_.store(true, std::memory_order_seq_cst);
    uint32_t t = UINT32_MAX;
    const bool popped = queue_.pop(t);
    if (popped || hasDeferred()) {
      queue_.setSleeping(false);
      sleeping_.store(false);
      if (popped) runToken(t);
    } else {
      pollFds(closing() ? 10 : -1);
      queue_.setSleeping(false);
      sleeping_.store(false);
    }
    lastWork_ = Clock::now();
  }

  void runToken(uint32_t token) {
    if (token < functions_.size() && functions_[token]) {
      auto fn = functions_[token];  // copy: the function may unregister itself
      fn();
    }
  }

  void wakeupEventLoop() override {
    if (sleeping_.load(std::memory_order_seq_cst)) {
      uint64_t one = 1;
      ssize_t r = ::write(eventFd_, &one, sizeof(one));
      (void)r;
    }
  }

 private:
  void pollFds(int timeoutMs) {
    epoll_event events[32];
    int n = ::epoll_wait(epollFd_, events, 32, timeoutMs);
    for (int i = 0; i < n; ++i) {
      uint64_t rec = events[i].data.u64;
      if (rec == 0) {
        uint64_t v;
        while (::read(eventFd_, &v, sizeof(v)) > 0) {}
        continue;
      }
      auto it = handlers_.find(rec);
      if (it == handlers_.end()) continue;
      auto h = it->second;
      h->handleFdEvents(static_cast<int>(events[i].events));
    }
  }

  ShmSegment segment_;
  ReactorQueue queue_;
  int eventFd_ = -1;
  int epollFd_ = -1;
  using Clock = std::chrono::steady_clock;
  long spinUs_ = 2000;
  Clock::time_point lastWork_ = Clock::now();
  std::atomic<bool> sleeping_{false};
  std::vector<std::function<void()>> functions_;
  std::vector<uint32_t> freeTokens_;
  uint64_t nextRecord_ = 1;
  std::unordered_map<int, uint64_t> fdRecords_;
  std::unordered_map<uint64_t, std::shared_ptr<FdHandler>> handlers_;
};

class ConnectionImpl;
class ListenerImpl;

class ContextImpl final : public std::enable_shared_from_this<ContextImpl> {
 public:
  ContextImpl(std::string dd) : domainDescriptor_(std::move(dd)) {}
  Reactor& reactor() { return reactor_; }
  const std::string& domainDescriptor() const { return domainDescriptor_; }
  bool closed() const { return closed_; }
  void enroll(std::shared_ptr<ConnectionImpl> c) { conns_.insert(std::move(c)); }
  void unenroll(const std::shared_ptr<ConnectionImpl>& c) { conns_.erase(c); }
  void enroll(std::shared_ptr<ListenerImpl> l) { listeners_.insert(std::move(l)); }
  void unenroll(const std::shared_ptr<ListenerImpl>& l) { listeners_.erase(l); }
  void close();
  void join() {
    close();
    if (!joined_.exchange(true)) reactor_.join();
  }

 private:
  Reactor reactor_;
  std::string domainDescriptor_;
  bool closed_ = false;
  std::atomic<bool> joined_{false};
  std::set<std::shared_ptr<ConnectionImpl>> conns_;
  std::set<std::shared_ptr<ListenerImpl>> listeners_;
};

// ---- connection -----------------------------------------------------------------------------
class ConnectionImpl final : public FdHandler, public std::enable_shared_from_this<ConnectionImpl> {
 public:
  enum State { kInitializing, kWaitingForPeer, kEstablished, kClosed };

  ConnectionImpl(std::shared_ptr<ContextImpl> ctx, Socket sock) : ctx_(std::move(ctx)), sock_(std::move(sock)) {}
  ConnectionImpl(std::shared_ptr<ContextImpl> ctx, std::string addr)
      : ctx_(std::move(ctx)), connectAddr_(std::move(addr)), isClient_(true) {}

  void init() {
    auto self = shared_from_this();
    ctx_->reactor().deferToLoop([self]() { self->initFromLoop(); });
  }
  void read(ReadOp op) {
    auto self = shared_from_this();
    ctx_->reactor().deferToLoop([self, op = std::move(op)]() mutable {
      if (self->error_) return op.fn(self->error_, nullptr, 0);
      self->reads_.push_back(std::move(op));
      if (self->state_ == kEstablished) self->processReads();
    });
  }
  void write(WriteOp op) {
    auto self = shared_from_this();
    {
      // Short cut: when nothing is queued ahead and the whole frame fits, the caller's own thread
      // copies it into the peer's inbox and pokes the peer; only the completion goes through the
      // reactor thread. This takes one thread hand-off out of every control message. Frames above
      // 64 KiB go to the reactor thread, which moves them in pieces so that the reader's copy
      // overlaps the writer's: there the hand-off costs nothing beside the copy, and a frame
      // written here in one go would keep the reader waiting until its last byte is in.
      std::unique_lock<std::mutex> lock(outboxMutex_);
      if (directWrites_ && queuedWrites_ == 0 && op.length <= directWriteMaxBytes() &&
          outbox_.freeBytes() >= sizeof(uint32_t) + op.length) {
        outbox_.write(&op.length, sizeof(uint32_t));
        if (op.length) outbox_.write(op.ptr, op.length);
        pokePeer(peerInboxToken_);
        lock.unlock();
        ctx_->reactor().deferToLoop([self, fn = std::move(op.fn)]() mutable { fn(Error::kSuccess); });
        return;
      }
      ++queuedWrites_;
    }
    ctx_->reactor().deferToLoop([self, op = std::move(op)]() mutable {
      if (self->error_) {
        self->forgetQueuedWrite();
        return op.fn(self->error_);
      }
      self->writes_.push_back(std::move(op));
      if (self->peerGone_) return self->closeFromLoop(TPB_CREATE_ERROR(EOFError));
      if (self->state_ == kEstablished) self->processWrites();
    });
  }
  void close() {
    auto self = shared_from_this();
    ctx_->reactor().deferToLoop([self]() { self->closeFromLoop(TPB_CREATE_ERROR(ConnectionClosedError)); });
  }
  void closeFromLoop(const Error& e);
  void handleFdEvents(int events) override;

 private:
  void initFromLoop();
  void onPeerBootstrap(const Bootstrap& b, int fds[3]);
  void processReads();
  void processWrites();
  // The outbox is too full to go on: say so in the ring header, so that the reader pokes our
  // outbox token once it has made room, and look once more (it may just have done so). Returns
  // true if there is room after all. Call with outboxMutex_ held.
  bool waitForSpace(uint64_t needed) {
    outbox_.setProducerStalled(true);
    stalled_ = true;
    return outbox_.freeBytes() >= needed;
  }
  void forgetQueuedWrite() {
    std::unique_lock<std::mutex> lock(outboxMutex_);
    --queuedWrites_;
  }
  void pokePeer(uint32_t token) {
    if (peerQueue_.push(token)) {
      uint64_t one = 1;
      ssize_t r = ::write(peerEventFd_, &one, sizeof(one));
      (void)r;
    }
  }

  std::shared_ptr<ContextImpl> ctx_;
  Socket sock_;
  std::string connectAddr_;
  bool isClient_ = false;
  State state_ = kInitializing;
  Error error_;
  ShmSegment inboxSeg_, outboxSeg_, peerReactorSeg_;
  Ring inbox_, outbox_;
  ReactorQueue peerQueue_;
  int peerEventFd_ = -1;
  uint32_t myInboxToken_ = 0, myOutboxToken_ = 0;
  uint32_t peerInboxToken_ = 0, peerOutboxToken_ = 0;
  bool tokensRegistered_ = false;
  bool watching_ = false;
  bool peerGone_ = false;
  std::deque<ReadOp> reads_;
  std::deque<WriteOp> writes_;
  // The outbox has one producer at a time: whoever holds this mutex, the reactor thread working
  // through writes_ or a caller taking the short cut in write().
  std::mutex outboxMutex_;
  bool directWrites_ = false;  // established, peer alive: callers may write the outbox themselves
  size_t queuedWrites_ = 0;    // writes handed to the reactor thread and not completed yet
  bool stalled_ = false;       // the ring header says we wait for space
};

void ConnectionImpl::initFromLoop() {
  auto self = shared_from_this();
  if (ctx_->closed()) {
    sock_.reset();
    error_ = TPB_CREATE_ERROR(ContextClosedError);
    state_ = kClosed;
    return;
  }
  ctx_->enroll(self);
  if (isClient_) {
    auto [created, sock] = Socket::createForFamily(AF_UNIX);
    if (created) return closeFromLoop(created);
    sock_ = std::move(sock);
    if (Error connected = sock_.connectAbstract(connectAddr_)) return closeFromLoop(connected);
  }
  if (Error e = sock_.setNonBlocking()) return closeFromLoop(e);

  auto [e, seg] = ShmSegment::create(Ring::bytesNeeded(kRingBytes));
  if (e) return closeFromLoop(e);
  inboxSeg_ = std::move(seg);
  inbox_ = Ring(inboxSeg_.ptr(), kRingBytes, true);

  std::weak_ptr<ConnectionImpl> weak = self;
  myInboxToken_ = ctx_->reactor().addToken([weak]() {
    if (auto c = weak.lock()) c->processReads();
  });
  myOutboxToken_ = ctx_->reactor().addToken([weak]() {
    if (auto c = weak.lock()) c->processWrites();
  });
  tokensRegistered_ = true;

  Bootstrap b{myInboxToken_, myOutboxToken_};
  int fds[3] = {ctx_->reactor().segmentFd(), ctx_->reactor().eventFd(), inboxSeg_.fd()};
  Error se = sock_.sendWithFds(b, fds);
  if (se) return closeFromLoop(se);
  state_ = kWaitingForPeer;
  ctx_->reactor().watchFd(sock_.fd(), EPOLLIN | EPOLLRDHUP, self);
  watching_ = true;
}

void ConnectionImpl::handleFdEvents(int events) {
  auto self = shared_from_this();
  if (state_ == kClosed) return;
  if (state_ == kWaitingForPeer && (events & EPOLLIN)) {
    Bootstrap b;
    int fds[3] = {-1, -1, -1};
    bool got = false;
    Error e = sock_.recvWithFds(b, fds, got);
    if (e) return closeFromLoop(e);
    if (got) onPeerBootstrap(b, fds);
    return;
  }
  if (events & (EPOLLIN | EPOLLRDHUP | EPOLLHUP | EPOLLERR)) {
    // Nothing legitimate arrives on the socket after bootstrap: this is the peer going away.
    // Frames it completed before leaving are still in the inbox and stay readable (as bytes in
    // a TCP socket buffer would); the connection fails once a read cannot be satisfied.
    if (state_ != kEstablished) return closeFromLoop(TPB_CREATE_ERROR(EOFError));
    peerGone_ = true;
    {
      std::unique_lock<std::mutex> lock(outboxMutex_);
      directWrites_ = false;
    }
    if (watching_) ctx_->reactor().unwatchFd(sock_.fd());
    watching_ = false;
    if (!writes_.empty()) return closeFromLoop(TPB_CREATE_ERROR(EOFError));
    processReads();
  }
}

void ConnectionImpl::onPeerBootstrap(const Bootstrap& b, int fds[3]) {
  peerInboxToken_ = b.inboxToken;
  peerOutboxToken_ = b.outboxToken;
  auto [e1, rseg] = ShmSegment::load(fds[0]);
  peerEventFd_ = fds[1];
  auto [e2, oseg] = ShmSegment::load(fds[2]);
  if (e1 || e2) return closeFromLoop(e1 ? e1 : e2);
  peerReactorSeg_ = std::move(rseg);
  outboxSeg_ = std::move(oseg);
  peerQueue_ = ReactorQueue(peerReactorSeg_.ptr(), false);
  outbox_ = Ring(outboxSeg_.ptr(), 0, false);
  if (!peerQueue_.valid(peerReactorSeg_.size()) || !outbox_.valid(outboxSeg_.size()))
    return closeFromLoop(TPB_CREATE_ERROR(ShortReadError, 0, 0));
  state_ = kEstablished;
  {
    std::unique_lock<std::mutex> lock(outboxMutex_);
    directWrites_ = true;
  }
  processWrites();
  if (state_ == kEstablished) processReads();
}

void ConnectionImpl::processReads() {
  if (state_ != kEstablished) return;
  auto self = shared_from_this();
  bool consumed = false;
  while (state_ == kEstablished && !reads_.empty()) {
    ReadOp& op = reads_.front();
    if (!op.haveHeader) {
      if (inbox_.usedBytes() < sizeof(uint32_t)) break;
      inbox_.read(&op.frameLen, sizeof(uint32_t));
      consumed = true;
      op.haveHeader = true;
      if (op.userBuffer) {
        if (op.frameLen != op.expected) {
          if (!peerGone_) pokePeer(peerOutboxToken_);
          closeFromLoop(TPB_CREATE_ERROR(ShortReadError, static_cast<ssize_t>(op.expected),
                                         static_cast<ssize_t>(op.frameLen)));
          return;
        }
      } else {
        // A length the peer chose: bound what is allocated on its word.
        if (op.frameLen > kMaxAllocatedFrame) {
          if (!peerGone_) pokePeer(peerOutboxToken_);
          closeFromLoop(TPB_CREATE_ERROR(MessageError, "incoming frame of " + std::to_string(op.frameLen) +
                                                           " bytes exceeds the limit for unsolicited frames"));
          return;
        }
        op.owned.resize(op.frameLen);
        op.ptr = op.owned.data();
      }
    }
    if (op.bodyRead < op.frameLen) {
      bool more = true;
      while (more && op.bodyRead < op.frameLen) {
        const uint64_t want = std::min<uint64_t>(op.frameLen - op.bodyRead, pieceBytes());
        const uint64_t n = inbox_.read(op.ptr + op.bodyRead, want);
        op.bodyRead += n;
        more = n == want;
        // Let the writer refill while the next piece is copied out.
        if (n > 0 && !peerGone_ && inbox_.producerStalled()) pokePeer(peerOutboxToken_);
      }
      if (op.bodyRead < op.frameLen) break;
    }
    ReadOp done = std::move(reads_.front());
    reads_.pop_front();
    done.fn(Error::kSuccess, done.ptr, done.frameLen);
  }
  if (peerGone_) {
    if (state_ == kEstablished && !reads_.empty()) closeFromLoop(TPB_CREATE_ERROR(EOFError));
    return;
  }
  // A writer that ran out of ring space waits for exactly this.
  if (consumed && state_ == kEstablished && inbox_.producerStalled()) pokePeer(peerOutboxToken_);
}

void ConnectionImpl::processWrites() {
  if (state_ != kEstablished) return;
  auto self = shared_from_this();
  std::vector<Connection::write_callback_fn> completed;
  {
    std::unique_lock<std::mutex> lock(outboxMutex_);
    bool produced = false;
    while (!writes_.empty()) {
      WriteOp& op = writes_.front();
      if (!op.headerWritten) {
        if (outbox_.freeBytes() < sizeof(uint32_t) && !waitForSpace(sizeof(uint32_t))) break;
        outbox_.write(&op.length, sizeof(uint32_t));
        op.headerWritten = true;
        produced = true;
      }
      if (op.bodyWritten < op.length) {
        const uint64_t want = std::min<uint64_t>(op.length - op.bodyWritten, pieceBytes());
        const uint64_t n = outbox_.write(op.ptr + op.bodyWritten, want);
        op.bodyWritten += n;
        if (op.bodyWritten < op.length) {
          // More to come: the reader may as well start on what is there.
          if (n > 0) pokePeer(peerInboxToken_);
          if (n == want || waitForSpace(1)) continue;
          break;
        }
        if (n > 0) produced = true;
      }
      completed.push_back(std::move(op.fn));
      writes_.pop_front();
      --queuedWrites_;
    }
    if (writes_.empty() && stalled_) {
      outbox_.setProducerStalled(false);
      stalled_ = false;
    }
    // Poke before the callbacks so the reader starts while we run user code.
    if (produced) pokePeer(peerInboxToken_);
  }
  for (auto& fn : completed) fn(Error::kSuccess);
}

void ConnectionImpl::closeFromLoop(const Error& e) {
  if (error_) return;
  error_ = e;
  auto self = shared_from_this();
  state_ = kClosed;
  {
    // No caller may be half way through the short cut of write() when the eventfd goes away.
    std::unique_lock<std::mutex> lock(outboxMutex_);
    directWrites_ = false;
    if (peerEventFd_ >= 0) ::close(peerEventFd_);
    peerEventFd_ = -1;
  }
  if (watching_) ctx_->reactor().unwatchFd(sock_.fd());
  watching_ = false;
  sock_.reset();
  if (tokensRegistered_) {
    ctx_->reactor().removeToken(myInboxToken_);
    ctx_->reactor().removeToken(myOutboxToken_);
    tokensRegistered_ = false;
  }
  ctx_->unenroll(self);
  auto reads = std::move(reads_);
  auto writes = std::move(writes_);
  reads_.clear();
  writes_.clear();
  {
    std::unique_lock<std::mutex> lock(outboxMutex_);
    queuedWrites_ -= writes.size();
  }
  for (auto& r : reads) r.fn(error_, nullptr, 0);
  for (auto& w : writes) w.fn(error_);
}

// ---- listener -------------------------------------------------------------------------------
class ConnectionShell final : public Connection {
 public:
  explicit ConnectionShell(std::shared_ptr<ConnectionImpl> impl) : impl_(std::move(impl)) {}
  ~ConnectionShell() override { impl_->close(); }
  void read(read_callback_fn fn) override {
    ReadOp op;
    op.fn = std::move(fn);
    impl_->read(std::move(op));
  }
  void read(void* ptr, size_t length, read_callback_fn fn) override {
    ReadOp op;
    op.userBuffer = true;
    op.ptr = static_cast<uint8_t*>(ptr);
    op.expected = length;
    op.fn = std::move(fn);
    impl_->read(std::move(op));
  }
  void write(const void* ptr, size_t length, write_callback_fn fn) override {
    if (length > UINT32_MAX) {
      // Frames carry a 32-bit length; larger writes are a caller bug (the pipe never does it
      // for control traffic, and the basic channel splits nothing — use uv for >4 GiB frames).
      throw std::runtime_error("shm transport: frame larger than 4 GiB");
    }
    WriteOp op;
    op.ptr = static_cast<const uint8_t*>(ptr);
    op.length = static_cast<uint32_t>(length);
    op.fn = std::move(fn);
    impl_->write(std::move(op));
  }
  void setId(std::string id) override { (void)id; }
  void close() override { impl_->close(); }

 private:
  std::shared_ptr<ConnectionImpl> impl_;
};

class ListenerImpl final : public FdHandler, public std::enable_shared_from_this<ListenerImpl> {
 public:
  ListenerImpl(std::shared_ptr<ContextImpl> ctx, const std::string& addr) : ctx_(std::move(ctx)) {
    auto [created, sock] = Socket::createForFamily(AF_UNIX, SOCK_NONBLOCK);
    TPB_THROW_SYSTEM_IF(bool(created), errno, "socket");
    sock_ = std::move(sock);
    // An empty address autobinds: the kernel picks a unique abstract name.
    TPB_THROW_SYSTEM_IF(bool(sock_.bindAbstract(addr)), errno, "bind");
    TPB_THROW_SYSTEM_IF(bool(sock_.listen(128)), errno, "listen");
    addr_ = sock_.boundAbstractName();
  }
  void init() {
    auto self = shared_from_this();
    ctx_->reactor().deferToLoop([self]() {
      if (self->ctx_->closed()) return self->closeFromLoop(TPB_CREATE_ERROR(ContextClosedError));
      self->ctx_->enroll(self);
    });
  }
  void accept(Listener::accept_callback_fn fn) {
    auto self = shared_from_this();
    ctx_->reactor().deferToLoop([self, fn = std::move(fn)]() mutable {
      if (self->error_) return fn(self->error_, nullptr);
      self->armed_.push_back(std::move(fn));
      // Accept-side backpressure: the listening socket is only watched while someone waits.
      if (!self->watching_) {
        self->ctx_->reactor().watchFd(self->sock_.fd(), EPOLLIN, self);
        self->watching_ = true;
      }
    });
  }
  std::string addr() const { return addr_; }
  void close() {
    auto self = shared_from_this();
    ctx_->reactor().deferToLoop([self]() { self->closeFromLoop(TPB_CREATE_ERROR(ListenerClosedError)); });
  }
  void closeFromLoop(const Error& e) {
    if (error_) return;
    error_ = e;
    auto self = shared_from_this();
    if (watching_) ctx_->reactor().unwatchFd(sock_.fd());
    watching_ = false;
    sock_.reset();
    ctx_->unenroll(self);
    auto armed = std::move(armed_);
    armed_.clear();
    for (auto& fn : armed) fn(error_, nullptr);
  }
  void handleFdEvents(int events) override {
    auto self = shared_from_this();
    (void)events;
    while (!armed_.empty() && sock_.hasValue()) {
      auto [failed, incoming] = sock_.accept();
      if (failed) return closeFromLoop(failed);
      if (!incoming.hasValue()) break;  // nobody waiting in the backlog
      auto impl = std::make_shared<ConnectionImpl>(ctx_, std::move(incoming));
      impl->init();
      auto fn = std::move(armed_.front());
      armed_.pop_front();
      fn(Error::kSuccess, std::make_shared<ConnectionShell>(std::move(impl)));
    }
    if (armed_.empty() && watching_ && sock_.hasValue()) {
      ctx_->reactor().unwatchFd(sock_.fd());
      watching_ = false;
    }
  }

 private:
  std::shared_ptr<ContextImpl> ctx_;
  Socket sock_;
  std::string addr_;
  Error error_;
  bool watching_ = false;
  std::deque<Listener::accept_callback_fn> armed_;
};

void ContextImpl::close() {
  auto self = shared_from_this();
  reactor_.deferToLoop([self]() {
    if (self->closed_) return;
    self->closed_ = true;
    auto conns = self->conns_;
    auto listeners = self->listeners_;
    Error e = TPB_CREATE_ERROR(ContextClosedError);
    for (auto& c : conns) c->closeFromLoop(e);
    for (auto& l : listeners) l->closeFromLoop(e);
  });
}

class ListenerShell final : public Listener {
 public:
  explicit ListenerShell(std::shared_ptr<ListenerImpl> impl) : impl_(std::move(impl)) {}
  ~ListenerShell() override { impl_->close(); }
  void accept(accept_callback_fn fn) override { impl_->accept(std::move(fn)); }
  std::string addr() const override { return impl_->addr(); }
  void setId(std::string id) override { (void)id; }
  void close() override { impl_->close(); }

 private:
  std::shared_ptr<ListenerImpl> impl_;
};

class ContextShell final : public Context {
 public:
  ContextShell() {
    auto boot = getBootID();
    auto netns = getLinuxNamespaceId(LinuxNamespace::kNet);
    if (!boot || !netns) {
      TPB_VLOG(7) << "shm transport not viable: cannot read boot id or network namespace";
      return;
    }
    // Probe: can we allocate shared memory at all (e.g. a full or missing /dev/shm)?
    auto [e, seg] = ShmSegment::create(1u << 20);
    if (e) {
      TPB_VLOG(7) << "shm transport not viable: " << e.what();
      return;
    }
    descriptor_ = "tpbshm1:" + *boot + "_" + *netns;
    impl_ = std::make_shared<ContextImpl>(descriptor_);
  }
  ~ContextShell() override {
    if (impl_) impl_->join();
  }
  std::shared_ptr<Connection> connect(std::string addr) override {
    TPB_THROW_ASSERT_IF(!impl_, "shm transport is not viable");
    auto c = std::make_shared<ConnectionImpl>(impl_, std::move(addr));
    c->init();
    return std::make_shared<ConnectionShell>(std::move(c));
  }
  std::shared_ptr<Listener> listen(std::string addr) override {
    TPB_THROW_ASSERT_IF(!impl_, "shm transport is not viable");
    auto l = std::make_shared<ListenerImpl>(impl_, addr);
    l->init();
    return std::make_shared<ListenerShell>(std::move(l));
  }
  bool isViable() const override { return impl_ != nullptr; }
  const std::string& domainDescriptor() const override { return descriptor_; }
  void setId(std::string id) override { (void)id; }
  void close() override {
    if (impl_) impl_->close();
  }
  void join() override {
    if (impl_) impl_->join();
  }

 private:
  std::shared_ptr<ContextImpl> impl_;
  std::string descriptor_;
};

}  // namespace

std::shared_ptr<Context> create() { return std::make_shared<ContextShell>(); }

}  // namespace shm
}  // namespace transport
}  // namespace tpb
