// The TCP transport: non-blocking sockets on one epoll thread per context.
//
// Wire format and naming match the reference's libuv transport so that the two interoperate
// (tensorpipe/transport/uv/connection_impl.cc:96-149, common/stream_read_write_ops.h:30-194,
// transport/uv/context_impl.cc:23-27): every frame is an 8-byte host-endian length followed by
// the payload, TCP_NODELAY is set, the domain descriptor is the constant "uv:*", and an idle
// connection (no read posted) stops watching its socket for readability — that is how
// backpressure reaches the kernel's socket buffers and, through them, the sender.
#include <arpa/inet.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <sys/uio.h>
#include <unistd.h>

#include <deque>
#include <set>
#include <vector>

#include <tpb/transport.h>

#include "common/defs.h"
#include "common/epoll_loop.h"

namespace tpb {
namespace transport {
namespace tcp {

namespace {

const std::string kDomainDescriptor = "uv:*";

struct SockAddr {
  sockaddr_storage ss{};
  socklen_t len = 0;
};

// "1.2.3.4", "1.2.3.4:80", "[::1]", "[::1]:80", "::1"
bool parseAddr(const std::string& s, SockAddr& out) {
  std::string host = s;
  uint16_t port = 0;
  bool v6 = false;
  if (!s.empty() && s[0] == '[') {
    auto close = s.find(']');
    if (close == std::string::npos) return false;
    host = s.substr(1, close - 1);
    v6 = true;
    if (close + 1 < s.size()) {
      if (s[close + 1] != ':') return false;
      port = static_cast<uint16_t>(std::strtoul(s.c_str() + close + 2, nullptr, 10));
    }
  } else {
    auto first = s.find(':');
    auto last = s.rfind(':');
    if (first != std::string::npos && first == last) {
      host = s.substr(0, first);
      port = static_cast<uint16_t>(std::strtoul(s.c_str() + first + 1, nullptr, 10));
    } else if (first != std::string::npos) {
      v6 = true;  // bare IPv6 without a port
    }
  }
  if (v6) {
    auto* a = reinterpret_cast<sockaddr_in6*>(&out.ss);
    a->sin6_family = AF_INET6;
    a->sin6_port = htons(port);
    if (::inet_pton(AF_INET6, host.c_str(), &a->sin6_addr) != 1) return false;
    out.len = sizeof(sockaddr_in6);
  } else {
    auto* a = reinterpret_cast<sockaddr_in*>(&out.ss);
    a->sin_family = AF_INET;
    a->sin_port = htons(port);
    if (::inet_pton(AF_INET, host.c_str(), &a->sin_addr) != 1) return false;
    out.len = sizeof(sockaddr_in);
  }
  return true;
}

std::string formatAddr(const sockaddr* sa, bool withPort = true) {
  char buf[INET6_ADDRSTRLEN] = {0};
  if (sa->sa_family == AF_INET) {
    auto* a = reinterpret_cast<const sockaddr_in*>(sa);
    ::inet_ntop(AF_INET, &a->sin_addr, buf, sizeof(buf));
    return withPort ? std::string(buf) + ":" + std::to_string(ntohs(a->sin_port)) : std::string(buf);
  }
  auto* a = reinterpret_cast<const sockaddr_in6*>(sa);
  ::inet_ntop(AF_INET6, &a->sin6_addr, buf, sizeof(buf));
  return withPort ? "[" + std::string(buf) + "]:" + std::to_string(ntohs(a->sin6_port))
                  : std::string(buf);
}

class ContextImpl;

struct ReadOp {
  bool userBuffer = false;
  uint8_t* ptr = nullptr;
  size_t expected = 0;
  Connection::read_callback_fn fn;
  uint64_t frameLen = 0;
  size_t headerRead = 0;
  size_t bodyRead = 0;
  std::vector<uint8_t> owned;
};

struct WriteOp {
  const uint8_t* ptr = nullptr;
  uint64_t length = 0;
  Connection::write_callback_fn fn;
  size_t written = 0;  // counts header + body
};

class ConnectionImpl final : public EpollEventHandler,
                             public std::enable_shared_from_this<ConnectionImpl> {
 public:
  enum State { kConnecting, kOpen, kClosed };

  ConnectionImpl(std::shared_ptr<ContextImpl> ctx, int fd, State st)
      : ctx_(std::move(ctx)), fd_(fd), state_(st) {}
  ConnectionImpl(std::shared_ptr<ContextImpl> ctx, std::string addr)
      : ctx_(std::move(ctx)), state_(kConnecting), connectAddr_(std::move(addr)) {}

  void init();
  void read(ReadOp op);
  void write(WriteOp op);
  void close();
  void setId(std::string id);
  void closeFromLoop(const Error& e);
  void handleEventsFromLoop(int events) override;

 private:
  void initFromLoop();
  void updateInterest();
  void processReads();
  void processWrites();
  void failAll();

  std::shared_ptr<ContextImpl> ctx_;
  int fd_ = -1;
  State state_;
  std::string connectAddr_;
  std::string id_ = "N/A";
  Error error_;
  std::deque<ReadOp> reads_;
  std::deque<WriteOp> writes_;
  int interest_ = 0;
  bool registered_ = false;
  // Bytes read from the socket ahead of the operation that will consume them: headers and small
  // frames come out of here, several per system call; large bodies are read straight into their
  // destination once this is empty.
  static constexpr size_t kReadAheadBytes = 64 * 1024;
  static constexpr size_t kDirectReadMinBytes = 16 * 1024;
  std::unique_ptr<uint8_t[]> readAhead_;
  size_t readAheadBegin_ = 0, readAheadEnd_ = 0;
  size_t takeReadAhead(uint8_t* dst, size_t n);
  enum class Fill { kGotBytes, kWouldBlock, kClosed };
  Fill fillReadAhead();
  // Writes queued during one pass of the loop leave in one sendmsg: the flush is itself a
  // closure deferred behind them.
  bool flushScheduled_ = false;
  bool socketFull_ = false;  // sendmsg said EAGAIN: the next attempt waits for EPOLLOUT
  bool flushingBeforeClose_ = false;
  bool interestUpdateScheduled_ = false;
};

class ListenerImpl final : public EpollEventHandler,
                           public std::enable_shared_from_this<ListenerImpl> {
 public:
  ListenerImpl(std::shared_ptr<ContextImpl> ctx, const std::string& addr);
  void init();
  void accept(Listener::accept_callback_fn fn);
  std::string addr() const { return addr_; }
  void close();
  void closeFromLoop(const Error& e);
  void setId(std::string id) { (void)id; }
  void handleEventsFromLoop(int events) override;

 private:
  void updateInterest();
  std::shared_ptr<ContextImpl> ctx_;
  int fd_ = -1;
  std::string addr_;
  Error error_;
  std::deque<Listener::accept_callback_fn> armed_;
  bool registered_ = false;
};

class ContextImpl final : public std::enable_shared_from_this<ContextImpl> {
 public:
  ContextImpl() : loop_("TP_UV_loop") {}
  EpollLoop& loop() { return loop_; }

  void enroll(std::shared_ptr<ConnectionImpl> c) { conns_.insert(std::move(c)); }
  void unenroll(const std::shared_ptr<ConnectionImpl>& c) { conns_.erase(c); }
  void enroll(std::shared_ptr<ListenerImpl> l) { listeners_.insert(std::move(l)); }
  void unenroll(const std::shared_ptr<ListenerImpl>& l) { listeners_.erase(l); }
  bool closed() const { return closed_; }

  void close() {
    auto self = shared_from_this();
    loop_.deferToLoop([self]() {
      if (self->closed_) return;
      self->closed_ = true;
      auto conns = self->conns_;
      auto listeners = self->listeners_;
      Error e = TPB_CREATE_ERROR(ContextClosedError);
      for (auto& c : conns) c->closeFromLoop(e);
      for (auto& l : listeners) l->closeFromLoop(e);
    });
  }
  void join() {
    close();
    if (!joined_.exchange(true)) loop_.join();
  }

 private:
  EpollLoop loop_;
  bool closed_ = false;
  std::atomic<bool> joined_{false};
  std::set<std::shared_ptr<ConnectionImpl>> conns_;
  std::set<std::shared_ptr<ListenerImpl>> listeners_;
};

// ---- connection -----------------------------------------------------------------------------
void ConnectionImpl::init() {
  auto self = shared_from_this();
  ctx_->loop().deferToLoop([self]() { self->initFromLoop(); });
}

void ConnectionImpl::initFromLoop() {
  if (ctx_->closed()) {
    error_ = TPB_CREATE_ERROR(ContextClosedError);
    if (fd_ >= 0) ::close(fd_);
    fd_ = -1;
    state_ = kClosed;
    return;
  }
  ctx_->enroll(shared_from_this());
  if (state_ == kConnecting) {
    SockAddr sa;
    if (!parseAddr(connectAddr_, sa)) {
      closeFromLoop(TPB_CREATE_ERROR(SystemError, "inet_pton", EINVAL));
      return;
    }
    fd_ = ::socket(sa.ss.ss_family, SOCK_STREAM | SOCK_NONBLOCK | SOCK_CLOEXEC, 0);
    if (fd_ < 0) {
      closeFromLoop(TPB_CREATE_ERROR(SystemError, "socket", errno));
      return;
    }
    int one = 1;
    ::setsockopt(fd_, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    int rv = ::connect(fd_, reinterpret_cast<sockaddr*>(&sa.ss), sa.len);
    if (rv == 0) {
      state_ = kOpen;
    } else if (errno != EINPROGRESS) {
      closeFromLoop(TPB_CREATE_ERROR(SystemError, "connect", errno));
      return;
    }
  }
  updateInterest();
  if (state_ == kOpen) {
    processWrites();
    processReads();
  }
}

void ConnectionImpl::updateInterest() {
  if (state_ == kClosed || fd_ < 0) return;
  int want = 0;
  if (state_ == kConnecting) want = EPOLLOUT;
  else {
    if (!reads_.empty()) want |= EPOLLIN;
    if (!writes_.empty()) want |= EPOLLOUT;
  }
  if (want == interest_ && (registered_ || want == 0)) return;
  interest_ = want;
  if (want == 0) {
    if (registered_) ctx_->loop().unregisterDescriptor(fd_);
    registered_ = false;
  } else {
    ctx_->loop().registerDescriptor(fd_, want, shared_from_this());
    registered_ = true;
  }
}

void ConnectionImpl::read(ReadOp op) {
  auto self = shared_from_this();
  ctx_->loop().deferToLoop([self, op = std::move(op)]() mutable {
    if (self->error_) {
      op.fn(self->error_, nullptr, 0);
      return;
    }
    self->reads_.push_back(std::move(op));
    if (self->state_ == kOpen && self->reads_.size() == 1) self->processReads();
    self->updateInterest();
  });
}

void ConnectionImpl::write(WriteOp op) {
  auto self = shared_from_this();
  ctx_->loop().deferToLoop([self, op = std::move(op)]() mutable {
    if (self->error_) {
      op.fn(self->error_);
      return;
    }
    self->writes_.push_back(std::move(op));
    if (self->state_ == kOpen && !self->flushScheduled_ && !self->socketFull_) {
      // A message is several frames (descriptor, payloads), written back to back by the pipe:
      // the closure below runs behind the ones that queue them.
      self->flushScheduled_ = true;
      self->ctx_->loop().deferToLoop([self]() {
        self->flushScheduled_ = false;
        if (self->state_ == kOpen) self->processWrites();
        self->updateInterest();
      });
    }
  });
}

size_t ConnectionImpl::takeReadAhead(uint8_t* dst, size_t n) {
  const size_t have = readAheadEnd_ - readAheadBegin_;
  if (n > have) n = have;
  if (n == 0) return 0;
  std::memcpy(dst, readAhead_.get() + readAheadBegin_, n);
  readAheadBegin_ += n;
  if (readAheadBegin_ == readAheadEnd_) readAheadBegin_ = readAheadEnd_ = 0;
  return n;
}

// Called with the read-ahead buffer empty.
ConnectionImpl::Fill ConnectionImpl::fillReadAhead() {
  if (!readAhead_) readAhead_.reset(new uint8_t[kReadAheadBytes]);
  for (;;) {
    ssize_t n = ::read(fd_, readAhead_.get(), kReadAheadBytes);
    if (n > 0) {
      readAheadBegin_ = 0;
      readAheadEnd_ = static_cast<size_t>(n);
      return Fill::kGotBytes;
    }
    if (n == 0) {
      closeFromLoop(TPB_CREATE_ERROR(EOFError));
      return Fill::kClosed;
    }
    if (errno == EAGAIN || errno == EWOULDBLOCK) return Fill::kWouldBlock;
    if (errno == EINTR) continue;
    closeFromLoop(TPB_CREATE_ERROR(SystemError, "read", errno));
    return Fill::kClosed;
  }
}

void ConnectionImpl::processReads() {
  while (state_ == kOpen && !reads_.empty()) {
    ReadOp& op = reads_.front();
    if (op.headerRead < sizeof(uint64_t)) {
      op.headerRead += takeReadAhead(reinterpret_cast<uint8_t*>(&op.frameLen) + op.headerRead,
                                     sizeof(uint64_t) - op.headerRead);
      if (op.headerRead < sizeof(uint64_t)) {
        if (fillReadAhead() != Fill::kGotBytes) return;
        continue;
      }
      if (op.userBuffer) {
        if (op.frameLen != op.expected) {
          closeFromLoop(TPB_CREATE_ERROR(ShortReadError, static_cast<ssize_t>(op.expected),
                                         static_cast<ssize_t>(op.frameLen)));
          return;
        }
      } else {
        // The length comes from the peer: a corrupt or hostile header must fail the connection,
        // not exhaust memory. Frames the library allocates for are control messages.
        if (op.frameLen > kMaxAllocatedFrame) {
          closeFromLoop(TPB_CREATE_ERROR(MessageError, "incoming frame of " + std::to_string(op.frameLen) +
                                                           " bytes exceeds the limit for unsolicited frames"));
          return;
        }
        op.owned.resize(op.frameLen);
        op.ptr = op.owned.data();
      }
    }
    while (op.bodyRead < op.frameLen) {
      op.bodyRead += takeReadAhead(op.ptr + op.bodyRead, op.frameLen - op.bodyRead);
      const size_t remaining = op.frameLen - op.bodyRead;
      if (remaining == 0) break;
      if (remaining < kDirectReadMinBytes) {
        // The rest of a small frame, and likely the frames behind it, in one system call.
        if (fillReadAhead() != Fill::kGotBytes) return;
        continue;
      }
      // A large body goes straight to where it belongs (the read-ahead buffer is empty here).
      ssize_t n = ::read(fd_, op.ptr + op.bodyRead, remaining);
      if (n == 0) { closeFromLoop(TPB_CREATE_ERROR(EOFError)); return; }
      if (n < 0) {
        if (errno == EAGAIN || errno == EWOULDBLOCK) return;
        if (errno == EINTR) continue;
        closeFromLoop(TPB_CREATE_ERROR(SystemError, "read", errno));
        return;
      }
      op.bodyRead += static_cast<size_t>(n);
    }
    ReadOp done = std::move(reads_.front());
    reads_.pop_front();
    done.fn(Error::kSuccess, done.ptr, done.frameLen);
  }
}

void ConnectionImpl::processWrites() {
  constexpr int kMaxVectors = 16;
  while (state_ == kOpen && !writes_.empty()) {
    // Gather what is left of the queued frames, oldest first, into one call.
    iovec iov[kMaxVectors];
    int cnt = 0;
    for (auto it = writes_.begin(); it != writes_.end() && cnt + 2 <= kMaxVectors; ++it) {
      WriteOp& op = *it;
      if (op.written < sizeof(uint64_t)) {
        iov[cnt].iov_base = reinterpret_cast<uint8_t*>(&op.length) + op.written;
        iov[cnt].iov_len = sizeof(uint64_t) - op.written;
        ++cnt;
        if (op.length > 0) {
          iov[cnt].iov_base = const_cast<uint8_t*>(op.ptr);
          iov[cnt].iov_len = op.length;
          ++cnt;
        }
      } else {
        const size_t off = op.written - sizeof(uint64_t);
        iov[cnt].iov_base = const_cast<uint8_t*>(op.ptr) + off;
        iov[cnt].iov_len = op.length - off;
        ++cnt;
      }
    }
    msghdr mh{};
    mh.msg_iov = iov;
    mh.msg_iovlen = cnt;
    ssize_t n = ::sendmsg(fd_, &mh, MSG_NOSIGNAL);
    if (n < 0) {
      if (errno == EAGAIN || errno == EWOULDBLOCK) {
        socketFull_ = true;
        return;
      }
      if (errno == EINTR) continue;
      closeFromLoop(TPB_CREATE_ERROR(SystemError, "sendmsg", errno));
      return;
    }
    socketFull_ = false;
    // Credit the bytes to the frames in order; the ones that are through call back.
    size_t sent = static_cast<size_t>(n);
    std::vector<Connection::write_callback_fn> completed;
    while (!writes_.empty()) {
      WriteOp& op = writes_.front();
      const size_t total = sizeof(uint64_t) + op.length;
      const size_t take = std::min(sent, total - op.written);
      op.written += take;
      sent -= take;
      if (op.written < total) break;
      completed.push_back(std::move(op.fn));
      writes_.pop_front();
    }
    for (auto& fn : completed) fn(Error::kSuccess);
  }
}

void ConnectionImpl::handleEventsFromLoop(int events) {
  auto self = shared_from_this();  // keep alive through callbacks that may drop the last ref
  if (state_ == kClosed) return;
  if (state_ == kConnecting) {
    int err = 0;
    socklen_t len = sizeof(err);
    ::getsockopt(fd_, SOL_SOCKET, SO_ERROR, &err, &len);
    if (err != 0 || (events & EPOLLERR)) {
      closeFromLoop(TPB_CREATE_ERROR(SystemError, "connect", err ? err : ECONNREFUSED));
      return;
    }
    if (events & EPOLLOUT) {
      state_ = kOpen;
      processWrites();
      if (state_ == kOpen) processReads();
      updateInterest();
    }
    return;
  }
  if (events & EPOLLIN) processReads();
  if (state_ == kOpen && (events & EPOLLOUT)) processWrites();
  if (state_ == kOpen && (events & (EPOLLERR | EPOLLHUP)) && !(events & EPOLLIN)) {
    int err = 0;
    socklen_t len = sizeof(err);
    ::getsockopt(fd_, SOL_SOCKET, SO_ERROR, &err, &len);
    if (err) closeFromLoop(TPB_CREATE_ERROR(SystemError, "socket", err));
    else closeFromLoop(TPB_CREATE_ERROR(EOFError));
    return;
  }
  // Not at once: the callback of the frame that just arrived has, as a rule, asked for the next
  // one, and that request is a closure queued behind us. Settling the interest after it has run
  // saves taking the descriptor out of the epoll set and putting it back for every frame.
  if (!interestUpdateScheduled_) {
    interestUpdateScheduled_ = true;
    ctx_->loop().deferToLoop([self]() {
      self->interestUpdateScheduled_ = false;
      self->updateInterest();
    });
  }
}

void ConnectionImpl::close() {
  auto self = shared_from_this();
  ctx_->loop().deferToLoop(
      [self]() { self->closeFromLoop(TPB_CREATE_ERROR(ConnectionClosedError)); });
}

void ConnectionImpl::closeFromLoop(const Error& e) {
  if (error_) return;
  // Frames that were handed over before the connection closes still go out if the socket takes
  // them (a channel writes its last acknowledgement and closes): their flush may still be queued
  // behind the closure that brought us here.
  if (flushScheduled_ && !flushingBeforeClose_ && state_ == kOpen && !writes_.empty() && !socketFull_) {
    flushingBeforeClose_ = true;
    processWrites();
    flushingBeforeClose_ = false;
    if (error_) return;  // the attempt itself failed and closed the connection
  }
  error_ = e;
  TPB_VLOG(7) << "Connection " << id_ << " is closing: " << e.what();
  auto self = shared_from_this();
  if (fd_ >= 0) {
    if (registered_) ctx_->loop().unregisterDescriptor(fd_);
    registered_ = false;
    ::close(fd_);
    fd_ = -1;
  }
  state_ = kClosed;
  ctx_->unenroll(self);
  failAll();
}

void ConnectionImpl::failAll() {
  auto reads = std::move(reads_);
  auto writes = std::move(writes_);
  reads_.clear();
  writes_.clear();
  for (auto& r : reads) r.fn(error_, nullptr, 0);
  for (auto& w : writes) w.fn(error_);
}

void ConnectionImpl::setId(std::string id) {
  auto self = shared_from_this();
  ctx_->loop().deferToLoop([self, id = std::move(id)]() mutable { self->id_ = std::move(id); });
}

// ---- listener -------------------------------------------------------------------------------
ListenerImpl::ListenerImpl(std::shared_ptr<ContextImpl> ctx, const std::string& addr)
    : ctx_(std::move(ctx)) {
  SockAddr sa;
  TPB_THROW_ASSERT_IF(!parseAddr(addr, sa), "cannot parse address " + addr);
  fd_ = ::socket(sa.ss.ss_family, SOCK_STREAM | SOCK_NONBLOCK | SOCK_CLOEXEC, 0);
  TPB_THROW_SYSTEM_IF(fd_ < 0, errno, "socket");
  int one = 1;
  ::setsockopt(fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  if (::bind(fd_, reinterpret_cast<sockaddr*>(&sa.ss), sa.len) < 0) {
    int e = errno;
    ::close(fd_);
    TPB_THROW_SYSTEM_IF(true, e, "bind " + addr);
  }
  if (::listen(fd_, 128) < 0) {
    int e = errno;
    ::close(fd_);
    TPB_THROW_SYSTEM_IF(true, e, "listen");
  }
  sockaddr_storage bound{};
  socklen_t len = sizeof(bound);
  ::getsockname(fd_, reinterpret_cast<sockaddr*>(&bound), &len);
  addr_ = formatAddr(reinterpret_cast<sockaddr*>(&bound));
}

void ListenerImpl::init() {
  auto self = shared_from_this();
  ctx_->loop().deferToLoop([self]() {
    if (self->ctx_->closed()) {
      self->closeFromLoop(TPB_CREATE_ERROR(ContextClosedError));
      return;
    }
    self->ctx_->enroll(self);
  });
}

void ListenerImpl::updateInterest() {
  if (fd_ < 0) return;
  bool want = !armed_.empty();
  if (want && !registered_) {
    ctx_->loop().registerDescriptor(fd_, EPOLLIN, shared_from_this());
    registered_ = true;
  } else if (!want && registered_) {
    ctx_->loop().unregisterDescriptor(fd_);
    registered_ = false;
  }
}

void ListenerImpl::accept(Listener::accept_callback_fn fn) {
  auto self = shared_from_this();
  ctx_->loop().deferToLoop([self, fn = std::move(fn)]() mutable {
    if (self->error_) {
      fn(self->error_, nullptr);
      return;
    }
    self->armed_.push_back(std::move(fn));
    self->updateInterest();
  });
}

void ListenerImpl::close() {
  auto self = shared_from_this();
  ctx_->loop().deferToLoop([self]() { self->closeFromLoop(TPB_CREATE_ERROR(ListenerClosedError)); });
}

void ListenerImpl::closeFromLoop(const Error& e) {
  if (error_) return;
  error_ = e;
  auto self = shared_from_this();
  if (fd_ >= 0) {
    if (registered_) ctx_->loop().unregisterDescriptor(fd_);
    registered_ = false;
    ::close(fd_);
    fd_ = -1;
  }
  ctx_->unenroll(self);
  auto armed = std::move(armed_);
  armed_.clear();
  for (auto& fn : armed) fn(error_, nullptr);
}

// ---- public shells --------------------------------------------------------------------------
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
    WriteOp op;
    op.ptr = static_cast<const uint8_t*>(ptr);
    op.length = length;
    op.fn = std::move(fn);
    impl_->write(std::move(op));
  }
  void setId(std::string id) override { impl_->setId(std::move(id)); }
  void close() override { impl_->close(); }

 private:
  std::shared_ptr<ConnectionImpl> impl_;
};

void ListenerImpl::handleEventsFromLoop(int events) {
  auto self = shared_from_this();
  if (events & (EPOLLERR | EPOLLHUP)) {
    closeFromLoop(TPB_CREATE_ERROR(SystemError, "accept", EIO));
    return;
  }
  while (!armed_.empty() && fd_ >= 0) {
    int cfd = ::accept4(fd_, nullptr, nullptr, SOCK_NONBLOCK | SOCK_CLOEXEC);
    if (cfd < 0) {
      if (errno == EAGAIN || errno == EWOULDBLOCK) break;
      if (errno == EINTR || errno == ECONNABORTED) continue;
      closeFromLoop(TPB_CREATE_ERROR(SystemError, "accept", errno));
      return;
    }
    int one = 1;
    ::setsockopt(cfd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    auto impl = std::make_shared<ConnectionImpl>(ctx_, cfd, ConnectionImpl::kOpen);
    impl->init();
    auto fn = std::move(armed_.front());
    armed_.pop_front();
    fn(Error::kSuccess, std::make_shared<ConnectionShell>(std::move(impl)));
  }
  updateInterest();
}

class ListenerShell final : public Listener {
 public:
  explicit ListenerShell(std::shared_ptr<ListenerImpl> impl) : impl_(std::move(impl)) {}
  ~ListenerShell() override { impl_->close(); }
  void accept(accept_callback_fn fn) override { impl_->accept(std::move(fn)); }
  std::string addr() const override { return impl_->addr(); }
  void setId(std::string id) override { impl_->setId(std::move(id)); }
  void close() override { impl_->close(); }

 private:
  std::shared_ptr<ListenerImpl> impl_;
};

class ContextShell final : public Context {
 public:
  ContextShell() : impl_(std::make_shared<ContextImpl>()) {}
  ~ContextShell() override { impl_->join(); }
  std::shared_ptr<Connection> connect(std::string addr) override {
    auto c = std::make_shared<ConnectionImpl>(impl_, std::move(addr));
    c->init();
    return std::make_shared<ConnectionShell>(std::move(c));
  }
  std::shared_ptr<Listener> listen(std::string addr) override {
    auto l = std::make_shared<ListenerImpl>(impl_, addr);
    l->init();
    return std::make_shared<ListenerShell>(std::move(l));
  }
  bool isViable() const override { return true; }
  const std::string& domainDescriptor() const override { return kDomainDescriptor; }
  void setId(std::string id) override { (void)id; }
  void close() override { impl_->close(); }
  void join() override { impl_->join(); }

 private:
  std::shared_ptr<ContextImpl> impl_;
};

}  // namespace

std::shared_ptr<Context> create() { return std::make_shared<ContextShell>(); }

std::pair<Error, std::string> lookupAddrForIface(const std::string& iface) {
  ifaddrs* list = nullptr;
  if (::getifaddrs(&list) < 0) return {TPB_CREATE_ERROR(SystemError, "getifaddrs", errno), ""};
  std::string found;
  for (ifaddrs* p = list; p; p = p->ifa_next) {
    if (!p->ifa_addr || iface != p->ifa_name) continue;
    if (p->ifa_addr->sa_family == AF_INET || p->ifa_addr->sa_family == AF_INET6) {
      found = formatAddr(p->ifa_addr, false);
      if (p->ifa_addr->sa_family == AF_INET) break;  // prefer v4
    }
  }
  ::freeifaddrs(list);
  if (found.empty()) return {TPB_CREATE_ERROR(NoAddrFoundError), ""};
  return {Error::kSuccess, found};
}

std::pair<Error, std::string> lookupAddrForHostname() {
  char host[256] = {0};
  if (::gethostname(host, sizeof(host) - 1) < 0)
    return {TPB_CREATE_ERROR(SystemError, "gethostname", errno), ""};
  addrinfo hints{};
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  addrinfo* res = nullptr;
  if (::getaddrinfo(host, nullptr, &hints, &res) != 0 || !res)
    return {TPB_CREATE_ERROR(NoAddrFoundError), ""};
  std::string found;
  for (addrinfo* p = res; p; p = p->ai_next) {
    // Only keep an address we can actually bind to.
    int fd = ::socket(p->ai_family, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) continue;
    bool ok = ::bind(fd, p->ai_addr, p->ai_addrlen) == 0;
    ::close(fd);
    if (ok) {
      found = formatAddr(p->ai_addr, false);
      break;
    }
  }
  ::freeaddrinfo(res);
  if (found.empty()) return {TPB_CREATE_ERROR(NoAddrFoundError), ""};
  return {Error::kSuccess, found};
}

// The address NCCL would pick for its sockets, so that both libraries of one job end up on the
// same network: the first interface that is up, not a loopback over IPv6 and (optionally) of the
// wanted family, ranked by name — "ib*" first (IP over InfiniBand), then anything else, then
// "docker*", then "lo*". Same ranking as tensorpipe/transport/uv/utility.cc:138-215.
std::pair<Error, std::string> lookupAddrLikeNccl(int family) {
  ifaddrs* list = nullptr;
  if (::getifaddrs(&list) < 0) return {TPB_CREATE_ERROR(SystemError, "getifaddrs", errno), ""};
  // rank 0: ib*, 1: unremarkable, 2: docker*, 3: lo*
  std::string best[4];
  for (ifaddrs* p = list; p; p = p->ifa_next) {
    if (!p->ifa_addr || !p->ifa_name) continue;
    const int fam = p->ifa_addr->sa_family;
    if (fam != AF_INET && fam != AF_INET6) continue;
    if (!(p->ifa_flags & IFF_UP) || !(p->ifa_flags & IFF_RUNNING)) continue;
    if (fam == AF_INET6 && (p->ifa_flags & IFF_LOOPBACK)) continue;
    if (family != AF_UNSPEC && fam != family) continue;
    const std::string name = p->ifa_name;
    const int rank = name.rfind("ib", 0) == 0 ? 0 : name.rfind("docker", 0) == 0 ? 2 : name.rfind("lo", 0) == 0 ? 3 : 1;
    if (best[rank].empty()) best[rank] = formatAddr(p->ifa_addr, false);
  }
  ::freeifaddrs(list);
  for (const std::string& addr : best)
    if (!addr.empty()) return {Error::kSuccess, addr};
  return {TPB_CREATE_ERROR(NoAddrFoundError), ""};
}

}  // namespace tcp
}  // namespace transport
}  // namespace tpb
