// mpt ("multiplexed transports"): a CPU channel that stripes every tensor over N lanes, each
// lane being a connection of its own transport context (typically N TCP loops), so that one
// large tensor is moved by N threads / sockets at once.
//
// As in the reference (tensorpipe/channel/mpt/channel_impl.cc:41-155,203-314, nop_types.h:22-43):
// the context is built from N transport contexts and N listeners; the listening endpoint of a
// channel sends ServerHello{(address, registration id) per lane} on the connection the pipe
// provided; the connecting endpoint dials every lane and identifies itself with
// ClientHello{registration id}; a tensor of L bytes is cut into N contiguous chunks at the byte offsets L*i/N
// (rounded down), chunk i travelling on lane i. The device descriptor is
// "N:<dd1>:<dd2>..." so both ends must have the same lane transports.
#include <deque>
#include <map>
#include <set>
#include <variant>

#include <tpb/channel.h>

#include "channel/nonviable.h"
#include "common/defs.h"
#include "common/loop.h"
#include "common/nop.h"
#include "transport/nop_io.h"

namespace tpb {
namespace channel {
namespace mpt {

namespace {

struct LaneAdvertisement {
  std::string address;
  uint64_t registrationId = 0;
  TPB_NOP_STRUCTURE(LaneAdvertisement, address, registrationId)
};
struct ServerHello {
  std::vector<LaneAdvertisement> laneAdvertisements;
  TPB_NOP_STRUCTURE(ServerHello, laneAdvertisements)
};
struct ClientHello {
  uint64_t registrationId = 0;
  TPB_NOP_STRUCTURE(ClientHello, registrationId)
};
using Packet = std::variant<ServerHello, ClientHello>;

class ContextImpl;

class ChannelImpl final : public Channel, public std::enable_shared_from_this<ChannelImpl> {
 public:
  ChannelImpl(std::shared_ptr<ContextImpl> ctx, std::shared_ptr<transport::Connection> conn, Endpoint ep)
      : ctx_(std::move(ctx)), conn_(std::move(conn)), endpoint_(ep) {}
  ~ChannelImpl() override {
    conn_->close();
    for (auto& l : lanes_)
      if (l) l->close();
  }
  void init();
  void send(Buffer buffer, size_t length, TSendCallback cb) override;
  void recv(Buffer buffer, size_t length, TRecvCallback cb) override;
  void setId(std::string id) override { (void)id; }
  void close() override;
  void closeFromLoop(const Error& e);
  void onLane(size_t lane, std::shared_ptr<transport::Connection> c);

 private:
  struct Op {
    bool isSend;
    uint8_t* ptr;
    size_t length;
    std::function<void(const Error&)> cb;
  };
  void flush();
  void issue(Op op);
  std::shared_ptr<ContextImpl> ctx_;
  std::shared_ptr<transport::Connection> conn_;
  Endpoint endpoint_;
  Error error_;
  std::vector<std::shared_ptr<transport::Connection>> lanes_;
  size_t lanesReady_ = 0;
  bool established_ = false;
  std::vector<uint64_t> registrationIds_;
  std::deque<Op> queued_;  // operations issued before all lanes exist
};

class ContextImpl final : public Context, public std::enable_shared_from_this<ContextImpl> {
 public:
  ContextImpl(std::vector<std::shared_ptr<transport::Context>> contexts,
              std::vector<std::shared_ptr<transport::Listener>> listeners)
      : contexts_(std::move(contexts)), listeners_(std::move(listeners)) {
    std::string d = std::to_string(contexts_.size());
    for (auto& c : contexts_) d += ":" + c->domainDescriptor();
    descriptors_[Device(kCpuDeviceType, 0)] = d;
    for (auto& l : listeners_) addresses_.push_back(l->addr());
  }
  void start() {
    for (size_t i = 0; i < listeners_.size(); ++i) armLane(i);
  }
  bool isViable() const override { return true; }
  const std::unordered_map<Device, std::string>& deviceDescriptors() const override { return descriptors_; }
  std::shared_ptr<Channel> createChannel(std::vector<std::shared_ptr<transport::Connection>> conns, Endpoint ep) override {
    TPB_THROW_ASSERT_IF(conns.size() != 1, "mpt needs exactly one connection from the pipe");
    auto ch = std::make_shared<ChannelImpl>(shared_from_this(), std::move(conns[0]), ep);
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
      for (auto& l : listeners_) l->close();
      for (auto& c : pendingLaneConnections_) c->close();
      pendingLaneConnections_.clear();
      for (auto& c : contexts_) c->close();
    });
  }
  void join() override {
    close();
    loop_.runInLoop([]() {});
    for (auto& c : contexts_) c->join();
    loop_.runInLoop([]() {});
  }

  size_t numLanes() const { return contexts_.size(); }
  const std::vector<std::string>& addresses() const { return addresses_; }
  std::shared_ptr<transport::Connection> connectLane(size_t lane, const std::string& addr) {
    return contexts_[lane]->connect(addr);
  }
  // From the loop.
  uint64_t registerLane(std::weak_ptr<ChannelImpl> ch, size_t lane) {
    uint64_t id = nextRegistration_++;
    registrations_[id] = {std::move(ch), lane};
    return id;
  }
  void unregisterLane(uint64_t id) { registrations_.erase(id); }

  OnDemandLoop loop_;
  bool closed_ = false;
  std::set<std::weak_ptr<ChannelImpl>, std::owner_less<std::weak_ptr<ChannelImpl>>> channels_;

 private:
  void armLane(size_t lane) {
    auto self = shared_from_this();
    listeners_[lane]->accept([self, lane](const Error& e, std::shared_ptr<transport::Connection> c) {
      self->loop_.deferToLoop([self, lane, e, c]() {
        if (e || self->closed_) return;
        self->armLane(lane);
        self->pendingLaneConnections_.insert(c);
        transport::readNop<Packet>(*c, [self, c](const Error& re, Packet p) {
          self->loop_.deferToLoop([self, c, re, p]() {
            self->pendingLaneConnections_.erase(c);
            if (re || self->closed_ || !std::holds_alternative<ClientHello>(p)) return;
            auto it = self->registrations_.find(std::get<ClientHello>(p).registrationId);
            if (it == self->registrations_.end()) return;
            auto reg = it->second;
            self->registrations_.erase(it);
            if (auto ch = reg.first.lock()) ch->onLane(reg.second, c);
          });
        });
      });
    });
  }
  std::vector<std::shared_ptr<transport::Context>> contexts_;
  std::vector<std::shared_ptr<transport::Listener>> listeners_;
  std::vector<std::string> addresses_;
  std::unordered_map<Device, std::string> descriptors_;
  uint64_t nextRegistration_ = 0;
  std::map<uint64_t, std::pair<std::weak_ptr<ChannelImpl>, size_t>> registrations_;
  std::set<std::shared_ptr<transport::Connection>> pendingLaneConnections_;
};

void ChannelImpl::init() {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self]() {
    if (self->ctx_->closed_) return self->closeFromLoop(TPB_CREATE_ERROR(ContextClosedError));
    self->ctx_->channels_.insert(self);
    const size_t n = self->ctx_->numLanes();
    self->lanes_.resize(n);
    if (self->endpoint_ == Endpoint::kListen) {
      ServerHello hello;
      for (size_t i = 0; i < n; ++i) {
        uint64_t id = self->ctx_->registerLane(self, i);
        self->registrationIds_.push_back(id);
        hello.laneAdvertisements.push_back({self->ctx_->addresses()[i], id});
      }
      Packet p = hello;
      transport::writeNop(*self->conn_, p, [self](const Error& e) {
        if (e) self->ctx_->loop_.deferToLoop([self, e]() { self->closeFromLoop(e); });
      });
    } else {
      transport::readNop<Packet>(*self->conn_, [self](const Error& e, Packet p) {
        self->ctx_->loop_.deferToLoop([self, e, p]() {
          if (self->error_) return;
          if (e) return self->closeFromLoop(e);
          if (!std::holds_alternative<ServerHello>(p))
            return self->closeFromLoop(TPB_CREATE_ERROR(LogicError, "mpt: expected a server hello"));
          const auto& ads = std::get<ServerHello>(p).laneAdvertisements;
          if (ads.size() != self->lanes_.size())
            return self->closeFromLoop(TPB_CREATE_ERROR(LogicError, "mpt: peer has a different number of lanes"));
          for (size_t i = 0; i < ads.size(); ++i) {
            auto c = self->ctx_->connectLane(i, ads[i].address);
            Packet hello = ClientHello{ads[i].registrationId};
            transport::writeNop(*c, hello, [self](const Error& we) {
              if (we) self->ctx_->loop_.deferToLoop([self, we]() { self->closeFromLoop(we); });
            });
            self->onLane(i, std::move(c));
          }
        });
      });
    }
  });
}

void ChannelImpl::onLane(size_t lane, std::shared_ptr<transport::Connection> c) {
  if (error_) {
    c->close();
    return;
  }
  lanes_[lane] = std::move(c);
  if (++lanesReady_ == lanes_.size()) {
    established_ = true;
    registrationIds_.clear();
    flush();
  }
}

void ChannelImpl::flush() {
  auto queued = std::move(queued_);
  queued_.clear();
  for (auto& op : queued) issue(std::move(op));
}

void ChannelImpl::issue(Op op) {
  if (error_) return op.cb(error_);
  if (!established_) {
    queued_.push_back(std::move(op));
    return;
  }
  const size_t n = lanes_.size();
  // Cut points at length * i / n, rounded down: what a reference peer's lanes expect
  // (tensorpipe/channel/mpt/channel_impl.cc:203-215), so the two libraries can share the channel.
  auto cut = [&](size_t i) { return static_cast<size_t>(static_cast<unsigned __int128>(op.length) * i / n); };
  struct Join {
    size_t remaining;
    Error error;
    std::function<void(const Error&)> cb;
  };
  auto join = std::make_shared<Join>();
  join->remaining = n;
  join->cb = std::move(op.cb);
  auto self = shared_from_this();
  for (size_t i = 0; i < n; ++i) {
    const size_t off = cut(i);
    const size_t len = cut(i + 1) - off;
    auto done = [self, join](const Error& e) {
      self->ctx_->loop_.deferToLoop([self, join, e]() {
        if (e && !join->error) join->error = e;
        if (--join->remaining == 0) join->cb(join->error);
      });
    };
    // Lanes always carry a frame, even an empty one, so the two ends stay in step.
    if (op.isSend) lanes_[i]->write(op.ptr + off, len, done);
    else lanes_[i]->read(op.ptr + off, len, [done](const Error& e, const void*, size_t) { done(e); });
  }
}

void ChannelImpl::send(Buffer buffer, size_t length, TSendCallback cb) {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self, buffer, length, cb = std::move(cb)]() mutable {
    if (self->error_) return cb(self->error_);
    if (length == 0) return cb(Error::kSuccess);
    self->issue({true, static_cast<uint8_t*>(buffer.unwrap<CpuBuffer>().ptr), length, std::move(cb)});
  });
}

void ChannelImpl::recv(Buffer buffer, size_t length, TRecvCallback cb) {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self, buffer, length, cb = std::move(cb)]() mutable {
    if (self->error_) return cb(self->error_);
    if (length == 0) return cb(Error::kSuccess);
    self->issue({false, static_cast<uint8_t*>(buffer.unwrap<CpuBuffer>().ptr), length, std::move(cb)});
  });
}

void ChannelImpl::close() {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self]() { self->closeFromLoop(TPB_CREATE_ERROR(ChannelClosedError)); });
}

void ChannelImpl::closeFromLoop(const Error& e) {
  if (error_) return;
  error_ = e;
  conn_->close();
  for (auto& l : lanes_)
    if (l) l->close();
  for (uint64_t id : registrationIds_) ctx_->unregisterLane(id);
  registrationIds_.clear();
  ctx_->channels_.erase(weak_from_this());
  auto queued = std::move(queued_);
  queued_.clear();
  for (auto& op : queued) op.cb(error_);
}

// What the user holds. The implementation is kept alive by the accept callbacks armed on its
// lanes, so without this its last reference could die on a lane's own I/O thread, whose
// destructor would then try to join itself. Dropping the shell joins from the caller's thread.
class ContextShell final : public Context {
 public:
  explicit ContextShell(std::shared_ptr<ContextImpl> impl) : impl_(std::move(impl)) {}
  ~ContextShell() override { impl_->join(); }
  bool isViable() const override { return impl_->isViable(); }
  size_t numConnectionsNeeded() const override { return impl_->numConnectionsNeeded(); }
  const std::unordered_map<Device, std::string>& deviceDescriptors() const override {
    return impl_->deviceDescriptors();
  }
  bool canCommunicateWithRemote(const std::string& local, const std::string& remote) const override {
    return impl_->canCommunicateWithRemote(local, remote);
  }
  std::shared_ptr<Channel> createChannel(std::vector<std::shared_ptr<transport::Connection>> connections,
                                         Endpoint endpoint) override {
    return impl_->createChannel(std::move(connections), endpoint);
  }
  void setId(std::string id) override { impl_->setId(std::move(id)); }
  void close() override { impl_->close(); }
  void join() override { impl_->join(); }

 private:
  std::shared_ptr<ContextImpl> impl_;
};

}  // namespace

std::shared_ptr<Context> create(std::vector<std::shared_ptr<transport::Context>> contexts,
                                std::vector<std::shared_ptr<transport::Listener>> listeners) {
  if (contexts.empty() || contexts.size() != listeners.size()) return std::make_shared<NonViableContext>();
  for (auto& c : contexts)
    if (!c->isViable()) return std::make_shared<NonViableContext>();
  auto ctx = std::make_shared<ContextImpl>(std::move(contexts), std::move(listeners));
  ctx->start();
  return std::make_shared<ContextShell>(std::move(ctx));
}

}  // namespace mpt
}  // namespace channel
}  // namespace tpb
