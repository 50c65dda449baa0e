// Setting a pipe up: what the two ends say to each other before the first message, and how the
// result is turned into connections and channels.
//
//   dialer                                     answerer (made by the listener)
//   ------                                     --------
//   Packet{"I am a new pipe from <context>"}
//   Brochure{my transports' domain descriptors,
//            my channels' device descriptors}
//                                              picks the transport (its own order of preference,
//                                              must be bound and compatible), picks a channel per
//                                              device pair, issues one ticket per connection it
//                                              now expects
//                                              BrochureAnswer{transport, address, tickets, its
//                                              channels' descriptors, its view of the routes}
//   dials the connections, each announcing
//   its ticket; checks that its own choice of
//   routes is the answerer's; creates channels
//                                              collects the connections, creates channels
//
// The frames and their order are what a reference peer speaks (tensorpipe/core/nop_types.h:38-64).
#include <algorithm>

#include "common/url.h"
#include "core/core.h"
#include "transport/nop_io.h"

namespace tpb {
namespace core {

namespace {
constexpr uint64_t kWireSlot = 0;       // key of the descriptor connection in the answer's ticket map
constexpr uint64_t kReplyWireSlot = 1;  // key of the descriptor-reply connection

Error badHandshake(const std::exception& ex) {
  return TPB_CREATE_ERROR(LogicError, std::string("inconsistent handshake from the peer: ") + ex.what());
}
}  // namespace

PipeCore::PipeCore(std::shared_ptr<ContextCore> context, std::string id, std::string remoteName, const std::string& url)
    : context_(std::move(context)), id_(std::move(id)), remoteName_(std::move(remoteName)), role_(Role::kDialer) {
  auto [scheme, address] = splitSchemeOfURL(url);
  wireTransport_ = scheme;
  wire_ = context_->transports().require(scheme)->connect(address);
  wire_->setId(id_ + "/wire@" + scheme);
}

PipeCore::PipeCore(std::shared_ptr<ContextCore> context, std::shared_ptr<ListenerCore> listener, std::string id,
                   std::string remoteName, std::string transport, std::shared_ptr<transport::Connection> wire)
    : context_(std::move(context)),
      listener_(std::move(listener)),
      id_(std::move(id)),
      remoteName_(std::move(remoteName)),
      role_(Role::kAnswerer),
      wireTransport_(std::move(transport)),
      wire_(std::move(wire)) {
  wire_->setId(id_ + "/wire@" + wireTransport_);
}

void PipeCore::start() {
  auto self = shared_from_this();
  context_->defer([self]() { self->startNow(); });
}

void PipeCore::startNow() {
  if (context_->closing()) return fail(TPB_CREATE_ERROR(ContextClosedError));
  auto self = shared_from_this();
  context_->adopt(self);
  if (role_ == Role::kDialer) {
    sendOffer();
    return;
  }
  phase_ = Phase::kAwaitingOffer;
  transport::readNop<Brochure>(*wire_, onLoopOf(self, [self](Brochure offer) {
    if (self->error_) return;
    // A well-formed brochure can still ask for the impossible; that fails this pipe only.
    try {
      self->onOffer(offer);
    } catch (const std::exception& ex) {
      self->fail(badHandshake(ex));
    }
  }));
}

void PipeCore::sendOffer() {
  auto self = shared_from_this();
  auto written = [self]() {};
  Packet hello = SpontaneousConnection{context_->name()};
  transport::writeNop(*wire_, hello, onLoopOf(self, written));

  Brochure offer;
  for (const auto& slot : context_->transports().bestFirst())
    offer.transportDomainDescriptors[slot.name] = slot.backend->domainDescriptor();
  for (const auto& slot : context_->channels().bestFirst())
    offer.channelDeviceDescriptors[slot.name] = slot.backend->deviceDescriptors();
  TPB_VLOG(3) << "Pipe " << id_ << " offers " << offer.transportDomainDescriptors.size() << " transports and "
              << offer.channelDeviceDescriptors.size() << " channels";
  transport::writeNop(*wire_, offer, onLoopOf(self, written));

  phase_ = Phase::kAwaitingAnswer;
  transport::readNop<BrochureAnswer>(*wire_, onLoopOf(self, [self](BrochureAnswer answer) {
    if (self->error_) return;
    try {
      self->onAnswer(answer);
    } catch (const std::exception& ex) {
      self->fail(badHandshake(ex));
    }
  }));
}

PipeCore::Routes PipeCore::chooseRoutes(const std::unordered_map<std::string, DeviceDescriptors>& theirs,
                                        std::vector<std::string>* used) {
  Routes routes;
  for (const auto& slot : context_->channels().bestFirst()) {
    auto peer = theirs.find(slot.name);
    if (peer == theirs.end()) continue;
    bool serves = false;
    for (const auto& mine : slot.backend->deviceDescriptors()) {
      for (const auto& other : peer->second) {
        const auto pair = std::make_pair(mine.first, other.first);
        if (routes.count(pair)) continue;  // a better channel already has this pair
        if (!slot.backend->canCommunicateWithRemote(mine.second, other.second)) continue;
        routes.emplace(pair, slot.name);
        serves = true;
      }
    }
    if (serves) used->push_back(slot.name);
  }
  return routes;
}

uint64_t PipeCore::expect(Expected what) {
  auto self = shared_from_this();
  auto ticketBox = std::make_shared<uint64_t>(0);
  const uint64_t ticket = listener_->issueTicket(
      onLoopOf(self, [self, ticketBox](std::string transport, std::shared_ptr<transport::Connection> conn) {
        if (!self->error_) self->onLink(*ticketBox, transport, std::move(conn));
      }));
  *ticketBox = ticket;
  expected_.emplace(ticket, std::move(what));
  return ticket;
}

void PipeCore::onOffer(const Brochure& offer) {
  BrochureAnswer answer;

  // The transport: my order of preference, among those the listener is bound on and the peer has.
  const Backends<transport::Context>::Slot* chosen = nullptr;
  const std::string* chosenAddress = nullptr;
  for (const auto& slot : context_->transports().bestFirst()) {
    auto bound = listener_->addresses().find(slot.name);
    if (bound == listener_->addresses().end()) continue;
    auto peer = offer.transportDomainDescriptors.find(slot.name);
    if (peer == offer.transportDomainDescriptors.end()) continue;
    if (!slot.backend->canCommunicateWithRemote(peer->second)) continue;
    chosen = &slot;
    chosenAddress = &bound->second;
    break;
  }
  TPB_THROW_ASSERT_IF(chosen == nullptr, "the two ends have no usable transport in common");
  answer.transport = chosen->name;
  answer.address = *chosenAddress;
  answer.transportDomainDescriptor = chosen->backend->domainDescriptor();
  if (chosen->name != wireTransport_) {
    // The dialer came in over something worse than what we can both do: it will redial.
    wireTransport_ = chosen->name;
    answer.transportRegistrationIds[kWireSlot] = expect({Expected::kWire, {}, 0});
  }
  answer.transportRegistrationIds[kReplyWireSlot] = expect({Expected::kReplyWire, {}, 0});

  std::vector<std::string> used;
  routes_ = chooseRoutes(offer.channelDeviceDescriptors, &used);
  answer.channelForDevicePair = routes_;
  for (const std::string& name : used) {
    auto backend = context_->channels().require(name);
    const size_t links = backend->numConnectionsNeeded();
    Mover& mover = movers_[name];
    mover.links.resize(links);
    mover.missing = links;
    std::vector<uint64_t>& tickets = answer.channelRegistrationIds[name];
    for (size_t i = 0; i < links; ++i) tickets.push_back(expect({Expected::kChannelLink, name, i}));
    answer.channelDeviceDescriptors[name] = backend->deviceDescriptors();
    if (links == 0) {
      mover.channel = backend->createChannel({}, channel::Endpoint::kListen);
      mover.channel->setId(id_ + "/" + name);
    }
  }

  TPB_VLOG(3) << "Pipe " << id_ << " answers: transport " << answer.transport << ", " << used.size()
              << " channels, " << expected_.size() << " connections expected";
  auto self = shared_from_this();
  transport::writeNop(*wire_, answer, onLoopOf(self, [self]() {}));
  if (expected_.empty()) becomeOpen();
  else phase_ = Phase::kAwaitingLinks;
}

void PipeCore::onLink(uint64_t ticket, const std::string& transport, std::shared_ptr<transport::Connection> conn) {
  auto it = expected_.find(ticket);
  if (it == expected_.end()) return;
  Expected what = std::move(it->second);
  expected_.erase(it);
  switch (what.kind) {
    case Expected::kWire:
      conn->setId(id_ + "/wire@" + transport);
      wire_ = std::move(conn);  // the connection that carried the handshake is let go
      break;
    case Expected::kReplyWire:
      conn->setId(id_ + "/reply@" + transport);
      replyWire_ = std::move(conn);
      break;
    case Expected::kChannelLink: {
      Mover& mover = movers_.at(what.channel);
      conn->setId(id_ + "/" + what.channel + "#" + std::to_string(what.index));
      mover.links[what.index] = std::move(conn);
      if (--mover.missing == 0) {
        mover.channel = context_->channels().require(what.channel)->createChannel(std::move(mover.links),
                                                                                 channel::Endpoint::kListen);
        mover.channel->setId(id_ + "/" + what.channel);
        mover.links.clear();
      }
      break;
    }
  }
  if (expected_.empty()) becomeOpen();
}

void PipeCore::presentTicket(transport::Connection& conn, uint64_t ticket) {
  Packet p = RequestedConnection{ticket};
  transport::writeNop(conn, p, onLoopOf(shared_from_this(), []() {}));
}

void PipeCore::onAnswer(const BrochureAnswer& answer) {
  auto transport = context_->transports().require(answer.transport);
  auto ticketFor = [&](uint64_t slot, const char* what) {
    auto it = answer.transportRegistrationIds.find(slot);
    TPB_THROW_ASSERT_IF(it == answer.transportRegistrationIds.end(), std::string("the peer named no ticket for the ") + what);
    return it->second;
  };
  if (answer.transport != wireTransport_) {
    auto conn = transport->connect(answer.address);
    conn->setId(id_ + "/wire@" + answer.transport);
    presentTicket(*conn, ticketFor(kWireSlot, "descriptor connection"));
    wireTransport_ = answer.transport;
    wire_ = std::move(conn);
  }
  {
    auto conn = transport->connect(answer.address);
    conn->setId(id_ + "/reply@" + answer.transport);
    presentTicket(*conn, ticketFor(kReplyWireSlot, "descriptor-reply connection"));
    replyWire_ = std::move(conn);
  }

  // Both ends choose routes on their own, each with its own priorities; the pipe only works if
  // they chose alike.
  std::vector<std::string> used;
  routes_ = chooseRoutes(answer.channelDeviceDescriptors, &used);
  bool agree = answer.channelForDevicePair.size() == routes_.size();
  for (auto it = routes_.begin(); agree && it != routes_.end(); ++it) {
    auto theirs = answer.channelForDevicePair.find({it->first.second, it->first.first});
    agree = theirs != answer.channelForDevicePair.end() && theirs->second == it->second;
  }
  TPB_THROW_ASSERT_IF(!agree, "the two ends chose different channels for the same device pairs "
                              "(are the channel priorities the same on both sides?)");

  for (const std::string& name : used) {
    auto backend = context_->channels().require(name);
    auto tickets = answer.channelRegistrationIds.find(name);
    TPB_THROW_ASSERT_IF(tickets == answer.channelRegistrationIds.end(), "the peer named no tickets for channel " + name);
    const size_t links = backend->numConnectionsNeeded();
    TPB_THROW_ASSERT_IF(links != tickets->second.size(),
                        "channel " + name + " wants " + std::to_string(links) + " connections here and " +
                            std::to_string(tickets->second.size()) + " at the peer");
    std::vector<std::shared_ptr<transport::Connection>> conns;
    for (size_t i = 0; i < links; ++i) {
      auto conn = transport->connect(answer.address);
      conn->setId(id_ + "/" + name + "#" + std::to_string(i));
      presentTicket(*conn, tickets->second[i]);
      conns.push_back(std::move(conn));
    }
    Mover& mover = movers_[name];
    mover.channel = backend->createChannel(std::move(conns), channel::Endpoint::kConnect);
    mover.channel->setId(id_ + "/" + name);
  }
  becomeOpen();
}

void PipeCore::becomeOpen() {
  TPB_VLOG(1) << "Pipe " << id_ << " is open over " << wireTransport_ << " with " << movers_.size() << " channels";
  phase_ = Phase::kOpen;
  pumpOutbound();
  pumpInbound();
}

channel::Channel* PipeCore::channelFor(const Device& local, const Device& remote, const std::string** name) {
  auto route = routes_.find({local, remote});
  if (route == routes_.end()) return nullptr;
  auto mover = movers_.find(route->second);
  if (mover == movers_.end() || !mover->second.channel) return nullptr;
  if (name) *name = &route->second;
  return mover->second.channel.get();
}

bool PipeCore::routeSupportsLayouts(const Device& local, const Device& remote) {
  bool yes = false;
  context_->runSync([&]() {
    if (channel::Channel* ch = channelFor(local, remote)) yes = ch->supportsLayouts();
  });
  return yes;
}

std::string PipeCore::transportName() {
  std::string name;
  context_->runSync([&]() { name = wireTransport_; });
  return name;
}

void PipeCore::close() {
  auto self = shared_from_this();
  context_->defer([self]() { self->fail(TPB_CREATE_ERROR(PipeClosedError)); });
}

void PipeCore::fail(const Error& e) {
  if (error_ || !e) return;
  error_ = e;
  phase_ = Phase::kFailed;
  TPB_VLOG(1) << "Pipe " << id_ << " fails: " << error_.what();
  auto self = shared_from_this();  // the context may hold the last reference
  if (wire_) wire_->close();
  if (replyWire_) replyWire_->close();
  for (auto& m : movers_) {
    if (m.second.channel) m.second.channel->close();
    for (auto& link : m.second.links)
      if (link) link->close();
  }
  if (listener_)
    for (auto& pending : expected_) listener_->revokeTicket(pending.first);
  expected_.clear();
  // Whatever is in flight comes back with an error and retires through these; what never
  // started retires now.
  pumpOutbound();
  pumpInbound();
  context_->release(this);
}

}  // namespace core

// ---- public shell ---------------------------------------------------------------------------
Pipe::Pipe(ConstructorToken, std::shared_ptr<core::PipeCore> impl) : impl_(std::move(impl)) {}
void Pipe::readDescriptor(read_descriptor_callback_fn fn) { impl_->readDescriptor(std::move(fn)); }
void Pipe::read(Allocation allocation, read_callback_fn fn) { impl_->read(std::move(allocation), std::move(fn)); }
void Pipe::write(Message message, write_callback_fn fn) { impl_->write(std::move(message), std::move(fn)); }
void Pipe::setTimeouts(PipeTimeouts timeouts) { impl_->setTimeouts(timeouts); }
const std::string& Pipe::getRemoteName() { return impl_->remoteName(); }
std::string Pipe::transportName() { return impl_->transportName(); }
bool Pipe::channelSupportsLayouts(const Device& local, const Device& remote) {
  return impl_->routeSupportsLayouts(local, remote);
}
void Pipe::close() { impl_->close(); }
Pipe::~Pipe() { close(); }

}  // namespace tpb
