// The listener: one transport listener per URL, a queue that pairs new pipes with accept()
// calls, and the ticket table through which a pipe under construction collects the extra
// connections its client opens. First frame on every accepted connection is a Packet
// (tensorpipe/core/nop_types.h:26-34,80): either "I am a new pipe from context X" or "I am the
// connection for ticket N".
#include "common/url.h"
#include "core/core.h"
#include "transport/nop_io.h"

namespace tpb {
namespace core {

ListenerCore::ListenerCore(std::shared_ptr<ContextCore> context, std::string id, const std::vector<std::string>& urls)
    : context_(std::move(context)), id_(std::move(id)) {
  for (const std::string& url : urls) {
    auto [scheme, address] = splitSchemeOfURL(url);
    auto socket = context_->transports().require(scheme)->listen(address);
    socket->setId(id_ + "@" + scheme);
    bound_[scheme] = socket->addr();
    sockets_[scheme] = std::move(socket);
  }
}

void ListenerCore::start() {
  auto self = shared_from_this();
  context_->defer([self]() {
    if (self->context_->closing()) return self->fail(TPB_CREATE_ERROR(ContextClosedError));
    self->context_->adopt(self);
    for (const auto& s : self->sockets_) self->watch(s.first);
  });
}

// Keep exactly one accept pending per transport listener.
void ListenerCore::watch(const std::string& transport) {
  auto socket = sockets_.find(transport);
  if (socket == sockets_.end() || error_) return;
  auto self = shared_from_this();
  socket->second->accept(onLoopOf(self, [self, transport](std::shared_ptr<transport::Connection> conn) {
    if (self->error_) return;
    self->greet(transport, std::move(conn));
    self->watch(transport);
  }));
}

void ListenerCore::greet(const std::string& transport, std::shared_ptr<transport::Connection> conn) {
  unidentified_.insert(conn);
  auto self = shared_from_this();
  std::weak_ptr<transport::Connection> weak = conn;
  transport::readNop<Packet>(*conn, onLoopOf(self, [self, transport, weak](Packet hello) {
    auto conn = weak.lock();
    if (!conn || self->unidentified_.erase(conn) == 0 || self->error_) return;
    self->admit(transport, std::move(conn), std::move(hello));
  }));
}

void ListenerCore::admit(const std::string& transport, std::shared_ptr<transport::Connection> conn, Packet hello) {
  if (auto* fresh = std::get_if<SpontaneousConnection>(&hello)) {
    std::string pipeId = id_ + ".p" + std::to_string(pipesMade_++);
    TPB_VLOG(1) << "Listener " << id_ << " opens pipe " << pipeId << " for " << fresh->contextName;
    auto core = std::make_shared<PipeCore>(context_, shared_from_this(), std::move(pipeId), fresh->contextName,
                                           transport, std::move(conn));
    core->startNow();
    waitingPipes_.push_back(std::make_shared<Pipe>(Pipe::kToken, std::move(core)));
    matchAccepts();
    return;
  }
  const uint64_t ticket = std::get<RequestedConnection>(hello).registrationId;
  auto holder = tickets_.find(ticket);
  if (holder == tickets_.end()) {
    // Whoever issued it has gone away; letting go of the connection closes it.
    TPB_VLOG(3) << "Listener " << id_ << " drops a connection presenting unknown ticket " << ticket;
    return;
  }
  TicketFn fn = std::move(holder->second);
  tickets_.erase(holder);
  fn(Error::kSuccess, transport, std::move(conn));
}

void ListenerCore::matchAccepts() {
  while (!waitingAccepts_.empty() && !waitingPipes_.empty()) {
    auto fn = std::move(waitingAccepts_.front());
    waitingAccepts_.pop_front();
    auto pipe = std::move(waitingPipes_.front());
    waitingPipes_.pop_front();
    fn(Error::kSuccess, std::move(pipe));
  }
}

void ListenerCore::accept(Listener::accept_callback_fn fn) {
  auto self = shared_from_this();
  context_->defer([self, fn = std::move(fn)]() mutable {
    if (self->error_) return fn(self->error_, nullptr);
    self->waitingAccepts_.push_back(std::move(fn));
    self->matchAccepts();
  });
}

const std::string& ListenerCore::address(const std::string& transport) const {
  auto it = bound_.find(transport);
  TPB_THROW_ASSERT_IF(it == bound_.end(), "the listener is not bound on transport " + transport);
  return it->second;
}

uint64_t ListenerCore::issueTicket(TicketFn fn) {
  const uint64_t ticket = ticketsIssued_++;
  if (error_) {
    const Error why = error_;
    context_->defer([fn = std::move(fn), why]() { fn(why, std::string(), nullptr); });
  } else {
    tickets_.emplace(ticket, std::move(fn));
  }
  return ticket;
}

void ListenerCore::revokeTicket(uint64_t ticket) { tickets_.erase(ticket); }

void ListenerCore::close() {
  auto self = shared_from_this();
  context_->defer([self]() { self->fail(TPB_CREATE_ERROR(ListenerClosedError)); });
}

void ListenerCore::fail(const Error& e) {
  if (error_ || !e) return;
  error_ = e;
  TPB_VLOG(1) << "Listener " << id_ << " fails: " << error_.what();
  auto self = shared_from_this();
  auto accepts = std::move(waitingAccepts_);
  waitingAccepts_.clear();
  for (auto& fn : accepts) fn(error_, nullptr);
  waitingPipes_.clear();
  auto tickets = std::move(tickets_);
  tickets_.clear();
  for (auto& t : tickets) t.second(error_, std::string(), nullptr);
  for (auto& s : sockets_) s.second->close();
  for (auto& c : unidentified_) c->close();
  unidentified_.clear();
  context_->release(this);
}

}  // namespace core

// ---- public shell ---------------------------------------------------------------------------
Listener::Listener(ConstructorToken, std::shared_ptr<core::ListenerCore> impl) : impl_(std::move(impl)) {}
void Listener::accept(accept_callback_fn fn) { impl_->accept(std::move(fn)); }
const std::map<std::string, std::string>& Listener::addresses() const { return impl_->addresses(); }
const std::string& Listener::address(const std::string& transport) const { return impl_->address(transport); }
std::string Listener::url(const std::string& transport) const { return transport + "://" + impl_->address(transport); }
void Listener::close() { impl_->close(); }
Listener::~Listener() { close(); }

}  // namespace tpb
