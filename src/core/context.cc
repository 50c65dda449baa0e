// Context and Listener implementation, plus the public shells.
// Behaviour follows tensorpipe/core/context_impl.cc:39-289 and listener_impl.cc:34-336:
// higher priority wins and is stored negated so iteration is best-first; duplicate names or
// priorities throw; non-viable backends are skipped; close() fans an error out to every pipe
// and listener from the loop; join() additionally waits for every backend thread.
#include <unistd.h>

#include <future>

#include "core/core_impl.h"
#include "transport/nop_io.h"

namespace tpb {

namespace {
std::pair<std::string, std::string> splitSchemeOfURL(const std::string& url) {
  auto pos = url.find("://");
  TPB_THROW_SYSTEM_IF(pos == std::string::npos, EINVAL, "url has no scheme: " + url);
  return {url.substr(0, pos), url.substr(pos + 3)};
}
std::atomic<uint64_t> contextCounter{0};
}  // namespace

// ---- ContextImpl ----------------------------------------------------------------------------
ContextImpl::ContextImpl(ContextOptions opts) : name_(std::move(opts.name_)) {
  id_ = name_.empty() ? std::to_string(::getpid()) + ":c" + std::to_string(contextCounter++) : name_;
  TPB_VLOG(1) << "Context " << id_ << " created";
}

std::string ContextImpl::makeChildId(const char* kind) {
  if (kind[0] == 'l') return id_ + "[l" + std::to_string(listenerCounter_++) + "]";
  return id_ + ".p" + std::to_string(pipeCounter_++);
}

void ContextImpl::registerTransport(int64_t priority, std::string name,
                                    std::shared_ptr<transport::Context> t) {
  TPB_THROW_ASSERT_IF(name.empty(), "transport name is empty");
  std::unique_lock<std::mutex> lock(registryMutex_);
  TPB_THROW_ASSERT_IF(transports_.count(name) != 0, "transport " + name + " already registered");
  TPB_THROW_ASSERT_IF(transportsByPriority_.count(-priority) != 0,
                      "transport with priority " + std::to_string(priority) + " already registered");
  if (!t->isViable()) {
    TPB_VLOG(1) << "Context " << id_ << " is not registering transport " << name
                << " because it is not viable";
    return;
  }
  TPB_VLOG(1) << "Context " << id_ << " is registering transport " << name;
  t->setId(id_ + ".tr_" + name);
  transports_.emplace(name, t);
  transportsByPriority_.emplace(-priority, std::make_pair(name, std::move(t)));
}

void ContextImpl::registerChannel(int64_t priority, std::string name,
                                  std::shared_ptr<channel::Context> c) {
  TPB_THROW_ASSERT_IF(name.empty(), "channel name is empty");
  std::unique_lock<std::mutex> lock(registryMutex_);
  TPB_THROW_ASSERT_IF(channels_.count(name) != 0, "channel " + name + " already registered");
  TPB_THROW_ASSERT_IF(channelsByPriority_.count(-priority) != 0,
                      "channel with priority " + std::to_string(priority) + " already registered");
  if (!c->isViable()) {
    TPB_VLOG(1) << "Context " << id_ << " is not registering channel " << name
                << " because it is not viable";
    return;
  }
  TPB_VLOG(1) << "Context " << id_ << " is registering channel " << name;
  c->setId(id_ + ".ch_" + name);
  channels_.emplace(name, c);
  channelsByPriority_.emplace(-priority, std::make_pair(name, std::move(c)));
}

std::shared_ptr<transport::Context> ContextImpl::getTransport(const std::string& name) {
  auto it = transports_.find(name);
  TPB_THROW_ASSERT_IF(it == transports_.end(), "unsupported transport " + name);
  return it->second;
}

std::shared_ptr<channel::Context> ContextImpl::getChannel(const std::string& name) {
  auto it = channels_.find(name);
  TPB_THROW_ASSERT_IF(it == channels_.end(), "unsupported channel " + name);
  return it->second;
}

std::shared_ptr<Listener> ContextImpl::listen(const std::vector<std::string>& urls) {
  std::string id = makeChildId("l");
  TPB_VLOG(1) << "Context " << id_ << " is opening listener " << id;
  return std::make_shared<Listener>(Listener::kToken, shared_from_this(), std::move(id), urls);
}

std::shared_ptr<Pipe> ContextImpl::connect(const std::string& url, PipeOptions opts) {
  std::string id = makeChildId("p");
  TPB_VLOG(1) << "Context " << id_ << " is opening pipe " << id;
  std::string remote = std::move(opts.remoteName_);
  return std::make_shared<Pipe>(Pipe::kToken, shared_from_this(), std::move(id), std::move(remote), url);
}

void ContextImpl::enroll(ListenerImpl& l) { listeners_.emplace(&l, l.shared_from_this()); }
void ContextImpl::enroll(PipeImpl& p) {
  pipes_.emplace(&p, p.shared_from_this());
  std::unique_lock<std::mutex> lock(statsMutex_);
  stats_.pipesCreated++;
}
void ContextImpl::unenroll(ListenerImpl& l) { listeners_.erase(&l); }
void ContextImpl::unenroll(PipeImpl& p) { pipes_.erase(&p); }

ContextStats ContextImpl::stats() {
  std::unique_lock<std::mutex> lock(statsMutex_);
  return stats_;
}

void ContextImpl::close() {
  auto self = shared_from_this();
  deferToLoop([self]() {
    if (self->closed_.exchange(true)) return;
    TPB_VLOG(1) << "Context " << self->id_ << " is closing";
    // Copy: closing unenrolls.
    auto listeners = self->listeners_;
    auto pipes = self->pipes_;
    Error e = TPB_CREATE_ERROR(ContextClosedError);
    for (auto& l : listeners) l.second->setError(e);
    for (auto& p : pipes) p.second->setError(e);
    for (auto& c : self->channels_) c.second->close();
    for (auto& t : self->transports_) t.second->close();
  });
}

void ContextImpl::join() {
  close();
  if (joined_.exchange(true)) return;
  // Barrier: everything deferred so far (including the close above) has run.
  std::promise<void> done;
  deferToLoop([&done]() { done.set_value(); });
  done.get_future().wait();
  for (auto& c : channels_) c.second->join();
  for (auto& t : transports_) t.second->join();
  // Backends may have deferred final callbacks into the loop while joining.
  std::promise<void> done2;
  deferToLoop([&done2]() { done2.set_value(); });
  done2.get_future().wait();
  TPB_VLOG(1) << "Context " << id_ << " joined";
}

// ---- ListenerImpl ---------------------------------------------------------------------------
ListenerImpl::ListenerImpl(std::shared_ptr<ContextImpl> context, std::string id,
                           const std::vector<std::string>& urls)
    : context_(std::move(context)), id_(std::move(id)) {
  for (const auto& url : urls) {
    auto [scheme, addr] = splitSchemeOfURL(url);
    std::shared_ptr<transport::Context> t = context_->getTransport(scheme);
    std::shared_ptr<transport::Listener> l = t->listen(addr);
    l->setId(id_ + ".tr_" + scheme);
    addresses_.emplace(scheme, l->addr());
    listeners_.emplace(scheme, std::move(l));
  }
}

void ListenerImpl::init() {
  auto self = shared_from_this();
  context_->deferToLoop([self]() { self->initFromLoop(); });
}

void ListenerImpl::initFromLoop() {
  if (context_->closed()) {
    setError(TPB_CREATE_ERROR(ContextClosedError));
    return;
  }
  context_->enroll(*this);
  for (const auto& l : listeners_) armListener(l.first);
}

void ListenerImpl::armListener(const std::string& transport) {
  auto it = listeners_.find(transport);
  if (it == listeners_.end()) return;
  it->second->accept(callbackWrapper_(
      [transport](ListenerImpl& impl, std::shared_ptr<transport::Connection> conn) {
        if (impl.error_) return;
        impl.onAccept(transport, std::move(conn));
        impl.armListener(transport);
      }));
}

void ListenerImpl::onAccept(const std::string& transport,
                            std::shared_ptr<transport::Connection> conn) {
  connectionsWaitingForHello_.insert(conn);
  std::weak_ptr<transport::Connection> weak = conn;
  transport::readNop<Packet>(
      *conn, callbackWrapper_([transport, weak](ListenerImpl& impl, Packet packet) {
        auto c = weak.lock();
        if (!c) return;
        impl.connectionsWaitingForHello_.erase(c);
        if (impl.error_) return;
        impl.onConnectionHelloRead(transport, std::move(c), packet);
      }));
}

void ListenerImpl::onConnectionHelloRead(const std::string& transport,
                                         std::shared_ptr<transport::Connection> conn,
                                         const Packet& packet) {
  if (std::holds_alternative<SpontaneousConnection>(packet)) {
    const auto& hello = std::get<SpontaneousConnection>(packet);
    std::string pipeId = id_ + ".p" + std::to_string(pipeCounter_++);
    TPB_VLOG(1) << "Listener " << id_ << " is opening pipe " << pipeId << " from "
                << hello.contextName;
    auto pipeImpl = std::make_shared<PipeImpl>(context_, shared_from_this(), pipeId,
                                               hello.contextName, transport, std::move(conn));
    pipeImpl->initFromLoop();
    acceptCallback_.trigger(Error::kSuccess, std::make_shared<Pipe>(Pipe::kToken, std::move(pipeImpl)));
  } else {
    uint64_t id = std::get<RequestedConnection>(packet).registrationId;
    auto it = connectionRequests_.find(id);
    if (it == connectionRequests_.end()) {
      TPB_VLOG(3) << "Listener " << id_ << " got a connection for unknown registration " << id;
      return;  // the pipe that wanted it is gone; dropping `conn` closes it
    }
    auto fn = std::move(it->second);
    connectionRequests_.erase(it);
    fn(Error::kSuccess, transport, std::move(conn));
  }
}

void ListenerImpl::accept(Listener::accept_callback_fn fn) {
  auto self = shared_from_this();
  context_->deferToLoop([self, fn = std::move(fn)]() mutable {
    if (self->error_) {
      fn(self->error_, nullptr);
      return;
    }
    self->acceptCallback_.arm(std::move(fn));
  });
}

const std::string& ListenerImpl::address(const std::string& transport) const {
  auto it = addresses_.find(transport);
  TPB_THROW_ASSERT_IF(it == addresses_.end(), "no address for transport " + transport);
  return it->second;
}

std::string ListenerImpl::url(const std::string& transport) const {
  return transport + "://" + address(transport);
}

uint64_t ListenerImpl::registerConnectionRequest(connection_request_callback_fn fn) {
  uint64_t id = nextConnectionRequestId_++;
  if (error_) {
    auto self = shared_from_this();
    Error e = error_;
    context_->deferToLoop([fn = std::move(fn), e]() { fn(e, std::string(), nullptr); });
  } else {
    connectionRequests_.emplace(id, std::move(fn));
  }
  return id;
}

void ListenerImpl::unregisterConnectionRequest(uint64_t id) { connectionRequests_.erase(id); }

void ListenerImpl::close() {
  auto self = shared_from_this();
  context_->deferToLoop([self]() { self->setError(TPB_CREATE_ERROR(ListenerClosedError)); });
}

void ListenerImpl::setError(const Error& e) {
  if (error_ || !e) return;
  error_ = e;
  handleError();
}

void ListenerImpl::handleError() {
  TPB_VLOG(1) << "Listener " << id_ << " is handling error " << error_.what();
  auto self = shared_from_this();
  Error e = error_;
  acceptCallback_.triggerAll([e]() { return std::make_tuple(e, std::shared_ptr<Pipe>()); });
  auto requests = std::move(connectionRequests_);
  connectionRequests_.clear();
  for (auto& r : requests) r.second(e, std::string(), nullptr);
  for (auto& l : listeners_) l.second->close();
  for (auto& c : connectionsWaitingForHello_) c->close();
  connectionsWaitingForHello_.clear();
  context_->unenroll(*this);
}

// ---- public shells --------------------------------------------------------------------------
Context::Context(ContextOptions opts) : impl_(std::make_shared<ContextImpl>(std::move(opts))) {}
void Context::registerTransport(int64_t p, std::string n, std::shared_ptr<transport::Context> t) {
  impl_->registerTransport(p, std::move(n), std::move(t));
}
void Context::registerChannel(int64_t p, std::string n, std::shared_ptr<channel::Context> c) {
  impl_->registerChannel(p, std::move(n), std::move(c));
}
std::shared_ptr<Listener> Context::listen(const std::vector<std::string>& urls) {
  return impl_->listen(urls);
}
std::shared_ptr<Pipe> Context::connect(const std::string& url, PipeOptions opts) {
  return impl_->connect(url, std::move(opts));
}
ContextStats Context::stats() const { return impl_->stats(); }
void Context::close() { impl_->close(); }
void Context::join() { impl_->join(); }
Context::~Context() { join(); }

Listener::Listener(ConstructorToken, std::shared_ptr<ContextImpl> context, std::string id,
                   const std::vector<std::string>& urls)
    : impl_(std::make_shared<ListenerImpl>(std::move(context), std::move(id), urls)) {
  impl_->init();
}
void Listener::accept(accept_callback_fn fn) { impl_->accept(std::move(fn)); }
const std::map<std::string, std::string>& Listener::addresses() const { return impl_->addresses(); }
const std::string& Listener::address(const std::string& t) const { return impl_->address(t); }
std::string Listener::url(const std::string& t) const { return impl_->url(t); }
void Listener::close() { impl_->close(); }
Listener::~Listener() { close(); }

}  // namespace tpb
