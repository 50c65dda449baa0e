// The context: the backends it was given, the loop that serialises every callback, and the set
// of live listeners and pipes that it fails when it closes. Contract as in
// tensorpipe/core/context.h:58-94 (close() starts closing and returns, join() is the one call
// that blocks).
#include <unistd.h>

#include <future>

#include "common/url.h"
#include "core/core.h"

namespace tpb {
namespace core {

namespace {
std::atomic<uint64_t> contextsMade{0};
}

ContextCore::ContextCore(std::string name) : name_(std::move(name)) {
  id_ = !name_.empty() ? name_ : std::to_string(::getpid()) + ":c" + std::to_string(contextsMade++);
  TPB_VLOG(1) << "Context " << id_ << " created";
}

void ContextCore::addTransport(int64_t priority, std::string name, std::shared_ptr<transport::Context> t) {
  std::unique_lock<std::mutex> lock(registrationMutex_);
  const std::string label = name;
  if (transports_.add(priority, std::move(name), t)) {
    t->setId(id_ + ".tr_" + label);
    TPB_VLOG(1) << "Context " << id_ << " has transport " << label << " at priority " << priority;
  } else {
    TPB_VLOG(1) << "Context " << id_ << " leaves out transport " << label << ": not viable here";
  }
}

void ContextCore::addChannel(int64_t priority, std::string name, std::shared_ptr<channel::Context> c) {
  std::unique_lock<std::mutex> lock(registrationMutex_);
  const std::string label = name;
  if (channels_.add(priority, std::move(name), c)) {
    c->setId(id_ + ".ch_" + label);
    TPB_VLOG(1) << "Context " << id_ << " has channel " << label << " at priority " << priority;
  } else {
    TPB_VLOG(1) << "Context " << id_ << " leaves out channel " << label << ": not viable here";
  }
}

std::shared_ptr<Listener> ContextCore::listen(const std::vector<std::string>& urls) {
  std::string id = id_ + "[l" + std::to_string(listenersMade_++) + "]";
  TPB_VLOG(1) << "Context " << id_ << " opens listener " << id;
  auto core = std::make_shared<ListenerCore>(shared_from_this(), std::move(id), urls);
  core->start();
  return std::make_shared<Listener>(Listener::kToken, std::move(core));
}

std::shared_ptr<Pipe> ContextCore::connect(const std::string& url, std::string remoteName) {
  std::string id = id_ + ".p" + std::to_string(pipesMade_++);
  TPB_VLOG(1) << "Context " << id_ << " opens pipe " << id << " to " << url;
  auto core = std::make_shared<PipeCore>(shared_from_this(), std::move(id), std::move(remoteName), url);
  core->start();
  return std::make_shared<Pipe>(Pipe::kToken, std::move(core));
}

void ContextCore::adopt(std::shared_ptr<PipeCore> p) {
  PipeCore* key = p.get();
  pipes_.emplace(key, std::move(p));
  counters.pipesCreated.fetch_add(1, std::memory_order_relaxed);
}
void ContextCore::adopt(std::shared_ptr<ListenerCore> l) {
  ListenerCore* key = l.get();
  listeners_.emplace(key, std::move(l));
}
void ContextCore::release(PipeCore* p) { pipes_.erase(p); }
void ContextCore::release(ListenerCore* l) { listeners_.erase(l); }

ContextStats ContextCore::snapshot() {
  ContextStats s;
  s.messagesWritten = counters.messagesWritten.load(std::memory_order_relaxed);
  s.messagesRead = counters.messagesRead.load(std::memory_order_relaxed);
  s.payloadBytesWritten = counters.payloadBytesWritten.load(std::memory_order_relaxed);
  s.payloadBytesRead = counters.payloadBytesRead.load(std::memory_order_relaxed);
  s.tensorBytesSent = counters.tensorBytesSent.load(std::memory_order_relaxed);
  s.tensorBytesReceived = counters.tensorBytesReceived.load(std::memory_order_relaxed);
  s.pipesCreated = counters.pipesCreated.load(std::memory_order_relaxed);
  std::unique_lock<std::mutex> lock(counters.perChannelMutex);
  s.bytesPerChannel = counters.bytesPerChannel;
  return s;
}

void ContextCore::close() {
  auto self = shared_from_this();
  defer([self]() {
    if (self->closing_.exchange(true)) return;
    TPB_VLOG(1) << "Context " << self->id_ << " is closing";
    const Error why = TPB_CREATE_ERROR(ContextClosedError);
    // Failing an object makes it leave the maps: walk copies.
    auto listeners = self->listeners_;
    auto pipes = self->pipes_;
    for (auto& l : listeners) l.second->fail(why);
    for (auto& p : pipes) p.second->fail(why);
    for (const auto& slot : self->channels_.bestFirst()) slot.backend->close();
    for (const auto& slot : self->transports_.bestFirst()) slot.backend->close();
  });
}

void ContextCore::join() {
  close();
  if (joined_.exchange(true)) return;
  // Everything deferred up to here, the close included, has run once this task has.
  auto drainLoop = [this]() {
    std::promise<void> reached;
    defer([&reached]() { reached.set_value(); });
    reached.get_future().wait();
  };
  drainLoop();
  for (const auto& slot : channels_.bestFirst()) slot.backend->join();
  for (const auto& slot : transports_.bestFirst()) slot.backend->join();
  // Backends hand their last completions to the loop while they wind down.
  drainLoop();
  TPB_VLOG(1) << "Context " << id_ << " joined";
}

}  // namespace core

// ---- public shell ---------------------------------------------------------------------------
Context::Context(ContextOptions opts) : impl_(std::make_shared<core::ContextCore>(std::move(opts.name_))) {}
void Context::registerTransport(int64_t priority, std::string name, std::shared_ptr<transport::Context> t) {
  impl_->addTransport(priority, std::move(name), std::move(t));
}
void Context::registerChannel(int64_t priority, std::string name, std::shared_ptr<channel::Context> c) {
  impl_->addChannel(priority, std::move(name), std::move(c));
}
std::shared_ptr<Listener> Context::listen(const std::vector<std::string>& urls) { return impl_->listen(urls); }
std::shared_ptr<Pipe> Context::connect(const std::string& url, PipeOptions opts) {
  return impl_->connect(url, std::move(opts.remoteName_));
}
ContextStats Context::stats() const { return impl_->snapshot(); }
void Context::close() { impl_->close(); }
void Context::join() { impl_->join(); }
Context::~Context() { join(); }

}  // namespace tpb
