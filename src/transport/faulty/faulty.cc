// Host-side fault injection: a transport decorator whose connections misbehave on purpose.
// The reference has no such facility (its tests only close objects mid-flight); here it is what
// failure-handling tests use instead of ever faulting a device: make a connection fail after N
// frames, swallow frames, or slow them down, and check that every pending callback still fires
// with an error and in order.
#include <atomic>
#include <chrono>
#include <random>
#include <thread>
#include <vector>

#include <tpb/transport.h>

namespace tpb {
namespace transport {

namespace {

class FaultyConnection final : public Connection {
 public:
  FaultyConnection(std::shared_ptr<Connection> inner, FaultPlan plan, std::shared_ptr<std::atomic<int>> writes)
      : inner_(std::move(inner)), plan_(plan), writes_(std::move(writes)) {}
  void read(read_callback_fn fn) override { inner_->read(std::move(fn)); }
  void read(void* ptr, size_t length, read_callback_fn fn) override { inner_->read(ptr, length, std::move(fn)); }
  void write(const void* ptr, size_t length, write_callback_fn fn) override {
    const int n = (*writes_)++;
    if (plan_.delayMs > 0) std::this_thread::sleep_for(std::chrono::milliseconds(plan_.delayMs));
    if (plan_.failAfterWrites >= 0 && n >= plan_.failAfterWrites) {
      // Fail this write through the normal path: close, then let the inner connection report.
      inner_->close();
      inner_->write(ptr, length, [fn = std::move(fn)](const Error& e) {
        fn(e ? e : TPB_CREATE_ERROR(InjectedFaultError));
      });
      return;
    }
    if (plan_.swallowFromWrite >= 0 && n >= plan_.swallowFromWrite) {
      // Nothing reaches the wire; the completion is reported from a short-lived thread so that it
      // never runs on the caller's stack.
      auto keep = inner_;
      std::thread([keep, fn = std::move(fn)]() mutable { fn(Error::kSuccess); }).detach();
      return;
    }
    if (n < plan_.dropWrites) {
      // Pretend success without sending anything; a zero-length read on our own side keeps the
      // callback off the caller's stack.
      inner_->write(nullptr, 0, [fn = std::move(fn)](const Error& e) { fn(e); });
      return;
    }
    if (plan_.corruptFromWrite >= 0 && n >= plan_.corruptFromWrite && length > 0) {
      // Same length on the wire, scrambled content; the copy lives until the write completes.
      auto copy = std::make_shared<std::vector<uint8_t>>(static_cast<const uint8_t*>(ptr),
                                                         static_cast<const uint8_t*>(ptr) + length);
      std::mt19937 rng(plan_.corruptSeed + static_cast<unsigned>(n));
      for (auto& b : *copy) b ^= static_cast<uint8_t>(rng());
      inner_->write(copy->data(), copy->size(), [fn = std::move(fn), copy](const Error& e) { fn(e); });
      return;
    }
    inner_->write(ptr, length, std::move(fn));
  }
  void setId(std::string id) override { inner_->setId(std::move(id)); }
  void close() override { inner_->close(); }

 private:
  std::shared_ptr<Connection> inner_;
  FaultPlan plan_;
  std::shared_ptr<std::atomic<int>> writes_;
};

class FaultyListener final : public Listener {
 public:
  FaultyListener(std::shared_ptr<Listener> inner, FaultPlan plan) : inner_(std::move(inner)), plan_(plan) {}
  void accept(accept_callback_fn fn) override {
    FaultPlan plan = plan_;
    inner_->accept([fn = std::move(fn), plan](const Error& e, std::shared_ptr<Connection> c) {
      if (e || !c) return fn(e, std::move(c));
      fn(e, std::make_shared<FaultyConnection>(std::move(c), plan, std::make_shared<std::atomic<int>>(0)));
    });
  }
  std::string addr() const override { return inner_->addr(); }
  void setId(std::string id) override { inner_->setId(std::move(id)); }
  void close() override { inner_->close(); }

 private:
  std::shared_ptr<Listener> inner_;
  FaultPlan plan_;
};

class FaultyContext final : public Context {
 public:
  FaultyContext(std::shared_ptr<Context> inner, FaultPlan plan) : inner_(std::move(inner)), plan_(plan) {}
  std::shared_ptr<Connection> connect(std::string addr) override {
    return std::make_shared<FaultyConnection>(inner_->connect(std::move(addr)), plan_,
                                              std::make_shared<std::atomic<int>>(0));
  }
  std::shared_ptr<Listener> listen(std::string addr) override {
    return std::make_shared<FaultyListener>(inner_->listen(std::move(addr)), plan_);
  }
  bool isViable() const override { return inner_->isViable(); }
  const std::string& domainDescriptor() const override { return inner_->domainDescriptor(); }
  bool canCommunicateWithRemote(const std::string& r) const override { return inner_->canCommunicateWithRemote(r); }
  void setId(std::string id) override { inner_->setId(std::move(id)); }
  void close() override { inner_->close(); }
  void join() override { inner_->join(); }

 private:
  std::shared_ptr<Context> inner_;
  FaultPlan plan_;
};

}  // namespace

std::shared_ptr<Context> wrapWithFaults(std::shared_ptr<Context> inner, FaultPlan plan) {
  return std::make_shared<FaultyContext>(std::move(inner), plan);
}

}  // namespace transport
}  // namespace tpb
