// The software fabric behind verbs::loopbackProvider(): queue pairs of one provider reach each
// other through memcpy, with the checks a NIC makes (queue-pair state, memory keys and bounds,
// a posted receive per arriving immediate, in-order delivery) and its failure behaviour (a bad
// key or a vanished peer fails the work request and puts the queue pair into the error state,
// after which everything posted is flushed with an error). One mutex guards the whole fabric:
// it exists to run the code above the verbs interface without InfiniBand hardware, not to be fast.
#include "common/verbs.h"

#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <stdexcept>

namespace tpb {
namespace verbs {
namespace {

struct Fabric;

struct Region {
  uint8_t* ptr;
  size_t length;
};

struct LoopCq final : CompletionQueue {
  explicit LoopCq(std::shared_ptr<Fabric> f) : fabric(std::move(f)) {}
  int poll(Completion* out, int max) override;
  std::shared_ptr<Fabric> fabric;
  std::deque<Completion> done;
};

struct LoopQp;

struct Arrival {
  LoopQp* to;
  Work work;
  uint32_t immediate;
  uint32_t byteLength;
  std::vector<uint8_t> payload;  // of a send that found no receive posted yet
};

struct LoopSrq final : SharedReceiveQueue {
  explicit LoopSrq(std::shared_ptr<Fabric> f) : fabric(std::move(f)) {}
  void postReceive(uint64_t id, ReceiveBuffer buffer) override;
  struct Posted {
    uint64_t id;
    ReceiveBuffer buffer;
  };
  std::shared_ptr<Fabric> fabric;
  std::deque<Posted> posted;
  std::deque<Arrival> waiting;  // arrived before a receive was posted (the wire would retry), in order
};

enum class State { kReset, kInit, kReadyToReceive, kReadyToSend, kError };

struct LoopQp final : QueuePair {
  LoopQp(std::shared_ptr<Fabric> f, LoopCq* cq, LoopSrq* srq, uint32_t number);
  ~LoopQp() override;
  uint32_t number() const override { return num; }
  void toInit() override;
  void toReadyToReceive(const Address& remote) override;
  void toReadyToSend(uint32_t) override;
  void toError() override;
  void postWriteWithImmediate(uint64_t id, const void* local, uint32_t length, uint32_t localKey, uint64_t remoteAddress,
                              uint32_t remoteKey, uint32_t immediate) override;
  void postSendWithImmediate(uint64_t id, const void* local, uint32_t length, uint32_t localKey, uint32_t immediate) override;

  std::shared_ptr<Fabric> fabric;
  LoopCq* cq;
  LoopSrq* srq;
  uint32_t num;
  uint32_t remote = 0;
  State state = State::kReset;
};

struct Fabric {
  std::mutex mu;
  CopyFn copy;
  uint32_t maxMessage = 1u << 30;
  uint32_t nextKey = 0x1000;
  uint32_t nextQp = 100;
  std::map<uint32_t, Region> regions;
  std::map<uint32_t, LoopQp*> qps;

  bool covers(uint32_t key, const void* ptr, size_t n) const {
    auto it = regions.find(key);
    if (it == regions.end()) return false;
    const uint8_t* p = static_cast<const uint8_t*>(ptr);
    return p >= it->second.ptr && n <= it->second.length && static_cast<size_t>(p - it->second.ptr) <= it->second.length - n;
  }
  void move(void* dst, const void* src, size_t n) const {
    if (n == 0) return;
    if (copy) copy(dst, src, n);
    else std::memcpy(dst, src, n);
  }
  // With the mutex held: hand `a` to its queue pair's receive side.
  void deliver(Arrival a) {
    LoopSrq* srq = a.to->srq;
    if (!srq->waiting.empty() || srq->posted.empty()) {
      srq->waiting.push_back(std::move(a));
      return;
    }
    complete(srq, std::move(a));
  }
  void complete(LoopSrq* srq, Arrival a) {
    LoopSrq::Posted r = srq->posted.front();
    srq->posted.pop_front();
    Completion c;
    c.id = r.id;
    c.work = a.work;
    c.immediate = a.immediate;
    c.byteLength = a.byteLength;
    c.queuePair = a.to->num;
    if (a.work == Work::kSendArrived && !a.payload.empty()) {
      if (a.payload.size() > r.buffer.length || !covers(r.buffer.localKey, r.buffer.ptr, a.payload.size())) {
        c.ok = false;
        c.error = "local length error";
        a.to->state = State::kError;
      } else {
        move(r.buffer.ptr, a.payload.data(), a.payload.size());
      }
    }
    a.to->cq->done.push_back(std::move(c));
  }
  void fail(LoopQp* qp, uint64_t id, Work work, const char* why) {
    Completion c;
    c.id = id;
    c.work = work;
    c.ok = false;
    c.error = why;
    c.queuePair = qp->num;
    qp->cq->done.push_back(std::move(c));
    qp->state = State::kError;
  }
  // The peer of `qp` if it can take traffic, else nullptr.
  LoopQp* peerOf(LoopQp* qp) {
    auto it = qps.find(qp->remote);
    if (it == qps.end()) return nullptr;
    LoopQp* p = it->second;
    if (p->remote != qp->num) return nullptr;
    if (p->state != State::kReadyToReceive && p->state != State::kReadyToSend) return nullptr;
    return p;
  }
};

int LoopCq::poll(Completion* out, int max) {
  std::unique_lock<std::mutex> l(fabric->mu);
  int n = 0;
  while (n < max && !done.empty()) {
    out[n++] = std::move(done.front());
    done.pop_front();
  }
  return n;
}

void LoopSrq::postReceive(uint64_t id, ReceiveBuffer buffer) {
  std::unique_lock<std::mutex> l(fabric->mu);
  posted.push_back({id, buffer});
  while (!waiting.empty() && !posted.empty()) {
    Arrival a = std::move(waiting.front());
    waiting.pop_front();
    fabric->complete(this, std::move(a));
  }
}

LoopQp::LoopQp(std::shared_ptr<Fabric> f, LoopCq* cq, LoopSrq* srq, uint32_t number)
    : fabric(std::move(f)), cq(cq), srq(srq), num(number) {}

LoopQp::~LoopQp() {
  std::unique_lock<std::mutex> l(fabric->mu);
  fabric->qps.erase(num);
  // Whatever still waits for a receive on behalf of this queue pair goes with it.
  for (auto it = srq->waiting.begin(); it != srq->waiting.end();) it = it->to == this ? srq->waiting.erase(it) : it + 1;
}

void LoopQp::toInit() {
  std::unique_lock<std::mutex> l(fabric->mu);
  if (state != State::kReset) throw std::runtime_error("queue pair: INIT is entered from RESET only");
  state = State::kInit;
}

void LoopQp::toReadyToReceive(const Address& r) {
  std::unique_lock<std::mutex> l(fabric->mu);
  if (state != State::kInit) throw std::runtime_error("queue pair: ready-to-receive is entered from INIT only");
  remote = r.queuePair;
  state = State::kReadyToReceive;
}

void LoopQp::toReadyToSend(uint32_t) {
  std::unique_lock<std::mutex> l(fabric->mu);
  if (state != State::kReadyToReceive) throw std::runtime_error("queue pair: ready-to-send is entered from ready-to-receive only");
  state = State::kReadyToSend;
}

void LoopQp::toError() {
  std::unique_lock<std::mutex> l(fabric->mu);
  state = State::kError;
}

void LoopQp::postWriteWithImmediate(uint64_t id, const void* local, uint32_t length, uint32_t localKey,
                                    uint64_t remoteAddress, uint32_t remoteKey, uint32_t immediate) {
  std::unique_lock<std::mutex> l(fabric->mu);
  if (state == State::kError) return fabric->fail(this, id, Work::kWrite, "work request flushed");
  if (state != State::kReadyToSend) throw std::runtime_error("queue pair: posting a write before ready-to-send");
  if (length > fabric->maxMessage) return fabric->fail(this, id, Work::kWrite, "local length error");
  if (!fabric->covers(localKey, local, length)) return fabric->fail(this, id, Work::kWrite, "local protection error");
  LoopQp* peer = fabric->peerOf(this);
  if (!peer) return fabric->fail(this, id, Work::kWrite, "transport retry counter exceeded");
  void* dst = reinterpret_cast<void*>(remoteAddress);
  if (!fabric->covers(remoteKey, dst, length)) return fabric->fail(this, id, Work::kWrite, "remote access error");
  fabric->move(dst, local, length);
  Arrival a{peer, Work::kWriteArrived, immediate, length, {}};
  fabric->deliver(std::move(a));
  Completion c;
  c.id = id;
  c.work = Work::kWrite;
  c.byteLength = length;
  c.queuePair = num;
  cq->done.push_back(std::move(c));
}

void LoopQp::postSendWithImmediate(uint64_t id, const void* local, uint32_t length, uint32_t localKey, uint32_t immediate) {
  std::unique_lock<std::mutex> l(fabric->mu);
  if (state == State::kError) return fabric->fail(this, id, Work::kSend, "work request flushed");
  if (state != State::kReadyToSend) throw std::runtime_error("queue pair: posting a send before ready-to-send");
  if (length > fabric->maxMessage) return fabric->fail(this, id, Work::kSend, "local length error");
  if (length != 0 && !fabric->covers(localKey, local, length)) return fabric->fail(this, id, Work::kSend, "local protection error");
  LoopQp* peer = fabric->peerOf(this);
  if (!peer) return fabric->fail(this, id, Work::kSend, "transport retry counter exceeded");
  Arrival a{peer, Work::kSendArrived, immediate, length, {}};
  if (length != 0) {
    // The payload is taken now (the sender may reuse its buffer once the send completes).
    a.payload.resize(length);
    fabric->move(a.payload.data(), local, length);
  }
  fabric->deliver(std::move(a));
  Completion c;
  c.id = id;
  c.work = Work::kSend;
  c.byteLength = length;
  c.queuePair = num;
  cq->done.push_back(std::move(c));
}

struct LoopRegion final : MemoryRegion {
  LoopRegion(std::shared_ptr<Fabric> f, uint32_t key) : fabric(std::move(f)), key(key) {}
  ~LoopRegion() override {
    std::unique_lock<std::mutex> l(fabric->mu);
    fabric->regions.erase(key);
  }
  uint32_t localKey() const override { return key; }
  uint32_t remoteKey() const override { return key; }
  std::shared_ptr<Fabric> fabric;
  uint32_t key;
};

struct LoopDevice final : Device {
  LoopDevice(std::shared_ptr<Fabric> f, std::string name, int index) : fabric(std::move(f)), name_(std::move(name)) {
    pci_ = "/sys/devices/loopback/nic" + std::to_string(index);
    address_.localId = static_cast<uint32_t>(index + 1);
    address_.gid[15] = static_cast<uint8_t>(index + 1);
    address_.mtu = 5;
  }
  const std::string& name() const override { return name_; }
  const std::string& pciPath() const override { return pci_; }
  Address portAddress() const override { return address_; }
  uint32_t maxMessageBytes() const override { return fabric->maxMessage; }
  std::unique_ptr<MemoryRegion> registerMemory(void* ptr, size_t length) override {
    std::unique_lock<std::mutex> l(fabric->mu);
    const uint32_t key = fabric->nextKey++;
    fabric->regions[key] = Region{static_cast<uint8_t*>(ptr), length};
    return std::make_unique<LoopRegion>(fabric, key);
  }
  std::unique_ptr<CompletionQueue> createCompletionQueue(int) override { return std::make_unique<LoopCq>(fabric); }
  std::unique_ptr<SharedReceiveQueue> createSharedReceiveQueue(int) override { return std::make_unique<LoopSrq>(fabric); }
  std::unique_ptr<QueuePair> createQueuePair(CompletionQueue& cq, SharedReceiveQueue& srq, int) override {
    std::unique_lock<std::mutex> l(fabric->mu);
    const uint32_t n = fabric->nextQp++;
    auto qp = std::make_unique<LoopQp>(fabric, static_cast<LoopCq*>(&cq), static_cast<LoopSrq*>(&srq), n);
    fabric->qps[n] = qp.get();
    return qp;
  }
  std::shared_ptr<Fabric> fabric;
  std::string name_, pci_;
  Address address_;
};

struct LoopProvider final : Provider {
  LoopProvider(int devices, CopyFn copy, uint32_t maxMessage) : fabric(std::make_shared<Fabric>()), count(devices) {
    fabric->copy = std::move(copy);
    fabric->maxMessage = maxMessage;
  }
  std::vector<std::string> deviceNames() override {
    std::vector<std::string> v;
    for (int i = 0; i < count; ++i) v.push_back("loop" + std::to_string(i));
    return v;
  }
  std::unique_ptr<Device> open(const std::string& name) override {
    for (int i = 0; i < count; ++i)
      if (name == "loop" + std::to_string(i)) return std::make_unique<LoopDevice>(fabric, name, i);
    throw std::runtime_error("no such loopback device: " + name);
  }
  std::shared_ptr<Fabric> fabric;
  int count;
};

}  // namespace

std::shared_ptr<Provider> loopbackProvider(int devices, CopyFn copy, uint32_t maxMessageBytes) {
  return std::make_shared<LoopProvider>(devices, std::move(copy), maxMessageBytes);
}

}  // namespace verbs
}  // namespace tpb
