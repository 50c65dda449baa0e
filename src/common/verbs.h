// RDMA verbs as this library uses them: reliable-connected queue pairs on one completion queue and
// one shared receive queue per user, memory regions, RDMA writes and sends that carry a 32-bit
// immediate. The ibv transport and the cuda_gdr channel are written against this interface only.
//
// Two providers implement it. systemProvider() loads libibverbs at run time (no link-time
// dependency, the verbs ABI it needs is declared in verbs_system.cc) and drives real NICs;
// loopbackProvider() is a software fabric inside the process (a "NIC" whose wire is memcpy),
// which lets everything above this interface run and be tested on a machine without InfiniBand.
//
// Role of tensorpipe/common/ibv_lib.h:20-704 (the dlopen'ed library) and
// tensorpipe/common/ibv.h:41-262 / ibv.cc:78-191 (RAII objects, queue-pair state transitions).
#pragma once

#include <array>
#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

namespace tpb {
namespace verbs {

// What two ends tell each other to connect their queue pairs.
struct Address {
  uint32_t localId = 0;            // LID (InfiniBand); 0 on RoCE
  std::array<uint8_t, 16> gid{};   // global id (RoCE, or routed InfiniBand)
  uint32_t queuePair = 0;
  uint32_t packetSequence = 0;
  uint8_t mtu = 0;                 // path MTU as the verbs enumeration (1..5)
};

enum class Work : uint8_t {
  kWrite,         // an RDMA write (with immediate) this side posted has completed
  kSend,          // a send (with immediate) this side posted has completed
  kWriteArrived,  // the peer's RDMA write with immediate landed; consumed one posted receive
  kSendArrived,   // the peer's send landed in (or, empty, consumed) one posted receive
};

struct Completion {
  uint64_t id = 0;         // what the poster passed
  Work work = Work::kWrite;
  bool ok = true;
  std::string error;       // provider's text for a failed completion
  uint32_t immediate = 0;  // for the two "arrived" kinds
  uint32_t byteLength = 0;
  uint32_t queuePair = 0;  // local queue-pair number the completion belongs to
};

class MemoryRegion {
 public:
  virtual uint32_t localKey() const = 0;
  virtual uint32_t remoteKey() const = 0;
  virtual ~MemoryRegion() = default;
};

class CompletionQueue {
 public:
  // Up to `max` completions; returns how many (0 = none now). Throws on a broken queue.
  virtual int poll(Completion* out, int max) = 0;
  virtual ~CompletionQueue() = default;
};

struct ReceiveBuffer {
  void* ptr = nullptr;  // may be null with length 0: only immediates are expected
  uint32_t length = 0;
  uint32_t localKey = 0;
};

class SharedReceiveQueue {
 public:
  virtual void postReceive(uint64_t id, ReceiveBuffer buffer = {}) = 0;
  virtual ~SharedReceiveQueue() = default;
};

class QueuePair {
 public:
  virtual uint32_t number() const = 0;
  // RESET -> INIT -> ready to receive (needs the peer's address) -> ready to send.
  virtual void toInit() = 0;
  virtual void toReadyToReceive(const Address& remote) = 0;
  virtual void toReadyToSend(uint32_t ownPacketSequence) = 0;
  // Flushes everything outstanding with failed completions.
  virtual void toError() = 0;
  virtual void postWriteWithImmediate(uint64_t id, const void* local, uint32_t length, uint32_t localKey,
                                      uint64_t remoteAddress, uint32_t remoteKey, uint32_t immediate) = 0;
  // A send; with length 0 it carries the immediate only.
  virtual void postSendWithImmediate(uint64_t id, const void* local, uint32_t length, uint32_t localKey,
                                     uint32_t immediate) = 0;
  virtual ~QueuePair() = default;
};

class Device {
 public:
  virtual const std::string& name() const = 0;
  // Where in the machine the NIC sits (sysfs PCI path), for matching GPUs to NICs; may be empty.
  virtual const std::string& pciPath() const = 0;
  // The address part that belongs to the port (local id, gid, MTU); queue pair and sequence
  // number are filled in per connection.
  virtual Address portAddress() const = 0;
  // Largest message one work request may carry.
  virtual uint32_t maxMessageBytes() const = 0;
  virtual std::unique_ptr<MemoryRegion> registerMemory(void* ptr, size_t length) = 0;
  virtual std::unique_ptr<CompletionQueue> createCompletionQueue(int entries) = 0;
  virtual std::unique_ptr<SharedReceiveQueue> createSharedReceiveQueue(int entries) = 0;
  virtual std::unique_ptr<QueuePair> createQueuePair(CompletionQueue& cq, SharedReceiveQueue& srq, int sendEntries) = 0;
  virtual ~Device() = default;
};

class Provider {
 public:
  virtual std::vector<std::string> deviceNames() = 0;
  virtual std::unique_ptr<Device> open(const std::string& name) = 0;
  // Why there is nothing to open, for logs.
  virtual std::string whyUnavailable() const { return std::string(); }
  virtual ~Provider() = default;
};

// libibverbs, loaded on first use. Never null; a machine without the library or without a device
// gets a provider with no devices (and whyUnavailable() says which).
std::shared_ptr<Provider> systemProvider();

// A software fabric with `devices` NICs named "loop0", "loop1", ... Queue pairs of one provider
// reach each other (same process only); memory keys are checked like a NIC checks them. With
// `copy` set, that function moves the bytes instead of memcpy (a test may copy between device
// pointers with it).
using CopyFn = std::function<void(void* dst, const void* src, size_t n)>;
std::shared_ptr<Provider> loopbackProvider(int devices = 1, CopyFn copy = nullptr, uint32_t maxMessageBytes = 1u << 30);

}  // namespace verbs
}  // namespace tpb
