// Abstract transport interfaces: a transport turns an address into connections that carry
// *framed* messages (every write is one frame, every read consumes exactly one frame) and wakes
// the reader up. Counterpart of tensorpipe/transport/{context,listener,connection}.h.
//
// Threading contract shared by every implementation: every method is non-blocking (except
// Listener::addr, Context::join); callbacks are one-shot, are always invoked (with an error
// after close), never from inside the call that registered them, and for one connection they
// fire in the order the operations were issued.
#pragma once

#include <cstddef>
#include <functional>
#include <memory>
#include <string>

#include <tpb/error.h>

namespace tpb {
namespace transport {

// Largest frame a transport allocates memory for on the peer's word (reads without a caller
// buffer: control messages). A longer one fails the connection instead of the allocation.
constexpr uint64_t kMaxAllocatedFrame = 1ull << 30;

class Connection {
 public:
  using read_callback_fn = std::function<void(const Error&, const void* ptr, size_t length)>;
  using write_callback_fn = std::function<void(const Error&)>;

  // Read the next frame into memory owned by the transport (valid during the callback only).
  virtual void read(read_callback_fn fn) = 0;
  // Read the next frame, which must be exactly `length` bytes, into caller memory.
  virtual void read(void* ptr, size_t length, read_callback_fn fn) = 0;
  // Write one frame. `ptr` must stay valid until the callback fires.
  virtual void write(const void* ptr, size_t length, write_callback_fn fn) = 0;

  virtual void setId(std::string id) = 0;
  virtual void close() = 0;
  virtual ~Connection() = default;
};

class Listener {
 public:
  using accept_callback_fn = std::function<void(const Error&, std::shared_ptr<Connection>)>;
  virtual void accept(accept_callback_fn fn) = 0;
  virtual std::string addr() const = 0;  // the address a peer can connect() to; may block briefly
  virtual void setId(std::string id) = 0;
  virtual void close() = 0;
  virtual ~Listener() = default;
};

class Context {
 public:
  virtual std::shared_ptr<Connection> connect(std::string addr) = 0;
  virtual std::shared_ptr<Listener> listen(std::string addr) = 0;
  // A context that cannot work on this machine says so instead of throwing; the core then
  // silently skips it at registration.
  virtual bool isViable() const = 0;
  // Two contexts can talk iff canCommunicateWithRemote(peer's descriptor).
  virtual const std::string& domainDescriptor() const = 0;
  virtual bool canCommunicateWithRemote(const std::string& remoteDomainDescriptor) const {
    return domainDescriptor() == remoteDomainDescriptor;
  }
  virtual void setId(std::string id) = 0;
  virtual void close() = 0;
  virtual void join() = 0;
  virtual ~Context() = default;
};

// ---- factories ------------------------------------------------------------------------------
namespace tcp {
// epoll TCP transport. Registered under the name "uv" for wire compatibility with reference
// peers (same 8-byte length framing and "uv:*" domain descriptor).
std::shared_ptr<Context> create();
// Address helpers (tensorpipe/transport/uv/utility.cc:20-215 counterparts).
std::pair<Error, std::string> lookupAddrForIface(const std::string& iface);
std::pair<Error, std::string> lookupAddrForHostname();
// The address NCCL's bootstrap would choose (interfaces named ib* first, docker* and lo* last);
// `family` is AF_INET, AF_INET6 or 0 for either.
std::pair<Error, std::string> lookupAddrLikeNccl(int family = 0);
}  // namespace tcp
namespace uv {
inline std::shared_ptr<Context> create() { return tcp::create(); }
}  // namespace uv
namespace shm {
std::shared_ptr<Context> create();
}
namespace ibv {
// Framed connections over RDMA writes into registered rings (libibverbs loaded at run time, TCP
// for the bootstrap). A machine without the library or without a NIC gets a non-viable context.
std::shared_ptr<Context> create();
}

// Host-side fault injection for tests: wraps a context so that the connections it hands out
// misbehave on purpose (fail after N frames, drop frames, delay).
struct FaultPlan {
  int failAfterWrites = -1;  // >=0: the (N+1)-th write and everything after fails and closes
  int dropWrites = 0;        // silently drop this many writes (callback still succeeds)
  int delayMs = 0;           // delay every write by this long
  int corruptFromWrite = -1; // >=0: from the N-th write on, frames are sent with their bytes scrambled
  unsigned corruptSeed = 1;  //      (same length, seeded noise XOR-ed over the content)
  int swallowFromWrite = -1; // >=0: from the N-th write of a connection on, frames vanish: the writer is told
                             //      they went out, the peer never sees them (a peer that has gone silent)
};
std::shared_ptr<Context> wrapWithFaults(std::shared_ptr<Context> inner, FaultPlan plan);

}  // namespace transport
}  // namespace tpb
