// What stands behind Context, Listener and Pipe. The public classes are shells over shared
// pointers to these; everything here is touched only from the context's loop (one callback
// "thread" per context, borrowed from whoever triggers work), except where a method says it may
// be called from any thread.
//
// The wire conversation is the one a reference peer expects (tensorpipe/core/nop_types.h:26-80
// and the order of frames described in tensorpipe/core/pipe_impl.cc): hello packet, brochure,
// brochure answer, extra connections announced by ticket, then per message a descriptor frame,
// the payload frames, and (only when the sender left a target device open) a descriptor reply on
// the second connection. How that conversation is driven is this library's own:
//
//   * a pipe keeps two queues of message records, outbound and inbound. A record counts what it
//     still waits for (frame writes, payload reads, tensor transfers); nothing else decides when
//     it is done. Records start in order, hand their tensors to channels in order, and retire
//     from the front of their queue only, which is what makes callbacks fire in issue order.
//   * failure is one sticky error per object. Failing closes every connection and channel of the
//     object; their completions come back carrying errors, the counters run down, and the queues
//     retire in order with the error. Records that never started retire right behind them.
#pragma once

#include <atomic>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <tuple>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include <tpb/context.h>

#include "common/defs.h"
#include "common/loop.h"
#include "core/backends.h"
#include "core/nop_types.h"

namespace tpb {
namespace core {

class ContextCore;
class ListenerCore;
class PipeCore;

// ---- context --------------------------------------------------------------------------------
class ContextCore final : public std::enable_shared_from_this<ContextCore> {
 public:
  explicit ContextCore(std::string name);

  const std::string& id() const { return id_; }
  const std::string& name() const { return name_; }

  // Any thread, before the backend is needed.
  void addTransport(int64_t priority, std::string name, std::shared_ptr<transport::Context> t);
  void addChannel(int64_t priority, std::string name, std::shared_ptr<channel::Context> c);
  const Backends<transport::Context>& transports() const { return transports_; }
  const Backends<channel::Context>& channels() const { return channels_; }

  std::shared_ptr<Listener> listen(const std::vector<std::string>& urls);
  std::shared_ptr<Pipe> connect(const std::string& url, std::string remoteName);

  // The loop.
  void defer(std::function<void()> fn) { loop_.deferToLoop(std::move(fn)); }
  bool onLoop() const { return loop_.inLoop(); }
  template <typename F>
  void runSync(F&& fn) {
    loop_.runInLoop(std::forward<F>(fn));
  }

  // Live pipes and listeners: the context keeps them alive and fails them when it closes.
  void adopt(std::shared_ptr<PipeCore> p);
  void adopt(std::shared_ptr<ListenerCore> l);
  void release(PipeCore* p);
  void release(ListenerCore* l);
  bool closing() const { return closing_.load(std::memory_order_acquire); }

  void close();
  void join();

  // Counters (any thread).
  struct Counters {
    std::atomic<uint64_t> messagesWritten{0}, messagesRead{0};
    std::atomic<uint64_t> payloadBytesWritten{0}, payloadBytesRead{0};
    std::atomic<uint64_t> tensorBytesSent{0}, tensorBytesReceived{0};
    std::atomic<uint64_t> pipesCreated{0};
    std::mutex perChannelMutex;
    std::map<std::string, uint64_t> bytesPerChannel;
  };
  Counters counters;
  ContextStats snapshot();

 private:
  OnDemandLoop loop_;
  std::string name_;
  std::string id_;
  std::atomic<bool> closing_{false};
  std::atomic<bool> joined_{false};
  std::atomic<uint64_t> listenersMade_{0}, pipesMade_{0};
  std::mutex registrationMutex_;
  Backends<transport::Context> transports_{"transport"};
  Backends<channel::Context> channels_{"channel"};
  std::unordered_map<PipeCore*, std::shared_ptr<PipeCore>> pipes_;
  std::unordered_map<ListenerCore*, std::shared_ptr<ListenerCore>> listeners_;
};

// Turns `fn(args...)` into a completion handler `(const Error&, args...)` that may be invoked on
// any thread: it moves to the subject's context loop, records the error on the subject (which
// fails it), and then runs fn in any case; the subject's own state tells fn what is left to do.
// An exception thrown by fn fails the subject instead of leaving the loop.
template <typename TSubject, typename F>
auto onLoopOf(std::shared_ptr<TSubject> subject, F fn) {
  return [subject = std::move(subject), fn = std::move(fn)](const Error& error, auto&&... args) mutable {
    auto task = [subject, fn = std::move(fn), error,
                 packed = std::make_tuple(std::decay_t<decltype(args)>(std::forward<decltype(args)>(args))...)]() mutable {
      if (error) subject->fail(error);
      subject->guarded([&]() { std::apply([&](auto&... a) { fn(std::move(a)...); }, packed); });
    };
    subject->context().defer(std::move(task));
  };
}

// ---- listener -------------------------------------------------------------------------------
// Besides handing new pipes to the user, a listener is the meeting point for the extra
// connections of a pipe being set up: the pipe's server end issues a ticket per connection it
// expects, tells the client the ticket numbers, and the client's connections present them.
class ListenerCore final : public std::enable_shared_from_this<ListenerCore> {
 public:
  using TicketFn =
      std::function<void(const Error&, const std::string& transport, std::shared_ptr<transport::Connection>)>;

  ListenerCore(std::shared_ptr<ContextCore> context, std::string id, const std::vector<std::string>& urls);
  void start();

  void accept(Listener::accept_callback_fn fn);
  const std::map<std::string, std::string>& addresses() const { return bound_; }
  const std::string& address(const std::string& transport) const;

  // Loop only.
  uint64_t issueTicket(TicketFn fn);
  void revokeTicket(uint64_t ticket);

  void close();
  void fail(const Error& e);
  template <typename F>
  void guarded(F&& fn);
  ContextCore& context() { return *context_; }
  const std::string& id() const { return id_; }

 private:
  void watch(const std::string& transport);
  void greet(const std::string& transport, std::shared_ptr<transport::Connection> conn);
  void admit(const std::string& transport, std::shared_ptr<transport::Connection> conn, Packet hello);
  void matchAccepts();

  std::shared_ptr<ContextCore> context_;
  std::string id_;
  Error error_;
  std::map<std::string, std::shared_ptr<transport::Listener>> sockets_;
  std::map<std::string, std::string> bound_;  // transport -> address a peer can dial
  std::deque<Listener::accept_callback_fn> waitingAccepts_;
  std::deque<std::shared_ptr<Pipe>> waitingPipes_;
  uint64_t ticketsIssued_ = 0;
  std::unordered_map<uint64_t, TicketFn> tickets_;
  std::unordered_set<std::shared_ptr<transport::Connection>> unidentified_;  // hello not read yet
  uint64_t pipesMade_ = 0;
};

// ---- pipe -----------------------------------------------------------------------------------
class PipeCore final : public std::enable_shared_from_this<PipeCore> {
 public:
  // The dialling end.
  PipeCore(std::shared_ptr<ContextCore> context, std::string id, std::string remoteName, const std::string& url);
  // The answering end, made by a listener around the connection that said hello.
  PipeCore(std::shared_ptr<ContextCore> context, std::shared_ptr<ListenerCore> listener, std::string id,
           std::string remoteName, std::string transport, std::shared_ptr<transport::Connection> wire);

  void start();      // any thread
  void startNow();   // loop only

  void readDescriptor(Pipe::read_descriptor_callback_fn fn);
  void read(Allocation allocation, Pipe::read_callback_fn fn);
  void write(Message message, Pipe::write_callback_fn fn);
  void setTimeouts(PipeTimeouts timeouts);
  bool routeSupportsLayouts(const Device& local, const Device& remote);
  std::string transportName();
  const std::string& remoteName() const { return remoteName_; }
  void close();

  void fail(const Error& e);
  template <typename F>
  void guarded(F&& fn);
  ContextCore& context() { return *context_; }

 private:
  // -- setup (pipe_setup.cc) --
  enum class Role : uint8_t { kDialer, kAnswerer };
  enum class Phase : uint8_t { kIdle, kAwaitingOffer, kAwaitingAnswer, kAwaitingLinks, kOpen, kFailed };
  // One channel in use by this pipe and the connections it was promised.
  struct Mover {
    std::shared_ptr<channel::Channel> channel;
    std::vector<std::shared_ptr<transport::Connection>> links;
    size_t missing = 0;
  };
  // What an expected connection is for.
  struct Expected {
    enum Kind : uint8_t { kWire, kReplyWire, kChannelLink } kind;
    std::string channel;
    size_t index = 0;
  };
  using DeviceDescriptors = std::unordered_map<Device, std::string>;
  using Routes = std::unordered_map<std::pair<Device, Device>, std::string>;

  void sendOffer();
  void onOffer(const Brochure& offer);
  void onAnswer(const BrochureAnswer& answer);
  void onLink(uint64_t ticket, const std::string& transport, std::shared_ptr<transport::Connection> conn);
  void presentTicket(transport::Connection& conn, uint64_t ticket);
  uint64_t expect(Expected what);
  // For every (local device, remote device): the best channel whose descriptors say it can serve
  // the pair; `used` receives the names of the channels that serve at least one pair.
  Routes chooseRoutes(const std::unordered_map<std::string, DeviceDescriptors>& theirs, std::vector<std::string>* used);
  void becomeOpen();
  channel::Channel* channelFor(const Device& local, const Device& remote, const std::string** name = nullptr);

  // -- traffic (pipe_traffic.cc) --
  struct Outbound {
    uint64_t seq = 0;
    Message message;
    Pipe::write_callback_fn done;
    std::vector<Device> targets;   // resolved target device per tensor (valid once !awaitingTargets)
    bool announced = false;        // descriptor and payload frames have been written
    bool awaitingTargets = false;  // the peer still owes the devices it picked
    bool dispatched = false;       // tensors have been handed to their channels
    uint32_t outstanding = 0;      // completions still owed: frame writes, the reply, tensor sends
  };
  struct Inbound {
    uint64_t seq = 0;
    enum Stage : uint8_t { kArmed, kDescriptorPosted, kOffered, kAnswered, kReceiving } stage = kArmed;
    Pipe::read_descriptor_callback_fn offer;
    Descriptor descriptor;
    Allocation allocation;
    Pipe::read_callback_fn done;
    uint32_t outstanding = 0;  // payload reads and tensor receives still owed
  };
  Outbound* outbound(uint64_t seq);
  Inbound* inbound(uint64_t seq);
  void pumpOutbound();
  void announce(Outbound& m);
  void awaitTargets(Outbound& m);
  void dispatch(Outbound& m);
  void settleOutbound(uint64_t seq);
  void pumpInbound();
  void postDescriptorRead(Inbound& m);
  void beginReceiving(Inbound& m);
  void settleInbound(uint64_t seq);
  enum class Deadline : uint8_t { kWrite, kRead, kDescriptor };
  void armDeadline(Deadline kind, uint64_t seq, std::chrono::milliseconds after);

  std::shared_ptr<ContextCore> context_;
  std::shared_ptr<ListenerCore> listener_;  // answering end only
  std::string id_;
  std::string remoteName_;
  Role role_;
  Phase phase_ = Phase::kIdle;
  Error error_;
  PipeTimeouts timeouts_;

  std::string wireTransport_;
  std::shared_ptr<transport::Connection> wire_;       // descriptors and payloads, both directions
  std::shared_ptr<transport::Connection> replyWire_;  // descriptor replies, both directions
  std::map<std::string, Mover> movers_;
  Routes routes_;
  std::map<uint64_t, Expected> expected_;  // ticket -> what the connection is for (answering end)

  std::deque<Outbound> outbound_;
  uint64_t outboundNext_ = 0;      // sequence number of the next write()
  uint64_t announceCursor_ = 0;    // first message not announced yet
  uint64_t dispatchCursor_ = 0;    // first message whose tensors are not with the channels yet
  std::deque<Inbound> inbound_;
  uint64_t inboundNext_ = 0;       // sequence number of the next readDescriptor()
  uint64_t postCursor_ = 0;        // first message whose descriptor read is not posted yet
  int64_t offered_ = -1;           // message whose descriptor the user holds and has not answered with read()
};

template <typename F>
void ListenerCore::guarded(F&& fn) {
  try {
    fn();
  } catch (const std::exception& ex) {
    fail(TPB_CREATE_ERROR(LogicError, std::string("while handling an incoming connection: ") + ex.what()));
  }
}

template <typename F>
void PipeCore::guarded(F&& fn) {
  try {
    fn();
  } catch (const std::exception& ex) {
    fail(TPB_CREATE_ERROR(LogicError, ex.what()));
  }
}

}  // namespace core
}  // namespace tpb
