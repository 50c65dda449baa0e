// Internal classes behind Context / Listener / Pipe. Every public object is a thin shell over a
// shared_ptr to one of these; all state is only touched from the context's on-demand loop.
// Counterparts: tensorpipe/core/context_impl.h:29-145, listener_impl.h:32-146,
// pipe_impl.h:37-306.
#pragma once

#include <atomic>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include <tpb/context.h>

#include "common/callback.h"
#include "common/defs.h"
#include "common/loop.h"
#include "common/ops.h"
#include "core/nop_types.h"

namespace tpb {

class ListenerImpl;
class PipeImpl;

class ContextImpl final : public std::enable_shared_from_this<ContextImpl> {
 public:
  using TOrderedTransports =
      std::map<int64_t, std::pair<std::string, std::shared_ptr<transport::Context>>>;
  using TOrderedChannels =
      std::map<int64_t, std::pair<std::string, std::shared_ptr<channel::Context>>>;

  explicit ContextImpl(ContextOptions opts);

  void registerTransport(int64_t priority, std::string name, std::shared_ptr<transport::Context> t);
  void registerChannel(int64_t priority, std::string name, std::shared_ptr<channel::Context> c);
  std::shared_ptr<Listener> listen(const std::vector<std::string>& urls);
  std::shared_ptr<Pipe> connect(const std::string& url, PipeOptions opts);

  std::shared_ptr<transport::Context> getTransport(const std::string& name);
  std::shared_ptr<channel::Context> getChannel(const std::string& name);
  const TOrderedTransports& getOrderedTransports() const { return transportsByPriority_; }
  const TOrderedChannels& getOrderedChannels() const { return channelsByPriority_; }
  const std::string& getName() const { return name_; }

  void enroll(ListenerImpl& l);
  void enroll(PipeImpl& p);
  void unenroll(ListenerImpl& l);
  void unenroll(PipeImpl& p);
  bool closed() const { return closed_; }

  DeferredExecutor& loop() { return loop_; }
  bool inLoop() const { return loop_.inLoop(); }
  void deferToLoop(std::function<void()> fn) { loop_.deferToLoop(std::move(fn)); }

  void close();
  void join();

  ContextStats stats();
  // Only from the loop.
  ContextStats stats_;
  std::mutex statsMutex_;

  std::string makeChildId(const char* kind);

 private:
  OnDemandLoop loop_;
  std::string id_;
  std::string name_;
  std::atomic<bool> closed_{false};
  std::atomic<bool> joined_{false};
  std::atomic<uint64_t> listenerCounter_{0}, pipeCounter_{0};
  std::mutex registryMutex_;  // registrations may come from any thread before use
  std::unordered_map<std::string, std::shared_ptr<transport::Context>> transports_;
  std::unordered_map<std::string, std::shared_ptr<channel::Context>> channels_;
  TOrderedTransports transportsByPriority_;
  TOrderedChannels channelsByPriority_;
  std::unordered_map<ListenerImpl*, std::shared_ptr<ListenerImpl>> listeners_;
  std::unordered_map<PipeImpl*, std::shared_ptr<PipeImpl>> pipes_;
};

class ListenerImpl final : public std::enable_shared_from_this<ListenerImpl> {
 public:
  using connection_request_callback_fn =
      std::function<void(const Error&, std::string, std::shared_ptr<transport::Connection>)>;

  ListenerImpl(std::shared_ptr<ContextImpl> context, std::string id,
               const std::vector<std::string>& urls);
  void init();
  void accept(Listener::accept_callback_fn fn);
  const std::map<std::string, std::string>& addresses() const { return addresses_; }
  const std::string& address(const std::string& transport) const;
  std::string url(const std::string& transport) const;

  // From the loop only.
  uint64_t registerConnectionRequest(connection_request_callback_fn fn);
  void unregisterConnectionRequest(uint64_t id);

  void close();

  DeferredExecutor& loop() { return context_->loop(); }
  void setError(const Error& e);

 private:
  void initFromLoop();
  void armListener(const std::string& transport);
  void onAccept(const std::string& transport, std::shared_ptr<transport::Connection> conn);
  void onConnectionHelloRead(const std::string& transport,
                             std::shared_ptr<transport::Connection> conn, const Packet& packet);
  void handleError();

  std::shared_ptr<ContextImpl> context_;
  std::string id_;
  Error error_;
  std::unordered_map<std::string, std::shared_ptr<transport::Listener>> listeners_;
  std::map<std::string, std::string> addresses_;
  RearmableCallback<const Error&, std::shared_ptr<Pipe>> acceptCallback_;
  uint64_t nextConnectionRequestId_ = 0;
  std::unordered_map<uint64_t, connection_request_callback_fn> connectionRequests_;
  std::unordered_set<std::shared_ptr<transport::Connection>> connectionsWaitingForHello_;
  uint64_t pipeCounter_ = 0;
  LoopCallback<ListenerImpl> callbackWrapper_{*this};
  friend class PipeImpl;
};

struct ReadOperation {
  enum State {
    UNINITIALIZED,
    READING_DESCRIPTOR,
    ASKING_FOR_ALLOCATION,
    ASKING_FOR_ALLOCATION_FIRST_IN_LINE,
    READING_PAYLOADS_AND_RECEIVING_TENSORS,
    FINISHED
  };
  int64_t sequenceNumber = -1;
  State state = UNINITIALIZED;
  bool doneReadingDescriptor = false;
  bool descriptorDelivered = false;  // the user got a descriptor (without error) for this op
  bool doneGettingAllocation = false;
  int64_t numPayloadsBeingRead = 0;
  int64_t numTensorsBeingReceived = 0;
  Pipe::read_descriptor_callback_fn readDescriptorCallback;
  Descriptor descriptor;
  Pipe::read_callback_fn readCallback;
  Allocation allocation;
};

struct WriteOperation {
  enum State {
    UNINITIALIZED,
    WRITING_PAYLOADS_AND_READING_TARGET_DEVICES,
    WRITING_PAYLOADS_AND_SENDING_TENSORS,
    FINISHED
  };
  int64_t sequenceNumber = -1;
  State state = UNINITIALIZED;
  int64_t numPayloadsBeingWritten = 0;  // includes the descriptor frame
  int64_t numTensorsBeingSent = 0;
  bool hasMissingTargetDevices = false;
  bool doneReadingDescriptorReply = false;
  Message message;
  std::vector<Device> sourceDevices;
  std::vector<std::optional<Device>> targetDevices;
  Pipe::write_callback_fn writeCallback;
};

class PipeImpl final : public std::enable_shared_from_this<PipeImpl> {
 public:
  enum State {
    INITIALIZING,
    CLIENT_ABOUT_TO_SEND_HELLO_AND_BROCHURE,
    SERVER_WAITING_FOR_BROCHURE,
    CLIENT_WAITING_FOR_BROCHURE_ANSWER,
    SERVER_WAITING_FOR_CONNECTIONS,
    ESTABLISHED
  };
  enum ConnectionId : uint64_t { DESCRIPTOR = 0, DESCRIPTOR_REPLY = 1 };

  // Client side.
  PipeImpl(std::shared_ptr<ContextImpl> context, std::string id, std::string remoteName,
           const std::string& url);
  // Server side.
  PipeImpl(std::shared_ptr<ContextImpl> context, std::shared_ptr<ListenerImpl> listener,
           std::string id, std::string remoteName, std::string transport,
           std::shared_ptr<transport::Connection> connection);

  void init();
  void initFromLoop();
  void readDescriptor(Pipe::read_descriptor_callback_fn fn);
  void read(Allocation allocation, Pipe::read_callback_fn fn);
  void write(Message message, Pipe::write_callback_fn fn);
  void setTimeouts(PipeTimeouts timeouts);
  const std::string& getRemoteName() { return remoteName_; }
  bool channelSupportsLayouts(const Device& local, const Device& remote);
  void close();

  DeferredExecutor& loop() { return context_->loop(); }
  void setError(const Error& e);

 private:
  void readDescriptorFromLoop(Pipe::read_descriptor_callback_fn fn);
  void readFromLoop(Allocation allocation, Pipe::read_callback_fn fn);
  void writeFromLoop(Message message, Pipe::write_callback_fn fn);
  void handleError();
  // Fails the pipe with TimeoutError if the operation is still pending after `delay`.
  enum class Deadline { kWrite, kRead, kDescriptor };
  void armDeadline(Deadline kind, int64_t seq, std::chrono::milliseconds delay);

  void advanceReadOperation(ReadOperation& op, ReadOperation::State prev);
  void advanceWriteOperation(WriteOperation& op, WriteOperation::State prev);

  void readDescriptorOfMessage(ReadOperation& op);
  void readPayloadsOfMessage(ReadOperation& op);
  void writeDescriptorReplyOfMessage(ReadOperation& op);
  void receiveTensorsOfMessage(ReadOperation& op);
  void writeDescriptorAndPayloadsOfMessage(WriteOperation& op);
  void readDescriptorReplyOfMessage(WriteOperation& op);
  void sendTensorsOfMessage(WriteOperation& op);

  void onReadWhileServerWaitingForBrochure(const Brochure& b);
  void onReadWhileClientWaitingForBrochureAnswer(const BrochureAnswer& a);
  void onAcceptWhileServerWaitingForConnection(ConnectionId id, std::string transport,
                                               std::shared_ptr<transport::Connection> c);
  void onAcceptWhileServerWaitingForChannel(const std::string& channel, size_t connId,
                                            std::string transport,
                                            std::shared_ptr<transport::Connection> c);
  uint64_t registerTransport(ConnectionId id);
  std::vector<uint64_t>& registerChannel(const std::string& name);
  void initConnection(transport::Connection& c, uint64_t token);
  bool pendingRegistrations() const;
  void establish();

  std::shared_ptr<ContextImpl> context_;
  std::shared_ptr<ListenerImpl> listener_;
  std::string id_;
  std::string remoteName_;
  State state_ = INITIALIZING;
  std::string transport_;
  std::shared_ptr<transport::Connection> descriptorConnection_;
  std::shared_ptr<transport::Connection> descriptorReplyConnection_;
  std::unordered_map<std::string, std::shared_ptr<channel::Channel>> channels_;
  std::unordered_map<std::pair<Device, Device>, std::string> channelForDevicePair_;
  std::unordered_map<uint64_t, uint64_t> registrationIds_;
  std::unordered_map<std::string, std::vector<uint64_t>> channelRegistrationIds_;
  std::unordered_map<std::string, std::vector<std::shared_ptr<transport::Connection>>>
      channelReceivedConnections_;
  Error error_;
  PipeTimeouts timeouts_;  // loop only

  OpQueue<ReadOperation> readOps_;
  OpQueue<WriteOperation> writeOps_;
  std::deque<int64_t> awaitingRead_;  // ops whose descriptor was delivered, oldest first

  LoopCallback<PipeImpl> callbackWrapper_{*this};
  friend class ContextImpl;
};

}  // namespace tpb
