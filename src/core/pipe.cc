// The pipe: handshake state machine, per-message read and write state machines, transport and
// channel selection, and error fan-out. The observable protocol (frames, their order, who
// opens which connection) is that of tensorpipe/core/pipe_impl.cc so that either end can be a
// reference peer; the code is organised around OpQueue transitions written for this library.
//
// Connections of a pipe: "descriptor" (both directions: descriptors followed by the payloads of
// each message) and "descriptor reply" (both directions: the target devices a receiver chose),
// plus numConnectionsNeeded() connections per selected channel.
#include <algorithm>

#include "core/core_impl.h"
#include "common/timer.h"
#include "common/trace.h"
#include "transport/nop_io.h"

namespace tpb {

namespace {

std::pair<std::string, std::string> splitSchemeOfURL(const std::string& url) {
  auto pos = url.find("://");
  TPB_THROW_SYSTEM_IF(pos == std::string::npos, EINVAL, "url has no scheme: " + url);
  return {url.substr(0, pos), url.substr(pos + 3)};
}

struct SelectedTransport {
  std::string name, address, domainDescriptor;
};

// First transport, by THIS side's priority, that both sides have, that the listener is bound
// on, and whose domain descriptors say the two ends can reach each other.
SelectedTransport selectTransport(
    const ContextImpl::TOrderedTransports& ordered,
    const std::unordered_map<std::string, std::string>& remoteDomainDescriptors,
    const std::map<std::string, std::string>& addresses) {
  for (const auto& it : ordered) {
    const std::string& name = it.second.first;
    const transport::Context& ctx = *it.second.second;
    auto addr = addresses.find(name);
    if (addr == addresses.end()) continue;
    auto remote = remoteDomainDescriptors.find(name);
    if (remote == remoteDomainDescriptors.end()) continue;
    if (!ctx.canCommunicateWithRemote(remote->second)) continue;
    return {name, addr->second, ctx.domainDescriptor()};
  }
  TPB_THROW_ASSERT_IF(true, "Could not find a viable transport");
  return {};
}

struct SelectedChannels {
  std::unordered_map<std::string, std::unordered_map<Device, std::string>> descriptorsMap;
  std::unordered_map<std::pair<Device, Device>, std::string> channelForDevicePair;
};

// For every (local device, remote device) pair, the highest-priority channel whose descriptors
// are compatible. Both ends run this with their own priorities and must agree.
SelectedChannels selectChannels(
    const ContextImpl::TOrderedChannels& ordered,
    const std::unordered_map<std::string, std::unordered_map<Device, std::string>>& remoteMap) {
  SelectedChannels result;
  for (const auto& it : ordered) {
    const std::string& name = it.second.first;
    const channel::Context& ctx = *it.second.second;
    auto remote = remoteMap.find(name);
    if (remote == remoteMap.end()) continue;
    const auto& local = ctx.deviceDescriptors();
    bool selected = false;
    for (const auto& l : local) {
      for (const auto& r : remote->second) {
        if (!ctx.canCommunicateWithRemote(l.second, r.second)) continue;
        auto key = std::make_pair(l.first, r.first);
        if (result.channelForDevicePair.count(key)) continue;
        result.channelForDevicePair[key] = name;
        selected = true;
      }
    }
    if (selected) result.descriptorsMap[name] = local;
  }
  return result;
}

void checkAllocationCompatibility(const Descriptor& d, const Allocation& a) {
  TPB_THROW_ASSERT_IF(a.payloads.size() != d.payloads.size(),
                      "allocation has a different number of payloads than the descriptor");
  TPB_THROW_ASSERT_IF(a.tensors.size() != d.tensors.size(),
                      "allocation has a different number of tensors than the descriptor");
  for (size_t i = 0; i < a.tensors.size(); ++i) {
    if (d.tensors[i].targetDevice.has_value()) {
      TPB_THROW_ASSERT_IF(!(a.tensors[i].buffer.device() == *d.tensors[i].targetDevice),
                          "tensor allocated on a device other than the requested target device");
    }
  }
}

}  // namespace

// ---- construction / handshake ---------------------------------------------------------------
PipeImpl::PipeImpl(std::shared_ptr<ContextImpl> context, std::string id, std::string remoteName,
                   const std::string& url)
    : context_(std::move(context)),
      id_(std::move(id)),
      remoteName_(std::move(remoteName)),
      state_(CLIENT_ABOUT_TO_SEND_HELLO_AND_BROCHURE),
      readOps_([this](ReadOperation& op, ReadOperation::State prev) { advanceReadOperation(op, prev); }),
      writeOps_([this](WriteOperation& op, WriteOperation::State prev) { advanceWriteOperation(op, prev); }) {
  auto [scheme, address] = splitSchemeOfURL(url);
  transport_ = scheme;
  descriptorConnection_ = context_->getTransport(transport_)->connect(address);
  descriptorConnection_->setId(id_ + ".d.tr_" + transport_);
}

PipeImpl::PipeImpl(std::shared_ptr<ContextImpl> context, std::shared_ptr<ListenerImpl> listener,
                   std::string id, std::string remoteName, std::string transport,
                   std::shared_ptr<transport::Connection> connection)
    : context_(std::move(context)),
      listener_(std::move(listener)),
      id_(std::move(id)),
      remoteName_(std::move(remoteName)),
      state_(SERVER_WAITING_FOR_BROCHURE),
      transport_(std::move(transport)),
      descriptorConnection_(std::move(connection)),
      readOps_([this](ReadOperation& op, ReadOperation::State prev) { advanceReadOperation(op, prev); }),
      writeOps_([this](WriteOperation& op, WriteOperation::State prev) { advanceWriteOperation(op, prev); }) {
  descriptorConnection_->setId(id_ + ".d.tr_" + transport_);
}

void PipeImpl::init() {
  auto self = shared_from_this();
  context_->deferToLoop([self]() { self->initFromLoop(); });
}

void PipeImpl::initFromLoop() {
  if (context_->closed()) {
    setError(TPB_CREATE_ERROR(ContextClosedError));
    return;
  }
  context_->enroll(*this);

  if (state_ == CLIENT_ABOUT_TO_SEND_HELLO_AND_BROCHURE) {
    Packet hello = SpontaneousConnection{context_->getName()};
    TPB_VLOG(3) << "Pipe " << id_ << " is writing nop object (spontaneous connection)";
    transport::writeNop(*descriptorConnection_, hello, callbackWrapper_([](PipeImpl&) {}));

    Brochure brochure;
    for (const auto& t : context_->getOrderedTransports())
      brochure.transportDomainDescriptors[t.second.first] = t.second.second->domainDescriptor();
    for (const auto& c : context_->getOrderedChannels())
      brochure.channelDeviceDescriptors[c.second.first] = c.second.second->deviceDescriptors();
    TPB_VLOG(3) << "Pipe " << id_ << " is writing nop object (brochure)";
    transport::writeNop(*descriptorConnection_, brochure, callbackWrapper_([](PipeImpl&) {}));

    state_ = CLIENT_WAITING_FOR_BROCHURE_ANSWER;
    transport::readNop<BrochureAnswer>(
        *descriptorConnection_, callbackWrapper_([](PipeImpl& impl, BrochureAnswer answer) {
          // What the peer says may be well formed and still make no sense (an unknown transport,
          // a channel map that contradicts ours): that fails this pipe, not the process.
          if (impl.error_) return;
          try {
            impl.onReadWhileClientWaitingForBrochureAnswer(answer);
          } catch (const std::exception& ex) {
            impl.setError(TPB_CREATE_ERROR(LogicError, std::string("inconsistent handshake from the peer: ") + ex.what()));
          }
        }));
  } else if (state_ == SERVER_WAITING_FOR_BROCHURE) {
    transport::readNop<Brochure>(
        *descriptorConnection_, callbackWrapper_([](PipeImpl& impl, Brochure brochure) {
          if (impl.error_) return;
          try {
            impl.onReadWhileServerWaitingForBrochure(brochure);
          } catch (const std::exception& ex) {
            impl.setError(TPB_CREATE_ERROR(LogicError, std::string("inconsistent handshake from the peer: ") + ex.what()));
          }
        }));
  }
}

void PipeImpl::onReadWhileServerWaitingForBrochure(const Brochure& brochure) {
  BrochureAnswer answer;
  SelectedTransport transport = selectTransport(
      context_->getOrderedTransports(), brochure.transportDomainDescriptors, listener_->addresses());
  if (transport.name != transport_) {
    transport_ = transport.name;
    answer.transportRegistrationIds[DESCRIPTOR] = registerTransport(DESCRIPTOR);
  }
  answer.transportRegistrationIds[DESCRIPTOR_REPLY] = registerTransport(DESCRIPTOR_REPLY);
  answer.transport = transport.name;
  answer.address = transport.address;
  answer.transportDomainDescriptor = transport.domainDescriptor;

  SelectedChannels selected =
      selectChannels(context_->getOrderedChannels(), brochure.channelDeviceDescriptors);
  channelForDevicePair_ = std::move(selected.channelForDevicePair);
  answer.channelForDevicePair = channelForDevicePair_;
  for (auto& d : selected.descriptorsMap) {
    answer.channelRegistrationIds[d.first] = registerChannel(d.first);
    answer.channelDeviceDescriptors[d.first] = std::move(d.second);
  }

  TPB_VLOG(3) << "Pipe " << id_ << " is writing nop object (brochure answer)";
  transport::writeNop(*descriptorConnection_, answer, callbackWrapper_([](PipeImpl&) {}));

  if (!pendingRegistrations()) establish();
  else state_ = SERVER_WAITING_FOR_CONNECTIONS;
}

uint64_t PipeImpl::registerTransport(ConnectionId connId) {
  uint64_t token = listener_->registerConnectionRequest(callbackWrapper_(
      [connId](PipeImpl& impl, std::string transport, std::shared_ptr<transport::Connection> c) {
        if (!impl.error_) impl.onAcceptWhileServerWaitingForConnection(connId, std::move(transport), std::move(c));
      }));
  registrationIds_[connId] = token;
  return token;
}

std::vector<uint64_t>& PipeImpl::registerChannel(const std::string& name) {
  const size_t n = context_->getChannel(name)->numConnectionsNeeded();
  auto& ids = channelRegistrationIds_[name];
  ids.resize(n);
  channelReceivedConnections_[name].resize(n);
  for (size_t i = 0; i < n; ++i) {
    ids[i] = listener_->registerConnectionRequest(callbackWrapper_(
        [name, i](PipeImpl& impl, std::string transport, std::shared_ptr<transport::Connection> c) {
          if (!impl.error_) impl.onAcceptWhileServerWaitingForChannel(name, i, std::move(transport), std::move(c));
        }));
  }
  return ids;
}

void PipeImpl::initConnection(transport::Connection& c, uint64_t token) {
  Packet p = RequestedConnection{token};
  transport::writeNop(c, p, callbackWrapper_([](PipeImpl&) {}));
}

void PipeImpl::onReadWhileClientWaitingForBrochureAnswer(const BrochureAnswer& answer) {
  const std::string& transport = answer.transport;
  std::shared_ptr<transport::Context> tctx = context_->getTransport(transport);

  if (transport != transport_) {
    auto conn = tctx->connect(answer.address);
    conn->setId(id_ + ".d.tr_" + transport);
    auto it = answer.transportRegistrationIds.find(DESCRIPTOR);
    TPB_THROW_ASSERT_IF(it == answer.transportRegistrationIds.end(), "peer did not register a descriptor connection");
    initConnection(*conn, it->second);
    transport_ = transport;
    descriptorConnection_ = std::move(conn);
  }
  {
    auto conn = tctx->connect(answer.address);
    conn->setId(id_ + ".r.tr_" + transport);
    auto it = answer.transportRegistrationIds.find(DESCRIPTOR_REPLY);
    TPB_THROW_ASSERT_IF(it == answer.transportRegistrationIds.end(), "peer did not register a descriptor-reply connection");
    initConnection(*conn, it->second);
    descriptorReplyConnection_ = std::move(conn);
  }

  SelectedChannels selected =
      selectChannels(context_->getOrderedChannels(), answer.channelDeviceDescriptors);
  channelForDevicePair_ = std::move(selected.channelForDevicePair);
  TPB_THROW_ASSERT_IF(answer.channelForDevicePair.size() != channelForDevicePair_.size(),
                      "Inconsistent channel selection");
  for (const auto& it : channelForDevicePair_) {
    auto peer = answer.channelForDevicePair.find({it.first.second, it.first.first});
    TPB_THROW_ASSERT_IF(peer == answer.channelForDevicePair.end() || peer->second != it.second,
                        "Inconsistent channel selection");
  }

  for (const auto& d : selected.descriptorsMap) {
    const std::string& name = d.first;
    auto cctx = context_->getChannel(name);
    const auto& ids = answer.channelRegistrationIds.at(name);
    const size_t n = cctx->numConnectionsNeeded();
    TPB_THROW_ASSERT_IF(n != ids.size(), "peer disagrees on the connections channel " + name + " needs");
    std::vector<std::shared_ptr<transport::Connection>> conns(n);
    for (size_t i = 0; i < n; ++i) {
      auto conn = tctx->connect(answer.address);
      conn->setId(id_ + ".ch_" + name + "_" + std::to_string(i));
      initConnection(*conn, ids[i]);
      conns[i] = std::move(conn);
    }
    auto ch = cctx->createChannel(std::move(conns), channel::Endpoint::kConnect);
    ch->setId(id_ + ".ch_" + name);
    channels_.emplace(name, std::move(ch));
  }
  establish();
}

void PipeImpl::onAcceptWhileServerWaitingForConnection(ConnectionId connId, std::string transport,
                                                       std::shared_ptr<transport::Connection> c) {
  registrationIds_.erase(connId);
  c->setId(id_ + (connId == DESCRIPTOR ? ".d.tr_" : ".r.tr_") + transport);
  if (connId == DESCRIPTOR) descriptorConnection_ = std::move(c);
  else descriptorReplyConnection_ = std::move(c);
  if (!pendingRegistrations()) establish();
}

void PipeImpl::onAcceptWhileServerWaitingForChannel(const std::string& name, size_t connId,
                                                    std::string transport,
                                                    std::shared_ptr<transport::Connection> c) {
  (void)transport;
  auto& ids = channelRegistrationIds_[name];
  auto& conns = channelReceivedConnections_[name];
  c->setId(id_ + ".ch_" + name + "_" + std::to_string(connId));
  conns[connId] = std::move(c);
  ids[connId] = UINT64_MAX;
  bool all = std::all_of(conns.begin(), conns.end(), [](const auto& p) { return p != nullptr; });
  if (all) {
    auto ch = context_->getChannel(name)->createChannel(std::move(conns), channel::Endpoint::kListen);
    ch->setId(id_ + ".ch_" + name);
    channels_.emplace(name, std::move(ch));
    channelRegistrationIds_.erase(name);
    channelReceivedConnections_.erase(name);
  }
  if (!pendingRegistrations()) establish();
}

bool PipeImpl::pendingRegistrations() const {
  return !registrationIds_.empty() || !channelRegistrationIds_.empty();
}

void PipeImpl::establish() {
  TPB_VLOG(1) << "Pipe " << id_ << " is established over transport " << transport_;
  state_ = ESTABLISHED;
  readOps_.advanceAllOperations();
  writeOps_.advanceAllOperations();
}

bool PipeImpl::channelSupportsLayouts(const Device& local, const Device& remote) {
  bool result = false;
  context_->loop().runInLoop([&]() {
    auto it = channelForDevicePair_.find({local, remote});
    if (it == channelForDevicePair_.end()) return;
    auto ch = channels_.find(it->second);
    if (ch != channels_.end()) result = ch->second->supportsLayouts();
  });
  return result;
}

// ---- user operations ------------------------------------------------------------------------
void PipeImpl::readDescriptor(Pipe::read_descriptor_callback_fn fn) {
  auto self = shared_from_this();
  context_->deferToLoop([self, fn = std::move(fn)]() mutable {
    try {
      self->readDescriptorFromLoop(std::move(fn));
    } catch (const std::exception& ex) {
      self->setError(TPB_CREATE_ERROR(LogicError, ex.what()));
    }
  });
}

void PipeImpl::readDescriptorFromLoop(Pipe::read_descriptor_callback_fn fn) {
  ReadOperation& op = readOps_.emplaceBack();
  trace::instant("pipe.readDescriptor", op.sequenceNumber);
  TPB_VLOG(1) << "Pipe " << id_ << " received a readDescriptor request (#" << op.sequenceNumber << ")";
  op.readDescriptorCallback = std::move(fn);
  if (timeouts_.descriptor.count() > 0) armDeadline(Deadline::kDescriptor, op.sequenceNumber, timeouts_.descriptor);
  readOps_.advanceOperation(op);
}

void PipeImpl::read(Allocation allocation, Pipe::read_callback_fn fn) {
  // Logic errors must surface in the caller's thread, so this part runs synchronously.
  context_->loop().runInLoop([&]() { readFromLoop(std::move(allocation), std::move(fn)); });
}

void PipeImpl::readFromLoop(Allocation allocation, Pipe::read_callback_fn fn) {
  if (awaitingRead_.empty()) {
    if (error_) {
      Error e = error_;
      context_->deferToLoop([fn = std::move(fn), e]() { fn(e); });
      return;
    }
    TPB_THROW_ASSERT_IF(true, "Pipe::read called while no message is waiting for an allocation");
  }
  ReadOperation* op = readOps_.findOperation(awaitingRead_.front());
  TPB_THROW_ASSERT_IF(op == nullptr, "internal: lost read operation");
  checkAllocationCompatibility(op->descriptor, allocation);
  awaitingRead_.pop_front();
  trace::instant("pipe.read", op->sequenceNumber);
  TPB_VLOG(1) << "Pipe " << id_ << " received a read request (#" << op->sequenceNumber << ")";
  op->allocation = std::move(allocation);
  op->readCallback = std::move(fn);
  op->doneGettingAllocation = true;
  if (timeouts_.read.count() > 0) armDeadline(Deadline::kRead, op->sequenceNumber, timeouts_.read);
  // Never call back from inside read(): advance from a fresh loop iteration.
  auto self = shared_from_this();
  int64_t seq = op->sequenceNumber;
  context_->deferToLoop([self, seq]() {
    try {
      self->readOps_.advanceOperation(seq);
    } catch (const std::exception& ex) {
      // E.g. a tensor between devices that no registered channel connects.
      self->setError(TPB_CREATE_ERROR(LogicError, ex.what()));
    }
  });
}

void PipeImpl::write(Message message, Pipe::write_callback_fn fn) {
  auto self = shared_from_this();
  context_->deferToLoop([self, message = std::move(message), fn = std::move(fn)]() mutable {
    try {
      self->writeFromLoop(std::move(message), std::move(fn));
    } catch (const std::exception& ex) {
      // E.g. a tensor on a device pair no registered channel serves: the pipe fails, the write's
      // callback (already queued) reports it.
      self->setError(TPB_CREATE_ERROR(LogicError, ex.what()));
    }
  });
}

void PipeImpl::writeFromLoop(Message message, Pipe::write_callback_fn fn) {
  WriteOperation& op = writeOps_.emplaceBack();
  trace::instant("pipe.write", op.sequenceNumber);
  TPB_VLOG(1) << "Pipe " << id_ << " received a write request (#" << op.sequenceNumber << ")";
  op.message = std::move(message);
  op.writeCallback = std::move(fn);
  const size_t n = op.message.tensors.size();
  op.sourceDevices.reserve(n);
  op.targetDevices.reserve(n);
  for (const auto& t : op.message.tensors) {
    op.sourceDevices.push_back(t.buffer.device());
    op.targetDevices.push_back(t.targetDevice);
    if (!t.targetDevice.has_value()) op.hasMissingTargetDevices = true;
  }
  if (timeouts_.write.count() > 0) armDeadline(Deadline::kWrite, op.sequenceNumber, timeouts_.write);
  writeOps_.advanceOperation(op);
}

void PipeImpl::setTimeouts(PipeTimeouts timeouts) {
  auto self = shared_from_this();
  context_->deferToLoop([self, timeouts]() { self->timeouts_ = timeouts; });
}

void PipeImpl::armDeadline(Deadline kind, int64_t seq, std::chrono::milliseconds delay) {
  std::weak_ptr<PipeImpl> weak = shared_from_this();
  TimerThread::get().schedule(delay, [weak, kind, seq]() {
    auto self = weak.lock();
    if (!self) return;
    self->context_->deferToLoop([self, kind, seq]() {
      if (self->error_) return;
      bool pending;
      if (kind == Deadline::kWrite) {
        WriteOperation* op = self->writeOps_.findOperation(seq);
        pending = op != nullptr && op->state != WriteOperation::FINISHED;
      } else {
        ReadOperation* op = self->readOps_.findOperation(seq);
        // A descriptor deadline is met once the descriptor has been handed to the user.
        pending = op != nullptr && op->state != ReadOperation::FINISHED &&
            (kind == Deadline::kRead || !op->descriptorDelivered);
      }
      if (!pending) return;
      TPB_VLOG(1) << "Pipe " << self->id_ << " gives up on "
                  << (kind == Deadline::kWrite ? "write" : kind == Deadline::kRead ? "read" : "readDescriptor") << " #"
                  << seq << ": deadline passed";
      self->setError(TPB_CREATE_ERROR(TimeoutError));
    });
  });
}

// ---- read state machine ---------------------------------------------------------------------
void PipeImpl::advanceReadOperation(ReadOperation& op, ReadOperation::State prev) {
  using Q = OpQueue<ReadOperation>;
  using R = ReadOperation;

  // Error before anything was read: report it through the descriptor callback, in order.
  Q::attemptTransition(op, R::UNINITIALIZED, R::ASKING_FOR_ALLOCATION,
                       bool(error_) && prev >= R::ASKING_FOR_ALLOCATION, [&]() {
                         auto fn = std::move(op.readDescriptorCallback);
                         op.readDescriptorCallback = nullptr;
                         fn(error_, Descriptor());
                       });
  // Wire order is descriptor N, payloads N, descriptor N+1: wait until the previous message
  // has posted its payload reads.
  Q::attemptTransition(op, R::UNINITIALIZED, R::READING_DESCRIPTOR,
                       !error_ && state_ == ESTABLISHED &&
                           prev >= R::READING_PAYLOADS_AND_RECEIVING_TENSORS,
                       [&]() { readDescriptorOfMessage(op); });
  Q::attemptTransition(op, R::READING_DESCRIPTOR, R::ASKING_FOR_ALLOCATION,
                       op.doneReadingDescriptor && prev >= R::ASKING_FOR_ALLOCATION, [&]() {
                         auto fn = std::move(op.readDescriptorCallback);
                         op.readDescriptorCallback = nullptr;
                         if (!error_) {
                           op.descriptorDelivered = true;
                           awaitingRead_.push_back(op.sequenceNumber);
                           fn(Error::kSuccess, op.descriptor);
                         } else {
                           fn(error_, Descriptor());
                         }
                       });
  // After an error: an op the user will never call read() for retires silently; one that did
  // get (or later gets) its read() call reports the error through the read callback.
  Q::attemptTransition(op, R::ASKING_FOR_ALLOCATION, R::FINISHED,
                       bool(error_) && prev == R::FINISHED &&
                           (!op.descriptorDelivered || op.doneGettingAllocation),
                       [&]() {
                         if (op.doneGettingAllocation) {
                           auto fn = std::move(op.readCallback);
                           fn(error_);
                         }
                       });
  Q::attemptTransition(op, R::ASKING_FOR_ALLOCATION, R::ASKING_FOR_ALLOCATION_FIRST_IN_LINE,
                       !error_ && prev >= R::READING_PAYLOADS_AND_RECEIVING_TENSORS);
  Q::attemptTransition(op, R::ASKING_FOR_ALLOCATION_FIRST_IN_LINE, R::FINISHED,
                       bool(error_) && op.doneGettingAllocation && prev == R::FINISHED, [&]() {
                         auto fn = std::move(op.readCallback);
                         fn(error_);
                       });
  Q::attemptTransition(op, R::ASKING_FOR_ALLOCATION_FIRST_IN_LINE,
                       R::READING_PAYLOADS_AND_RECEIVING_TENSORS,
                       !error_ && op.doneGettingAllocation, [&]() {
                         readPayloadsOfMessage(op);
                         writeDescriptorReplyOfMessage(op);
                         receiveTensorsOfMessage(op);
                       });
  Q::attemptTransition(op, R::READING_PAYLOADS_AND_RECEIVING_TENSORS, R::FINISHED,
                       op.numPayloadsBeingRead == 0 && op.numTensorsBeingReceived == 0 &&
                           prev == R::FINISHED,
                       [&]() {
                         trace::instant("pipe.read.done", op.sequenceNumber);
                         TPB_VLOG(1) << "Pipe " << id_ << " is calling a read callback (#"
                                     << op.sequenceNumber << ")";
                         if (!error_) {
                           std::unique_lock<std::mutex> lock(context_->statsMutex_);
                           context_->stats_.messagesRead++;
                         }
                         auto fn = std::move(op.readCallback);
                         fn(error_);
                       });
}

void PipeImpl::readDescriptorOfMessage(ReadOperation& op) {
  int64_t seq = op.sequenceNumber;
  TPB_VLOG(3) << "Pipe " << id_ << " is reading nop object (message descriptor #" << seq << ")";
  transport::readNop<Descriptor>(
      *descriptorConnection_, callbackWrapper_([seq](PipeImpl& impl, Descriptor d) {
        ReadOperation* op = impl.readOps_.findOperation(seq);
        if (!op) return;
        op->doneReadingDescriptor = true;
        if (!impl.error_) op->descriptor = std::move(d);
        impl.readOps_.advanceOperation(*op);
      }));
}

void PipeImpl::readPayloadsOfMessage(ReadOperation& op) {
  int64_t seq = op.sequenceNumber;
  for (size_t i = 0; i < op.allocation.payloads.size(); ++i) {
    size_t len = op.descriptor.payloads[i].length;
    {
      std::unique_lock<std::mutex> lock(context_->statsMutex_);
      context_->stats_.payloadBytesRead += len;
    }
    ++op.numPayloadsBeingRead;
    descriptorConnection_->read(
        op.allocation.payloads[i].data, len,
        callbackWrapper_([seq](PipeImpl& impl, const void*, size_t) {
          ReadOperation* op = impl.readOps_.findOperation(seq);
          if (!op) return;
          --op->numPayloadsBeingRead;
          impl.readOps_.advanceOperation(*op);
        }));
  }
}

void PipeImpl::writeDescriptorReplyOfMessage(ReadOperation& op) {
  bool missing = false;
  DescriptorReply reply;
  for (size_t i = 0; i < op.descriptor.tensors.size(); ++i) {
    if (!op.descriptor.tensors[i].targetDevice.has_value()) {
      missing = true;
      reply.targetDevices.push_back(op.allocation.tensors[i].buffer.device());
    }
  }
  if (!missing) return;
  TPB_VLOG(3) << "Pipe " << id_ << " is writing nop object (descriptor reply #" << op.sequenceNumber << ")";
  transport::writeNop(*descriptorReplyConnection_, reply, callbackWrapper_([](PipeImpl&) {}));
}

void PipeImpl::receiveTensorsOfMessage(ReadOperation& op) {
  int64_t seq = op.sequenceNumber;
  // Group the tensors by channel (keeping message order inside a group) so that a channel sees
  // everything it carries for this message at once.
  std::vector<std::pair<std::string, std::vector<channel::RecvItem>>> groups;
  for (size_t i = 0; i < op.descriptor.tensors.size(); ++i) {
    const auto& td = op.descriptor.tensors[i];
    const auto& ta = op.allocation.tensors[i];
    Device local = ta.buffer.device();
    auto it = channelForDevicePair_.find({local, td.sourceDevice});
    TPB_THROW_ASSERT_IF(it == channelForDevicePair_.end(),
                        "Could not find suitable channel for receiving from " +
                            td.sourceDevice.toString() + " to " + local.toString());
    {
      std::unique_lock<std::mutex> lock(context_->statsMutex_);
      context_->stats_.tensorBytesReceived += td.length;
      context_->stats_.bytesPerChannel[it->second] += td.length;
    }
    channel::RecvItem item;
    item.buffer = ta.buffer;
    item.length = td.length;
    item.castTo = ta.castTo;
    item.srcDtype = ta.sourceDtype;
    item.sourceDevice = td.sourceDevice;
    ++op.numTensorsBeingReceived;
    item.callback = callbackWrapper_([seq](PipeImpl& impl) {
      ReadOperation* op = impl.readOps_.findOperation(seq);
      if (!op) return;
      --op->numTensorsBeingReceived;
      impl.readOps_.advanceOperation(*op);
    });
    auto g = std::find_if(groups.begin(), groups.end(), [&](const auto& p) { return p.first == it->second; });
    if (g == groups.end()) {
      groups.emplace_back(it->second, std::vector<channel::RecvItem>());
      g = groups.end() - 1;
    }
    g->second.push_back(std::move(item));
  }
  for (auto& g : groups) channels_.at(g.first)->recvBatch(std::move(g.second));
}

// ---- write state machine --------------------------------------------------------------------
void PipeImpl::advanceWriteOperation(WriteOperation& op, WriteOperation::State prev) {
  using Q = OpQueue<WriteOperation>;
  using W = WriteOperation;

  Q::attemptTransition(op, W::UNINITIALIZED, W::FINISHED, bool(error_) && prev == W::FINISHED, [&]() {
    auto fn = std::move(op.writeCallback);
    fn(error_);
  });
  Q::attemptTransition(op, W::UNINITIALIZED, W::WRITING_PAYLOADS_AND_SENDING_TENSORS,
                       !error_ && state_ == ESTABLISHED && !op.hasMissingTargetDevices &&
                           prev >= W::WRITING_PAYLOADS_AND_SENDING_TENSORS,
                       [&]() {
                         writeDescriptorAndPayloadsOfMessage(op);
                         sendTensorsOfMessage(op);
                       });
  Q::attemptTransition(op, W::UNINITIALIZED, W::WRITING_PAYLOADS_AND_READING_TARGET_DEVICES,
                       !error_ && state_ == ESTABLISHED && op.hasMissingTargetDevices &&
                           prev >= W::WRITING_PAYLOADS_AND_READING_TARGET_DEVICES,
                       [&]() {
                         writeDescriptorAndPayloadsOfMessage(op);
                         readDescriptorReplyOfMessage(op);
                       });
  Q::attemptTransition(op, W::WRITING_PAYLOADS_AND_READING_TARGET_DEVICES, W::FINISHED,
                       bool(error_) && op.numPayloadsBeingWritten == 0 &&
                           op.doneReadingDescriptorReply && prev == W::FINISHED,
                       [&]() {
                         auto fn = std::move(op.writeCallback);
                         fn(error_);
                       });
  Q::attemptTransition(op, W::WRITING_PAYLOADS_AND_READING_TARGET_DEVICES,
                       W::WRITING_PAYLOADS_AND_SENDING_TENSORS,
                       !error_ && op.doneReadingDescriptorReply &&
                           prev >= W::WRITING_PAYLOADS_AND_SENDING_TENSORS,
                       [&]() { sendTensorsOfMessage(op); });
  Q::attemptTransition(op, W::WRITING_PAYLOADS_AND_SENDING_TENSORS, W::FINISHED,
                       op.numPayloadsBeingWritten == 0 && op.numTensorsBeingSent == 0 &&
                           prev == W::FINISHED,
                       [&]() {
                         trace::instant("pipe.write.done", op.sequenceNumber);
                         TPB_VLOG(1) << "Pipe " << id_ << " is calling a write callback (#"
                                     << op.sequenceNumber << ")";
                         if (!error_) {
                           std::unique_lock<std::mutex> lock(context_->statsMutex_);
                           context_->stats_.messagesWritten++;
                         }
                         auto fn = std::move(op.writeCallback);
                         fn(error_);
                       });
}

void PipeImpl::writeDescriptorAndPayloadsOfMessage(WriteOperation& op) {
  int64_t seq = op.sequenceNumber;
  Descriptor d;
  d.metadata = op.message.metadata;
  for (const auto& p : op.message.payloads) d.payloads.push_back({p.length, p.metadata});
  for (size_t i = 0; i < op.message.tensors.size(); ++i) {
    const auto& t = op.message.tensors[i];
    Descriptor::Tensor dt;
    dt.length = t.length;
    dt.sourceDevice = op.sourceDevices[i];
    dt.targetDevice = t.targetDevice;
    dt.metadata = t.metadata;
    d.tensors.push_back(std::move(dt));
  }
  auto done = [seq](PipeImpl& impl) {
    WriteOperation* op = impl.writeOps_.findOperation(seq);
    if (!op) return;
    --op->numPayloadsBeingWritten;
    impl.writeOps_.advanceOperation(*op);
  };
  TPB_VLOG(3) << "Pipe " << id_ << " is writing nop object (message descriptor #" << seq << ")";
  ++op.numPayloadsBeingWritten;
  transport::writeNop(*descriptorConnection_, d, callbackWrapper_(done));
  for (const auto& p : op.message.payloads) {
    {
      std::unique_lock<std::mutex> lock(context_->statsMutex_);
      context_->stats_.payloadBytesWritten += p.length;
    }
    ++op.numPayloadsBeingWritten;
    descriptorConnection_->write(p.data, p.length, callbackWrapper_(done));
  }
}

void PipeImpl::readDescriptorReplyOfMessage(WriteOperation& op) {
  int64_t seq = op.sequenceNumber;
  transport::readNop<DescriptorReply>(
      *descriptorReplyConnection_, callbackWrapper_([seq](PipeImpl& impl, DescriptorReply reply) {
        WriteOperation* op = impl.writeOps_.findOperation(seq);
        if (!op) return;
        op->doneReadingDescriptorReply = true;
        if (!impl.error_) {
          size_t k = 0;
          for (size_t i = 0; i < op->targetDevices.size(); ++i) {
            if (!op->targetDevices[i].has_value() && k < reply.targetDevices.size())
              op->targetDevices[i] = reply.targetDevices[k++];
          }
          if (k != reply.targetDevices.size() ||
              std::any_of(op->targetDevices.begin(), op->targetDevices.end(),
                          [](const auto& d) { return !d.has_value(); })) {
            impl.setError(TPB_CREATE_ERROR(LogicError, "peer sent a descriptor reply of the wrong size"));
            return;
          }
        }
        impl.writeOps_.advanceOperation(*op);
      }));
}

void PipeImpl::sendTensorsOfMessage(WriteOperation& op) {
  int64_t seq = op.sequenceNumber;
  std::vector<std::pair<std::string, std::vector<channel::SendItem>>> groups;
  for (size_t i = 0; i < op.message.tensors.size(); ++i) {
    const auto& t = op.message.tensors[i];
    const Device& local = op.sourceDevices[i];
    const Device& remote = *op.targetDevices[i];
    auto it = channelForDevicePair_.find({local, remote});
    TPB_THROW_ASSERT_IF(it == channelForDevicePair_.end(),
                        "Could not find suitable channel for sending from " + local.toString() +
                            " to " + remote.toString());
    {
      std::unique_lock<std::mutex> lock(context_->statsMutex_);
      context_->stats_.tensorBytesSent += t.length;
    }
    channel::SendItem item;
    item.buffer = t.buffer;
    item.length = t.length;
    item.dtype = t.dtype;
    item.view = t.view;
    item.targetDevice = remote;
    ++op.numTensorsBeingSent;
    item.callback = callbackWrapper_([seq](PipeImpl& impl) {
      WriteOperation* op = impl.writeOps_.findOperation(seq);
      if (!op) return;
      --op->numTensorsBeingSent;
      impl.writeOps_.advanceOperation(*op);
    });
    auto g = std::find_if(groups.begin(), groups.end(), [&](const auto& p) { return p.first == it->second; });
    if (g == groups.end()) {
      groups.emplace_back(it->second, std::vector<channel::SendItem>());
      g = groups.end() - 1;
    }
    g->second.push_back(std::move(item));
  }
  for (auto& g : groups) channels_.at(g.first)->sendBatch(std::move(g.second));
}

// ---- errors ---------------------------------------------------------------------------------
void PipeImpl::close() {
  auto self = shared_from_this();
  context_->deferToLoop([self]() { self->setError(TPB_CREATE_ERROR(PipeClosedError)); });
}

void PipeImpl::setError(const Error& e) {
  if (error_ || !e) return;
  error_ = e;
  handleError();
}

void PipeImpl::handleError() {
  TPB_VLOG(1) << "Pipe " << id_ << " is handling error " << error_.what();
  auto self = shared_from_this();
  if (descriptorConnection_) descriptorConnection_->close();
  if (descriptorReplyConnection_) descriptorReplyConnection_->close();
  for (auto& c : channels_) c.second->close();
  for (auto& conns : channelReceivedConnections_)
    for (auto& c : conns.second)
      if (c) c->close();
  if (listener_) {
    for (auto& r : registrationIds_) listener_->unregisterConnectionRequest(r.second);
    for (auto& ids : channelRegistrationIds_)
      for (uint64_t id : ids.second)
        if (id != UINT64_MAX) listener_->unregisterConnectionRequest(id);
  }
  registrationIds_.clear();
  channelRegistrationIds_.clear();
  channelReceivedConnections_.clear();
  readOps_.advanceAllOperations();
  writeOps_.advanceAllOperations();
  context_->unenroll(*this);
}

// ---- public shell ---------------------------------------------------------------------------
Pipe::Pipe(ConstructorToken, std::shared_ptr<ContextImpl> context, std::string id,
           std::string remoteName, const std::string& url)
    : impl_(std::make_shared<PipeImpl>(std::move(context), std::move(id), std::move(remoteName), url)) {
  impl_->init();
}
Pipe::Pipe(ConstructorToken, std::shared_ptr<PipeImpl> impl) : impl_(std::move(impl)) {}
void Pipe::readDescriptor(read_descriptor_callback_fn fn) { impl_->readDescriptor(std::move(fn)); }
void Pipe::read(Allocation allocation, read_callback_fn fn) { impl_->read(std::move(allocation), std::move(fn)); }
void Pipe::write(Message message, write_callback_fn fn) { impl_->write(std::move(message), std::move(fn)); }
void Pipe::setTimeouts(PipeTimeouts timeouts) { impl_->setTimeouts(timeouts); }
const std::string& Pipe::getRemoteName() { return impl_->getRemoteName(); }
bool Pipe::channelSupportsLayouts(const Device& l, const Device& r) { return impl_->channelSupportsLayouts(l, r); }
void Pipe::close() { impl_->close(); }
Pipe::~Pipe() { close(); }

}  // namespace tpb
