// Messages through an open pipe.
//
// On the wire (what a reference peer expects, tensorpipe/core/nop_types.h:66-78): per message one
// Descriptor frame followed by one frame per payload on the first connection; a DescriptorReply
// on the second connection, from the receiver, for messages whose sender left a target device
// open. Tensors travel on channels, the k-th send of a channel meeting the k-th receive.
//
// Each direction is a queue of records with three cursors that only move forward:
//
//   outbound   announce (frames written)  ->  dispatch (tensors with the channels)  ->  retire
//   inbound    post (descriptor read armed) -> offered to the user -> receiving     ->  retire
//
// A record carries a count of completions it is still owed; it retires when the count is zero,
// it has been through its last stage, and it is at the front of its queue. That is all the
// ordering there is: callbacks of one kind fire in the order their operations were issued.
#include <algorithm>

#include "common/timer.h"
#include "common/trace.h"
#include "core/core.h"
#include "transport/nop_io.h"

namespace tpb {
namespace core {

namespace {

// Hands the tensors of one message to the channels that carry them, one batch per channel, in
// message order within a batch.
template <typename TItem>
class Batches {
 public:
  std::vector<TItem>& of(channel::Channel* ch) {
    for (auto& b : batches_)
      if (b.first == ch) return b.second;
    batches_.emplace_back(ch, std::vector<TItem>());
    return batches_.back().second;
  }
  template <typename F>
  void forEach(F&& fn) {
    for (auto& b : batches_) fn(b.first, std::move(b.second));
  }

 private:
  std::vector<std::pair<channel::Channel*, std::vector<TItem>>> batches_;
};

void requireFit(const Descriptor& d, const Allocation& a) {
  TPB_THROW_ASSERT_IF(a.payloads.size() != d.payloads.size(),
                      "the allocation has " + std::to_string(a.payloads.size()) + " payloads, the message " +
                          std::to_string(d.payloads.size()));
  TPB_THROW_ASSERT_IF(a.tensors.size() != d.tensors.size(),
                      "the allocation has " + std::to_string(a.tensors.size()) + " tensors, the message " +
                          std::to_string(d.tensors.size()));
  for (size_t i = 0; i < a.tensors.size(); ++i) {
    const auto& wanted = d.tensors[i].targetDevice;
    TPB_THROW_ASSERT_IF(wanted.has_value() && !(a.tensors[i].buffer.device() == *wanted),
                        "tensor " + std::to_string(i) + " must be received on " + wanted->toString());
  }
}

}  // namespace

PipeCore::Outbound* PipeCore::outbound(uint64_t seq) {
  if (outbound_.empty() || seq < outbound_.front().seq) return nullptr;
  const uint64_t at = seq - outbound_.front().seq;
  return at < outbound_.size() ? &outbound_[at] : nullptr;
}

PipeCore::Inbound* PipeCore::inbound(uint64_t seq) {
  if (inbound_.empty() || seq < inbound_.front().seq) return nullptr;
  const uint64_t at = seq - inbound_.front().seq;
  return at < inbound_.size() ? &inbound_[at] : nullptr;
}

// ---- writing --------------------------------------------------------------------------------
void PipeCore::write(Message message, Pipe::write_callback_fn fn) {
  auto self = shared_from_this();
  context_->defer([self, message = std::move(message), fn = std::move(fn)]() mutable {
    Outbound m;
    m.seq = self->outboundNext_++;
    m.message = std::move(message);
    m.done = std::move(fn);
    m.targets.reserve(m.message.tensors.size());
    for (const auto& t : m.message.tensors) {
      if (t.targetDevice) m.targets.push_back(*t.targetDevice);
      else {
        m.targets.emplace_back();
        m.awaitingTargets = true;
      }
    }
    trace::instant("pipe.write", m.seq);
    TPB_VLOG(2) << "Pipe " << self->id_ << " queues message #" << m.seq << " (" << m.message.payloads.size()
                << " payloads, " << m.message.tensors.size() << " tensors)";
    const uint64_t seq = m.seq;
    self->outbound_.push_back(std::move(m));
    if (self->timeouts_.write.count() > 0) self->armDeadline(Deadline::kWrite, seq, self->timeouts_.write);
    // A tensor between devices that no channel connects surfaces here: it fails the pipe and the
    // write reports it.
    self->guarded([&]() { self->pumpOutbound(); });
  });
}

void PipeCore::pumpOutbound() {
  if (phase_ == Phase::kOpen && !error_) {
    while (!error_ && announceCursor_ < outboundNext_) announce(*outbound(announceCursor_++));
    while (!error_ && dispatchCursor_ < announceCursor_) {
      Outbound& m = *outbound(dispatchCursor_);
      if (m.awaitingTargets) break;  // later messages queue behind: channels pair sends by order
      ++dispatchCursor_;
      dispatch(m);
    }
  }
  while (!outbound_.empty()) {
    Outbound& front = outbound_.front();
    if (front.outstanding != 0 || !(front.dispatched || error_)) break;
    auto done = std::move(front.done);
    const uint64_t seq = front.seq;
    outbound_.pop_front();
    if (!error_) context_->counters.messagesWritten.fetch_add(1, std::memory_order_relaxed);
    trace::instant("pipe.write.done", seq);
    TPB_VLOG(2) << "Pipe " << id_ << " reports message #" << seq << " written";
    done(error_);
  }
}

void PipeCore::announce(Outbound& m) {
  auto self = shared_from_this();
  const uint64_t seq = m.seq;
  Descriptor d;
  d.metadata = m.message.metadata;
  d.payloads.reserve(m.message.payloads.size());
  for (const auto& p : m.message.payloads) d.payloads.push_back({p.length, p.metadata});
  d.tensors.reserve(m.message.tensors.size());
  for (const auto& t : m.message.tensors) {
    Descriptor::Tensor dt;
    dt.length = t.length;
    dt.sourceDevice = t.buffer.device();
    dt.targetDevice = t.targetDevice;
    dt.metadata = t.metadata;
    d.tensors.push_back(std::move(dt));
  }
  auto frameWritten = onLoopOf(self, [self, seq]() { self->settleOutbound(seq); });
  ++m.outstanding;
  transport::writeNop(*wire_, d, frameWritten);
  uint64_t payloadBytes = 0;
  for (const auto& p : m.message.payloads) {
    ++m.outstanding;
    payloadBytes += p.length;
    wire_->write(p.data, p.length, frameWritten);
  }
  context_->counters.payloadBytesWritten.fetch_add(payloadBytes, std::memory_order_relaxed);
  m.announced = true;
  trace::instant("pipe.announced", seq);
  if (m.awaitingTargets) awaitTargets(m);
}

void PipeCore::awaitTargets(Outbound& m) {
  auto self = shared_from_this();
  const uint64_t seq = m.seq;
  ++m.outstanding;
  transport::readNop<DescriptorReply>(*replyWire_, onLoopOf(self, [self, seq](DescriptorReply reply) {
    Outbound* m = self->outbound(seq);
    if (!m) return;
    --m->outstanding;
    if (!self->error_) {
      size_t next = 0;
      for (size_t i = 0; i < m->targets.size(); ++i) {
        if (m->message.tensors[i].targetDevice) continue;
        if (next == reply.targetDevices.size()) {
          next = SIZE_MAX;
          break;
        }
        m->targets[i] = reply.targetDevices[next++];
      }
      if (next != reply.targetDevices.size())
        return self->fail(TPB_CREATE_ERROR(LogicError, "the peer's descriptor reply names the wrong number of devices"));
      m->awaitingTargets = false;
    }
    self->pumpOutbound();
  }));
}

void PipeCore::dispatch(Outbound& m) {
  auto self = shared_from_this();
  const uint64_t seq = m.seq;
  // Every tensor needs a route before any of them is handed over: a record only counts
  // completions that will certainly come back.
  std::vector<channel::Channel*> carriers(m.message.tensors.size());
  for (size_t i = 0; i < m.message.tensors.size(); ++i) {
    const Device local = m.message.tensors[i].buffer.device();
    carriers[i] = channelFor(local, m.targets[i]);
    TPB_THROW_ASSERT_IF(carriers[i] == nullptr, "no registered channel moves tensors from " + local.toString() +
                                                    " to " + m.targets[i].toString() + " of this peer");
  }
  Batches<channel::SendItem> batches;
  uint64_t bytes = 0;
  for (size_t i = 0; i < m.message.tensors.size(); ++i) {
    const auto& t = m.message.tensors[i];
    channel::Channel* ch = carriers[i];
    channel::SendItem item;
    item.buffer = t.buffer;
    item.length = t.length;
    item.dtype = t.dtype;
    item.view = t.view;
    item.targetDevice = m.targets[i];
    item.callback = onLoopOf(self, [self, seq]() { self->settleOutbound(seq); });
    ++m.outstanding;
    bytes += t.length;
    batches.of(ch).push_back(std::move(item));
  }
  m.dispatched = true;
  context_->counters.tensorBytesSent.fetch_add(bytes, std::memory_order_relaxed);
  batches.forEach([](channel::Channel* ch, std::vector<channel::SendItem> items) { ch->sendBatch(std::move(items)); });
}

void PipeCore::settleOutbound(uint64_t seq) {
  if (Outbound* m = outbound(seq)) {
    --m->outstanding;
    pumpOutbound();
  }
}

// ---- reading --------------------------------------------------------------------------------
void PipeCore::readDescriptor(Pipe::read_descriptor_callback_fn fn) {
  auto self = shared_from_this();
  context_->defer([self, fn = std::move(fn)]() mutable {
    Inbound m;
    m.seq = self->inboundNext_++;
    m.offer = std::move(fn);
    trace::instant("pipe.readDescriptor", m.seq);
    const uint64_t seq = m.seq;
    self->inbound_.push_back(std::move(m));
    if (self->timeouts_.descriptor.count() > 0) self->armDeadline(Deadline::kDescriptor, seq, self->timeouts_.descriptor);
    self->guarded([&]() { self->pumpInbound(); });
  });
}

void PipeCore::pumpInbound() {
  // Arm the next descriptor read. The peer writes descriptor, payloads, descriptor, ...: the read
  // for the next descriptor may only be queued behind the payload reads of the message before it,
  // i.e. once that message is past the user's read() call.
  if (phase_ == Phase::kOpen && !error_ && postCursor_ < inboundNext_) {
    Inbound* prev = postCursor_ > 0 ? inbound(postCursor_ - 1) : nullptr;
    if (prev == nullptr || prev->stage == Inbound::kReceiving) postDescriptorRead(*inbound(postCursor_++));
  }
  while (!inbound_.empty()) {
    Inbound& front = inbound_.front();
    if (front.stage == Inbound::kReceiving || (front.stage == Inbound::kAnswered && error_)) {
      if (front.outstanding != 0) break;
      auto done = std::move(front.done);
      const uint64_t seq = front.seq;
      inbound_.pop_front();
      if (!error_) context_->counters.messagesRead.fetch_add(1, std::memory_order_relaxed);
      trace::instant("pipe.read.done", seq);
      TPB_VLOG(2) << "Pipe " << id_ << " reports message #" << seq << " read";
      done(error_);
      continue;
    }
    if (!error_) break;
    // After a failure. A posted descriptor read is still owed by the connection; an armed
    // readDescriptor that never reached the wire reports the failure now; a descriptor the user
    // holds without having called read() has nothing left to report.
    if (front.stage == Inbound::kDescriptorPosted) break;
    auto offer = std::move(front.offer);
    const bool armedOnly = front.stage == Inbound::kArmed;
    if (static_cast<int64_t>(front.seq) == offered_) offered_ = -1;
    if (postCursor_ <= front.seq) postCursor_ = front.seq + 1;
    inbound_.pop_front();
    if (armedOnly) offer(error_, Descriptor());
  }
}

void PipeCore::postDescriptorRead(Inbound& m) {
  auto self = shared_from_this();
  const uint64_t seq = m.seq;
  m.stage = Inbound::kDescriptorPosted;
  transport::readNop<Descriptor>(*wire_, onLoopOf(self, [self, seq](Descriptor d) {
    Inbound* m = self->inbound(seq);
    if (!m) return;
    auto offer = std::move(m->offer);
    m->offer = nullptr;
    if (self->error_) {
      // Leaves the queue through the failure path of pumpInbound, as a record with nothing to say.
      m->stage = Inbound::kOffered;
      offer(self->error_, Descriptor());
      self->pumpInbound();
      return;
    }
    trace::instant("pipe.descriptor", seq);
    m->descriptor = std::move(d);
    m->stage = Inbound::kOffered;
    self->offered_ = static_cast<int64_t>(seq);
    offer(Error::kSuccess, m->descriptor);
  }));
}

void PipeCore::read(Allocation allocation, Pipe::read_callback_fn fn) {
  // Runs to the point where the call is known to be legitimate before returning, so that a
  // misuse throws in the caller's thread.
  auto self = shared_from_this();
  context_->runSync([&]() {
    Inbound* m = offered_ >= 0 ? inbound(static_cast<uint64_t>(offered_)) : nullptr;
    if (m == nullptr) {
      if (error_) {
        const Error why = error_;
        context_->defer([fn = std::move(fn), why]() { fn(why); });
        return;
      }
      TPB_THROW_ASSERT_IF(true, "Pipe::read needs a message whose descriptor was delivered and not yet read");
    }
    requireFit(m->descriptor, allocation);
    offered_ = -1;
    m->stage = Inbound::kAnswered;
    m->allocation = std::move(allocation);
    m->done = std::move(fn);
    const uint64_t seq = m->seq;
    trace::instant("pipe.read", seq);
    if (timeouts_.read.count() > 0) armDeadline(Deadline::kRead, seq, timeouts_.read);
    // The rest happens in a turn of its own: no callback ever runs inside read().
    context_->defer([self, seq]() {
      self->guarded([&]() {
        if (Inbound* m = self->inbound(seq)) self->beginReceiving(*m);
      });
    });
  });
}

void PipeCore::beginReceiving(Inbound& m) {
  auto self = shared_from_this();
  const uint64_t seq = m.seq;
  if (error_) return pumpInbound();  // retires as an answered record carrying the error
  // Every tensor needs a route before anything is posted: a record only counts completions that
  // will certainly come back.
  std::vector<std::pair<channel::Channel*, const std::string*>> carriers(m.descriptor.tensors.size());
  for (size_t i = 0; i < m.descriptor.tensors.size(); ++i) {
    const Device local = m.allocation.tensors[i].buffer.device();
    const Device& source = m.descriptor.tensors[i].sourceDevice;
    carriers[i].first = channelFor(local, source, &carriers[i].second);
    TPB_THROW_ASSERT_IF(carriers[i].first == nullptr, "no registered channel moves tensors from " + source.toString() +
                                                          " of this peer to " + local.toString());
  }
  m.stage = Inbound::kReceiving;

  uint64_t payloadBytes = 0;
  for (size_t i = 0; i < m.allocation.payloads.size(); ++i) {
    const size_t length = m.descriptor.payloads[i].length;
    payloadBytes += length;
    ++m.outstanding;
    wire_->read(m.allocation.payloads[i].data, length,
                onLoopOf(self, [self, seq](const void*, size_t) { self->settleInbound(seq); }));
  }
  context_->counters.payloadBytesRead.fetch_add(payloadBytes, std::memory_order_relaxed);

  // Tell the sender where the tensors it left open are going.
  DescriptorReply reply;
  bool owed = false;
  for (size_t i = 0; i < m.descriptor.tensors.size(); ++i) {
    if (m.descriptor.tensors[i].targetDevice) continue;
    owed = true;
    reply.targetDevices.push_back(m.allocation.tensors[i].buffer.device());
  }
  if (owed) transport::writeNop(*replyWire_, reply, onLoopOf(self, [self]() {}));

  Batches<channel::RecvItem> batches;
  uint64_t bytes = 0;
  for (size_t i = 0; i < m.descriptor.tensors.size(); ++i) {
    const auto& announced = m.descriptor.tensors[i];
    const auto& given = m.allocation.tensors[i];
    channel::Channel* ch = carriers[i].first;
    channel::RecvItem item;
    item.buffer = given.buffer;
    item.length = announced.length;
    item.castTo = given.castTo;
    item.srcDtype = given.sourceDtype;
    item.sourceDevice = announced.sourceDevice;
    item.callback = onLoopOf(self, [self, seq]() { self->settleInbound(seq); });
    ++m.outstanding;
    bytes += announced.length;
    batches.of(ch).push_back(std::move(item));
  }
  context_->counters.tensorBytesReceived.fetch_add(bytes, std::memory_order_relaxed);
  if (!carriers.empty()) {
    std::unique_lock<std::mutex> lock(context_->counters.perChannelMutex);
    for (size_t i = 0; i < carriers.size(); ++i)
      context_->counters.bytesPerChannel[*carriers[i].second] += m.descriptor.tensors[i].length;
  }
  batches.forEach([](channel::Channel* ch, std::vector<channel::RecvItem> items) { ch->recvBatch(std::move(items)); });
  pumpInbound();
}

void PipeCore::settleInbound(uint64_t seq) {
  if (Inbound* m = inbound(seq)) {
    --m->outstanding;
    pumpInbound();
  }
}

// ---- deadlines ------------------------------------------------------------------------------
void PipeCore::setTimeouts(PipeTimeouts timeouts) {
  auto self = shared_from_this();
  context_->defer([self, timeouts]() { self->timeouts_ = timeouts; });
}

void PipeCore::armDeadline(Deadline kind, uint64_t seq, std::chrono::milliseconds after) {
  std::weak_ptr<PipeCore> weak = shared_from_this();
  TimerThread::get().schedule(after, [weak, kind, seq]() {
    auto self = weak.lock();
    if (!self) return;
    self->context_->defer([self, kind, seq]() {
      if (self->error_) return;
      bool late;
      if (kind == Deadline::kWrite) {
        late = self->outbound(seq) != nullptr;
      } else {
        Inbound* m = self->inbound(seq);
        // A descriptor deadline is met once the user holds the descriptor.
        late = m != nullptr && (kind == Deadline::kRead || m->stage < Inbound::kOffered);
      }
      if (!late) return;
      TPB_VLOG(1) << "Pipe " << self->id_ << " gives up on "
                  << (kind == Deadline::kWrite ? "write" : kind == Deadline::kRead ? "read" : "readDescriptor") << " #"
                  << seq << ": deadline passed";
      self->fail(TPB_CREATE_ERROR(TimeoutError));
    });
  });
}

}  // namespace core
}  // namespace tpb
