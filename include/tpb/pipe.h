// A pipe: one end of a bidirectional, ordered message conduit between two contexts.
// Counterpart of tensorpipe/core/pipe.h:39-96. All callbacks are one-shot, are always called
// (with an error after close), run on the owning context's single callback thread, and for a
// given pipe fire in the order the operations were issued.
#pragma once

#include <chrono>
#include <functional>
#include <memory>
#include <string>

#include <tpb/error.h>
#include <tpb/message.h>

namespace tpb {

namespace core {
class ContextCore;
class ListenerCore;
class PipeCore;
}  // namespace core

// Optional deadlines (not in the reference, where a silent peer hangs an operation forever).
// Zero means "wait forever". When a deadline passes the pipe fails with TimeoutError: the late
// operation and everything queued behind it get that error, as after any other pipe error.
struct PipeTimeouts {
  std::chrono::milliseconds write{0};       // write() call -> its callback
  std::chrono::milliseconds read{0};        // read() call -> its callback
  std::chrono::milliseconds descriptor{0};  // readDescriptor() call -> its callback (an idle limit)
};

class Pipe final {
  // Only the context and the listener create pipes.
  enum ConstructorToken { kToken };

 public:
  Pipe(ConstructorToken, std::shared_ptr<core::PipeCore> impl);

  using read_descriptor_callback_fn = std::function<void(const Error&, Descriptor)>;
  using read_callback_fn = std::function<void(const Error&)>;
  using write_callback_fn = std::function<void(const Error&)>;

  // Ask for the descriptor of the next incoming message. Not arming this is how a receiver
  // exerts backpressure.
  void readDescriptor(read_descriptor_callback_fn fn);
  // Provide memory for the message whose descriptor was just delivered and receive it.
  // Throws if no message is waiting for an allocation or if the allocation does not fit.
  void read(Allocation allocation, read_callback_fn fn);
  // Send a message. The memory it points to must stay valid until the callback fires.
  void write(Message message, write_callback_fn fn);

  // Applies to operations issued after the call.
  void setTimeouts(PipeTimeouts timeouts);

  // Name the peer gave to its context (or the name passed to connect()).
  const std::string& getRemoteName();

  // Name of the transport the two ends settled on for descriptors and payloads ("uv", "shm",
  // ...), once the pipe is established; before that, the one the handshake travels over.
  std::string transportName();

  // True when the channel selected for (localDevice -> remoteDevice) tensors understands
  // strided views and receiver-requested casts. Valid once the pipe is established.
  bool channelSupportsLayouts(const Device& local, const Device& remote);

  void close();
  ~Pipe();

 private:
  std::shared_ptr<core::PipeCore> impl_;
  friend class core::ContextCore;
  friend class core::ListenerCore;
};

}  // namespace tpb
