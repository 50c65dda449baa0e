// The context: registry of transports and channels, factory of listeners and pipes, and owner of
// the single callback "thread" (an on-demand loop borrowed from whichever thread triggers work).
// Counterpart of tensorpipe/core/context.h:26-94.
#pragma once

#include <map>
#include <memory>
#include <string>
#include <vector>

#include <tpb/channel.h>
#include <tpb/listener.h>
#include <tpb/pipe.h>
#include <tpb/transport.h>

namespace tpb {

namespace core {
class ContextCore;
}

class ContextOptions {
 public:
  // Human-readable name used in log lines and told to peers.
  ContextOptions&& name(std::string name) && {
    name_ = std::move(name);
    return std::move(*this);
  }
  std::string name_;
};

class PipeOptions {
 public:
  ContextOptions dummy_;
  PipeOptions&& remoteName(std::string remoteName) && {
    remoteName_ = std::move(remoteName);
    return std::move(*this);
  }
  std::string remoteName_;
};

// Counters kept by a context (not in the reference; exported to Python as Context.stats()).
struct ContextStats {
  uint64_t messagesWritten = 0, messagesRead = 0;
  uint64_t payloadBytesWritten = 0, payloadBytesRead = 0;
  uint64_t tensorBytesSent = 0, tensorBytesReceived = 0;
  uint64_t pipesCreated = 0;
  std::map<std::string, uint64_t> bytesPerChannel;
};

class Context final {
 public:
  explicit Context(ContextOptions opts = ContextOptions());

  // Higher priority wins. Names and priorities must be unique. A backend that is not viable on
  // this machine is silently skipped.
  void registerTransport(int64_t priority, std::string name, std::shared_ptr<transport::Context> t);
  void registerChannel(int64_t priority, std::string name, std::shared_ptr<channel::Context> c);

  std::shared_ptr<Listener> listen(const std::vector<std::string>& urls);
  std::shared_ptr<Pipe> connect(const std::string& url, PipeOptions opts = PipeOptions());

  ContextStats stats() const;

  // Start closing everything; every pending callback fires with an error.
  void close();
  // close() and wait for every backend thread. The only blocking call of the API.
  void join();

  ~Context();

 private:
  std::shared_ptr<core::ContextCore> impl_;
};

}  // namespace tpb
