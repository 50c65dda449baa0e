// A listener accepts incoming pipes on the addresses it was bound to (one per transport).
// Counterpart of tensorpipe/core/listener.h:36-94.
#pragma once

#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include <tpb/error.h>
#include <tpb/pipe.h>

namespace tpb {

namespace core {
class ContextCore;
class ListenerCore;
}  // namespace core

class Listener final {
  enum ConstructorToken { kToken };

 public:
  // Only a context creates listeners.
  Listener(ConstructorToken, std::shared_ptr<core::ListenerCore> impl);

  using accept_callback_fn = std::function<void(const Error&, std::shared_ptr<Pipe>)>;
  // One-shot: re-arm to accept the next pipe. Unclaimed pipes queue up.
  void accept(accept_callback_fn fn);

  // transport name -> address the listener is actually bound to (ports resolved).
  const std::map<std::string, std::string>& addresses() const;
  const std::string& address(const std::string& transport) const;
  // "<transport>://<address>"
  std::string url(const std::string& transport) const;

  void close();
  ~Listener();

 private:
  std::shared_ptr<core::ListenerCore> impl_;
  friend class core::ContextCore;
};

}  // namespace tpb
