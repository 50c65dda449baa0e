// The backends a context knows, best first. One instance holds the transports, another the
// channels. Registration rules (tensorpipe/core/context_impl.cc:66-110 states them for the
// reference): a higher priority wins, a name or a priority may be used once, and a backend that
// says it cannot work on this machine is dropped without complaint.
#pragma once

#include <algorithm>
#include <memory>
#include <string>
#include <vector>

#include "common/defs.h"

namespace tpb {
namespace core {

template <typename TBackend>
class Backends {
 public:
  struct Slot {
    int64_t priority;
    std::string name;
    std::shared_ptr<TBackend> backend;
  };

  explicit Backends(const char* kind) : kind_(kind) {}

  // Returns false when the backend was skipped because it is not viable.
  bool add(int64_t priority, std::string name, std::shared_ptr<TBackend> backend) {
    TPB_THROW_ASSERT_IF(name.empty(), std::string(kind_) + " needs a name");
    TPB_THROW_ASSERT_IF(backend == nullptr, std::string(kind_) + " " + name + " is null");
    for (const Slot& s : slots_) {
      TPB_THROW_ASSERT_IF(s.name == name, std::string(kind_) + " " + name + " is registered twice");
      TPB_THROW_ASSERT_IF(s.priority == priority, std::string(kind_) + " " + name + " has the priority (" +
                                                      std::to_string(priority) + ") of " + s.name);
    }
    if (!backend->isViable()) return false;
    Slot slot{priority, std::move(name), std::move(backend)};
    auto at = std::find_if(slots_.begin(), slots_.end(), [&](const Slot& s) { return s.priority < slot.priority; });
    slots_.insert(at, std::move(slot));
    return true;
  }

  // nullptr when nothing of that name is registered.
  std::shared_ptr<TBackend> find(const std::string& name) const {
    for (const Slot& s : slots_)
      if (s.name == name) return s.backend;
    return nullptr;
  }
  std::shared_ptr<TBackend> require(const std::string& name) const {
    auto b = find(name);
    TPB_THROW_ASSERT_IF(b == nullptr, "no " + std::string(kind_) + " named " + name + " is registered");
    return b;
  }

  // Highest priority first.
  const std::vector<Slot>& bestFirst() const { return slots_; }

 private:
  const char* kind_;
  std::vector<Slot> slots_;
};

}  // namespace core
}  // namespace tpb
