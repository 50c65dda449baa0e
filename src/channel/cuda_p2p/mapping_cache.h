// Process-wide cache of peer allocations opened through CUDA IPC, keyed by (handle, accessing
// device). Declared here so that its bookkeeping (keys, idle eviction, pinning) can be tested on
// a machine without a GPU by swapping the two driver calls for counters.
#pragma once

#include <array>
#include <atomic>
#include <cstdint>
#include <functional>
#include <map>
#include <mutex>
#include <string>

namespace tpb {
namespace channel {
namespace cuda_p2p {

class MappingCache {
 public:
  using Handle = std::array<uint8_t, 64>;
  using Opener = std::function<void*(const Handle&, int device, size_t* size)>;
  using Closer = std::function<void(void* base, int device)>;

  static MappingCache& get();
  MappingCache();

  // Local address of the peer allocation's base as seen from `device` (which must be current),
  // opening it on first use; `size` receives the size of the allocation when known (0 if not).
  // A pinned mapping is never closed by the cache (channel arenas, whose addresses are kept).
  // Callers that keep an address must call this again at least every kRefreshNs while they use it,
  // and whenever generation() has changed.
  void* open(const Handle& handle, int device, size_t* size, std::string* err, bool pin = false);
  // Changes whenever a mapping was closed: addresses obtained earlier must be looked up again.
  uint64_t generation() const { return generation_.load(std::memory_order_acquire); }
  static constexpr uint64_t kRefreshNs = 100'000'000ull;

  // For tests.
  void setBackendForTesting(Opener opener, Closer closer);
  void setLimits(size_t maxMappings, uint64_t idleNs);
  size_t size();
  uint64_t closedCount();

 private:
  using Key = std::pair<Handle, int>;
  struct Entry {
    void* base;
    size_t size;
    uint64_t lastUseNs;
    bool pinned;
  };
  void evictIdle();
  std::mutex m_;
  std::map<Key, Entry> map_;
  size_t limit_;
  uint64_t idleNs_ = 2'000'000'000ull;
  std::atomic<uint64_t> generation_{0};
  uint64_t closed_ = 0;
  Opener opener_;
  Closer closer_;
};

}  // namespace cuda_p2p
}  // namespace channel
}  // namespace tpb
