// Fixed pool of equally sized chunks carved out of caller-provided memory, handed out in request
// order. A request that cannot be served waits in a FIFO; a chunk comes back to the pool when the
// last copy of its handle dies, which immediately serves the oldest waiter. close() fails every
// waiter (and every later request) with AllocatorClosedError. This is the staging-slot
// back-pressure primitive of the reference (tensorpipe/common/allocator.h:28-56,
// allocator.cc:16-79). Not thread-safe by itself: use it from one loop.
#pragma once

#include <cstddef>
#include <cstdint>
#include <deque>
#include <functional>
#include <memory>
#include <vector>

#include <tpb/error.h>

namespace tpb {

class Allocator {
 public:
  // The chunk is released when the shared_ptr (and all its copies) are gone.
  using TChunk = std::shared_ptr<uint8_t>;
  using TAllocCallback = std::function<void(const Error&, TChunk)>;

  Allocator(uint8_t* data, size_t numChunks, size_t chunkSize)
      : state_(std::make_shared<State>()) {
    state_->data = data;
    state_->chunkSize = chunkSize;
    for (size_t i = 0; i < numChunks; ++i) state_->available.push_back(numChunks - 1 - i);
    state_->numChunks = numChunks;
  }
  ~Allocator() { close(); }
  Allocator(const Allocator&) = delete;
  Allocator& operator=(const Allocator&) = delete;

  void alloc(size_t size, TAllocCallback callback) {
    if (size > state_->chunkSize) {
      callback(TPB_CREATE_ERROR(LogicError, "allocation larger than the pool's chunk size"), nullptr);
      return;
    }
    state_->pending.push_back(std::move(callback));
    State::pump(state_);
  }
  size_t getChunkLength() const { return state_->chunkSize; }
  size_t numAvailable() const { return state_->available.size(); }
  size_t numPending() const { return state_->pending.size(); }

  void close() {
    if (state_->closed) return;
    state_->closed = true;
    State::pump(state_);
  }

 private:
  struct State {
    uint8_t* data = nullptr;
    size_t chunkSize = 0, numChunks = 0;
    std::vector<size_t> available;  // stack of free chunk indices
    std::deque<TAllocCallback> pending;
    bool closed = false;

    static void pump(const std::shared_ptr<State>& st) {
      while (!st->pending.empty()) {
        if (st->closed) {
          auto cb = std::move(st->pending.front());
          st->pending.pop_front();
          cb(TPB_CREATE_ERROR(AllocatorClosedError), nullptr);
          continue;
        }
        if (st->available.empty()) return;
        const size_t idx = st->available.back();
        st->available.pop_back();
        auto cb = std::move(st->pending.front());
        st->pending.pop_front();
        // The deleter keeps the pool's state alive, so a chunk may outlive the Allocator object.
        TChunk chunk(st->data + idx * st->chunkSize, [st, idx](uint8_t*) {
          st->available.push_back(idx);
          pump(st);
        });
        cb(Error::kSuccess, std::move(chunk));
      }
    }
  };
  std::shared_ptr<State> state_;
};

}  // namespace tpb
