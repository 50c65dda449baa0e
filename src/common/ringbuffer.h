// Single-producer / single-consumer byte ring over caller-provided memory (typically a shared
// memory segment mapped in two processes). The header holds two free-running 64-bit cursors on
// separate cache lines; the data area is a power of two so positions wrap with a mask. The
// producer publishes with a release store of `tail` after copying bytes in, the consumer
// acquires `tail` before copying out and releases `head` after, which is all the ordering two
// processes need (same reasoning as tensorpipe/common/ringbuffer.h:83-117, reduced to the two
// roles the shm transport uses).
#pragma once

#include <atomic>
#include <cstdint>
#include <cstring>

namespace tpb {

struct alignas(64) RingHeader {
  uint64_t size;  // data bytes, power of two
  uint64_t magic;
  // Set by a producer that found the ring too full to go on; a consumer that frees space while
  // it is set owes the producer a wake-up (how it delivers it is the transport's business).
  std::atomic<uint32_t> producerStalled;
  alignas(64) std::atomic<uint64_t> head;  // consumer cursor
  alignas(64) std::atomic<uint64_t> tail;  // producer cursor
};
static_assert(sizeof(RingHeader) == 192, "ring header layout is part of the shm protocol");

class Ring {
 public:
  static constexpr uint64_t kMagic = 0x7470625f72696e32ull;  // "tpb_rin2"
  Ring() = default;
  Ring(void* mem, uint64_t dataBytes, bool init) : h_(static_cast<RingHeader*>(mem)) {
    data_ = reinterpret_cast<uint8_t*>(h_ + 1);
    if (init) {
      h_->size = dataBytes;
      h_->magic = kMagic;
      h_->producerStalled.store(0, std::memory_order_relaxed);
      h_->head.store(0, std::memory_order_relaxed);
      h_->tail.store(0, std::memory_order_release);
    }
  }
  static size_t bytesNeeded(uint64_t dataBytes) { return sizeof(RingHeader) + dataBytes; }
  bool valid(size_t segmentBytes) const {
    return h_ && h_->magic == kMagic && (h_->size & (h_->size - 1)) == 0 &&
        sizeof(RingHeader) + h_->size <= segmentBytes;
  }
  uint64_t capacity() const { return h_->size; }

  // Producer side.
  uint64_t freeBytes() const {
    return h_->size - (h_->tail.load(std::memory_order_relaxed) - h_->head.load(std::memory_order_acquire));
  }
  // Copies up to n bytes in; returns how many were accepted.
  uint64_t write(const void* src, uint64_t n) {
    uint64_t tail = h_->tail.load(std::memory_order_relaxed);
    uint64_t space = h_->size - (tail - h_->head.load(std::memory_order_acquire));
    if (n > space) n = space;
    if (n == 0) return 0;
    uint64_t off = tail & (h_->size - 1);
    uint64_t first = n < h_->size - off ? n : h_->size - off;
    std::memcpy(data_ + off, src, first);
    if (n > first) std::memcpy(data_, static_cast<const uint8_t*>(src) + first, n - first);
    h_->tail.store(tail + n, std::memory_order_release);
    return n;
  }
  // Producer: announce (or withdraw) that it waits for space. After announcing, look at
  // freeBytes() once more before going idle: the consumer may have freed space in between.
  void setProducerStalled(bool stalled) {
    h_->producerStalled.store(stalled ? 1 : 0, std::memory_order_seq_cst);
    std::atomic_thread_fence(std::memory_order_seq_cst);
  }
  // Consumer: call after read() freed space; true means the producer must be woken.
  bool producerStalled() const {
    std::atomic_thread_fence(std::memory_order_seq_cst);
    return h_->producerStalled.load(std::memory_order_seq_cst) != 0;
  }

  // Consumer side.
  uint64_t usedBytes() const {
    return h_->tail.load(std::memory_order_acquire) - h_->head.load(std::memory_order_relaxed);
  }
  uint64_t read(void* dst, uint64_t n) {
    uint64_t head = h_->head.load(std::memory_order_relaxed);
    uint64_t avail = h_->tail.load(std::memory_order_acquire) - head;
    if (n > avail) n = avail;
    if (n == 0) return 0;
    uint64_t off = head & (h_->size - 1);
    uint64_t first = n < h_->size - off ? n : h_->size - off;
    std::memcpy(dst, data_ + off, first);
    if (n > first) std::memcpy(static_cast<uint8_t*>(dst) + first, data_, n - first);
    h_->head.store(head + n, std::memory_order_release);
    return n;
  }

 private:
  RingHeader* h_ = nullptr;
  uint8_t* data_ = nullptr;
};

}  // namespace tpb
