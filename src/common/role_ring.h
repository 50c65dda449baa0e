// A byte ring that N parties chase each other around, with transactions. Party 0 (the producer)
// puts bytes in; party 1 works on what party 0 has released, party 2 on what party 1 has
// released, and so on; what the last party releases is free again for party 0. Two parties make
// the classic producer / consumer ring; three make a staging ring for an asynchronous device:
// the producer copies bytes in, the poster hands them to the device, the reclaimer frees them
// when the device reports that it is done with them.
//
// Every party works through a transaction: begin() says how many bytes lie ahead of it, span()
// gives them as at most two contiguous runs (the ring may wrap), advance() moves the private
// position, commit() publishes it (release) and cancel() forgets it. One transaction per party at
// a time, enforced by a flag in the header, so that two threads (or processes, when the memory is
// a shared segment) acting as the same party by mistake are caught instead of corrupting it.
//
// Same job as tensorpipe/common/ringbuffer.h:53-175 and ringbuffer_role.h:25-283 (N roles,
// startTx / commitTx / cancelTx, at most two spans per access); the layout and the interface are
// this library's own.
#pragma once

#include <atomic>
#include <cstdint>
#include <cstring>

#include "common/defs.h"

namespace tpb {

template <int N>
struct alignas(64) RoleRingHeader {
  static_assert(N >= 2 && N <= 8, "between two and eight parties");
  uint64_t size = 0;  // data bytes, a power of two
  uint64_t magic = 0;
  struct alignas(64) Party {
    std::atomic<uint64_t> cursor;   // free-running count of bytes this party has released
    std::atomic<uint32_t> inTransaction;
  };
  Party party[N];
};

template <int N>
class RoleRing {
 public:
  static constexpr uint64_t kMagic = 0x7470625f726f6c30ull + N;  // "tpb_rol0" + N
  using Header = RoleRingHeader<N>;

  RoleRing() = default;
  // `header` and `data` may live apart (a device writes only the data area); `dataBytes` must be
  // a power of two.
  RoleRing(Header* header, uint8_t* data, uint64_t dataBytes, bool init) : h_(header), data_(data) {
    if (init) {
      TPB_ARG_CHECK(dataBytes != 0 && (dataBytes & (dataBytes - 1)) == 0, "ring size must be a power of two");
      h_->size = dataBytes;
      h_->magic = kMagic;
      for (int i = 0; i < N; ++i) {
        h_->party[i].inTransaction.store(0, std::memory_order_relaxed);
        h_->party[i].cursor.store(0, std::memory_order_release);
      }
    }
  }
  bool valid() const { return h_ && h_->magic == kMagic && h_->size != 0 && (h_->size & (h_->size - 1)) == 0; }
  uint64_t capacity() const { return h_->size; }
  uint8_t* data() const { return data_; }
  // Bytes released by `party` so far (free-running).
  uint64_t released(int party) const { return h_->party[party].cursor.load(std::memory_order_acquire); }

  struct Span {
    uint8_t* ptr = nullptr;
    uint64_t length = 0;
  };

  class Transaction {
   public:
    Transaction() = default;
    Transaction(Transaction&& o) noexcept { *this = std::move(o); }
    Transaction& operator=(Transaction&& o) noexcept {
      if (this != &o) {
        cancel();
        ring_ = o.ring_;
        party_ = o.party_;
        start_ = o.start_;
        position_ = o.position_;
        limit_ = o.limit_;
        o.ring_ = nullptr;
      }
      return *this;
    }
    Transaction(const Transaction&) = delete;
    Transaction& operator=(const Transaction&) = delete;
    ~Transaction() { cancel(); }

    // False when another transaction of the same party was open: nothing can be done with this one.
    bool open() const { return ring_ != nullptr; }
    // Bytes still ahead of this party inside the transaction.
    uint64_t available() const { return limit_ - position_; }
    // Free-running stream position of the next byte this party would touch.
    uint64_t position() const { return position_; }
    // The next `n` bytes (n <= available()) as up to two runs; returns how many runs.
    int span(uint64_t n, Span out[2]) const {
      TPB_DCHECK(n <= available());
      if (n == 0) return 0;
      const uint64_t size = ring_->h_->size;
      const uint64_t off = position_ & (size - 1);
      const uint64_t first = n < size - off ? n : size - off;
      out[0] = Span{ring_->data_ + off, first};
      if (first == n) return 1;
      out[1] = Span{ring_->data_, n - first};
      return 2;
    }
    void advance(uint64_t n) {
      TPB_DCHECK(n <= available());
      position_ += n;
    }
    // Copy helpers over span() + advance(): all or nothing.
    bool write(const void* src, uint64_t n) {
      if (n > available()) return false;
      Span s[2];
      const int runs = span(n, s);
      const uint8_t* p = static_cast<const uint8_t*>(src);
      for (int i = 0; i < runs; ++i) {
        std::memcpy(s[i].ptr, p, s[i].length);
        p += s[i].length;
      }
      advance(n);
      return true;
    }
    bool read(void* dst, uint64_t n) {
      if (n > available()) return false;
      Span s[2];
      const int runs = span(n, s);
      uint8_t* p = static_cast<uint8_t*>(dst);
      for (int i = 0; i < runs; ++i) {
        std::memcpy(p, s[i].ptr, s[i].length);
        p += s[i].length;
      }
      advance(n);
      return true;
    }
    // Publish what was advanced and end the transaction.
    void commit() {
      if (!ring_) return;
      auto& me = ring_->h_->party[party_];
      me.cursor.store(position_, std::memory_order_release);
      me.inTransaction.store(0, std::memory_order_release);
      ring_ = nullptr;
    }
    // End the transaction as if nothing had been advanced.
    void cancel() {
      if (!ring_) return;
      ring_->h_->party[party_].inTransaction.store(0, std::memory_order_release);
      ring_ = nullptr;
    }

   private:
    friend class RoleRing;
    RoleRing* ring_ = nullptr;
    int party_ = 0;
    uint64_t start_ = 0, position_ = 0, limit_ = 0;
  };

  // Opens a transaction for `party`. The bytes ahead of it are those the party before it has
  // released and it has not (for party 0: the space the last party has freed).
  Transaction begin(int party) {
    TPB_DCHECK(party >= 0 && party < N);
    Transaction t;
    auto& me = h_->party[party];
    uint32_t expected = 0;
    if (!me.inTransaction.compare_exchange_strong(expected, 1, std::memory_order_acquire)) return t;
    t.ring_ = this;
    t.party_ = party;
    t.start_ = t.position_ = me.cursor.load(std::memory_order_relaxed);
    if (party == 0) t.limit_ = h_->party[N - 1].cursor.load(std::memory_order_acquire) + h_->size;
    else t.limit_ = h_->party[party - 1].cursor.load(std::memory_order_acquire);
    return t;
  }

  // How many bytes lie ahead of `party` right now (what begin() would offer).
  uint64_t ahead(int party) const {
    const uint64_t mine = h_->party[party].cursor.load(std::memory_order_relaxed);
    if (party == 0) return h_->party[N - 1].cursor.load(std::memory_order_acquire) + h_->size - mine;
    return h_->party[party - 1].cursor.load(std::memory_order_acquire) - mine;
  }

 private:
  Header* h_ = nullptr;
  uint8_t* data_ = nullptr;
};

}  // namespace tpb
