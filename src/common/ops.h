// Ordered operation queue: the ordering backbone of the pipe and of every channel.
// Each operation has a sequence number and a state (an enum whose first value is the initial
// state and whose last value is FINISHED). An operation may move forward one transition at a
// time, a transition may be gated on how far the *previous* operation got, advancing one
// operation retries its successors, and finished operations retire from the front only.
// Counterpart of tensorpipe/common/state_machine.h:18-146, expressed with a transition callback
// instead of CRTP.
#pragma once

#include <cstdint>
#include <deque>
#include <functional>
#include <initializer_list>

namespace tpb {

template <typename TOp>
class OpQueue {
 public:
  using TState = decltype(TOp::state);
  // advance(op, prevOpState) must call attemptTransition() for each edge, in order.
  using TAdvanceFn = std::function<void(TOp&, TState)>;

  explicit OpQueue(TAdvanceFn advance) : advance_(std::move(advance)) {}

  template <typename... Args>
  TOp& emplaceBack(Args&&... args) {
    ops_.emplace_back(std::forward<Args>(args)...);
    ops_.back().sequenceNumber = nextSeq_++;
    return ops_.back();
  }

  TOp* findOperation(int64_t seq) {
    if (ops_.empty()) return nullptr;
    int64_t off = seq - ops_.front().sequenceNumber;
    if (off < 0 || off >= static_cast<int64_t>(ops_.size())) return nullptr;
    return &ops_[off];
  }

  void advanceOperation(TOp& initial) {
    for (int64_t seq = initial.sequenceNumber;; ++seq) {
      TOp* op = findOperation(seq);
      if (!op) break;
      if (!advanceOne(*op)) break;
    }
  }
  void advanceOperation(int64_t seq) {
    if (TOp* op = findOperation(seq)) advanceOperation(*op);
  }

  void advanceAllOperations() {
    if (ops_.empty()) return;
    for (int64_t seq = ops_.front().sequenceNumber;; ++seq) {
      TOp* op = findOperation(seq);
      if (!op) break;
      advanceOne(*op);
    }
  }

  // One edge: if op is in `from` and cond holds, run actions and move to `to`.
  template <typename TActions>
  static void attemptTransition(TOp& op, TState from, TState to, bool cond, TActions&& actions) {
    if (op.state == from && cond) {
      actions();
      op.state = to;
    }
  }
  static void attemptTransition(TOp& op, TState from, TState to, bool cond) {
    if (op.state == from && cond) op.state = to;
  }

  bool empty() const { return ops_.empty(); }
  size_t size() const { return ops_.size(); }
  int64_t nextSequenceNumber() const { return nextSeq_; }

 private:
  // Returns whether the state changed (so that successors deserve a retry).
  bool advanceOne(TOp& op) {
    int64_t seq = op.sequenceNumber;
    TState before = op.state;
    TOp* prev = findOperation(seq - 1);
    TState prevState = prev ? prev->state : TOp::FINISHED;
    advance_(op, prevState);
    // `op` may have been retired by a nested call; re-look it up.
    TOp* again = findOperation(seq);
    bool changed = !again || again->state != before;
    if (again && again->state == TOp::FINISHED) {
      while (!ops_.empty() && ops_.front().state == TOp::FINISHED) ops_.pop_front();
    }
    return changed;
  }

  TAdvanceFn advance_;
  std::deque<TOp> ops_;
  int64_t nextSeq_ = 0;
};

}  // namespace tpb
