// Bounded blocking multi-producer / multi-consumer queue (mutex + condition variables), the
// hand-off primitive between a loop and a worker thread (tensorpipe/common/queue.h:18-47).
#pragma once

#include <condition_variable>
#include <deque>
#include <mutex>

namespace tpb {

template <typename T>
class Queue {
 public:
  explicit Queue(size_t capacity = 1) : capacity_(capacity) {}
  void push(T t) {
    std::unique_lock<std::mutex> l(mu_);
    notFull_.wait(l, [&] { return items_.size() < capacity_; });
    items_.push_back(std::move(t));
    notEmpty_.notify_one();
  }
  T pop() {
    std::unique_lock<std::mutex> l(mu_);
    notEmpty_.wait(l, [&] { return !items_.empty(); });
    T t = std::move(items_.front());
    items_.pop_front();
    notFull_.notify_one();
    return t;
  }
  size_t size() const {
    std::unique_lock<std::mutex> l(mu_);
    return items_.size();
  }

 private:
  mutable std::mutex mu_;
  std::condition_variable notFull_, notEmpty_;
  std::deque<T> items_;
  const size_t capacity_;
};

}  // namespace tpb
