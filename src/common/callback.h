// Callback plumbing.
//  * RearmableCallback pairs stored callbacks with stored results: whichever comes first waits
//    for the other (tensorpipe/common/callback.h:54-83 counterpart).
//  * LoopCallback wraps a member-style closure so that, when fired from any thread, it hops to
//    the subject's loop, records the error on the subject first (setError), and then ALWAYS
//    runs the closure — the subject decides what to do with its own sticky error
//    (tensorpipe/common/callback.h:119-148 counterpart).
#pragma once

#include <deque>
#include <functional>
#include <memory>
#include <tuple>
#include <utility>

#include <tpb/error.h>

#include "common/loop.h"

namespace tpb {

template <typename... Args>
class RearmableCallback {
  using TFn = std::function<void(Args...)>;
  using TStored = std::tuple<std::decay_t<Args>...>;

 public:
  void arm(TFn fn) {
    if (!args_.empty()) {
      TStored a = std::move(args_.front());
      args_.pop_front();
      std::apply(fn, std::move(a));
    } else {
      callbacks_.push_back(std::move(fn));
    }
  }
  void trigger(Args... args) {
    if (!callbacks_.empty()) {
      TFn fn = std::move(callbacks_.front());
      callbacks_.pop_front();
      fn(std::forward<Args>(args)...);
    } else {
      args_.emplace_back(std::forward<Args>(args)...);
    }
  }
  // Fire every armed callback with the same arguments (used on close/error).
  void triggerAll(std::function<TStored()> gen) {
    while (!callbacks_.empty()) {
      TFn fn = std::move(callbacks_.front());
      callbacks_.pop_front();
      std::apply(fn, gen());
    }
  }
  size_t numArmed() const { return callbacks_.size(); }
  size_t numStored() const { return args_.size(); }

 private:
  std::deque<TFn> callbacks_;
  std::deque<TStored> args_;
};

// TSubject must provide: DeferredExecutor& loop(); void setError(const Error&).
template <typename TSubject>
class LoopCallback {
 public:
  explicit LoopCallback(std::enable_shared_from_this<TSubject>& subject) : subject_(subject) {}

  // fn(TSubject&, args...) ; resulting callable has signature (const Error&, args...).
  template <typename F>
  auto operator()(F fn) {
    std::shared_ptr<TSubject> subject = subject_.shared_from_this();
    return [subject = std::move(subject), fn = std::move(fn)](const Error& error, auto&&... args) mutable {
      auto bound = [subject, fn = std::move(fn), error,
                    tup = std::make_tuple(std::decay_t<decltype(args)>(std::forward<decltype(args)>(args))...)]() mutable {
        if (error) subject->setError(error);
        // Whatever a peer makes this object do, an exception on the loop thread would end the
        // process: it becomes the object's error instead (every pending callback then fires).
        try {
          std::apply([&](auto&... a) { fn(*subject, std::move(a)...); }, tup);
        } catch (const std::exception& ex) {
          subject->setError(TPB_CREATE_ERROR(LogicError, std::string("while handling a peer's message: ") + ex.what()));
        }
      };
      subject->loop().deferToLoop(std::move(bound));
    };
  }

 private:
  std::enable_shared_from_this<TSubject>& subject_;
};

}  // namespace tpb
