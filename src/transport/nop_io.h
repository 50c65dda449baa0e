// Typed control messages over a transport connection: one nop-encoded object per frame.
// (The reference reaches the same wire bytes through AbstractNopHolder overloads of
// Connection::read/write, tensorpipe/transport/connection.h:44-58.)
#pragma once

#include <functional>
#include <memory>
#include <vector>

#include <tpb/transport.h>

#include "common/nop.h"

namespace tpb {
namespace transport {

TPB_SIMPLE_ERROR(NopDecodeError, "malformed control message");

template <typename T>
void writeNop(Connection& conn, const T& obj, Connection::write_callback_fn fn) {
  auto buf = std::make_shared<std::vector<uint8_t>>(nop::encode(obj));
  conn.write(buf->data(), buf->size(), [buf, fn = std::move(fn)](const Error& e) { fn(e); });
}

template <typename T>
void readNop(Connection& conn, std::function<void(const Error&, T)> fn) {
  conn.read([fn = std::move(fn)](const Error& e, const void* ptr, size_t len) {
    T obj{};
    if (e) {
      fn(e, std::move(obj));
      return;
    }
    if (!nop::decode(ptr, len, obj)) {
      fn(TPB_CREATE_ERROR(NopDecodeError), T{});
      return;
    }
    fn(Error::kSuccess, std::move(obj));
  });
}

}  // namespace transport
}  // namespace tpb
