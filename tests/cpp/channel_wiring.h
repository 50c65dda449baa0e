// Raw connections for channel-level tests: the two peers open N TCP connections tagged with an
// index and hand them to createChannel on both sides (the reference's channel tests are wired the
// same way, tensorpipe/test/channel/channel_test.h:41-298).
#pragma once

#include <cstring>
#include <future>
#include <memory>
#include <string>
#include <vector>

#include <tpb/tpb.h>

#include "test_util.h"

namespace tpbtest {

using tpb::Error;
namespace transport = tpb::transport;

// Opens `n` tagged connections between two transport contexts. The server side sorts them by tag.
struct Wiring {
  std::shared_ptr<transport::Context> tctx = transport::uv::create();
  std::shared_ptr<transport::Listener> listener;
  std::string listen() {
    listener = tctx->listen("127.0.0.1");
    return listener->addr();
  }
  std::vector<std::shared_ptr<transport::Connection>> acceptAll(size_t n) {
    std::vector<std::shared_ptr<transport::Connection>> out(n);
    for (size_t i = 0; i < n; ++i) {
      std::promise<std::shared_ptr<transport::Connection>> pc;
      listener->accept([&](const Error& e, std::shared_ptr<transport::Connection> c) { pc.set_value(e ? nullptr : c); });
      auto fc = pc.get_future();
      auto c = waitFor(fc);
      if (!c) throw TestFailure("accept failed");
      std::promise<uint64_t> tag;
      c->read([&](const Error& e, const void* p, size_t len) {
        uint64_t v = UINT64_MAX;
        if (!e && len == 8) std::memcpy(&v, p, 8);
        tag.set_value(v);
      });
      auto ft = tag.get_future();
      uint64_t idx = waitFor(ft);
      if (idx >= n) throw TestFailure("bad connection tag");
      out[idx] = c;
    }
    return out;
  }
  std::vector<std::shared_ptr<transport::Connection>> connectAll(const std::string& addr, size_t n) {
    std::vector<std::shared_ptr<transport::Connection>> out;
    for (size_t i = 0; i < n; ++i) {
      auto c = tctx->connect(addr);
      auto tag = std::make_shared<uint64_t>(i);
      std::promise<Error> pw;
      c->write(tag.get(), 8, [&, tag](const Error& e) { pw.set_value(e); });
      auto fw = pw.get_future();
      if (waitFor(fw)) throw TestFailure("tag write failed");
      out.push_back(std::move(c));
    }
    return out;
  }
};


}  // namespace tpbtest
