// Interoperability peer built ONLY from the reference library as PyTorch ships it
// (torch/include/tensorpipe + libtorch_cpu.so): an echo server and an echo-checking client over
// the reference's uv transport and basic channel. The test suite runs this library's pipes against
// it in both directions to prove that the handshake and the descriptor wire format are compatible.
//
//   ref_interop server <port> [full]          listen on 127.0.0.1:<port>, echo every message, forever
//   ref_interop client <address> <n> [full]   connect to uv://<address>, send n messages, check echoes
// With "full" the context carries every CPU backend the way PyTorch's RPC agent registers them
// (transports uv and shm; channels basic, cma, mpt_uv over three lanes), so that the other side's negotiation has to
// steer clear of everything the two libraries do not really share.
#include <cstring>
#include <future>
#include <iostream>
#include <memory>
#include <string>
#include <vector>

#include <tensorpipe/tensorpipe.h>

namespace tp = tensorpipe;

bool gFull = false;

std::shared_ptr<tp::Context> makeContext(const std::string& name) {
  auto ctx = std::make_shared<tp::Context>(tp::ContextOptions().name(name));
  ctx->registerTransport(0, "uv", tp::transport::uv::create());
  ctx->registerChannel(0, "basic", tp::channel::basic::create());
  if (gFull) {
    ctx->registerTransport(10, "shm", tp::transport::shm::create());
    ctx->registerChannel(10, "cma", tp::channel::cma::create());
    std::vector<std::shared_ptr<tp::transport::Context>> lanes;
    std::vector<std::shared_ptr<tp::transport::Listener>> laneListeners;
    for (int i = 0; i < 3; ++i) {
      lanes.push_back(tp::transport::uv::create());
      laneListeners.push_back(lanes.back()->listen("127.0.0.1"));
    }
    ctx->registerChannel(5, "mpt_uv", tp::channel::mpt::create(std::move(lanes), std::move(laneListeners)));
  }
  return ctx;
}

struct Owned {
  std::string metadata;
  std::vector<std::pair<std::string, std::vector<uint8_t>>> payloads, tensors;
};

void echoLoop(std::shared_ptr<tp::Pipe> pipe) {
  pipe->readDescriptor([pipe](const tp::Error& e, tp::Descriptor d) {
    if (e) return;
    auto msg = std::make_shared<Owned>();
    msg->metadata = d.metadata;
    tp::Allocation a;
    for (auto& p : d.payloads) {
      msg->payloads.emplace_back(p.metadata, std::vector<uint8_t>(p.length));
      a.payloads.push_back({msg->payloads.back().second.data()});
    }
    for (auto& t : d.tensors) {
      msg->tensors.emplace_back(t.metadata, std::vector<uint8_t>(t.length));
      tp::Allocation::Tensor at;
      at.buffer = tp::CpuBuffer{msg->tensors.back().second.data()};
      a.tensors.push_back(at);
    }
    pipe->read(std::move(a), [pipe, msg](const tp::Error& e2) {
      if (e2) return;
      tp::Message out;
      out.metadata = msg->metadata;
      for (auto& p : msg->payloads) {
        tp::Message::Payload op;
        op.data = p.second.data();
        op.length = p.second.size();
        op.metadata = p.first;
        out.payloads.push_back(op);
      }
      for (auto& t : msg->tensors) {
        tp::Message::Tensor ot;
        ot.buffer = tp::CpuBuffer{t.second.data()};
        ot.length = t.second.size();
        ot.metadata = t.first;
        out.tensors.push_back(ot);
      }
      pipe->write(std::move(out), [pipe, msg](const tp::Error&) {});
      echoLoop(pipe);
    });
  });
}

int main(int argc, char** argv) {
  if (argc < 3) return 2;
  std::string mode = argv[1];
  gFull = std::string(argv[argc - 1]) == "full";
  if (mode == "server") {
    auto ctx = makeContext("ref-server");
    std::vector<std::string> urls = {std::string("uv://127.0.0.1:") + argv[2]};
    if (gFull) urls.push_back("shm://");
    auto listener = ctx->listen(urls);
    std::function<void()> arm = [&]() {
      listener->accept([&](const tp::Error& e, std::shared_ptr<tp::Pipe> pipe) {
        if (e) return;
        echoLoop(pipe);
        arm();
      });
    };
    arm();
    std::cout << "listening " << listener->url("uv") << std::endl;
    std::string line;
    std::getline(std::cin, line);  // runs until stdin closes
    ctx->join();
    return 0;
  }
  if (mode == "client" && argc >= 4) {
    auto ctx = makeContext("ref-client");
    auto pipe = ctx->connect(std::string("uv://") + argv[2]);
    int n = std::stoi(argv[3]);
    for (int i = 0; i < n; ++i) {
      std::vector<uint8_t> payload(100 + i), tensor(5000 * (i + 1));
      for (size_t b = 0; b < payload.size(); ++b) payload[b] = static_cast<uint8_t>(b * 3 + i);
      for (size_t b = 0; b < tensor.size(); ++b) tensor[b] = static_cast<uint8_t>(b * 7 + i);
      tp::Message m;
      m.metadata = "ref-msg-" + std::to_string(i);
      tp::Message::Payload p;
      p.data = payload.data();
      p.length = payload.size();
      p.metadata = "pm";
      m.payloads.push_back(p);
      tp::Message::Tensor t;
      t.buffer = tp::CpuBuffer{tensor.data()};
      t.length = tensor.size();
      t.metadata = "tm";
      if (i % 2) t.targetDevice = tp::Device(tp::kCpuDeviceType, 0);
      m.tensors.push_back(t);
      std::promise<bool> wrote;
      pipe->write(std::move(m), [&](const tp::Error& e) { wrote.set_value(!e); });
      std::promise<bool> ok;
      std::vector<uint8_t> gotPayload, gotTensor;
      pipe->readDescriptor([&](const tp::Error& e, tp::Descriptor d) {
        if (e || d.metadata != "ref-msg-" + std::to_string(i) || d.payloads.size() != 1 || d.tensors.size() != 1 ||
            d.payloads[0].metadata != "pm" || d.tensors[0].metadata != "tm") {
          ok.set_value(false);
          return;
        }
        gotPayload.resize(d.payloads[0].length);
        gotTensor.resize(d.tensors[0].length);
        tp::Allocation a;
        a.payloads.push_back({gotPayload.data()});
        tp::Allocation::Tensor at;
        at.buffer = tp::CpuBuffer{gotTensor.data()};
        a.tensors.push_back(at);
        pipe->read(std::move(a), [&](const tp::Error& e2) { ok.set_value(!e2); });
      });
      if (!wrote.get_future().get() || !ok.get_future().get() || gotPayload != payload || gotTensor != tensor) {
        std::cout << "mismatch at message " << i << std::endl;
        return 1;
      }
    }
    std::cout << "ok " << n << std::endl;
    pipe.reset();
    ctx->join();
    return 0;
  }
  return 2;
}
