// A channel context that reports "not viable": what a factory returns when the hardware or
// system support its channel needs is absent, so that registration is silently skipped.
#pragma once

#include <tpb/channel.h>

namespace tpb {
namespace channel {

class NonViableContext final : public Context {
 public:
  bool isViable() const override { return false; }
  const std::unordered_map<Device, std::string>& deviceDescriptors() const override { return empty_; }
  std::shared_ptr<Channel> createChannel(std::vector<std::shared_ptr<transport::Connection>>, Endpoint) override {
    throw std::runtime_error("channel context is not viable");
  }
  void setId(std::string) override {}
  void close() override {}
  void join() override {}

 private:
  std::unordered_map<Device, std::string> empty_;
};

}  // namespace channel
}  // namespace tpb
