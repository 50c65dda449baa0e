// The "basic" channel: tensor bytes simply travel as frames on the one transport connection the
// pipe hands over. Always viable, cpu -> cpu only, device descriptor "any" (same strings as
// tensorpipe/channel/basic/context_impl.cc:20-24 so a reference peer selects it with us).
#include <atomic>
#include <set>

#include <tpb/channel.h>

#include "common/defs.h"
#include "common/loop.h"

namespace tpb {
namespace channel {
namespace basic {

namespace {

class ContextImpl;

class ChannelImpl final : public Channel, public std::enable_shared_from_this<ChannelImpl> {
 public:
  ChannelImpl(std::shared_ptr<ContextImpl> ctx, std::shared_ptr<transport::Connection> conn)
      : ctx_(std::move(ctx)), conn_(std::move(conn)) {}

  void send(Buffer buffer, size_t length, TSendCallback cb) override;
  void recv(Buffer buffer, size_t length, TRecvCallback cb) override;
  void setId(std::string id) override { (void)id; }
  void close() override;
  void closeFromLoop(const Error& e);
  ~ChannelImpl() override { conn_->close(); }

 private:
  std::shared_ptr<ContextImpl> ctx_;
  std::shared_ptr<transport::Connection> conn_;
  Error error_;
};

class ContextImpl final : public Context, public std::enable_shared_from_this<ContextImpl> {
 public:
  ContextImpl() { descriptors_[Device(kCpuDeviceType, 0)] = "any"; }
  bool isViable() const override { return true; }
  const std::unordered_map<Device, std::string>& deviceDescriptors() const override { return descriptors_; }
  std::shared_ptr<Channel> createChannel(std::vector<std::shared_ptr<transport::Connection>> conns,
                                         Endpoint) override {
    TPB_THROW_ASSERT_IF(conns.size() != 1, "basic channel needs exactly one connection");
    auto ch = std::make_shared<ChannelImpl>(shared_from_this(), std::move(conns[0]));
    std::weak_ptr<ChannelImpl> weak = ch;
    loop_.deferToLoop([this, self = shared_from_this(), weak]() {
      if (auto c = weak.lock()) {
        if (closed_) c->closeFromLoop(TPB_CREATE_ERROR(ContextClosedError));
        else channels_.insert(weak);
      }
    });
    return ch;
  }
  void setId(std::string id) override { (void)id; }
  void close() override {
    loop_.deferToLoop([this, self = shared_from_this()]() {
      if (closed_) return;
      closed_ = true;
      for (auto& w : channels_)
        if (auto c = w.lock()) c->closeFromLoop(TPB_CREATE_ERROR(ContextClosedError));
      channels_.clear();
    });
  }
  void join() override {
    close();
    loop_.runInLoop([]() {});
  }
  OnDemandLoop loop_;

 private:
  std::unordered_map<Device, std::string> descriptors_;
  bool closed_ = false;
  std::set<std::weak_ptr<ChannelImpl>, std::owner_less<std::weak_ptr<ChannelImpl>>> channels_;
};

void ChannelImpl::send(Buffer buffer, size_t length, TSendCallback cb) {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self, buffer, length, cb = std::move(cb)]() mutable {
    if (self->error_) return cb(self->error_);
    if (length == 0) return cb(Error::kSuccess);  // nothing travels for an empty tensor
    self->conn_->write(buffer.unwrap<CpuBuffer>().ptr, length,
                       [self, cb = std::move(cb)](const Error& e) { cb(e); });
  });
}

void ChannelImpl::recv(Buffer buffer, size_t length, TRecvCallback cb) {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self, buffer, length, cb = std::move(cb)]() mutable {
    if (self->error_) return cb(self->error_);
    if (length == 0) return cb(Error::kSuccess);
    self->conn_->read(buffer.unwrap<CpuBuffer>().ptr, length,
                      [self, cb = std::move(cb)](const Error& e, const void*, size_t) { cb(e); });
  });
}

void ChannelImpl::close() {
  auto self = shared_from_this();
  ctx_->loop_.deferToLoop([self]() { self->closeFromLoop(TPB_CREATE_ERROR(ChannelClosedError)); });
}

void ChannelImpl::closeFromLoop(const Error& e) {
  if (error_) return;
  error_ = e;
  conn_->close();  // pending reads/writes fail through their own callbacks
}

}  // namespace

std::shared_ptr<Context> create() { return std::make_shared<ContextImpl>(); }

}  // namespace basic
}  // namespace channel
}  // namespace tpb
