// ibv: InfiniBand verbs transport. Its job in the reference is to carry control traffic between
// hosts (tensorpipe/transport/ibv/*); this library targets one NVSwitch box where TCP loopback
// and shared memory cover every pair of processes. The factory probes like the reference does
// (libibverbs loadable and at least one device, tensorpipe/transport/ibv/context_impl.cc:36-66)
// and returns a context that is not viable; there is no data path behind it.
#include <dlfcn.h>

#include <tpb/transport.h>

#include "common/defs.h"

namespace tpb {
namespace transport {
namespace ibv {

namespace {
class NonViable final : public Context {
 public:
  std::shared_ptr<Connection> connect(std::string) override { throw std::runtime_error("ibv transport is not viable"); }
  std::shared_ptr<Listener> listen(std::string) override { throw std::runtime_error("ibv transport is not viable"); }
  bool isViable() const override { return false; }
  const std::string& domainDescriptor() const override { return dd_; }
  void setId(std::string) override {}
  void close() override {}
  void join() override {}

 private:
  std::string dd_ = "ibv:*";
};
}  // namespace

std::shared_ptr<Context> create() {
  void* verbs = ::dlopen("libibverbs.so.1", RTLD_LOCAL | RTLD_LAZY);
  int numDevices = 0;
  if (verbs) {
    using GetList = void** (*)(int*);
    using FreeList = void (*)(void**);
    auto getList = reinterpret_cast<GetList>(::dlsym(verbs, "ibv_get_device_list"));
    auto freeList = reinterpret_cast<FreeList>(::dlsym(verbs, "ibv_free_device_list"));
    if (getList && freeList) {
      void** list = getList(&numDevices);
      if (list) freeList(list);
    }
    ::dlclose(verbs);
  }
  TPB_VLOG(7) << "ibv transport is not viable (libibverbs " << (verbs ? "present" : "absent") << ", " << numDevices
              << " devices; the verbs data path is not built)";
  return std::make_shared<NonViable>();
}

}  // namespace ibv
}  // namespace transport
}  // namespace tpb
