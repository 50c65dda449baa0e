// cuda_gdr: GPUDirect RDMA between hosts (GPU memory registered with an InfiniBand NIC). A single
// NVSwitch box has no such requirement: every GPU pair is reached over NVLink by cuda_p2p. The
// factory keeps the reference's behaviour on a machine without the prerequisites — it probes for
// libibverbs and the peer-memory kernel module and reports a context that is not viable
// (tensorpipe/channel/cuda_gdr/context_impl.cc:452-520) — and there is no data path behind it.
#include <dlfcn.h>
#include <unistd.h>

#include "channel/nonviable.h"
#include "common/defs.h"

namespace tpb {
namespace channel {
namespace cuda_gdr {

std::shared_ptr<Context> create() {
  void* verbs = ::dlopen("libibverbs.so.1", RTLD_LOCAL | RTLD_LAZY);
  const bool peerMem = ::access("/sys/kernel/mm/memory_peers/nv_mem/version", F_OK) == 0 ||
      ::access("/sys/module/nvidia_peermem/version", F_OK) == 0;
  if (verbs) ::dlclose(verbs);
  TPB_VLOG(4) << "cuda_gdr is not viable (libibverbs " << (verbs ? "present" : "absent") << ", peer memory module "
              << (peerMem ? "present" : "absent") << "; cross-host GPUDirect RDMA is not built)";
  return std::make_shared<NonViableContext>();
}

}  // namespace cuda_gdr
}  // namespace channel
}  // namespace tpb
