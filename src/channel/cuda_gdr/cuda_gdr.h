// The cuda_gdr channel over a given verbs provider (channel::cuda_gdr::create() in the public
// header uses the system's libibverbs and insists on the GPU peer-memory kernel module), and the
// GPU-to-NIC matching it uses, exposed for tests.
#pragma once

#include <memory>
#include <string>
#include <vector>

#include <tpb/channel.h>

#include "common/verbs.h"

namespace tpb {
namespace channel {
namespace cuda_gdr {

struct Options {
  // A real NIC can only reach GPU memory when the nvidia-peermem (nv_peer_mem) module is loaded.
  bool requirePeerMemoryModule = true;
  // Bytes of one tensor a lane keeps posted at a time (work requests are at most the NIC's
  // message size each).
  size_t maxPostedBytes = 64u << 20;
};

std::shared_ptr<Context> createWithProvider(std::shared_ptr<verbs::Provider> provider, Options options = Options());

// For every GPU (by its sysfs PCI path) the index of the NIC that shares the longest run of
// leading path components with it, i.e. the one behind the same PCIe switch when there is one.
// GPUs that share nothing with any NIC are dealt round robin.
std::vector<int> matchGpusToNics(const std::vector<std::string>& gpuPciPaths, const std::vector<std::string>& nicPciPaths);

}  // namespace cuda_gdr
}  // namespace channel
}  // namespace tpb
