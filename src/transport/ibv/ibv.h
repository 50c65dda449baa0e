// The ibv transport over a given verbs provider. transport::ibv::create() (public header) uses the
// system's libibverbs; tests hand in the software fabric.
#pragma once

#include <memory>

#include <tpb/transport.h>

#include "common/verbs.h"

namespace tpb {
namespace transport {
namespace ibv {

std::shared_ptr<Context> createWithProvider(std::shared_ptr<verbs::Provider> provider);

}  // namespace ibv
}  // namespace transport
}  // namespace tpb
