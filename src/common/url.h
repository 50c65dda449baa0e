// "<scheme>://<rest>" -> (scheme, rest). A string without a scheme is a caller bug and throws
// EINVAL (same contract as tensorpipe/common/address.cc:15-22).
#pragma once

#include <string>
#include <utility>

#include "common/defs.h"

namespace tpb {

inline std::pair<std::string, std::string> splitSchemeOfURL(const std::string& url) {
  const auto at = url.find("://");
  TPB_THROW_SYSTEM_IF(at == std::string::npos, EINVAL, "url has no scheme: " + url);
  return {url.substr(0, at), url.substr(at + 3)};
}

}  // namespace tpb
