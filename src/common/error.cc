#include <tpb/error.h>

namespace tpb {
const Error Error::kSuccess = Error();
}  // namespace tpb
