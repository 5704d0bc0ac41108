// Stand-in for the CUDA backend in host-only builds (sanitizer runs of the daemon and
// the client library): reports that no CUDA device is usable, so the daemon takes the
// host backend.
#include "../device/backend.h"

namespace mccs {
Backend* make_cuda_backend(const BackendOptions&, std::string* why) {
  if (why) *why = "built without the CUDA backend";
  return nullptr;
}
}  // namespace mccs
