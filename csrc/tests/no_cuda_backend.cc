// Stand-in for the CUDA backend in host-only builds (sanitizer runs of the daemon and
// the client library): reports that no CUDA device is usable, so the daemon takes the
// host backend.
#include "../device/backend.h"
#include "../device/emulated_kernels.h"

namespace mccs {
Backend* make_cuda_backend(const BackendOptions&, std::string* why) {
  if (why) *why = "built without the CUDA backend";
  return nullptr;
}
// The emulated kernels switch stacks with ucontext, which the sanitizers do not follow;
// sanitizer builds run the host backend's plain loops only.
bool emulated_launch(int, const CollArgs&, LaunchDims) { return false; }
bool emulated_launch_batch(const BatchArgs&, LaunchDims) { return false; }
bool emulated_launch_rank(int, const CollArgs&, LaunchDims) { return false; }
bool emulated_launch_batch_rank(const BatchArgs&, LaunchDims) { return false; }
void emulated_mc_add(uint64_t, size_t, const std::vector<void*>&) {}
void emulated_mc_remove(uint64_t) {}
}  // namespace mccs
