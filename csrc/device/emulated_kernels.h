// Host-side entry to the kernels as compiled for the SIMT emulator (emulated_kernels.cc).
// Both run the launch to completion on the calling thread's behalf (they spawn one OS
// thread per CTA and join them) and return false for a variant that has no emulated form
// (the NVLS variants: the host has no multicast mappings).
#pragma once
#include "../kernels/dev_types.h"

namespace mccs {
bool emulated_launch(int kind, const CollArgs& args, LaunchDims dims);
bool emulated_launch_batch(const BatchArgs& args, LaunchDims dims);
// One rank's part of a collective (args.rank), to completion; the other ranks' parts run
// concurrently elsewhere and are met through the shared signal pads.
bool emulated_launch_rank(int kind, const CollArgs& args, LaunchDims dims);
}  // namespace mccs
