// Host-side entry to the kernels as compiled for the SIMT emulator (emulated_kernels.cc).
// Both run the launch to completion on the calling thread's behalf (they spawn one OS
// thread per CTA and join them) and return false for a variant that has no emulated form.
// The in-switch (NVLS) variants work on emulated multicast regions: an address range that
// stands for the same offsets of every rank's buffer, registered with emulated_mc_add.
#pragma once
#include <stddef.h>

#include <vector>

#include "../kernels/dev_types.h"

namespace mccs {
bool emulated_launch(int kind, const CollArgs& args, LaunchDims dims);
bool emulated_launch_batch(const BatchArgs& args, LaunchDims dims);
// One rank's part of a collective (args.rank), to completion; the other ranks' parts run
// concurrently elsewhere and are met through the shared signal pads.
bool emulated_launch_rank(int kind, const CollArgs& args, LaunchDims dims);
bool emulated_launch_batch_rank(const BatchArgs& args, LaunchDims dims);
// [base, base + size) becomes a multicast address range over `backing` (one pointer per
// rank); the range itself is never dereferenced, only looked up.
void emulated_mc_add(uint64_t base, size_t size, const std::vector<void*>& backing);
void emulated_mc_remove(uint64_t base);
}  // namespace mccs
