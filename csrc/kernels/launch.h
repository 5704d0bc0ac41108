// Host-side entry to the collective kernels: kernel lookup by (variant, type, op)
// and the launch itself. The reference picks among five precompiled symbols
// (src/mccs/src/proxy/plan.rs:142-166) and launches grid = channels
// (plan.rs:637-669); here the grid is CTAs per rank, times ranks when one
// cooperative launch emulates every rank on a single GPU.
#pragma once
#include <cuda_runtime.h>

#include "dev_types.h"

namespace mccs {

const void* kernel_function(int variant, int dtype, int op);
cudaError_t launch_collective(int kind, const CollArgs& args, LaunchDims dims, void* stream);
// Largest CTA count per rank that keeps an emulated (cooperative) launch resident.
int max_cooperative_ctas(int variant, int dtype, int op, int threads, int nranks);

// Fused AllReduce (several members in one launch, see batch.cuh). Only the two-shot
// variants have a fused form; returns null / cudaErrorInvalidDeviceFunction otherwise.
const void* batch_kernel_function(int variant, int dtype, int op);
cudaError_t launch_batch(const BatchArgs& args, LaunchDims dims, void* stream);
int max_cooperative_batch_ctas(int variant, int dtype, int op, int threads, int nranks);

}  // namespace mccs
