// Entry points of libmccs_kernels.so: the collective kernels in a library of their own,
// which the client library loads on demand when a communicator is in client-side launch
// mode on a GPU. The client library itself stays free of the CUDA runtime (it talks to
// the driver through dlopen); this library carries the kernels' device code and a static
// copy of the runtime, which launches into whatever context is current: the primary
// context of the caller's device, i.e. the one PyTorch and the caller's stream live in.
//
// The reference always launches from its service (src/mccs/src/proxy/plan.rs:637-669).
#include <cuda_runtime.h>

#include "launch.h"

extern "C" {

// Layout check between the two libraries: both must have been built from the same
// dev_types.h.
unsigned long long mccs_kernels_abi(void) {
  return (unsigned long long)sizeof(mccs::CollArgs) | ((unsigned long long)sizeof(mccs::BatchArgs) << 32);
}

// Launches one rank's kernel of the collective described by `args` on `stream` of the
// current context. Returns 0 or a cudaError_t; `*err` then points to its static text.
int mccs_kernels_launch(int kind, const mccs::CollArgs* args, int ctas, int threads, void* stream, const char** err) {
  if (err) *err = nullptr;
  if (!args || args->emulated) {
    if (err) *err = "invalid arguments";
    return (int)cudaErrorInvalidValue;
  }
  mccs::LaunchDims dims;
  dims.ctas = ctas;
  dims.threads = threads;
  cudaError_t e = mccs::launch_collective(kind, *args, dims, stream);
  if (e != cudaSuccess) {
    if (err) *err = cudaGetErrorString(e);
    cudaGetLastError();
  }
  return (int)e;
}

// Same for a fused launch of several AllReduces (kernels/batch.cuh).
int mccs_kernels_launch_batch(const mccs::BatchArgs* args, int ctas, int threads, void* stream, const char** err) {
  if (err) *err = nullptr;
  if (!args || args->base.emulated) {
    if (err) *err = "invalid arguments";
    return (int)cudaErrorInvalidValue;
  }
  mccs::LaunchDims dims;
  dims.ctas = ctas;
  dims.threads = threads;
  cudaError_t e = mccs::launch_batch(*args, dims, stream);
  if (e != cudaSuccess) {
    if (err) *err = cudaGetErrorString(e);
    cudaGetLastError();
  }
  return (int)e;
}

}  // extern "C"
