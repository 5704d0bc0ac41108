// Allocation-free local AllReduce (see csrc/include/mccs_noalloc.h for who needs it
// and the rules). The synchronisation scratch that the service normally allocates per
// communicator — one signal pad and one status block per rank — sits here in a
// file-scope device array, so the call path contains no cudaMalloc, cudaHostAlloc or
// any other allocating routine.
#include "../include/mccs_noalloc.h"

#include <cuda_runtime.h>
#include <string.h>

#include "dev_types.h"
#include "launch.h"

namespace {

constexpr size_t kSlot = 5120;   // one rank's share: SignalPad (4736 B) + StatusBlock (64 B), rounded up
static_assert(sizeof(mccs::SignalPad) + sizeof(mccs::StatusBlock) <= kSlot, "scratch slot too small");
static_assert(MCCS_NOALLOC_SCRATCH_BYTES == MCCS_NOALLOC_MAX_RANKS * kSlot, "header and source disagree");
static_assert(MCCS_NOALLOC_MAX_RANKS <= mccs::kMaxRanks, "more ranks than the kernels support");

// In host code this name is only a stand-in for the device array: its device address
// comes from cudaGetSymbolAddress below, once per device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[MCCS_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
unsigned char* g_scratch_addr[kMaxDevices];   // per device, filled on that device's first call

}  // namespace

extern "C" int mccsLocalAllReduceNoAlloc(const void* const* in, void* const* out, int nranks, size_t count, int dtype,
                                         void* stream) {
  using namespace mccs;
  if (!in || !out || nranks < 1 || nranks > MCCS_NOALLOC_MAX_RANKS) return (int)cudaErrorInvalidValue;
  if (dtype != kFloat32 && dtype != kFloat16 && dtype != kBfloat16) return (int)cudaErrorInvalidValue;
  if (count == 0) return (int)cudaSuccess;
  for (int r = 0; r < nranks; r++)
    if (!in[r] || !out[r]) return (int)cudaErrorInvalidValue;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
  if (!g_scratch_addr[dev]) {
    // Set-up, first call on this device (which is current): resolve the array's address.
    unsigned char* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_scratch_addr[dev] = p;
  }
  unsigned char* scratch = g_scratch_addr[dev];
  cudaStream_t s = (cudaStream_t)stream;
  // The barrier counters and status words must start at zero: the array still holds
  // what the previous call left.
  e = cudaMemsetAsync(scratch, 0, (size_t)nranks * kSlot, s);
  if (e != cudaSuccess) return (int)e;

  CollArgs a;
  memset(&a, 0, sizeof a);
  a.rank = 0;
  a.nranks = nranks;
  a.emulated = nranks > 1 ? 1 : 0;
  a.dtype = dtype;
  a.op = kSum;
  a.variant = nranks > 1 ? kArTwoShot : kLocalCopy;
  a.count = count;
  a.seq = 1;
  a.scale = 1.0f;
  a.epoch = 1;
  a.timeout_ns = 10ull * 1000000000ull;
  for (int r = 0; r < nranks; r++) {
    a.send[r] = in[r];
    a.recv[r] = out[r];
    a.pad[r] = (SignalPad*)(scratch + (size_t)r * kSlot);
    a.status[r] = (StatusBlock*)(scratch + (size_t)r * kSlot + sizeof(SignalPad));
  }
  const uint64_t bytes = (uint64_t)count * (uint64_t)dtype_size(dtype);
  LaunchDims dims;
  dims.threads = 512;
  dims.ctas = bytes <= (256u << 10) ? 2 : bytes <= (8u << 20) ? 8 : 16;
  if (nranks > 1) {
    // All ranks' CTAs wait on one another inside one cooperative launch: stay resident.
    int fit = max_cooperative_ctas(a.variant, dtype, kSum, dims.threads, nranks);
    if (fit < 1) return (int)cudaErrorLaunchOutOfResources;
    if (dims.ctas > fit) dims.ctas = fit;
  } else {
    dims.ctas = 64;
  }
  return (int)launch_collective(kAllReduce, a, dims, s);
}
