// Allocation-free local AllReduce (see csrc/include/mccs_noalloc.h for who needs it
// and the rules). The synchronisation scratch that the service normally allocates per
// communicator — one signal pad and one status block per rank — sits here in a
// file-scope device array, so the call path contains no cudaMalloc, cudaHostAlloc or
// any other allocating routine.
#include "../include/mccs_noalloc.h"

#include <cuda_runtime.h>
#include <string.h>

#include <atomic>

#include "dev_types.h"
#include "launch.h"

namespace {

constexpr size_t kSlot = 5632;   // one rank's share: SignalPad (5376 B) + StatusBlock (64 B), rounded up to 256
static_assert(sizeof(mccs::SignalPad) + sizeof(mccs::StatusBlock) <= kSlot, "scratch slot too small");
static_assert(MCCS_NOALLOC_SCRATCH_BYTES == MCCS_NOALLOC_MAX_RANKS * kSlot, "header and source disagree");
static_assert(MCCS_NOALLOC_MAX_RANKS <= mccs::kMaxRanks, "more ranks than the kernels support");
static_assert(offsetof(mccs::StatusBlock, error) == 0 && offsetof(mccs::StatusBlock, error_peer) == 4,
              "the status copy below reads the first two words of a status block");

// In host code this name is only a stand-in for the device array: its device address
// comes from cudaGetSymbolAddress below, once per device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[MCCS_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
// Per device, filled on that device's first call. Two threads that make the first call
// together both resolve the same address and store the same value.
std::atomic<unsigned char*> g_scratch_addr[kMaxDevices];

cudaError_t scratch_for_current_device(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  unsigned char* p = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (!p) {
    // Set-up, first call on this device (which is current): resolve the array's address.
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_addr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return cudaSuccess;
}

bool overlap_without_identity(const void* a, const void* b, size_t bytes) {
  if (a == b) return false;
  const uintptr_t x = (uintptr_t)a, y = (uintptr_t)b;
  return x < y ? y - x < bytes : x - y < bytes;
}

}  // namespace

extern "C" int mccsLocalAllReduceNoAllocPrepare(void) {
  using namespace mccs;
  unsigned char* scratch = nullptr;
  cudaError_t e = scratch_for_current_device(&scratch);
  if (e != cudaSuccess) return (int)e;
  // Asking for a kernel's attributes makes the runtime load its code now instead of at the
  // first launch.
  const int variants[2] = {kArTwoShot, kLocalCopy};
  const int dtypes[3] = {kFloat32, kFloat16, kBfloat16};
  for (int v : variants)
    for (int dt : dtypes) {
      const void* fn = kernel_function(v, dt, kSum);
      if (!fn) return (int)cudaErrorInvalidDeviceFunction;
      cudaFuncAttributes attr;
      e = cudaFuncGetAttributes(&attr, fn);
      if (e != cudaSuccess) return (int)e;
      (void)max_cooperative_ctas(v, dt, kSum, 512, 2);
    }
  return (int)cudaSuccess;
}

extern "C" int mccsLocalAllReduceNoAllocStatus(mccsNoAllocStatus_t* status, void* stream) {
  if (!status) return (int)cudaErrorInvalidValue;
  unsigned char* scratch = nullptr;
  cudaError_t e = scratch_for_current_device(&scratch);
  if (e != cudaSuccess) return (int)e;
  e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  // One strided copy: the first two words (error, peer) of each slot's status block.
  unsigned words[MCCS_NOALLOC_MAX_RANKS][2];
  e = cudaMemcpy2D(words, sizeof words[0], scratch + sizeof(mccs::SignalPad), kSlot, sizeof words[0], MCCS_NOALLOC_MAX_RANKS,
                   cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return (int)e;
  for (int r = 0; r < MCCS_NOALLOC_MAX_RANKS; r++) {
    status->error[r] = words[r][0];
    status->peer[r] = words[r][1];
  }
  return (int)cudaSuccess;
}

extern "C" int mccsLocalAllReduceNoAlloc(const void* const* in, void* const* out, int nranks, size_t count, int dtype,
                                         void* stream) {
  using namespace mccs;
  if (!in || !out || nranks < 1 || nranks > MCCS_NOALLOC_MAX_RANKS) return (int)cudaErrorInvalidValue;
  if (dtype != kFloat32 && dtype != kFloat16 && dtype != kBfloat16) return (int)cudaErrorInvalidValue;
  if (count == 0) return (int)cudaSuccess;
  const uint64_t bytes = (uint64_t)count * (uint64_t)dtype_size(dtype);
  for (int r = 0; r < nranks; r++)
    if (!in[r] || !out[r]) return (int)cudaErrorInvalidValue;
  // Identical buffers are fine (see the header); anything that overlaps partly is not.
  for (int r = 0; r < nranks; r++)
    for (int q = 0; q < nranks; q++) {
      if (overlap_without_identity(out[r], in[q], (size_t)bytes)) return (int)cudaErrorInvalidValue;
      if (q > r && (out[r] == out[q] || overlap_without_identity(out[r], out[q], (size_t)bytes))) return (int)cudaErrorInvalidValue;
    }
  unsigned char* scratch = nullptr;
  cudaError_t e = scratch_for_current_device(&scratch);
  if (e != cudaSuccess) return (int)e;
  cudaStream_t s = (cudaStream_t)stream;
  // The barrier counters and status words must start at zero: the array still holds
  // what the previous call left. All slots, so that the status query sees no stale words.
  e = cudaMemsetAsync(scratch, 0, MCCS_NOALLOC_SCRATCH_BYTES, s);
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
  LaunchDims dims;
  dims.threads = 512;
  dims.ctas = bytes <= (256u << 10) ? 2 : bytes <= (8u << 20) ? 8 : 16;
  if (nranks > 1) {
    // All ranks' CTAs wait on one another inside one cooperative launch: stay resident.
    int fit = max_cooperative_ctas(a.variant, dtype, kSum, dims.threads, nranks);
    if (fit < 1) return (int)cudaErrorLaunchOutOfResources;
    if (dims.ctas > fit) dims.ctas = fit;
  }
  return (int)launch_collective(kAllReduce, a, dims, s);
}
