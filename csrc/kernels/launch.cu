#include "launch.h"

#include <stdio.h>

extern "C" {
const void* mccs_kfn_i8(int, int);
const void* mccs_kfn_u8(int, int);
const void* mccs_kfn_i32(int, int);
const void* mccs_kfn_u32(int, int);
const void* mccs_kfn_i64(int, int);
const void* mccs_kfn_u64(int, int);
const void* mccs_kfn_f16(int, int);
const void* mccs_kfn_f32(int, int);
const void* mccs_kfn_f64(int, int);
const void* mccs_kfn_bf16(int, int);
const void* mccs_kfn_untyped(int);
const void* mccs_kfn_batch_i8(int, int);
const void* mccs_kfn_batch_u8(int, int);
const void* mccs_kfn_batch_i32(int, int);
const void* mccs_kfn_batch_u32(int, int);
const void* mccs_kfn_batch_i64(int, int);
const void* mccs_kfn_batch_u64(int, int);
const void* mccs_kfn_batch_f16(int, int);
const void* mccs_kfn_batch_f32(int, int);
const void* mccs_kfn_batch_f64(int, int);
const void* mccs_kfn_batch_bf16(int, int);
}

namespace mccs {

const void* batch_kernel_function(int variant, int dtype, int op);

const void* kernel_function(int variant, int dtype, int op) {
  if (variant == kArHybrid || variant == kRsDirect || variant == kRsNvls)
    return batch_kernel_function(variant, dtype, op);   // live with the newer kernels
  switch (variant) {
    case kAgPull: case kAgPush: case kAgNvls: case kAgRing: case kLocalCopy:
      return mccs_kfn_untyped(variant);
    default: break;
  }
  switch (dtype) {
    case kInt8: return mccs_kfn_i8(variant, op);
    case kUint8: return mccs_kfn_u8(variant, op);
    case kInt32: return mccs_kfn_i32(variant, op);
    case kUint32: return mccs_kfn_u32(variant, op);
    case kInt64: return mccs_kfn_i64(variant, op);
    case kUint64: return mccs_kfn_u64(variant, op);
    case kFloat16: return mccs_kfn_f16(variant, op);
    case kFloat32: return mccs_kfn_f32(variant, op);
    case kFloat64: return mccs_kfn_f64(variant, op);
    case kBfloat16: return mccs_kfn_bf16(variant, op);
  }
  return nullptr;
}

const void* batch_kernel_function(int variant, int dtype, int op) {
  switch (dtype) {
    case kInt8: return mccs_kfn_batch_i8(variant, op);
    case kUint8: return mccs_kfn_batch_u8(variant, op);
    case kInt32: return mccs_kfn_batch_i32(variant, op);
    case kUint32: return mccs_kfn_batch_u32(variant, op);
    case kInt64: return mccs_kfn_batch_i64(variant, op);
    case kUint64: return mccs_kfn_batch_u64(variant, op);
    case kFloat16: return mccs_kfn_batch_f16(variant, op);
    case kFloat32: return mccs_kfn_batch_f32(variant, op);
    case kFloat64: return mccs_kfn_batch_f64(variant, op);
    case kBfloat16: return mccs_kfn_batch_bf16(variant, op);
  }
  return nullptr;
}

static int cooperative_fit(const void* fn, int threads, int nranks) {
  if (!fn || nranks <= 0) return 0;
  int dev = 0, sms = 0, per_sm = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, threads, 0) != cudaSuccess) return 0;
  return sms * per_sm / nranks;
}

int max_cooperative_batch_ctas(int variant, int dtype, int op, int threads, int nranks) {
  return cooperative_fit(batch_kernel_function(variant, dtype, op), threads, nranks);
}

cudaError_t launch_batch(const BatchArgs& args, LaunchDims dims, void* stream) {
  const CollArgs& a = args.base;
  const void* fn = batch_kernel_function(a.variant, a.dtype, a.op);
  if (!fn) return cudaErrorInvalidDeviceFunction;
  if (args.nops < 1 || args.nops > kMaxBatch) return cudaErrorInvalidValue;
  if (dims.ctas < 1 || dims.ctas > kMaxCtas || dims.threads < 32 || dims.threads > 512)
    return cudaErrorInvalidConfiguration;
  dim3 grid((unsigned)dims.ctas, a.emulated ? (unsigned)a.nranks : 1u, 1u);
  dim3 block((unsigned)dims.threads, 1u, 1u);
  BatchArgs b = args;
  void* params[] = {(void*)&b};
  if (a.emulated && a.nranks > 1) return cudaLaunchCooperativeKernel(fn, grid, block, params, 0, (cudaStream_t)stream);
  return cudaLaunchKernel(fn, grid, block, params, 0, (cudaStream_t)stream);
}

int max_cooperative_ctas(int variant, int dtype, int op, int threads, int nranks) {
  const void* fn = kernel_function(variant, dtype, op);
  if (!fn || nranks <= 0) return 0;
  int dev = 0, sms = 0, per_sm = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, threads, 0) != cudaSuccess) return 0;
  return sms * per_sm / nranks;
}

cudaError_t launch_collective(int kind, const CollArgs& args, LaunchDims dims, void* stream) {
  CollArgs a = args;
  if (a.variant == kLocalCopy && kind_reduces(kind)) a.count = args.count * (uint64_t)dtype_size(args.dtype);
  const void* fn = kernel_function(a.variant, a.dtype, a.op);
  if (!fn) return cudaErrorInvalidDeviceFunction;
  if (dims.ctas < 1 || dims.ctas > kMaxCtas || dims.threads < 32 || dims.threads > 512)
    return cudaErrorInvalidConfiguration;
  if (variant_is_ring(a.variant) && dims.ctas > kMaxRingChannels) return cudaErrorInvalidConfiguration;
  if (a.variant == kLocalCopy) {
    // No CTA of a copy waits for another one, so the grid follows the message instead of the
    // plan: one CTA per tile (see local_copy_kernel), bounded so that the tile loop takes over
    // for messages beyond 16 GiB.
    const uint64_t tile = kCopyTileBytes;
    uint64_t ctas = (a.count + tile - 1) / tile;
    dims.ctas = (int32_t)(ctas < 1 ? 1 : ctas > (1u << 20) ? (1u << 20) : ctas);
    dims.threads = kCopyThreads;
  }
  dim3 grid((unsigned)dims.ctas, a.emulated ? (unsigned)a.nranks : 1u, 1u);
  dim3 block((unsigned)dims.threads, 1u, 1u);
  void* params[] = {(void*)&a};
  if (a.emulated && a.nranks > 1) {
    // All ranks' CTAs wait on one another, so they must be resident together.
    return cudaLaunchCooperativeKernel(fn, grid, block, params, 0, (cudaStream_t)stream);
  }
  return cudaLaunchKernel(fn, grid, block, params, 0, (cudaStream_t)stream);
}

}  // namespace mccs
