// The collective kernels, compiled for the host against the SIMT emulator of
// tests/sim/simt_sim.h, behind two plain functions. The host backend uses them when the
// configuration asks for `[b200] host_kernels = "emulated"`, so that the whole service —
// client library, daemon, proxies, planner, argument filling (barrier epochs, tickets, ring
// step counters, FIFO placement, slices, fused launches) — can be tested on a machine
// without a GPU against the very kernel sources the GPU build compiles, instead of
// against the host backend's plain loops.
#include "../tests/sim/simt_sim.h"

// The GPU build's host stubs of the same kernels live in mccs::dev of this library (their
// addresses are what cudaLaunchKernel is given). The host-compiled copies get a namespace
// of their own so that the two can never be confused by the linker.
#define dev dev_emulated
#define MCCS_UNTYPED_KERNELS 1
#include "../kernels/batch.cuh"
#include "../kernels/hybrid.cuh"
#include "../kernels/scatter.cuh"

#include "emulated_kernels.h"

namespace mccs {

namespace {

using namespace mccs::dev;

// When set, a launch covers one rank only (grid.y = 1, the rank comes with the
// arguments): the other ranks' kernels run elsewhere, in other threads or processes, and
// meet this one through the shared signal pads. Used by client-side launch.
thread_local bool g_single_rank = false;

template <typename Kernel, typename Args>
void run_grid(Kernel kernel, const Args& a, int nranks, int ctas, int threads) {
  std::vector<std::thread> pool;
  sim::Dim3 grid;
  grid.x = (unsigned)ctas;
  grid.y = g_single_rank ? 1u : (unsigned)nranks;   // else one launch carries every rank, as on a single GPU
  sim::launch(kernel, grid, (unsigned)threads, a, &pool);
  sim::join_all(&pool);
}

template <typename T>
bool typed_allreduce(const CollArgs& a, int ctas, int threads) {
  auto by_op = [&](auto op_tag) {
    using Op = decltype(op_tag);
    switch (a.variant) {
      case kArOneShot: run_grid(ar_oneshot_kernel<T, Op>, a, a.nranks, ctas, threads); return true;
      case kArTwoShot: run_grid(ar_twoshot_kernel<T, Op>, a, a.nranks, ctas, threads); return true;
      case kArRing: run_grid(ar_ring_kernel<T, Op>, a, a.nranks, ctas, threads); return true;
    }
    return false;
  };
  // The in-switch variants: sums of the three floating-point types that multimem reduces.
  if constexpr (std::is_same<T, float>::value || std::is_same<T, __half>::value || std::is_same<T, __nv_bfloat16>::value) {
    if (a.op == kSum || a.op == kPreMulSum || a.op == kSumPostDiv) {
      switch (a.variant) {
        case kArNvlsOne: run_grid(ar_nvls_kernel<T, false>, a, a.nranks, ctas, threads); return true;
        case kArNvlsTwo: run_grid(ar_nvls_kernel<T, true>, a, a.nranks, ctas, threads); return true;
        case kArHybrid: run_grid(ar_hybrid_kernel<T>, a, a.nranks, ctas, threads); return true;
      }
    }
  }
  switch (a.op) {
    case kSum: case kPreMulSum: case kSumPostDiv: return by_op(OpSum{});
    case kProd: return by_op(OpProd{});
    case kMax: return by_op(OpMax{});
    case kMin: return by_op(OpMin{});
  }
  return false;
}

template <typename T>
bool typed_reduce_scatter(const CollArgs& a, int ctas, int threads) {
  if constexpr (std::is_same<T, float>::value || std::is_same<T, __half>::value || std::is_same<T, __nv_bfloat16>::value) {
    if (a.variant == kRsNvls && (a.op == kSum || a.op == kSumPostDiv)) {
      run_grid(rs_nvls_kernel<T>, a, a.nranks, ctas, threads);
      return true;
    }
  }
  if (a.variant != kRsDirect) return false;
  switch (a.op) {
    case kSum: case kPreMulSum: case kSumPostDiv: run_grid(rs_direct_kernel<T, OpSum>, a, a.nranks, ctas, threads); return true;
    case kProd: run_grid(rs_direct_kernel<T, OpProd>, a, a.nranks, ctas, threads); return true;
    case kMax: run_grid(rs_direct_kernel<T, OpMax>, a, a.nranks, ctas, threads); return true;
    case kMin: run_grid(rs_direct_kernel<T, OpMin>, a, a.nranks, ctas, threads); return true;
  }
  return false;
}

template <typename T>
bool typed_batch(const BatchArgs& b, int ctas, int threads) {
  const int n = b.base.nranks;
  if constexpr (std::is_same<T, float>::value || std::is_same<T, __half>::value || std::is_same<T, __nv_bfloat16>::value) {
    if (b.base.variant == kArNvlsTwo && (b.base.op == kSum || b.base.op == kPreMulSum || b.base.op == kSumPostDiv)) {
      run_grid(ar_nvls_batch_kernel<T>, b, n, ctas, threads);
      return true;
    }
  }
  if (b.base.variant != kArTwoShot) return false;
  switch (b.base.op) {
    case kSum: case kPreMulSum: case kSumPostDiv: run_grid(ar_twoshot_batch_kernel<T, OpSum>, b, n, ctas, threads); return true;
    case kProd: run_grid(ar_twoshot_batch_kernel<T, OpProd>, b, n, ctas, threads); return true;
    case kMax: run_grid(ar_twoshot_batch_kernel<T, OpMax>, b, n, ctas, threads); return true;
    case kMin: run_grid(ar_twoshot_batch_kernel<T, OpMin>, b, n, ctas, threads); return true;
  }
  return false;
}

template <typename Fn>
bool by_dtype(int dtype, Fn fn) {
  switch (dtype) {
    case kInt8: return fn((int8_t*)nullptr);
    case kUint8: return fn((uint8_t*)nullptr);
    case kInt32: return fn((int32_t*)nullptr);
    case kUint32: return fn((uint32_t*)nullptr);
    case kInt64: return fn((int64_t*)nullptr);
    case kUint64: return fn((uint64_t*)nullptr);
    case kFloat16: return fn((__half*)nullptr);
    case kFloat32: return fn((float*)nullptr);
    case kFloat64: return fn((double*)nullptr);
    case kBfloat16: return fn((__nv_bfloat16*)nullptr);
  }
  return false;
}

// The emulator runs every CUDA thread as a fiber: keep the shapes small.
void clamp(int* ctas, int* threads, bool ring) {
  if (*threads > 64) *threads = 64;
  if (*threads < 32) *threads = 32;
  if (!ring && *ctas > 4) *ctas = 4;
  if (*ctas < 1) *ctas = 1;
}

}  // namespace

void emulated_mc_add(uint64_t base, size_t size, const std::vector<void*>& backing) {
  std::vector<char*> b;
  for (void* p : backing) b.push_back((char*)p);
  sim_mc_add((uintptr_t)base, size, b);
}

void emulated_mc_remove(uint64_t base) { sim_mc_remove((uintptr_t)base); }

bool emulated_launch_rank(int kind, const CollArgs& args, LaunchDims dims) {
  g_single_rank = true;
  const bool ok = emulated_launch(kind, args, dims);
  g_single_rank = false;
  return ok;
}

bool emulated_launch(int kind, const CollArgs& args, LaunchDims dims) {
  CollArgs a = args;
  a.emulated = g_single_rank ? 0 : 1;
  int ctas = dims.ctas, threads = dims.threads;
  clamp(&ctas, &threads, variant_is_ring(a.variant));
  if (a.variant == kLocalCopy) {
    if (kind_reduces(kind)) a.count = args.count * (uint64_t)dtype_size(args.dtype);
    run_grid(local_copy_kernel, a, a.nranks, ctas, threads);
    return true;
  }
  if (kind == kAllGather) {
    switch (a.variant) {
      case kAgPull: run_grid(ag_direct_kernel<kAgModePull>, a, a.nranks, ctas, threads); return true;
      case kAgPush: run_grid(ag_direct_kernel<kAgModePush>, a, a.nranks, ctas, threads); return true;
      case kAgRing: run_grid(ag_ring_kernel, a, a.nranks, ctas, threads); return true;
      case kAgNvls: run_grid(ag_direct_kernel<kAgModeNvls>, a, a.nranks, ctas, threads); return true;
    }
    return false;
  }
  if (kind == kReduceScatter)
    return by_dtype(a.dtype, [&](auto* tag) {
      using T = typename std::remove_pointer<decltype(tag)>::type;
      return typed_reduce_scatter<T>(a, ctas, threads);
    });
  return by_dtype(a.dtype, [&](auto* tag) {
    using T = typename std::remove_pointer<decltype(tag)>::type;
    return typed_allreduce<T>(a, ctas, threads);
  });
}

bool emulated_launch_batch_rank(const BatchArgs& args, LaunchDims dims) {
  g_single_rank = true;
  const bool ok = emulated_launch_batch(args, dims);
  g_single_rank = false;
  return ok;
}

bool emulated_launch_batch(const BatchArgs& args, LaunchDims dims) {
  BatchArgs b = args;
  b.base.emulated = g_single_rank ? 0 : 1;
  int ctas = dims.ctas, threads = dims.threads;
  clamp(&ctas, &threads, false);
  return by_dtype(b.base.dtype, [&](auto* tag) {
    using T = typename std::remove_pointer<decltype(tag)>::type;
    return typed_batch<T>(b, ctas, threads);
  });
}

}  // namespace mccs
