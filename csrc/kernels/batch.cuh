// Fused AllReduce: several collectives of one communicator in one launch.
//
// The reference chains consecutive queued AllReduce tasks with equal element type and
// operator into one kernel launch (src/mccs/src/proxy/plan.rs:122-141); its kernel then
// walks the work elements one after another (src/collectives/src/common.h:130-179), each
// with its own ring hand-shakes. Here the members share the two cross-rank barriers: one
// before the first member (every rank's inputs exist, every rank's outputs may be
// overwritten) and one after the last (every remote store has landed). Between them each
// member is the two-shot exchange of collectives.cuh: rank r reduces shard r of the
// member from all ranks and stores it into every rank's output.
//
// In place is safe for the same reason as in the single kernel: a rank only overwrites
// shard r of its peers' buffers, which those peers never read (they read their own shard
// of every buffer), and members are independent buffers.
#pragma once
#include "collectives.cuh"

namespace mccs {
namespace dev {

// Start of a fused launch: the cross-rank barrier, unless the host vouches for it.
__device__ __forceinline__ bool batch_begin(const BatchArgs& b, int rank) {
  trace_begin(b.base, rank);
  if (b.flags & kBatchSkipStartBarrier) return true;
  return rank_barrier<false>(b.base, rank, b.base.epoch, kDevTimeoutStart);
}

// End of a fused launch, after this CTA's closing barrier: bookkeeping for the daemon,
// and, if asked for, the caller's completion word once ALL CTAs of this rank are through
// (every CTA's barrier only covers the CTAs with its own index on the peers).
__device__ __forceinline__ void batch_end(const BatchArgs& b, int rank) {
  finish(b.base, rank);
  if (b.done_ptr[rank] == nullptr) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    // Release pattern on the way in (everything this CTA observed and wrote is ordered
    // before its count), acquire pattern for the CTA that sees the full count, so that the
    // completion word is ordered after what ALL CTAs of this rank observed.
    fence_sys();
    const unsigned last = gridDim.x - 1;
    if (atomicInc(b.done_counter[rank], last) == last) {
      fence_sys();
      st_release_sys_u64(b.done_ptr[rank], b.done_value[rank]);
    }
  }
}

__device__ __forceinline__ bool batch_aligned16(const BatchArgs& b, int k) {
  uint64_t bits = 0;
  for (int r = 0; r < b.base.nranks; r++) bits |= (uint64_t)b.send[k][r] | (uint64_t)b.recv[k][r];
  return (bits & 15u) == 0;
}

// The members are walked twice: first the whole 16-byte packs of every member whose buffers
// are 16-byte aligned, then what is left of each member (less than a pack, or all of it when a
// buffer is not aligned) element by element. One walk doing both per member kept the second
// part's operands live across the pack loop, beyond 128 registers. The pack loop is the "eight
// sources, unroll 2" form: the "four sources, unroll 4" form of the single kernel does not
// fit next to the member loop either.
template <typename T, typename Op>
__global__ void __launch_bounds__(kMaxThreads) ar_twoshot_batch_kernel(const __grid_constant__ BatchArgs b) {
  const CollArgs& a = b.base;
  const int rank = a.emulated ? (int)blockIdx.y : a.rank;
  __shared__ const char* s_src[kMaxRanks];
  __shared__ char* s_dst[kMaxRanks];
  if (!batch_begin(b, rank)) return;
  constexpr uint64_t kN = 16 / sizeof(T);

#pragma unroll 1
  for (int k = 0; k < b.nops; k++) {
    if (!batch_aligned16(b, k) || b.count[k] < kN) continue;   // the same answer in every thread
    __syncthreads();   // the previous member's users of s_src / s_dst are done
    if (threadIdx.x < a.nranks) {
      s_src[threadIdx.x] = (const char*)b.send[k][threadIdx.x];
      s_dst[threadIdx.x] = (char*)b.recv[k][threadIdx.x];
    }
    __syncthreads();
    Scaler<typename AccOf<T>::type> sc{scaler_mode(a.op), a.scale};
    const Range mine = split_range(b.count[k] / kN, a.nranks, rank);
    reduce_store<T, Op, 16, 2, kMaxRanks>(s_src, a.nranks, s_dst, a.nranks, mine.beg, mine.end, blockIdx.x, gridDim.x, sc);
  }
#pragma unroll 1
  for (int k = 0; k < b.nops; k++) {
    const uint64_t count = b.count[k];
    const uint64_t done = batch_aligned16(b, k) ? count / kN * kN : 0;
    if (done == count) continue;
    __syncthreads();
    if (threadIdx.x < a.nranks) {
      s_src[threadIdx.x] = (const char*)b.send[k][threadIdx.x];
      s_dst[threadIdx.x] = (char*)b.recv[k][threadIdx.x];
    }
    __syncthreads();
    Scaler<typename AccOf<T>::type> sc{scaler_mode(a.op), a.scale};
    const Range mine = split_range(count - done, a.nranks, rank);
    reduce_store<T, Op, sizeof(T), 1, kMaxRanks>(s_src, a.nranks, s_dst, a.nranks, done + mine.beg, done + mine.end,
                                                 blockIdx.x, gridDim.x, sc);
  }
  if (!rank_barrier<true>(a, rank, a.epoch + 1, kDevTimeoutEnd)) return;
  batch_end(b, rank);
}

// Same, with the sum done by the switch (`multimem.ld_reduce`) and the broadcast by
// `multimem.st`. Every member must be 16-byte aligned and bound to a multicast mapping;
// the host only forms such batches.
template <typename T>
__global__ void __launch_bounds__(kMaxThreads) ar_nvls_batch_kernel(const __grid_constant__ BatchArgs b) {
  const CollArgs& a = b.base;
  const int rank = a.emulated ? (int)blockIdx.y : a.rank;
  using P = Pack<T, 16>;
  using Acc = typename P::Acc;
  __shared__ const char* s_src[kMaxRanks];
  __shared__ char* s_dst[kMaxRanks];
  if (!batch_begin(b, rank)) return;

  Scaler<Acc> sc{scaler_mode(a.op), a.scale};
  constexpr int kN = P::kN;
  constexpr int U = 4;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (int k = 0; k < b.nops; k++) {
    const uint64_t count = b.count[k];
    const uint64_t nv = count / kN;
    const Range mine = split_range(nv, a.nranks, rank);
    const char* mc_in = (const char*)b.mc_send[k];
    char* mc_out = (char*)b.mc_recv[k];
    auto emit = [&](uint64_t idx, Raw<16> v) {
      if (sc.mode == 2) {
        Acc acc[kN];
        P::unpack(v, acc);
#pragma unroll
        for (int e = 0; e < kN; e++) acc[e] = sc.div(acc[e]);
        v = P::pack(acc);
      }
      multimem_st16(mc_out + idx * 16, v);
    };
    uint64_t i = mine.beg + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + (uint64_t)(U - 1) * stride < mine.end; i += (uint64_t)U * stride) {
      Raw<16> v[U];
#pragma unroll
      for (int u = 0; u < U; u++) v[u] = Multimem<T>::ld_reduce_add(mc_in + (i + u * stride) * 16);
#pragma unroll
      for (int u = 0; u < U; u++) emit(i + u * stride, v[u]);
    }
    for (; i < mine.end; i += stride) emit(i, Multimem<T>::ld_reduce_add(mc_in + i * 16));
    // Sub-16-byte remainder of this member: plain peer loads/stores by rank 0.
    if (nv * kN < count) {
      __syncthreads();
      if (threadIdx.x < a.nranks) {
        s_src[threadIdx.x] = (const char*)b.send[k][threadIdx.x];
        s_dst[threadIdx.x] = (char*)b.recv[k][threadIdx.x];
      }
      __syncthreads();
      if (rank == 0)
        reduce_store_auto<T, OpSum, sizeof(T)>(s_src, a.nranks, s_dst, a.nranks, nv * kN, count,
                                               blockIdx.x, gridDim.x, sc);
    }
  }
  if (!rank_barrier<true>(a, rank, a.epoch + 1, kDevTimeoutEnd)) return;
  batch_end(b, rank);
}

}  // namespace dev
}  // namespace mccs
