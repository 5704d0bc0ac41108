// ReduceScatter: every rank contributes nranks * count elements and keeps the reduction
// of block `rank` (count elements). The reference offers AllReduce and AllGather only
// (src/ipc/mccs/src/command.rs:88-112); frameworks that shard optimizer state or
// gradients (ZeRO / FSDP style) need this half of an AllReduce by itself, at half its
// traffic.
//
//   rs_direct : rank r loads block r from every rank over NVLink, reduces in registers
//               (fp32 accumulation for 16-bit floats) and stores locally: the first phase
//               of the two-shot AllReduce with a local destination.
//   rs_nvls   : `multimem.ld_reduce` of block r, the sum happens in the NVSwitch.
//
// Both are safe in place (recv == send + rank * count): a rank overwrites only its own
// block of its own input, which no other rank reads.
#pragma once
#include "collectives.cuh"

namespace mccs {
namespace dev {

template <typename T, typename Op>
__global__ void __launch_bounds__(kMaxThreads) rs_direct_kernel(const __grid_constant__ CollArgs a) {
  const int rank = a.emulated ? (int)blockIdx.y : a.rank;
  __shared__ const char* s_src[kMaxRanks];
  __shared__ char* s_dst[1];
  const uint64_t block_bytes = a.count * sizeof(T);
  if (threadIdx.x < a.nranks) s_src[threadIdx.x] = (const char*)a.send[threadIdx.x] + (uint64_t)rank * block_bytes;
  if (threadIdx.x == 0) s_dst[0] = (char*)a.recv[rank];
  trace_begin(a, rank);
  if (!rank_barrier<false>(a, rank, a.epoch, kDevTimeoutStart)) return;

  Scaler<typename AccOf<T>::type> sc{scaler_mode(a.op), a.scale};
  constexpr int kN = 16 / (int)sizeof(T);
  uint64_t done = 0;
  if (all_aligned16(a, block_bytes)) {   // the blocks start on 16-byte boundaries too
    const uint64_t nv = a.count / kN;
    reduce_store_auto<T, Op, 16>(s_src, a.nranks, s_dst, 1, 0, nv, blockIdx.x, gridDim.x, sc);
    done = nv * kN;
  }
  reduce_store_auto<T, Op, sizeof(T)>(s_src, a.nranks, s_dst, 1, done, a.count, blockIdx.x, gridDim.x, sc);
  // Nobody may leave (and let its caller reuse the input) while a peer still reads it.
  rank_barrier<false>(a, rank, a.epoch + 1, kDevTimeoutEnd);
  finish(a, rank);
}

// Sum (and average) of f32 / f16 / bf16; the planner selects it only for 16-byte aligned
// buffers and block sizes bound to a multicast mapping.
template <typename T>
__global__ void __launch_bounds__(kMaxThreads) rs_nvls_kernel(const __grid_constant__ CollArgs a) {
  const int rank = a.emulated ? (int)blockIdx.y : a.rank;
  using P = Pack<T, 16>;
  using Acc = typename P::Acc;
  constexpr int kN = P::kN;
  trace_begin(a, rank);
  if (!rank_barrier<false>(a, rank, a.epoch, kDevTimeoutStart)) return;

  const uint64_t block_bytes = a.count * sizeof(T);
  if ((a.count % kN) != 0 || !all_aligned16(a, block_bytes)) {
    if (threadIdx.x == 0 && blockIdx.x == 0) report_error(a.status[rank], kDevBadArgs, 0);
  } else {
    Scaler<Acc> sc{scaler_mode(a.op), a.scale};
    const char* mc_in = (const char*)a.mc_send + (uint64_t)rank * block_bytes;
    char* out = (char*)a.recv[rank];
    const uint64_t nv = a.count / kN;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    constexpr int U = 4;
    auto emit = [&](uint64_t idx, Raw<16> v) {
      if (sc.mode == 2) {
        Acc acc[kN];
        P::unpack(v, acc);
#pragma unroll
        for (int e = 0; e < kN; e++) acc[e] = sc.div(acc[e]);
        v = P::pack(acc);
      }
      st_data<16>(out + idx * 16, v);
    };
    for (; i + (uint64_t)(U - 1) * stride < nv; i += (uint64_t)U * stride) {
      Raw<16> v[U];
#pragma unroll
      for (int u = 0; u < U; u++) v[u] = Multimem<T>::ld_reduce_add(mc_in + (i + u * stride) * 16);
#pragma unroll
      for (int u = 0; u < U; u++) emit(i + u * stride, v[u]);
    }
    for (; i < nv; i += stride) emit(i, Multimem<T>::ld_reduce_add(mc_in + i * 16));
  }
  rank_barrier<false>(a, rank, a.epoch + 1, kDevTimeoutEnd);
  finish(a, rank);
}

}  // namespace dev
}  // namespace mccs
