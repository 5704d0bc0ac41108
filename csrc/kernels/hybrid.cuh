// AllReduce through the switch AND around it at the same time.
//
// Measured on 8 x B200, the in-switch reduction (`multimem.ld_reduce` + `multimem.st`)
// moves only one byte per message byte over each GPU's links but tops out at 0.63 of the
// links' copy rate, while the plain two-shot exchange needs 1.75 bytes per byte and runs
// the links at 0.85. If the first limit sits in the switch's reduction/multicast path and
// not in the links, the two can run side by side: this kernel gives the head of the
// buffer to a few CTAs that use the multimem path and the rest to the other CTAs, which
// exchange it with ordinary peer loads and stores. Both parts share the kernel's two
// cross-rank barriers. Where to cut and how many CTAs each part gets come with the
// launch (`CollArgs::unroll_hint`: low 16 bits = share of the message for the multimem
// part in 1/1000, high 16 bits = its CTA count).
//
// Sum (and average) of f32 / f16 / bf16 on 16-byte aligned buffers bound to multicast
// mappings, like the NVLS variants. The reference has no counterpart (one ring algorithm).
#pragma once
#include "collectives.cuh"

namespace mccs {
namespace dev {

template <typename T>
__global__ void __launch_bounds__(kMaxThreads) ar_hybrid_kernel(const __grid_constant__ CollArgs a) {
  const int rank = a.emulated ? (int)blockIdx.y : a.rank;
  using P = Pack<T, 16>;
  using Acc = typename P::Acc;
  __shared__ const char* s_src[kMaxRanks];
  __shared__ char* s_dst[kMaxRanks];
  if (threadIdx.x < a.nranks) {
    s_src[threadIdx.x] = (const char*)a.send[threadIdx.x];
    s_dst[threadIdx.x] = (char*)a.recv[threadIdx.x];
  }
  trace_begin(a, rank);
  if (!rank_barrier<false>(a, rank, a.epoch, kDevTimeoutStart)) return;

  Scaler<Acc> sc{scaler_mode(a.op), a.scale};
  constexpr int kN = P::kN;
  const uint64_t nv = a.count / kN;   // 16-byte packs in the message
  int nvls_ctas = (int)(((uint32_t)a.unroll_hint) >> 16);
  const uint32_t permille = ((uint32_t)a.unroll_hint) & 0xffffu;
  if (nvls_ctas > (int)gridDim.x) nvls_ctas = (int)gridDim.x;
  // Packs [0, cut) go through the switch, [cut, nv) around it. Either part may be empty;
  // a part without CTAs gets no packs.
  uint64_t cut = nv * (uint64_t)(permille > 1000u ? 1000u : permille) / 1000u;
  if (nvls_ctas == 0) cut = 0;
  if (nvls_ctas == (int)gridDim.x) cut = nv;

  if ((int)blockIdx.x < nvls_ctas) {
    Range part = split_range(cut, a.nranks, rank);   // rank r reduces and broadcasts shard r of the head
    const char* mc_in = (const char*)a.mc_send;
    char* mc_out = (char*)a.mc_recv;
    const uint64_t stride = (uint64_t)nvls_ctas * blockDim.x;
    uint64_t i = part.beg + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    constexpr int U = 4;
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
    for (; i + (uint64_t)(U - 1) * stride < part.end; i += (uint64_t)U * stride) {
      Raw<16> v[U];
#pragma unroll
      for (int u = 0; u < U; u++) v[u] = Multimem<T>::ld_reduce_add(mc_in + (i + u * stride) * 16);
#pragma unroll
      for (int u = 0; u < U; u++) emit(i + u * stride, v[u]);
    }
    for (; i < part.end; i += stride) emit(i, Multimem<T>::ld_reduce_add(mc_in + i * 16));
  } else {
    const int cta = (int)blockIdx.x - nvls_ctas;
    const int nctas = (int)gridDim.x - nvls_ctas;
    Range part = split_range(nv - cut, a.nranks, rank);   // rank r's shard of the tail
    reduce_store_auto<T, OpSum, 16>(s_src, a.nranks, s_dst, a.nranks, cut + part.beg, cut + part.end, cta, nctas, sc);
  }
  // Elements beyond the last full pack: plain loads and stores by rank 0, spread over all CTAs.
  if (nv * kN < a.count && rank == 0)
    reduce_store_auto<T, OpSum, sizeof(T)>(s_src, a.nranks, s_dst, a.nranks, nv * kN, a.count, blockIdx.x, gridDim.x, sc);
  rank_barrier<true>(a, rank, a.epoch + 1, kDevTimeoutEnd);
  finish(a, rank);
}

}  // namespace dev
}  // namespace mccs
