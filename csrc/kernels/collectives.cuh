// sm_100a collective kernels: AllReduce (one-shot, two-shot, NVLS one-/two-shot,
// FIFO ring) and AllGather (pull, push, NVLS, FIFO ring). Every kernel moves the
// data itself with peer loads/stores or multimem instructions and fuses the
// reduction, the optional scaling and the cast back to the element type into that
// transfer; no copy or elementwise kernel runs before or after it.
//
// Reference counterpart: the single ring/Simple algorithm of
// src/collectives/src/all_reduce.h:6-87 and all_gather.h:6-71, whose every hop
// stages through an 8-slot FIFO. The ring variants here keep that scheme (they are
// what the host-staged transport and ring re-ordering use); the other variants
// have no counterpart there because the reference has no peer-memory transport.
#pragma once
#include <type_traits>

#include "dev_prims.cuh"

namespace mccs {
namespace dev {

constexpr int kMaxThreads = 512;  // 128 registers per thread available

struct Range { uint64_t beg, end; };
__device__ __forceinline__ Range split_range(uint64_t n, int parts, int idx) {
  uint64_t per = (n + (uint64_t)parts - 1) / (uint64_t)parts;
  Range r;
  r.beg = per * (uint64_t)idx; if (r.beg > n) r.beg = n;
  r.end = r.beg + per; if (r.end > n) r.end = n;
  return r;
}

// dst[d][i] = post(op_s pre(src[s][i])) for packs i in [pbeg, pend), distributed over
// `nparts` CTAs. Source 0..nsrc-1 are accumulated in index order, so every rank that
// evaluates the same element gets bit-identical results. `pre_mask` selects which
// sources get the PreMulSum multiplier (FIFO partial sums already carry it).
template <typename T, typename Op, int BYTES, int U, int MAXS>
__device__ __forceinline__ void reduce_store(const char* const* src, int nsrc, char* const* dst,
                                             int ndst, uint64_t pbeg, uint64_t pend, int part,
                                             int nparts,
                                             Scaler<typename AccOf<T>::type> sc,
                                             uint32_t pre_mask = 0xffffffffu) {
  using P = Pack<T, BYTES>;
  using Acc = typename P::Acc;
  const uint64_t stride = (uint64_t)nparts * blockDim.x;
  uint64_t i = pbeg + (uint64_t)part * blockDim.x + threadIdx.x;

  auto body = [&](auto uc, uint64_t base) {
    constexpr int UU = decltype(uc)::value;
    Raw<BYTES> v[UU][MAXS];
#pragma unroll
    for (int u = 0; u < UU; u++) {
#pragma unroll
      for (int s = 0; s < MAXS; s++) {
        if (s < nsrc) v[u][s] = ld_data<BYTES>(src[s] + (base + (uint64_t)u * stride) * BYTES);
      }
    }
#pragma unroll
    for (int u = 0; u < UU; u++) {
      Acc acc[P::kN];
      P::unpack(v[u][0], acc);
      if (sc.mode == 1 && (pre_mask & 1u)) {
#pragma unroll
        for (int e = 0; e < P::kN; e++) acc[e] = sc.mul(acc[e]);
      }
#pragma unroll
      for (int s = 1; s < MAXS; s++) {
        if (s < nsrc) {
          Acc x[P::kN];
          P::unpack(v[u][s], x);
          const bool pre = sc.mode == 1 && ((pre_mask >> s) & 1u);
#pragma unroll
          for (int e = 0; e < P::kN; e++) acc[e] = Op::apply(acc[e], pre ? sc.mul(x[e]) : x[e]);
        }
      }
      Raw<BYTES> out;
      if (nsrc == 1 && sc.mode == 0) {
        out = v[u][0];  // pure copy: keep the bits
      } else {
        if (sc.mode == 2) {
#pragma unroll
          for (int e = 0; e < P::kN; e++) acc[e] = sc.div(acc[e]);
        }
        out = P::pack(acc);
      }
#pragma unroll
      for (int d = 0; d < kMaxRanks; d++) {
        if (d < ndst) st_data<BYTES>(dst[d] + (base + (uint64_t)u * stride) * BYTES, out);
      }
    }
  };

  for (; i + (uint64_t)(U - 1) * stride < pend; i += (uint64_t)U * stride)
    body(std::integral_constant<int, U>{}, i);
  for (; i < pend; i += stride) body(std::integral_constant<int, 1>{}, i);
}

// Picks the unroll/source-count instantiation from the communicator size.
template <typename T, typename Op, int BYTES>
__device__ __forceinline__ void reduce_store_auto(const char* const* src, int nsrc,
                                                  char* const* dst, int ndst, uint64_t pbeg,
                                                  uint64_t pend, int part, int nparts,
                                                  Scaler<typename AccOf<T>::type> sc,
                                                  uint32_t pre_mask = 0xffffffffu) {
  if (BYTES < 16) {
    reduce_store<T, Op, BYTES, 1, kMaxRanks>(src, nsrc, dst, ndst, pbeg, pend, part, nparts, sc, pre_mask);
  } else if (nsrc > 4) {
    reduce_store<T, Op, BYTES, 2, kMaxRanks>(src, nsrc, dst, ndst, pbeg, pend, part, nparts, sc, pre_mask);
  } else {
    reduce_store<T, Op, BYTES, 4, 4>(src, nsrc, dst, ndst, pbeg, pend, part, nparts, sc, pre_mask);
  }
}

__device__ __forceinline__ bool all_aligned16(const CollArgs& a, uint64_t extra = 0) {
  uint64_t bits = extra;
  for (int r = 0; r < a.nranks; r++) bits |= (uint64_t)a.send[r] | (uint64_t)a.recv[r];
  return (bits & 15u) == 0;
}

__device__ __forceinline__ bool all_aligned32(const CollArgs& a) {
  uint64_t bits = 0;
  for (int r = 0; r < a.nranks; r++) bits |= (uint64_t)a.send[r] | (uint64_t)a.recv[r];
  return (bits & 31u) == 0;
}

__device__ __forceinline__ void trace_begin(const CollArgs& a, int rank) {
  if (a.trace && blockIdx.x == 0 && threadIdx.x == 0)
    st_relaxed_sys_u64(&a.status[rank]->start_ns, globaltimer_ns());
}
// End of a kernel, called by every thread of every CTA after its last store and its
// closing barrier. The rank's completion word (StatusBlock::done_seq) is what the host
// side reasons with (how much is queued on the GPU, when a tenant's admission credit is
// returned, when buffers may go away in client-side launch), so it must not be written
// while another CTA of the rank is still storing: each CTA's closing barrier only covers
// the CTAs with its own index on the peers. The CTAs therefore count themselves off and
// the last one publishes the word.
__device__ __forceinline__ void finish(const CollArgs& a, int rank) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();   // this CTA's stores are ordered before its count
    const unsigned last = gridDim.x - 1;
    if (atomicInc(&a.pad[rank]->pad_[kPadCtaCounter], last) == last) {
      fence_sys();     // ... and, through the counts, before the completion word
      if (a.trace) st_relaxed_sys_u64(&a.status[rank]->end_ns, globaltimer_ns());
      st_release_sys_u64(&a.status[rank]->done_seq, a.seq);
    }
  }
}

// ----------------------------------------------------------------------------
// AllReduce, one-shot: each rank reads every rank's whole input and keeps the
// result. Lowest latency; out-of-place only (a rank would otherwise overwrite
// input its peers still have to read).
// ----------------------------------------------------------------------------
template <typename T, typename Op>
__global__ void __launch_bounds__(kMaxThreads) ar_oneshot_kernel(const __grid_constant__ CollArgs a) {
  const int rank = a.emulated ? (int)blockIdx.y : a.rank;
  __shared__ const char* s_src[kMaxRanks];
  __shared__ char* s_dst[1];
  if (threadIdx.x < a.nranks) s_src[threadIdx.x] = (const char*)a.send[threadIdx.x];
  if (threadIdx.x == 0) s_dst[0] = (char*)a.recv[rank];
  trace_begin(a, rank);
  if (!rank_barrier<false>(a, rank, a.epoch, kDevTimeoutStart)) return;

  Scaler<typename AccOf<T>::type> sc{scaler_mode(a.op), a.scale};
  constexpr int kN = 16 / (int)sizeof(T);
  uint64_t done = 0;
  if (all_aligned16(a)) {
    const uint64_t nv = a.count / kN;
    reduce_store_auto<T, Op, 16>(s_src, a.nranks, s_dst, 1, 0, nv, blockIdx.x, gridDim.x, sc);
    done = nv * kN;
  }
  reduce_store_auto<T, Op, sizeof(T)>(s_src, a.nranks, s_dst, 1, done, a.count, blockIdx.x,
                                      gridDim.x, sc);
  // Nobody may leave (and let its caller reuse the input) while a peer still reads it.
  rank_barrier<false>(a, rank, a.epoch + 1, kDevTimeoutEnd);
  finish(a, rank);
}

// ----------------------------------------------------------------------------
// AllReduce, two-shot: rank r reduces shard r from all peers (reduce-scatter by
// loads) and stores the result into every rank's output (all-gather by stores).
// Safe in place: an element is read and then overwritten by the same thread only.
// ----------------------------------------------------------------------------
template <typename T, typename Op>
__global__ void __launch_bounds__(kMaxThreads) ar_twoshot_kernel(const __grid_constant__ CollArgs a) {
  const int rank = a.emulated ? (int)blockIdx.y : a.rank;
  __shared__ const char* s_src[kMaxRanks];
  __shared__ char* s_dst[kMaxRanks];
  if (threadIdx.x < a.nranks) {
    s_src[threadIdx.x] = (const char*)a.send[threadIdx.x];
    s_dst[threadIdx.x] = (char*)a.recv[threadIdx.x];
  }
  trace_begin(a, rank);
  if (!rank_barrier<false>(a, rank, a.epoch, kDevTimeoutStart)) return;

  Scaler<typename AccOf<T>::type> sc{scaler_mode(a.op), a.scale};
  constexpr int kN = 16 / (int)sizeof(T);
  uint64_t done = 0;
  // 256-bit packs (the daemon's `pack_bytes = 32`): 1 KiB per warp and instruction. Not for
  // 8-bit elements, whose 32 accumulators per pack would not fit the register budget.
  if (sizeof(T) >= 2 && a.unroll_hint == 32 && all_aligned32(a)) {
    constexpr int kN32 = sizeof(T) >= 2 ? 32 / (int)sizeof(T) : 16;
    const uint64_t nv = a.count / kN32;
    Range mine = split_range(nv, a.nranks, rank);
    if constexpr (sizeof(T) >= 2) {
      if (a.nranks > 4)
        reduce_store<T, Op, 32, 1, kMaxRanks>(s_src, a.nranks, s_dst, a.nranks, mine.beg, mine.end, blockIdx.x, gridDim.x, sc);
      else
        reduce_store<T, Op, 32, 2, 4>(s_src, a.nranks, s_dst, a.nranks, mine.beg, mine.end, blockIdx.x, gridDim.x, sc);
    }
    done = nv * kN32;
  } else if (all_aligned16(a)) {
    const uint64_t nv = a.count / kN;
    Range mine = split_range(nv, a.nranks, rank);
    reduce_store_auto<T, Op, 16>(s_src, a.nranks, s_dst, a.nranks, mine.beg, mine.end,
                                 blockIdx.x, gridDim.x, sc);
    done = nv * kN;
  }
  {
    // Leftover elements (or everything, when a buffer is not 16-byte aligned).
    Range mine = split_range(a.count - done, a.nranks, rank);
    reduce_store_auto<T, Op, sizeof(T)>(s_src, a.nranks, s_dst, a.nranks, done + mine.beg,
                                        done + mine.end, blockIdx.x, gridDim.x, sc);
  }
  rank_barrier<true>(a, rank, a.epoch + 1, kDevTimeoutEnd);
  finish(a, rank);
}

// ----------------------------------------------------------------------------
// AllReduce through NVLS. The switch performs the sum (`multimem.ld_reduce`, fp32
// accumulation for 16-bit types) and the broadcast (`multimem.st`).
// kTwoShot: rank r handles shard r and broadcasts it. Otherwise every rank reduces
// the whole buffer for itself (out-of-place only).
// ----------------------------------------------------------------------------
template <typename T, bool kTwoShot>
__global__ void __launch_bounds__(kMaxThreads) ar_nvls_kernel(const __grid_constant__ CollArgs a) {
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
  const uint64_t nv = a.count / kN;
  Range mine = kTwoShot ? split_range(nv, a.nranks, rank) : Range{0, nv};
  const char* mc_in = (const char*)a.mc_send;
  char* mc_out = (char*)a.mc_recv;
  char* local_out = (char*)a.recv[rank];
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  uint64_t i = mine.beg + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  auto emit = [&](uint64_t idx, Raw<16> v) {
    if (sc.mode == 2) {
      Acc acc[kN];
      P::unpack(v, acc);
#pragma unroll
      for (int e = 0; e < kN; e++) acc[e] = sc.div(acc[e]);
      v = P::pack(acc);
    }
    if (kTwoShot) multimem_st16(mc_out + idx * 16, v);
    else st_data<16>(local_out + idx * 16, v);
  };
  // In-switch loads in flight per thread before the first store (CollArgs::unroll_hint: 8,
  // anything else means 4).
  auto sweep = [&](auto uc) {
    constexpr int U = decltype(uc)::value;
    for (; i + (uint64_t)(U - 1) * stride < mine.end; i += (uint64_t)U * stride) {
      Raw<16> v[U];
#pragma unroll
      for (int u = 0; u < U; u++) v[u] = Multimem<T>::ld_reduce_add(mc_in + (i + u * stride) * 16);
#pragma unroll
      for (int u = 0; u < U; u++) emit(i + u * stride, v[u]);
    }
  };
  if (a.unroll_hint == 8) sweep(std::integral_constant<int, 8>{});
  else sweep(std::integral_constant<int, 4>{});
  for (; i < mine.end; i += stride) emit(i, Multimem<T>::ld_reduce_add(mc_in + i * 16));

  // Sub-16-byte remainder: plain peer loads/stores.
  if (nv * kN < a.count) {
    if (kTwoShot) {
      if (rank == 0)
        reduce_store_auto<T, OpSum, sizeof(T)>(s_src, a.nranks, s_dst, a.nranks, nv * kN, a.count,
                                               blockIdx.x, gridDim.x, sc);
    } else {
      reduce_store_auto<T, OpSum, sizeof(T)>(s_src, a.nranks, s_dst + rank, 1, nv * kN, a.count,
                                             blockIdx.x, gridDim.x, sc);
    }
  }
  if (kTwoShot) rank_barrier<true>(a, rank, a.epoch + 1, kDevTimeoutEnd);
  else rank_barrier<false>(a, rank, a.epoch + 1, kDevTimeoutEnd);
  finish(a, rank);
}

// ----------------------------------------------------------------------------
// Ring connection state of one channel (= one CTA) on one rank.
// ----------------------------------------------------------------------------
struct RingChan {
  char* recv_fifo;            // my receive FIFO for this channel
  char* send_fifo;            // successor's receive FIFO
  const uint64_t* my_tail;    // slots the predecessor has filled for me
  const uint64_t* my_head;    // slots of mine the successor has consumed
  uint64_t* next_tail;        // successor's tail (I publish my sends here)
  uint64_t* prev_head;        // predecessor's head (I return credits here)
  const uint32_t* abort_word;
  StatusBlock* status;
  uint64_t slot_bytes;
  uint64_t step;              // cumulative step counter (sends and receives advance together)
  uint64_t sends, recvs;      // per-launch counters on top of `step`
  uint64_t timeout_ns;
  int pos;                    // my position in this channel's ring
  bool failed;
};

__device__ __forceinline__ RingChan ring_open(const CollArgs& a, int rank) {
  RingChan ch;
  const int c = blockIdx.x;
  int pos = 0;
  for (int i = 0; i < a.nranks; i++) if (a.ring[c][i] == rank) pos = i;
  ch.pos = pos;
  const int next = a.ring[c][(pos + 1) % a.nranks];
  const int prev = a.ring[c][(pos + a.nranks - 1) % a.nranks];
  const uint64_t chan_bytes = a.fifo_slot_bytes * kRingSlots;
  ch.recv_fifo = a.fifo[rank] + (uint64_t)c * chan_bytes;
  ch.send_fifo = a.fifo[next] + (uint64_t)c * chan_bytes;
  ch.my_tail = &a.pad[rank]->ring_tail[c];
  ch.my_head = &a.pad[rank]->ring_head[c];
  ch.next_tail = &a.pad[next]->ring_tail[c];
  ch.prev_head = &a.pad[prev]->ring_head[c];
  ch.abort_word = &a.status[rank]->abort;
  ch.status = a.status[rank];
  ch.slot_bytes = a.fifo_slot_bytes;
  ch.step = a.ring_step_base[c];
  ch.sends = ch.recvs = 0;
  ch.timeout_ns = a.timeout_ns;
  ch.failed = false;
  return ch;
}

// One ring step. Inputs: the next FIFO slot from the predecessor (kRecv) and/or a
// local buffer; outputs: the successor's next FIFO slot (kSend) and/or a local
// buffer. `nbytes` may be zero (flags still advance so that all channels and ranks
// stay in lock-step).
template <typename T, typename Op, bool kRecv, bool kSend>
__device__ __forceinline__ void ring_step(RingChan& ch, const char* local_in, char* local_out,
                                          uint64_t nbytes, Scaler<typename AccOf<T>::type> sc,
                                          bool post) {
  if (ch.failed) return;
  __shared__ const char* s_src[2];
  __shared__ char* s_dst[2];
  uint32_t err = kDevOk;
  if (threadIdx.x == 0) {
    const uint64_t deadline = globaltimer_ns() + ch.timeout_ns;
    int ns = 0, nd = 0;
    if (kRecv) {
      const uint64_t s = ch.step + ch.recvs;
      err = wait_ge_u64(ch.my_tail, s + 1, deadline, ch.abort_word, kDevTimeoutRing);
      s_src[ns++] = ch.recv_fifo + (s % kRingSlots) * ch.slot_bytes;
    }
    if (local_in) s_src[ns++] = local_in;
    if (kSend && err == kDevOk) {
      const uint64_t s = ch.step + ch.sends;
      if (s + 1 > kRingSlots)
        err = wait_ge_u64(ch.my_head, s + 1 - kRingSlots, deadline, ch.abort_word, kDevTimeoutRing);
      s_dst[nd++] = ch.send_fifo + (s % kRingSlots) * ch.slot_bytes;
    }
    if (local_out) s_dst[nd++] = local_out;
    if (err != kDevOk) report_error(ch.status, err, (uint32_t)(ch.step + ch.recvs));
  }
  if (__syncthreads_or(err != kDevOk)) { ch.failed = true; return; }

  const int nsrc = (kRecv ? 1 : 0) + (local_in ? 1 : 0);
  const int ndst = (kSend ? 1 : 0) + (local_out ? 1 : 0);
  Scaler<typename AccOf<T>::type> s2 = sc;
  if (!post && s2.mode == 2) s2.mode = 0;
  // Only the local contribution gets the PreMulSum factor; a FIFO partial sum has it.
  const uint32_t pre_mask = kRecv ? 2u : 1u;
  if (nbytes > 0 && nsrc > 0 && ndst > 0) {
    uint64_t bits = (uint64_t)s_src[0] | (uint64_t)s_dst[0] | nbytes;
    if (nsrc > 1) bits |= (uint64_t)s_src[1];
    if (ndst > 1) bits |= (uint64_t)s_dst[1];
    if ((bits & 15u) == 0)
      reduce_store<T, Op, 16, 4, 2>(s_src, nsrc, s_dst, ndst, 0, nbytes / 16, 0, 1, s2, pre_mask);
    else
      reduce_store<T, Op, sizeof(T), 4, 2>(s_src, nsrc, s_dst, ndst, 0, nbytes / sizeof(T), 0, 1, s2, pre_mask);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (kSend) {
      fence_sys();
      st_release_sys_u64(ch.next_tail, ch.step + ch.sends + 1);
    }
    if (kRecv) st_release_sys_u64(ch.prev_head, ch.step + ch.recvs + 1);
  }
  if (kSend) ch.sends++;
  if (kRecv) ch.recvs++;
}

// ----------------------------------------------------------------------------
// AllReduce, FIFO ring (reduce-scatter then all-gather around the ring).
// ----------------------------------------------------------------------------
template <typename T, typename Op>
__global__ void __launch_bounds__(kMaxThreads) ar_ring_kernel(const __grid_constant__ CollArgs a) {
  const int rank = a.emulated ? (int)blockIdx.y : a.rank;
  const int n = a.nranks;
  trace_begin(a, rank);
  // Start barrier: every rank has left its previous collective, so FIFO counters
  // and the ring order may differ from the previous launch.
  if (!rank_barrier<false>(a, rank, a.epoch, kDevTimeoutStart)) return;
  RingChan ch = ring_open(a, rank);
  using Acc = typename AccOf<T>::type;
  Scaler<Acc> sc{scaler_mode(a.op), a.scale};
  const int pos = ch.pos;
  const int nch = gridDim.x;
  const uint64_t slot_elems = a.fifo_slot_bytes / sizeof(T);
  const uint64_t per_loop = slot_elems * (uint64_t)nch * (uint64_t)n;
  const uint64_t align = 16 / sizeof(T);
  const char* in = (const char*)a.send[rank];
  char* out = (char*)a.recv[rank];

  for (uint64_t base = 0; base < a.count; base += per_loop) {
    const uint64_t remaining = a.count - base;
    uint64_t chunk = (remaining + (uint64_t)(nch * n) - 1) / (uint64_t)(nch * n);
    chunk = (chunk + align - 1) / align * align;
    if (chunk > slot_elems) chunk = slot_elems;
    const uint64_t chan_base = base + (uint64_t)blockIdx.x * (uint64_t)n * chunk;
    auto span = [&](int j, uint64_t& off, uint64_t& len) {
      off = chan_base + (uint64_t)j * chunk;
      if (off >= a.count) { off = a.count; len = 0; }
      else { len = a.count - off; if (len > chunk) len = chunk; }
      off *= sizeof(T); len *= sizeof(T);
    };
    uint64_t off, len;
    // 1. push my copy of chunk (pos-1)
    span((pos + n - 1) % n, off, len);
    ring_step<T, Op, false, true>(ch, in + off, nullptr, len, sc, false);
    // 2. n-2 times: receive a partial sum, add mine, pass it on
    for (int j = 2; j < n; j++) {
      span((pos + n - j) % n, off, len);
      ring_step<T, Op, true, true>(ch, in + off, nullptr, len, sc, false);
    }
    // 3. chunk `pos` completes here: final value to my output and onwards
    span(pos, off, len);
    ring_step<T, Op, true, true>(ch, in + off, out + off, len, sc, true);
    // 4. n-2 times: receive a final chunk, keep it, pass it on
    for (int j = 1; j < n - 1; j++) {
      span((pos + n - j) % n, off, len);
      ring_step<T, Op, true, true>(ch, nullptr, out + off, len, sc, false);
    }
    // 5. last final chunk
    span((pos + 1) % n, off, len);
    ring_step<T, Op, true, false>(ch, nullptr, out + off, len, sc, false);
  }
  finish(a, rank);
}

// ----------------------------------------------------------------------------
// AllGather kernels. `count` is the per-rank byte count; rank r's data lands at
// recv + r*count on every rank.
// ----------------------------------------------------------------------------
enum AgMode { kAgModePull = 0, kAgModePush = 1, kAgModeNvls = 2 };

template <int MODE>
__global__ void __launch_bounds__(kMaxThreads) ag_direct_kernel(const __grid_constant__ CollArgs a) {
  const int rank = a.emulated ? (int)blockIdx.y : a.rank;
  const int n = a.nranks;
  __shared__ const char* s_src[kMaxRanks];
  __shared__ char* s_dst[kMaxRanks];
  if (threadIdx.x < n) {
    const int r = threadIdx.x;
    if (MODE == kAgModePull) {
      s_src[r] = (const char*)a.send[r];
      s_dst[r] = (char*)a.recv[rank] + (uint64_t)r * a.count;
    } else {
      s_src[r] = (const char*)a.send[rank];
      s_dst[r] = (char*)a.recv[r] + (uint64_t)rank * a.count;
    }
  }
  trace_begin(a, rank);
  if (!rank_barrier<false>(a, rank, a.epoch, kDevTimeoutStart)) return;

  const bool in_place = (const char*)a.send[rank] == (const char*)a.recv[rank] + (uint64_t)rank * a.count;
  const bool aligned = all_aligned16(a, a.count);
  // 256-bit packs (CollArgs::unroll_hint == 32, set by the daemon's `pack_bytes`): half as
  // many instructions and 1 KiB per warp and store, for buffers and sizes that allow it.
  uint64_t bits32 = a.count;
  for (int r = 0; r < n; r++) bits32 |= (uint64_t)a.send[r] | (uint64_t)a.recv[r];
  const bool wide = MODE != kAgModeNvls && a.unroll_hint == 32 && (bits32 & 31u) == 0;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const uint64_t first = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;

  auto run = [&](auto bytes_c) {
    constexpr int B = decltype(bytes_c)::value;
    const uint64_t np = a.count / B;
    if (MODE == kAgModePull) {
      for (uint64_t i = first; i < np; i += stride) {
        Raw<B> v[kMaxRanks];
#pragma unroll
        for (int s = 0; s < kMaxRanks; s++)
          if (s < n && !(in_place && s == rank)) v[s] = ld_data<B>(s_src[s] + i * B);
#pragma unroll
        for (int s = 0; s < kMaxRanks; s++)
          if (s < n && !(in_place && s == rank)) st_data<B>(s_dst[s] + i * B, v[s]);
      }
    } else {
      constexpr int U = B == 16 ? 4 : B == 32 ? 2 : 1;
      uint64_t i = first;
      auto emit = [&](uint64_t idx, Raw<B> v) {
        if (MODE == kAgModeNvls) {
          if constexpr (B == 16)
            multimem_st16((char*)a.mc_recv + (uint64_t)rank * a.count + idx * 16, v);
        } else {
#pragma unroll
          for (int d = 0; d < kMaxRanks; d++)
            if (d < n && !(in_place && d == rank)) st_data<B>(s_dst[d] + idx * B, v);
        }
      };
      for (; i + (uint64_t)(U - 1) * stride < np; i += (uint64_t)U * stride) {
        Raw<B> v[U];
#pragma unroll
        for (int u = 0; u < U; u++) v[u] = ld_data<B>(s_src[0] + (i + u * stride) * B);
#pragma unroll
        for (int u = 0; u < U; u++) emit(i + u * stride, v[u]);
      }
      for (; i < np; i += stride) emit(i, ld_data<B>(s_src[0] + i * B));
    }
  };
  // The planner only selects the NVLS mode for 16-byte aligned buffers and sizes.
  if (wide) run(std::integral_constant<int, 32>{});
  else if (aligned) run(std::integral_constant<int, 16>{});
  else if (MODE != kAgModeNvls) run(std::integral_constant<int, 1>{});
  else if (threadIdx.x == 0) report_error(a.status[rank], kDevBadArgs, 0);

  if (MODE == kAgModePull) rank_barrier<false>(a, rank, a.epoch + 1, kDevTimeoutEnd);
  else rank_barrier<true>(a, rank, a.epoch + 1, kDevTimeoutEnd);
  finish(a, rank);
}

#ifdef MCCS_UNTYPED_KERNELS
__global__ void __launch_bounds__(kMaxThreads) ag_ring_kernel(const __grid_constant__ CollArgs a) {
  const int rank = a.emulated ? (int)blockIdx.y : a.rank;
  const int n = a.nranks;
  trace_begin(a, rank);
  if (!rank_barrier<false>(a, rank, a.epoch, kDevTimeoutStart)) return;
  RingChan ch = ring_open(a, rank);
  Scaler<uint32_t> sc{0, 1.0f};
  const int pos = ch.pos;
  const int nch = gridDim.x;
  const uint64_t per_loop = a.fifo_slot_bytes * (uint64_t)nch;
  const char* in = (const char*)a.send[rank];
  char* out = (char*)a.recv[rank];
  const bool in_place = in == out + (uint64_t)rank * a.count;

  for (uint64_t base = 0; base < a.count; base += per_loop) {
    const uint64_t remaining = a.count - base;
    uint64_t chunk = (remaining + (uint64_t)nch - 1) / (uint64_t)nch;
    chunk = (chunk + 15) / 16 * 16;
    if (chunk > a.fifo_slot_bytes) chunk = a.fifo_slot_bytes;
    uint64_t off = base + (uint64_t)blockIdx.x * chunk;
    uint64_t len = 0;
    if (off >= a.count) off = a.count;
    else { len = a.count - off; if (len > chunk) len = chunk; }
    // my shard: to the successor, and into my own output when out of place
    ring_step<uint8_t, OpSum, false, true>(ch, in + off,
                                           in_place ? nullptr : out + (uint64_t)rank * a.count + off,
                                           len, sc, false);
    for (int j = 1; j < n - 1; j++) {
      const int src_rank = a.ring[blockIdx.x][(pos + n - j) % n];
      ring_step<uint8_t, OpSum, true, true>(ch, nullptr, out + (uint64_t)src_rank * a.count + off,
                                            len, sc, false);
    }
    const int last_rank = a.ring[blockIdx.x][(pos + 1) % n];
    ring_step<uint8_t, OpSum, true, false>(ch, nullptr, out + (uint64_t)last_rank * a.count + off,
                                           len, sc, false);
  }
  finish(a, rank);
}

// Single-rank communicator: the collective degenerates to a device copy (nothing at all
// in place). Both buffers are local by construction, so plain loads and stores are used,
// and the launcher sizes the grid from the message: one CTA per kCopyTileBytes, far more
// CTAs than SMs for a large message. Measured on a B200 with 512 MiB: this shape moves
// 6.7 TB/s (read + write), a persistent grid of one to eight CTAs per SM with the same
// inner loop 5.8-6.2 TB/s, the driver's own device-to-device copy 6.3 TB/s. Any grid
// works (the tile loop strides by the grid), which is what the CPU emulation uses.
__global__ void __launch_bounds__(kMaxThreads) local_copy_kernel(const __grid_constant__ CollArgs a) {
  const int rank = a.emulated ? (int)blockIdx.y : a.rank;
  trace_begin(a, rank);
  const char* in = (const char*)a.send[rank];
  char* out = (char*)a.recv[rank];
  const uint64_t bytes = a.count;  // the launcher converts elements to bytes
  if (in != out) {
    uint64_t done = 0;
    if ((((uint64_t)in | (uint64_t)out) & 15u) == 0) {
      const uint64_t nv = bytes / 16;
      const uint64_t tile = (uint64_t)blockDim.x * kCopyUnroll;
      const Raw<16>* src = (const Raw<16>*)in;
      Raw<16>* dst = (Raw<16>*)out;
      for (uint64_t base = (uint64_t)blockIdx.x * tile; base < nv; base += (uint64_t)gridDim.x * tile) {
        const uint64_t i = base + threadIdx.x;
        if (base + tile <= nv) {
          Raw<16> v[kCopyUnroll];
#pragma unroll
          for (int u = 0; u < kCopyUnroll; u++) v[u] = src[i + (uint64_t)u * blockDim.x];
#pragma unroll
          for (int u = 0; u < kCopyUnroll; u++) dst[i + (uint64_t)u * blockDim.x] = v[u];
        } else {
          for (uint64_t j = i; j < nv; j += blockDim.x) dst[j] = src[j];
        }
      }
      done = nv * 16;
    }
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = done + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < bytes; i += stride) out[i] = in[i];
  }
  finish(a, rank);
}

#endif  // MCCS_UNTYPED_KERNELS

}  // namespace dev
}  // namespace mccs
