// Runs the collective kernels — the very source the GPU build compiles — on the CPU
// through the SIMT emulator of sim/simt_sim.h and checks every variant against a plain
// reduction: AllReduce one-shot / two-shot / NVLS one- and two-shot / FIFO ring, AllGather
// pull / push / NVLS / ring, the single-rank copy and the fused (batch) kernels with their
// options, for 2, 3, 4 and 8 ranks, odd sizes, unaligned buffers, in place, several
// element types and operators, back-to-back launches that reuse the signal pads, ranks on
// one "device" (grid.y = rank) or one launch per rank; and the error path: a peer that
// never shows up makes the others give up within the bound and report it.
//
// The reference has no test of its device code at all.
#include "sim/simt_sim.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include <random>
#include <string>

#define MCCS_UNTYPED_KERNELS 1
#include "../kernels/batch.cuh"
#include "../kernels/hybrid.cuh"
#include "../kernels/scatter.cuh"

using namespace mccs;
using namespace mccs::dev;

namespace {

int g_checks = 0, g_failed = 0;
#define CHECK(cond)                                                                  \
  do {                                                                               \
    g_checks++;                                                                      \
    if (!(cond)) { g_failed++; fprintf(stderr, "%s:%d: CHECK(%s) failed\n", __FILE__, __LINE__, #cond); } \
  } while (0)

template <typename T> struct Dt;
template <> struct Dt<float> { static constexpr int id = kFloat32; static float to(double v) { return (float)v; } static double from(float v) { return v; } };
template <> struct Dt<double> { static constexpr int id = kFloat64; static double to(double v) { return v; } static double from(double v) { return v; } };
template <> struct Dt<int32_t> { static constexpr int id = kInt32; static int32_t to(double v) { return (int32_t)v; } static double from(int32_t v) { return v; } };
template <> struct Dt<uint8_t> { static constexpr int id = kUint8; static uint8_t to(double v) { return (uint8_t)v; } static double from(uint8_t v) { return v; } };
template <> struct Dt<int64_t> { static constexpr int id = kInt64; static int64_t to(double v) { return (int64_t)v; } static double from(int64_t v) { return (double)v; } };
template <> struct Dt<__nv_bfloat16> {
  static constexpr int id = kBfloat16;
  static __nv_bfloat16 to(double v) { return __float2bfloat16_rn((float)v); }
  static double from(__nv_bfloat16 v) { return __bfloat162float(v); }
};
template <> struct Dt<__half> {
  static constexpr int id = kFloat16;
  static __half to(double v) { return __float2half_rn((float)v); }
  static double from(__half v) { return __half2float(v); }
};

// What one communicator owns: pads, status blocks, FIFOs, and the running counters the
// daemon keeps (barrier epoch, tickets, ring steps).
// CollArgs::unroll_hint for the cases that follow (0 = the kernels' default paths; 32 = 256-bit
// packs in two-shot and pull/push; 8 = deeper unroll of the in-switch kernels).
static int g_unroll_hint = 0;

struct World {
  int n;
  std::vector<SignalPad*> pad;
  std::vector<StatusBlock*> status;
  std::vector<char*> fifo;
  uint64_t fifo_slot_bytes = 4096;
  uint32_t epoch = 1;
  uint64_t ticket = 0;
  uint64_t ring_steps[kMaxRingChannels] = {0};
  explicit World(int nranks) : n(nranks) {
    for (int r = 0; r < n; r++) {
      pad.push_back((SignalPad*)aligned_alloc(128, sizeof(SignalPad)));
      memset(pad.back(), 0, sizeof(SignalPad));
      status.push_back((StatusBlock*)aligned_alloc(64, sizeof(StatusBlock)));
      memset(status.back(), 0, sizeof(StatusBlock));
      fifo.push_back((char*)aligned_alloc(128, fifo_slot_bytes * kRingSlots * 4));
    }
  }
  ~World() {
    for (int r = 0; r < n; r++) { free(pad[(size_t)r]); free(status[(size_t)r]); free(fifo[(size_t)r]); }
  }
  CollArgs base(int dtype, int op, int variant, uint64_t count, bool emulated) {
    CollArgs a;
    memset(&a, 0, sizeof a);
    a.nranks = n;
    a.emulated = emulated ? 1 : 0;
    a.dtype = dtype; a.op = op; a.variant = variant;
    a.count = count;
    a.seq = ++ticket;
    a.scale = op == kSumPostDiv ? 1.0f / (float)n : 1.0f;
    a.epoch = epoch;
    epoch += 2;
    a.timeout_ns = 20ull * 1000 * 1000 * 1000;
    a.unroll_hint = g_unroll_hint;
    for (int r = 0; r < n; r++) { a.pad[r] = pad[(size_t)r]; a.status[r] = status[(size_t)r]; a.fifo[r] = fifo[(size_t)r]; }
    a.fifo_slot_bytes = fifo_slot_bytes;
    for (int ch = 0; ch < kMaxRingChannels; ch++) {
      for (int i = 0; i < n; i++) a.ring[ch][i] = (int8_t)((ch % 2) ? (n - 1 - i) : i);   // odd channels run the ring backwards
      a.ring_step_base[ch] = ring_steps[ch];
    }
    return a;
  }
  // After a kernel that ran to its end: no error, the completion word names this launch,
  // and the counter of finished CTAs is back at zero (it wraps at the grid size).
  int finished_cleanly(int r, uint64_t seq) const {
    return status[(size_t)r]->error == 0 && status[(size_t)r]->done_seq == seq && pad[(size_t)r]->pad_[kPadCtaCounter] == 0 ? 0 : 1;
  }
  void account_ring(int kind, uint64_t count, int esz, int nch) {
    const uint64_t steps = ring_steps_per_channel(kind, count, esz, n, nch, fifo_slot_bytes);
    for (int ch = 0; ch < nch; ch++) ring_steps[ch] += steps;
  }
};

// Launches `kernel` for all ranks: one grid with grid.y = rank ("emulated" placement) or
// one grid per rank, all running concurrently either way.
template <typename Kernel, typename Args>
void run_all(Kernel kernel, Args a, int n, int ctas, int threads, bool emulated, int skip_rank = -1) {
  std::vector<std::thread> pool;
  CollArgs* base = (CollArgs*)&a;   // CollArgs itself, or the first member of BatchArgs
  if (emulated) {
    sim::Dim3 grid; grid.x = (unsigned)ctas; grid.y = (unsigned)n;
    sim::launch(kernel, grid, (unsigned)threads, a, &pool);
  } else {
    for (int r = 0; r < n; r++) {
      if (r == skip_rank) continue;
      base->rank = r;
      sim::Dim3 grid; grid.x = (unsigned)ctas;
      sim::launch(kernel, grid, (unsigned)threads, a, &pool);
    }
  }
  sim::join_all(&pool);
}

template <typename T>
struct Buffers {
  int n; size_t count; size_t offset;   // offset in elements: buffers start `offset` elements into a 16-byte aligned block
  std::vector<T*> send_block, recv_block;
  Buffers(int nranks, size_t cnt, size_t off, size_t recv_factor = 1) : n(nranks), count(cnt), offset(off) {
    for (int r = 0; r < n; r++) {
      send_block.push_back((T*)aligned_alloc(64, ((cnt + off) * sizeof(T) + 127) / 64 * 64));
      recv_block.push_back((T*)aligned_alloc(64, ((cnt * recv_factor + off) * sizeof(T) + 127) / 64 * 64));
      memset(recv_block.back(), 0xEE, (cnt * recv_factor + off) * sizeof(T));
    }
  }
  ~Buffers() { for (int r = 0; r < n; r++) { free(send_block[(size_t)r]); free(recv_block[(size_t)r]); } }
  T* send(int r) { return send_block[(size_t)r] + offset; }
  T* recv(int r) { return recv_block[(size_t)r] + offset; }
};

double reduce_ref(int op, const std::vector<double>& xs, int n) {
  double acc = xs[0];
  for (size_t i = 1; i < xs.size(); i++) {
    switch (op) {
      case kProd: acc *= xs[i]; break;
      case kMax: acc = acc > xs[i] ? acc : xs[i]; break;
      case kMin: acc = acc < xs[i] ? acc : xs[i]; break;
      default: acc += xs[i]; break;
    }
  }
  if (op == kSumPostDiv) acc /= n;
  return acc;
}

template <typename T> double tolerance(int n) {
  if (std::is_same<T, __nv_bfloat16>::value) return 0.02 * n;
  if (std::is_same<T, __half>::value) return 0.004 * n;
  if (std::is_same<T, float>::value) return 1e-5 * n;
  return 0.0;
}

// One AllReduce through `variant`, checked on every rank.
template <typename T, typename Op>
void allreduce_case(World& w, int variant, int op, size_t count, int ctas, int threads, bool emulated, size_t offset,
                    bool in_place, const char* what) {
  const int n = w.n;
  Buffers<T> b(n, count, offset);
  std::mt19937 rng((unsigned)(count * 31 + (size_t)variant * 7 + (size_t)n));
  std::vector<std::vector<double>> in((size_t)n, std::vector<double>(count));
  for (int r = 0; r < n; r++)
    for (size_t i = 0; i < count; i++) {
      double v = op == kProd ? 1.0 + (double)(rng() % 3) * 0.25 : (double)((int)(rng() % 17) - 8);
      if (std::is_same<T, uint8_t>::value) v = (double)(rng() % 9);
      b.send(r)[i] = Dt<T>::to(v);
      in[(size_t)r][i] = Dt<T>::from(b.send(r)[i]);
    }
  CollArgs a = w.base(Dt<T>::id, op, variant, count, emulated);
  for (int r = 0; r < n; r++) {
    a.send[r] = b.send(r);
    a.recv[r] = in_place ? (void*)b.send(r) : (void*)b.recv(r);
  }
  const bool nvls = variant == kArNvlsOne || variant == kArNvlsTwo;
  if (nvls) {
    // emulated multicast mappings of the send and the receive buffers
    sim_mc_regions().clear();
    SimMcRegion ms{0x100000000000ull, (count * sizeof(T) + 15) / 16 * 16, {}}, mr{0x200000000000ull, (count * sizeof(T) + 15) / 16 * 16, {}};
    for (int r = 0; r < n; r++) { ms.backing.push_back((char*)a.send[r]); mr.backing.push_back((char*)a.recv[r]); }
    sim_mc_regions().push_back(ms);
    sim_mc_regions().push_back(mr);
    a.mc_send = (const void*)ms.base;
    a.mc_recv = (void*)mr.base;
  }
  switch (variant) {
    case kArOneShot: run_all(ar_oneshot_kernel<T, Op>, a, n, ctas, threads, emulated); break;
    case kArTwoShot: run_all(ar_twoshot_kernel<T, Op>, a, n, ctas, threads, emulated); break;
    case kArRing: run_all(ar_ring_kernel<T, Op>, a, n, ctas, threads, emulated); w.account_ring(kAllReduce, count, sizeof(T), ctas); break;
    default: break;
  }
  if constexpr (std::is_same<T, float>::value || std::is_same<T, __nv_bfloat16>::value || std::is_same<T, __half>::value) {
    if (variant == kArNvlsOne) run_all(ar_nvls_kernel<T, false>, a, n, ctas, threads, emulated);
    if (variant == kArNvlsTwo) run_all(ar_nvls_kernel<T, true>, a, n, ctas, threads, emulated);
  }
  const double tol = tolerance<T>(n);
  int bad = 0;
  for (size_t i = 0; i < count && bad < 4; i++) {
    std::vector<double> xs;
    for (int r = 0; r < n; r++) xs.push_back(in[(size_t)r][i]);
    const double want = reduce_ref(op, xs, n);
    for (int r = 0; r < n; r++) {
      const double got = Dt<T>::from(((T*)a.recv[r])[i]);
      if (fabs(got - want) > tol + 1e-3 * fabs(want) * (tol > 0 ? 1 : 0)) {
        if (bad++ < 3) fprintf(stderr, "  %s: rank %d elem %zu: got %g want %g\n", what, r, i, got, want);
      }
    }
  }
  // every rank holds bit-identical results
  for (int r = 1; r < n; r++) bad += memcmp(a.recv[0], a.recv[r], count * sizeof(T)) != 0;
  for (int r = 0; r < n; r++) bad += w.finished_cleanly(r, a.seq);
  if (bad) fprintf(stderr, "FAILED %s (n=%d count=%zu ctas=%d emulated=%d offset=%zu in_place=%d)\n", what, n, count, ctas,
                   (int)emulated, offset, (int)in_place);
  CHECK(bad == 0);
}

// One ReduceScatter: rank r must end up with the reduction of block r, and nothing else of
// anybody's buffers may change (apart from the rank's own block when it works in place).
template <typename T, typename Op>
void reduce_scatter_case(World& w, int variant, int op, size_t count, int ctas, int threads, bool emulated, size_t offset,
                         bool in_place, const char* what) {
  const int n = w.n;
  Buffers<T> b(n, count * (size_t)n, offset);
  std::mt19937 rng((unsigned)(count * 13 + (size_t)variant * 5 + (size_t)n));
  std::vector<std::vector<double>> in((size_t)n, std::vector<double>(count * (size_t)n));
  for (int r = 0; r < n; r++)
    for (size_t i = 0; i < count * (size_t)n; i++) {
      double v = (double)((int)(rng() % 17) - 8);
      if (std::is_same<T, uint8_t>::value) v = (double)(rng() % 9);   // no wrap-around in the sum
      b.send(r)[i] = Dt<T>::to(v);
      in[(size_t)r][i] = Dt<T>::from(b.send(r)[i]);
    }
  CollArgs a = w.base(Dt<T>::id, op, variant, count, emulated);
  for (int r = 0; r < n; r++) {
    a.send[r] = b.send(r);
    a.recv[r] = in_place ? (void*)(b.send(r) + (size_t)r * count) : (void*)b.recv(r);
  }
  if (variant == kRsNvls) {
    sim_mc_regions().clear();
    SimMcRegion ms{0x100000000000ull, (count * (size_t)n * sizeof(T) + 15) / 16 * 16, {}};
    for (int r = 0; r < n; r++) ms.backing.push_back((char*)a.send[r]);
    sim_mc_regions().push_back(ms);
    a.mc_send = (const void*)ms.base;
  }
  if (variant == kRsDirect) run_all(rs_direct_kernel<T, Op>, a, n, ctas, threads, emulated);
  if constexpr (std::is_same<T, float>::value || std::is_same<T, __nv_bfloat16>::value || std::is_same<T, __half>::value) {
    if (variant == kRsNvls) run_all(rs_nvls_kernel<T>, a, n, ctas, threads, emulated);
  }
  const double tol = tolerance<T>(n);
  int bad = 0;
  for (int r = 0; r < n; r++) {
    for (size_t i = 0; i < count && bad < 4; i++) {
      std::vector<double> xs;
      for (int q = 0; q < n; q++) xs.push_back(in[(size_t)q][(size_t)r * count + i]);
      const double want = reduce_ref(op, xs, n);
      const double got = Dt<T>::from(((T*)a.recv[r])[i]);
      if (fabs(got - want) > tol + 1e-3 * fabs(want) * (tol > 0 ? 1 : 0)) {
        if (bad++ < 3) fprintf(stderr, "  %s: rank %d elem %zu: got %g want %g\n", what, r, i, got, want);
      }
    }
    // the inputs outside the rank's own block are untouched
    for (size_t i = 0; i < count * (size_t)n; i++) {
      if (in_place && i / count == (size_t)r) continue;
      if (Dt<T>::from(b.send(r)[i]) != in[(size_t)r][i]) { bad++; break; }
    }
    bad += w.status[(size_t)r]->error != 0;
  }
  if (bad) fprintf(stderr, "FAILED %s (n=%d count=%zu ctas=%d emulated=%d offset=%zu in_place=%d)\n", what, n, count, ctas,
                   (int)emulated, offset, (int)in_place);
  CHECK(bad == 0);
}

void allgather_case(World& w, int variant, size_t bytes, int ctas, int threads, bool emulated, size_t offset, bool in_place,
                    const char* what) {
  const int n = w.n;
  Buffers<uint8_t> b(n, bytes, offset, (size_t)n);
  for (int r = 0; r < n; r++)
    for (size_t i = 0; i < bytes; i++) b.send(r)[i] = (uint8_t)(r * 37 + i * 11 + 1);
  CollArgs a = w.base(kUint8, kSum, variant, bytes, emulated);
  for (int r = 0; r < n; r++) {
    a.recv[r] = b.recv(r);
    if (in_place) {
      memcpy(b.recv(r) + (size_t)r * bytes, b.send(r), bytes);
      a.send[r] = b.recv(r) + (size_t)r * bytes;
    } else {
      a.send[r] = b.send(r);
    }
  }
  if (variant == kAgNvls) {
    sim_mc_regions().clear();
    SimMcRegion mr{0x200000000000ull, (bytes * (size_t)n + 15) / 16 * 16, {}};
    for (int r = 0; r < n; r++) mr.backing.push_back((char*)a.recv[r]);
    sim_mc_regions().push_back(mr);
    a.mc_recv = (void*)mr.base;
  }
  switch (variant) {
    case kAgPull: run_all(ag_direct_kernel<kAgModePull>, a, n, ctas, threads, emulated); break;
    case kAgPush: run_all(ag_direct_kernel<kAgModePush>, a, n, ctas, threads, emulated); break;
    case kAgNvls: run_all(ag_direct_kernel<kAgModeNvls>, a, n, ctas, threads, emulated); break;
    case kAgRing: run_all(ag_ring_kernel, a, n, ctas, threads, emulated); w.account_ring(kAllGather, bytes, 1, ctas); break;
  }
  int bad = 0;
  for (int r = 0; r < n; r++) {
    for (int s = 0; s < n; s++)
      for (size_t i = 0; i < bytes; i++)
        if (b.recv(r)[(size_t)s * bytes + i] != (uint8_t)(s * 37 + i * 11 + 1)) { bad++; break; }
    bad += w.finished_cleanly(r, a.seq);
  }
  if (bad) fprintf(stderr, "FAILED %s (n=%d bytes=%zu ctas=%d emulated=%d offset=%zu in_place=%d)\n", what, n, bytes, ctas,
                   (int)emulated, offset, (int)in_place);
  CHECK(bad == 0);
}

// The hybrid kernel: `permille` of the message through the (emulated) switch on the first
// `nvls_ctas` CTAs, the rest by peer loads/stores on the others.
template <typename T>
void hybrid_case(World& w, size_t count, int ctas, int nvls_ctas, int permille, int threads, bool emulated, bool in_place, int op) {
  const int n = w.n;
  Buffers<T> b(n, count, 0);
  std::vector<std::vector<double>> in((size_t)n, std::vector<double>(count));
  for (int r = 0; r < n; r++)
    for (size_t i = 0; i < count; i++) {
      b.send(r)[i] = Dt<T>::to((double)((int)((i * 5 + (size_t)r * 7) % 13) - 6));
      in[(size_t)r][i] = Dt<T>::from(b.send(r)[i]);
    }
  CollArgs a = w.base(Dt<T>::id, op, kArHybrid, count, emulated);
  a.unroll_hint = (int32_t)(((uint32_t)nvls_ctas << 16) | (uint32_t)permille);
  for (int r = 0; r < n; r++) { a.send[r] = b.send(r); a.recv[r] = in_place ? (void*)b.send(r) : (void*)b.recv(r); }
  sim_mc_regions().clear();
  SimMcRegion ms{0x100000000000ull, (count * sizeof(T) + 15) / 16 * 16, {}}, mr{0x200000000000ull, (count * sizeof(T) + 15) / 16 * 16, {}};
  for (int r = 0; r < n; r++) { ms.backing.push_back((char*)a.send[r]); mr.backing.push_back((char*)a.recv[r]); }
  sim_mc_regions().push_back(ms);
  sim_mc_regions().push_back(mr);
  a.mc_send = (const void*)ms.base;
  a.mc_recv = (void*)mr.base;
  run_all(ar_hybrid_kernel<T>, a, n, ctas, threads, emulated);
  int bad = 0;
  const double tol = tolerance<T>(n);
  for (size_t i = 0; i < count && bad < 4; i++) {
    double want = 0;
    for (int r = 0; r < n; r++) want += in[(size_t)r][i];
    if (op == kSumPostDiv) want /= n;
    for (int r = 0; r < n; r++)
      if (fabs(Dt<T>::from(((T*)a.recv[r])[i]) - want) > tol + (tol > 0 ? 1e-3 * fabs(want) : 0)) bad++;
  }
  for (int r = 1; r < n; r++) bad += memcmp(a.recv[0], a.recv[r], count * sizeof(T)) != 0;
  for (int r = 0; r < n; r++) bad += w.status[(size_t)r]->error != 0 || w.status[(size_t)r]->done_seq != a.seq;
  if (bad) fprintf(stderr, "FAILED hybrid (n=%d count=%zu ctas=%d nvls_ctas=%d permille=%d emulated=%d in_place=%d)\n", n, count, ctas,
                   nvls_ctas, permille, (int)emulated, (int)in_place);
  CHECK(bad == 0);
}

// A fused launch of `nops` independent AllReduces, optionally without the start barrier
// and with the in-kernel completion word.
template <typename T>
void batch_case(World& w, bool nvls, int nops, int ctas, int threads, bool emulated, bool skip_start, bool kernel_done) {
  const int n = w.n;
  const size_t counts[kMaxBatch] = {1000, 16, 4099, 7, 256, 33, 2048, 1};
  std::vector<std::unique_ptr<Buffers<T>>> bufs;
  BatchArgs b;
  memset(&b, 0, sizeof b);
  b.base = w.base(Dt<T>::id, kSum, nvls ? kArNvlsTwo : kArTwoShot, 0, emulated);
  b.nops = nops;
  if (skip_start) b.flags |= kBatchSkipStartBarrier;
  std::vector<uint64_t> done_words((size_t)n, 0);
  if (kernel_done)
    for (int r = 0; r < n; r++) {
      b.done_ptr[r] = &done_words[(size_t)r];
      b.done_value[r] = 1000 + (uint64_t)r;
      b.done_counter[r] = &w.pad[(size_t)r]->pad_[0];
    }
  sim_mc_regions().clear();
  for (int k = 0; k < nops; k++) {
    size_t count = counts[k];
    if (nvls) count = (count + 7) / 8 * 8 + (k == 2 ? 3 : 0);   // one member with a sub-16-byte tail
    bufs.emplace_back(new Buffers<T>(n, count, !nvls && k == 4 ? 1 : 0));   // one member that is not 16-byte aligned
    b.count[k] = count;
    for (int r = 0; r < n; r++) {
      for (size_t i = 0; i < count; i++) bufs.back()->send(r)[i] = Dt<T>::to((double)((int)((i * 7 + (size_t)r * 3 + (size_t)k) % 9) - 4));
      b.send[k][r] = bufs.back()->send(r);
      b.recv[k][r] = (k % 2) ? (void*)bufs.back()->send(r) : (void*)bufs.back()->recv(r);   // odd members in place
    }
    if (nvls) {
      SimMcRegion ms{0x100000000000ull + (uintptr_t)k * 0x10000000ull, (count * sizeof(T) + 15) / 16 * 16, {}};
      SimMcRegion mr{0x200000000000ull + (uintptr_t)k * 0x10000000ull, (count * sizeof(T) + 15) / 16 * 16, {}};
      for (int r = 0; r < n; r++) { ms.backing.push_back((char*)b.send[k][r]); mr.backing.push_back((char*)b.recv[k][r]); }
      sim_mc_regions().push_back(ms);
      sim_mc_regions().push_back(mr);
      b.mc_send[k] = (const void*)ms.base;
      b.mc_recv[k] = (void*)mr.base;
    }
  }
  // expected values before anything is overwritten in place
  std::vector<std::vector<double>> want((size_t)nops);
  for (int k = 0; k < nops; k++)
    for (size_t i = 0; i < b.count[k]; i++) {
      double acc = 0;
      for (int r = 0; r < n; r++) acc += Dt<T>::from(((const T*)b.send[k][r])[i]);
      want[(size_t)k].push_back(acc);
    }
  if constexpr (std::is_same<T, float>::value || std::is_same<T, __nv_bfloat16>::value) {
    if (nvls) run_all(ar_nvls_batch_kernel<T>, b, n, ctas, threads, emulated);
  }
  if (!nvls) run_all(ar_twoshot_batch_kernel<T, OpSum>, b, n, ctas, threads, emulated);
  int bad = 0;
  const double tol = tolerance<T>(n);
  for (int k = 0; k < nops; k++)
    for (int r = 0; r < n; r++)
      for (size_t i = 0; i < b.count[k]; i++)
        if (fabs(Dt<T>::from(((T*)b.recv[k][r])[i]) - want[(size_t)k][i]) > tol) { bad++; break; }
  for (int r = 0; r < n; r++) {
    bad += w.status[(size_t)r]->error != 0;
    bad += w.status[(size_t)r]->done_seq != b.base.seq;
    if (kernel_done) bad += done_words[(size_t)r] != 1000 + (uint64_t)r;
    if (kernel_done) bad += w.pad[(size_t)r]->pad_[0] != 0;   // the CTA counter wrapped back to zero
  }
  if (bad) fprintf(stderr, "FAILED batch (nvls=%d nops=%d n=%d ctas=%d emulated=%d skip=%d done=%d)\n", (int)nvls, nops, n, ctas,
                   (int)emulated, (int)skip_start, (int)kernel_done);
  CHECK(bad == 0);
}

// A peer that never launches: the others must give up within the bound, say so in their
// status blocks and return (no hang), and the host-raised abort word must end a wait at once.
void missing_peer_case() {
  World w(3);
  Buffers<float> b(3, 256, 0);
  CollArgs a = w.base(kFloat32, kSum, kArTwoShot, 256, false);
  for (int r = 0; r < 3; r++) { a.send[r] = b.send(r); a.recv[r] = b.recv(r); }
  a.timeout_ns = 200ull * 1000 * 1000;   // 200 ms
  const uint64_t t0 = sim::now_ns();
  run_all(ar_twoshot_kernel<float, OpSum>, a, 3, 2, 32, false, /*skip_rank=*/2);
  const double ms = (double)(sim::now_ns() - t0) / 1e6;
  CHECK(ms >= 150 && ms < 5000);
  CHECK(w.status[0]->error == kDevTimeoutStart && w.status[1]->error == kDevTimeoutStart);
  CHECK(w.status[0]->error_peer == 2 && w.status[1]->error_peer == 2);
  CHECK(w.status[0]->done_seq == 0);
  // abort word: rank 0 alone, long bound, the "host" raises abort after 50 ms
  World w2(2);
  CollArgs a2 = w2.base(kFloat32, kSum, kArTwoShot, 256, false);
  for (int r = 0; r < 2; r++) { a2.send[r] = b.send(r); a2.recv[r] = b.recv(r); }
  a2.timeout_ns = 30ull * 1000 * 1000 * 1000;
  std::thread host([&] {
    struct timespec ts = {0, 50 * 1000 * 1000};
    nanosleep(&ts, nullptr);
    __atomic_store_n(&w2.status[0]->abort, 1u, __ATOMIC_SEQ_CST);
  });
  const uint64_t t1 = sim::now_ns();
  run_all(ar_twoshot_kernel<float, OpSum>, a2, 2, 1, 32, false, /*skip_rank=*/1);
  host.join();
  CHECK((double)(sim::now_ns() - t1) / 1e6 < 5000);
  CHECK(w2.status[0]->error == kDevAborted);
}

// Stream order per rank, nothing else: every rank runs its own sequence of kernels (one
// launch after the other, like a backend stream) with its own random delays, so a fast
// rank is already in collective k+1 while a slow one still finishes k. Signal pads, ring
// counters and FIFO slots are reused from one collective to the next without any reset.
void pipelined_case(int n, int rounds) {
  World w(n);
  const size_t count = 3000;
  struct Step { int variant; CollArgs a; };
  std::vector<std::unique_ptr<Buffers<float>>> bufs;
  std::vector<Step> steps;
  const int variants[] = {kArTwoShot, kArRing, kArOneShot, kArTwoShot, kArRing, kArNvlsTwo};
  sim_mc_regions().clear();
  for (int k = 0; k < rounds; k++) {
    const int v = variants[k % 6];
    bufs.emplace_back(new Buffers<float>(n, count, 0));
    Step s;
    s.variant = v;
    s.a = w.base(kFloat32, kSum, v, count, false);
    for (int r = 0; r < n; r++) {
      for (size_t i = 0; i < count; i++) bufs.back()->send(r)[i] = (float)((int)((i + (size_t)r * 5 + (size_t)k) % 11) - 5);
      s.a.send[r] = bufs.back()->send(r);
      s.a.recv[r] = bufs.back()->recv(r);
    }
    if (v == kArRing) w.account_ring(kAllReduce, count, 4, 2);
    if (v == kArNvlsTwo) {
      SimMcRegion ms{0x100000000000ull + (uintptr_t)k * 0x10000000ull, count * 4, {}}, mr{0x200000000000ull + (uintptr_t)k * 0x10000000ull, count * 4, {}};
      for (int r = 0; r < n; r++) { ms.backing.push_back((char*)s.a.send[r]); mr.backing.push_back((char*)s.a.recv[r]); }
      sim_mc_regions().push_back(ms);
      sim_mc_regions().push_back(mr);
      s.a.mc_send = (const void*)ms.base;
      s.a.mc_recv = (void*)mr.base;
    }
    steps.push_back(s);
  }
  std::vector<std::thread> streams;
  for (int r = 0; r < n; r++)
    streams.emplace_back([&, r] {
      std::mt19937 rng((unsigned)r * 977u + 5u);
      for (const Step& s : steps) {
        struct timespec ts = {0, (long)(rng() % 300) * 1000};
        nanosleep(&ts, nullptr);
        CollArgs a = s.a;
        a.rank = r;
        std::vector<std::thread> pool;
        sim::Dim3 grid; grid.x = 2;
        switch (s.variant) {
          case kArTwoShot: sim::launch(ar_twoshot_kernel<float, OpSum>, grid, 32, a, &pool); break;
          case kArOneShot: sim::launch(ar_oneshot_kernel<float, OpSum>, grid, 32, a, &pool); break;
          case kArRing: sim::launch(ar_ring_kernel<float, OpSum>, grid, 32, a, &pool); break;
          case kArNvlsTwo: sim::launch(ar_nvls_kernel<float, true>, grid, 32, a, &pool); break;
        }
        sim::join_all(&pool);
      }
    });
  for (auto& t : streams) t.join();
  int bad = 0;
  for (int k = 0; k < rounds; k++)
    for (int r = 0; r < n; r++)
      for (size_t i = 0; i < count; i++) {
        float want = 0;
        for (int q = 0; q < n; q++) want += (float)((int)((i + (size_t)q * 5 + (size_t)k) % 11) - 5);
        if (((float*)steps[(size_t)k].a.recv[r])[i] != want) { bad++; break; }
      }
  for (int r = 0; r < n; r++) bad += w.status[(size_t)r]->error != 0;
  if (bad) fprintf(stderr, "FAILED pipelined case (n=%d rounds=%d)\n", n, rounds);
  CHECK(bad == 0);
}

// The start barrier may be dropped when the host holds every launch back until all
// clients have arrived. Worst case for that claim: every rank's stream runs the same
// in-place AllReduce on the same buffer again and again, with no barrier before the first
// load and nothing but stream order between the launches of one rank; a rank may be in
// launch k+1 while a peer is still inside launch k. The closing barrier of launch k
// (which every rank passed before its launch k+1 could start) is what keeps this correct.
void skip_start_chain_case(int n, int rounds, bool nvls) {
  World w(n);
  const size_t count = 2048 + 8;
  Buffers<float> b(n, count, 0);
  for (int r = 0; r < n; r++)
    for (size_t i = 0; i < count; i++) b.send(r)[i] = (float)(1 + (i + (size_t)r) % 3);
  std::vector<BatchArgs> launches;
  sim_mc_regions().clear();
  SimMcRegion ms{0x100000000000ull, count * 4, {}};
  for (int r = 0; r < n; r++) ms.backing.push_back((char*)b.send(r));
  sim_mc_regions().push_back(ms);
  for (int k = 0; k < rounds; k++) {
    BatchArgs a;
    memset(&a, 0, sizeof a);
    a.base = w.base(kFloat32, kSum, nvls ? kArNvlsTwo : kArTwoShot, 0, false);
    a.nops = 1;
    a.flags = kBatchSkipStartBarrier;
    // Odd launches reduce only the first half: their shards cut across the shards of the
    // even launches, so a rank does read what OTHER ranks wrote one launch earlier.
    a.count[0] = (k % 2) ? count / 2 : count;
    for (int r = 0; r < n; r++) { a.send[0][r] = b.send(r); a.recv[0][r] = b.send(r); }
    a.mc_send[0] = (const void*)ms.base;
    a.mc_recv[0] = (void*)ms.base;
    launches.push_back(a);
  }
  // every launch multiplies the common value by n (fp32 sums in rank order, as the kernels
  // do), so a launch that read a peer's buffer one round too early or too late shows up
  std::vector<float> want(count);
  for (size_t i = 0; i < count; i++) {
    float acc = 0;
    for (int r = 0; r < n; r++) acc += (float)(1 + (i + (size_t)r) % 3);
    for (int k = 1; k < rounds; k++) {
      if ((k % 2) && i >= count / 2) continue;
      float next = acc;
      for (int r = 1; r < n; r++) next += acc;
      acc = next;
    }
    want[i] = acc;
  }
  std::vector<std::thread> streams;
  for (int r = 0; r < n; r++)
    streams.emplace_back([&, r] {
      std::mt19937 rng((unsigned)r * 31u + 7u);
      for (const BatchArgs& l : launches) {
        struct timespec ts = {0, (long)(rng() % 200) * 1000};
        nanosleep(&ts, nullptr);
        BatchArgs a = l;
        a.base.rank = r;
        std::vector<std::thread> pool;
        sim::Dim3 grid; grid.x = 3;
        if (nvls) sim::launch(ar_nvls_batch_kernel<float>, grid, 32, a, &pool);
        else sim::launch(ar_twoshot_batch_kernel<float, OpSum>, grid, 32, a, &pool);
        sim::join_all(&pool);
      }
    });
  for (auto& t : streams) t.join();
  int bad = 0;
  for (int r = 0; r < n; r++) {
    for (size_t i = 0; i < count; i++)
      if (b.send(r)[i] != want[i]) { bad++; break; }
    bad += w.status[(size_t)r]->error != 0;
  }
  if (bad) fprintf(stderr, "FAILED skip-start chain (n=%d rounds=%d nvls=%d)\n", n, rounds, (int)nvls);
  CHECK(bad == 0);
}

// Random shapes within what the planner would allow: rank count, CTAs, threads, size,
// start offset (scalar path), placement, in place, variant, element type.
void random_cases(unsigned seed, int iterations) {
  std::mt19937 rng(seed);
  for (int it = 0; it < iterations; it++) {
    const int n = 2 + (int)(rng() % 7);
    World w(n);
    const int rounds = 1 + (int)(rng() % 3);   // pads and ring counters are reused within a world
    for (int k = 0; k < rounds; k++) {
      const int ctas = 1 + (int)(rng() % 4);
      const int threads = (rng() % 2) ? 32 : 64;
      const bool emulated = rng() % 2;
      const size_t count = 1 + rng() % ((rng() % 4 == 0) ? 30000 : 3000);
      const size_t offset = rng() % 4;
      const bool in_place = rng() % 2;
      const bool bf16 = rng() % 2;
      switch (rng() % 9) {
        case 0:
          if (bf16) allreduce_case<__nv_bfloat16, OpSum>(w, kArOneShot, kSum, count, ctas, threads, emulated, offset, false, "rnd oneshot bf16");
          else allreduce_case<float, OpSum>(w, kArOneShot, kSum, count, ctas, threads, emulated, offset, false, "rnd oneshot f32");
          break;
        case 1:
          if (bf16) allreduce_case<__nv_bfloat16, OpSum>(w, kArTwoShot, kSum, count, ctas, threads, emulated, offset, in_place, "rnd twoshot bf16");
          else allreduce_case<float, OpSum>(w, kArTwoShot, kSumPostDiv, count, ctas, threads, emulated, offset, in_place, "rnd twoshot f32 avg");
          break;
        case 2:
          if (bf16) allreduce_case<__nv_bfloat16, OpSum>(w, kArRing, kSum, count, ctas, threads, emulated, offset, in_place, "rnd ring bf16");
          else allreduce_case<float, OpSum>(w, kArRing, kSum, count, ctas, threads, emulated, offset, in_place, "rnd ring f32");
          break;
        case 3:
          if (bf16) allreduce_case<__nv_bfloat16, OpSum>(w, kArNvlsTwo, kSum, count, ctas, threads, emulated, 0, in_place, "rnd nvls2 bf16");
          else allreduce_case<float, OpSum>(w, kArNvlsTwo, kSum, count, ctas, threads, emulated, 0, in_place, "rnd nvls2 f32");
          break;
        case 4:
          allreduce_case<float, OpSum>(w, kArNvlsOne, kSum, count, ctas, threads, emulated, 0, false, "rnd nvls1 f32");
          break;
        case 5: allgather_case(w, (rng() % 2) ? kAgPull : kAgPush, count, ctas, threads, emulated, offset, in_place, "rnd ag direct"); break;
        case 6: allgather_case(w, kAgRing, count, ctas, threads, emulated, offset, in_place, "rnd ag ring"); break;
        case 7: allgather_case(w, kAgNvls, (count + 15) / 16 * 16, ctas, threads, emulated, 0, false, "rnd ag nvls"); break;
        case 8:
          if (bf16) batch_case<__nv_bfloat16>(w, rng() % 2, 1 + (int)(rng() % 8), ctas, threads, emulated, rng() % 2, rng() % 2);
          else batch_case<float>(w, rng() % 2, 1 + (int)(rng() % 8), ctas, threads, emulated, rng() % 2, rng() % 2);
          break;
      }
    }
  }
}

}  // namespace

int main() {

  // The wide-pack and deep-unroll forms of the kernels: 256-bit loads and stores in two-shot,
  // pull and push (sizes that are and are not multiples of 32 bytes, in place, every rank
  // count), eight in-switch loads in flight in the NVLS kernels.
  for (int hint : {32, 8}) {
    g_unroll_hint = hint;
    for (int n : {2, 3, 4, 8})
      for (bool emulated : {true, false}) {
        World w(n);
        for (size_t count : {(size_t)8, (size_t)1000, (size_t)4099, (size_t)65536 + 24}) {
          if (hint == 32) {
            allreduce_case<float, OpSum>(w, kArTwoShot, kSum, count, 3, 64, emulated, 0, false, "twoshot f32 wide");
            allreduce_case<__nv_bfloat16, OpSum>(w, kArTwoShot, kSumPostDiv, count, 2, 96, emulated, 0, true, "twoshot bf16 wide in place avg");
            allreduce_case<int32_t, OpMax>(w, kArTwoShot, kMax, count, 4, 32, emulated, 0, false, "twoshot i32 wide max");
            allgather_case(w, kAgPush, count * 4, 3, 64, emulated, 0, false, "ag push wide");
            allgather_case(w, kAgPull, count * 4, 2, 64, emulated, 0, true, "ag pull wide in place");
            allgather_case(w, kAgPush, count * 4 + 16, 2, 64, emulated, 0, false, "ag push, 16-byte multiple only");
          } else {
            allreduce_case<float, OpSum>(w, kArNvlsTwo, kSum, count, 2, 64, emulated, 0, false, "nvls twoshot f32 unroll 8");
            allreduce_case<__nv_bfloat16, OpSum>(w, kArNvlsOne, kSum, count, 3, 32, emulated, 0, false, "nvls oneshot bf16 unroll 8");
          }
        }
      }
  }
  g_unroll_hint = 0;
  const int threads = 32;
  // --- AllReduce: every variant, several rank counts, both placements ------------------
  for (int n : {2, 3, 4, 8}) {
    World w(n);
    for (bool emulated : {true, false}) {
      const int ctas = n == 8 ? 1 : 2;
      for (size_t count : {(size_t)1, (size_t)37, (size_t)1000, (size_t)4099}) {
        allreduce_case<float, OpSum>(w, kArOneShot, kSum, count, ctas, threads, emulated, 0, false, "oneshot f32");
        allreduce_case<float, OpSum>(w, kArTwoShot, kSum, count, ctas, threads, emulated, 0, false, "twoshot f32");
        allreduce_case<float, OpSum>(w, kArTwoShot, kSum, count, ctas, threads, emulated, 0, true, "twoshot f32 in place");
        allreduce_case<float, OpSum>(w, kArRing, kSum, count, ctas, threads, emulated, 0, false, "ring f32");
        allreduce_case<float, OpSum>(w, kArNvlsTwo, kSum, count, ctas, threads, emulated, 0, false, "nvls twoshot f32");
        allreduce_case<float, OpSum>(w, kArNvlsOne, kSum, count, ctas, threads, emulated, 0, false, "nvls oneshot f32");
      }
      // 16-bit types (fp32 accumulation), unaligned starts (scalar path), other operators and types
      allreduce_case<__nv_bfloat16, OpSum>(w, kArTwoShot, kSum, 3001, ctas, threads, emulated, 3, false, "twoshot bf16 +6B");
      allreduce_case<__nv_bfloat16, OpSum>(w, kArOneShot, kSum, 515, ctas, threads, emulated, 0, false, "oneshot bf16");
      allreduce_case<__nv_bfloat16, OpSum>(w, kArNvlsTwo, kSum, 2051, ctas, threads, emulated, 0, true, "nvls twoshot bf16 in place");
      allreduce_case<__half, OpSum>(w, kArRing, kSum, 2500, ctas, threads, emulated, 0, true, "ring f16 in place");
      allreduce_case<__half, OpSum>(w, kArNvlsOne, kSum, 1024, ctas, threads, emulated, 0, false, "nvls oneshot f16");
      allreduce_case<int32_t, OpMax>(w, kArTwoShot, kMax, 777, ctas, threads, emulated, 1, false, "twoshot i32 max +4B");
      allreduce_case<int32_t, OpMin>(w, kArOneShot, kMin, 130, ctas, threads, emulated, 0, false, "oneshot i32 min");
      allreduce_case<double, OpProd>(w, kArTwoShot, kProd, 99, ctas, threads, emulated, 0, false, "twoshot f64 prod");
      allreduce_case<uint8_t, OpSum>(w, kArRing, kSum, 5000, ctas, threads, emulated, 0, false, "ring u8");
      allreduce_case<int64_t, OpSum>(w, kArTwoShot, kSum, 301, ctas, threads, emulated, 0, true, "twoshot i64 in place");
      allreduce_case<float, OpSum>(w, kArTwoShot, kSumPostDiv, 1000, ctas, threads, emulated, 0, false, "twoshot f32 avg");
      allreduce_case<float, OpSum>(w, kArNvlsTwo, kSumPostDiv, 1000, ctas, threads, emulated, 0, false, "nvls twoshot f32 avg");
      // several FIFO loops per channel (ring slots are 4 KiB here)
      allreduce_case<float, OpSum>(w, kArRing, kSum, 40000, ctas, threads, emulated, 0, false, "ring f32, many loops");
      // --- ReduceScatter -----------------------------------------------------------------
      for (size_t count : {(size_t)1, (size_t)37, (size_t)1000, (size_t)4100}) {
        reduce_scatter_case<float, OpSum>(w, kRsDirect, kSum, count, ctas, threads, emulated, 0, false, "rs direct f32");
        reduce_scatter_case<float, OpSum>(w, kRsDirect, kSum, count, ctas, threads, emulated, 0, true, "rs direct f32 in place");
        if (count % 4 == 0) reduce_scatter_case<float, OpSum>(w, kRsNvls, kSum, count, ctas, threads, emulated, 0, false, "rs nvls f32");
      }
      reduce_scatter_case<__nv_bfloat16, OpSum>(w, kRsDirect, kSum, 3001, ctas, threads, emulated, 3, false, "rs direct bf16 +6B");
      reduce_scatter_case<__nv_bfloat16, OpSum>(w, kRsNvls, kSumPostDiv, 2048, ctas, threads, emulated, 0, true, "rs nvls bf16 avg in place");
      reduce_scatter_case<__half, OpSum>(w, kRsNvls, kSum, 1024, ctas, threads, emulated, 0, false, "rs nvls f16");
      reduce_scatter_case<int32_t, OpMax>(w, kRsDirect, kMax, 777, ctas, threads, emulated, 1, false, "rs direct i32 max +4B");
      reduce_scatter_case<double, OpSum>(w, kRsDirect, kSum, 99, ctas, threads, emulated, 0, false, "rs direct f64");
      reduce_scatter_case<float, OpSum>(w, kRsDirect, kSumPostDiv, 1000, ctas, threads, emulated, 0, false, "rs direct f32 avg");
      reduce_scatter_case<uint8_t, OpSum>(w, kRsDirect, kSum, 5000, ctas, threads, emulated, 0, true, "rs direct u8 in place");
      // --- AllGather ---------------------------------------------------------------------
      for (size_t bytes : {(size_t)16, (size_t)1000, (size_t)4112}) {
        allgather_case(w, kAgPull, bytes, ctas, threads, emulated, 0, false, "ag pull");
        allgather_case(w, kAgPush, bytes, ctas, threads, emulated, 0, true, "ag push in place");
        allgather_case(w, kAgRing, bytes, ctas, threads, emulated, 0, false, "ag ring");
        allgather_case(w, kAgRing, bytes, ctas, threads, emulated, 0, true, "ag ring in place");
      }
      allgather_case(w, kAgNvls, 4096, ctas, threads, emulated, 0, false, "ag nvls");
      allgather_case(w, kAgPull, 333, ctas, threads, emulated, 5, false, "ag pull unaligned");
      allgather_case(w, kAgPush, 333, ctas, threads, emulated, 5, false, "ag push unaligned");
      allgather_case(w, kAgRing, 60000, ctas, threads, emulated, 0, false, "ag ring, many loops");
      // --- hybrid: part through the switch, part around it ----------------------------------------
      for (int permille : {0, 250, 750, 1000}) {
        hybrid_case<float>(w, 4099, 4, 1, permille, threads, emulated, false, kSum);
        hybrid_case<__nv_bfloat16>(w, 10007, 4, 2, permille, threads, emulated, true, kSum);
      }
      hybrid_case<float>(w, 3, 3, 1, 750, threads, emulated, false, kSum);            // less than one pack
      hybrid_case<float>(w, 2048, 4, 0, 750, threads, emulated, false, kSumPostDiv);  // no CTA feeds the switch
      hybrid_case<float>(w, 2048, 2, 2, 750, threads, emulated, true, kSumPostDiv);   // every CTA feeds the switch
      hybrid_case<__half>(w, 8191, 5, 2, 600, threads, emulated, false, kSum);
      // --- fused launches --------------------------------------------------------------------
      batch_case<float>(w, false, 5, ctas, threads, emulated, false, false);
      batch_case<float>(w, false, 8, ctas, threads, emulated, true, true);
      batch_case<__nv_bfloat16>(w, false, 3, ctas, threads, emulated, false, true);
      batch_case<float>(w, true, 4, ctas, threads, emulated, false, false);
      batch_case<__nv_bfloat16>(w, true, 6, ctas, threads, emulated, true, true);
      batch_case<float>(w, false, 1, ctas, threads, emulated, true, true);
    }
  }
  // empty collectives (only the hand-shakes run), a full-size CTA, and more CTAs than work
  {
    World w(4);
    for (int v : {kArOneShot, kArTwoShot, kArRing, kArNvlsOne, kArNvlsTwo})
      allreduce_case<float, OpSum>(w, v, kSum, 0, 2, threads, false, 0, false, "empty all-reduce");
    for (int v : {kAgPull, kAgPush, kAgRing, kAgNvls}) allgather_case(w, v, 0, 2, threads, true, 0, false, "empty all-gather");
    allreduce_case<__nv_bfloat16, OpSum>(w, kArTwoShot, kSum, 20011, 2, 512, true, 0, false, "twoshot bf16, 512 threads");
    allreduce_case<float, OpSum>(w, kArRing, kSum, 9000, 4, 512, false, 0, true, "ring f32, 512 threads");
    allreduce_case<float, OpSum>(w, kArTwoShot, kSum, 5, 16, threads, false, 0, false, "twoshot, 16 CTAs for 5 elements");
    allgather_case(w, kAgPush, 48, 12, threads, false, 0, false, "ag push, 12 CTAs for 48 bytes");
    batch_case<float>(w, false, 8, 16, threads, false, false, true);
  }
  // a variant the planner must never pick for these arguments reports that instead of
  // touching memory: NVLS all-gather of a size that is not a multiple of 16 bytes
  {
    World w(2);
    Buffers<uint8_t> b(2, 40, 0, 2);
    CollArgs a = w.base(kUint8, kSum, kAgNvls, 40, false);
    for (int r = 0; r < 2; r++) { a.send[r] = b.send(r); a.recv[r] = b.recv(r); }
    a.mc_recv = (void*)0x200000000000ull;   // never dereferenced
    run_all(ag_direct_kernel<kAgModeNvls>, a, 2, 1, threads, false);
    CHECK(w.status[0]->error == kDevBadArgs && w.status[1]->error == kDevBadArgs);
  }
  // single-rank copy
  {
    World w(1);
    Buffers<uint8_t> b(1, 5000, 0);
    for (size_t i = 0; i < 5000; i++) b.send(0)[i] = (uint8_t)(i * 3);
    CollArgs a = w.base(kUint8, kSum, kLocalCopy, 5000, false);
    a.send[0] = b.send(0); a.recv[0] = b.recv(0);
    run_all(local_copy_kernel, a, 1, 3, threads, false);
    CHECK(memcmp(b.send(0), b.recv(0), 5000) == 0 && w.status[0]->done_seq == a.seq);
  }
  random_cases(20240611u, 250);
  // from here on the emulated kernels are perturbed (see sim::chaos_point)
  sim::g_chaos = true;
  skip_start_chain_case(2, 30, false);
  skip_start_chain_case(5, 20, false);
  skip_start_chain_case(4, 20, true);
  skip_start_chain_case(8, 12, true);
  pipelined_case(4, 24);
  pipelined_case(8, 12);
  random_cases(777u, 60);
  sim::g_chaos = false;
  missing_peer_case();
  // MCCS_SIM_SOAK=N: N more seeds of random shapes, every second one perturbed (a longer soak
  // than the default run, for changes to the kernels).
  if (const char* soak = getenv("MCCS_SIM_SOAK"))
    for (int i = 0; i < atoi(soak); i++) {
      sim::g_chaos = i % 2 == 1;
      random_cases(1000u + (unsigned)i, 100);
    }
  sim::g_chaos = false;
  printf("kernel_sim_test: %d checks, %d failed\n", g_checks, g_failed);
  return g_failed ? 1 : 0;
}
