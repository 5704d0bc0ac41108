// A small SIMT emulator so that the collective kernels (the same source the GPU build
// compiles) run on CPU threads in tests: every CTA is one OS thread, every CUDA thread of
// the CTA a cooperative fiber (ucontext) of that OS thread.
//
//  * `__shared__` becomes `static thread_local`: one copy per OS thread = per CTA.
//  * `__syncthreads()` parks a fiber until all live fibers of the CTA have arrived; a
//    fiber that returned from the kernel no longer counts, as on the GPU.
//  * spin waits call `__nanosleep`, which here yields to the CTA's other fibers and to
//    the other CTAs' OS threads, so cross-CTA and cross-rank flag protocols make progress.
//  * blockIdx / threadIdx / blockDim / gridDim are macros over the current fiber.
//  * system-scope loads/stores and `multimem` instructions are in sim_prims.h.
//
// It checks the kernels' logic (indexing, barrier use, flow control, error paths), not the
// GPU memory model: the host's sequentially consistent atomics are stronger than what
// the PTX asks for.
#pragma once
// CUDA's own headers first (they use the words that become macros below).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <math.h>
#include <sched.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <ucontext.h>

#include <functional>
#include <memory>
#include <thread>
#include <vector>

#define MCCS_HOST_SIM 1
#undef __global__
#undef __device__
#undef __host__
#undef __forceinline__
#undef __launch_bounds__
#undef __grid_constant__
#undef __shared__
#define __global__
#define __device__
#define __host__
#define __forceinline__ inline __attribute__((always_inline))
#define __launch_bounds__(...)
#define __grid_constant__
#define __shared__ static thread_local

namespace sim {

struct Dim3 { unsigned x = 1, y = 1, z = 1; };

enum FiberState { kRunnable, kAtBarrier, kDone };

struct Fiber {
  ucontext_t ctx;
  std::unique_ptr<char[]> stack;
  FiberState state = kRunnable;
  Dim3 tid;
};

struct Cta {
  ucontext_t main;
  std::vector<Fiber> fibers;
  int current = 0;
  int alive = 0;
  int at_barrier = 0;
  unsigned generation = 0;
  int or_acc[2] = {0, 0};
  Dim3 bid, bdim, gdim;
  std::function<void()> body;
};

inline thread_local Cta* g_cta = nullptr;

inline Fiber& self() { return g_cta->fibers[(size_t)g_cta->current]; }
inline void to_scheduler() { swapcontext(&self().ctx, &g_cta->main); }

inline void release_barrier(Cta& c) {
  for (Fiber& f : c.fibers)
    if (f.state == kAtBarrier) f.state = kRunnable;
  c.at_barrier = 0;
  c.generation++;
  c.or_acc[c.generation & 1] = 0;   // accumulator of the barrier after this one
}

inline void syncthreads() {
  Cta& c = *g_cta;
  Fiber& f = self();
  c.at_barrier++;
  if (c.at_barrier == c.alive) {
    release_barrier(c);   // last to arrive: everybody (including this fiber) goes on
    return;
  }
  f.state = kAtBarrier;
  to_scheduler();
}

inline int syncthreads_or(int pred) {
  Cta& c = *g_cta;
  const unsigned gen = c.generation;
  c.or_acc[gen & 1] |= pred ? 1 : 0;
  syncthreads();
  return c.or_acc[gen & 1];
}

// A spinning fiber lets its siblings and the other OS threads run.
inline void spin_yield() { to_scheduler(); }

inline void fiber_entry() {
  Cta& c = *g_cta;
  c.body();
  Fiber& f = self();
  f.state = kDone;
  c.alive--;
  if (c.alive > 0 && c.at_barrier == c.alive) release_barrier(c);
  to_scheduler();   // never resumed
}

// Runs one CTA to completion on the calling OS thread.
inline void run_cta(Dim3 bid, Dim3 bdim, Dim3 gdim, std::function<void()> body) {
  Cta c;
  c.bid = bid; c.bdim = bdim; c.gdim = gdim;
  c.body = std::move(body);
  const size_t kStack = 256 * 1024;
  c.fibers.resize(bdim.x);
  c.alive = (int)bdim.x;
  g_cta = &c;
  for (unsigned t = 0; t < bdim.x; t++) {
    Fiber& f = c.fibers[t];
    f.tid.x = t;
    f.stack.reset(new char[kStack]);
    getcontext(&f.ctx);
    f.ctx.uc_stack.ss_sp = f.stack.get();
    f.ctx.uc_stack.ss_size = kStack;
    f.ctx.uc_link = &c.main;
    makecontext(&f.ctx, (void (*)())fiber_entry, 0);
  }
  while (c.alive > 0) {
    for (unsigned t = 0; t < bdim.x; t++) {
      if (c.fibers[t].state != kRunnable) continue;
      c.current = (int)t;
      swapcontext(&c.main, &c.fibers[t].ctx);
    }
    sched_yield();
  }
  g_cta = nullptr;
}

// One kernel launch: grid.x * grid.y CTAs, each on its own OS thread, `threads` fibers each.
template <typename Kernel, typename Args>
void launch(Kernel kernel, Dim3 grid, unsigned threads, const Args& args, std::vector<std::thread>* pool) {
  Dim3 bdim; bdim.x = threads;
  for (unsigned by = 0; by < grid.y; by++)
    for (unsigned bx = 0; bx < grid.x; bx++) {
      Dim3 bid; bid.x = bx; bid.y = by;
      pool->emplace_back([=] { run_cta(bid, bdim, grid, [&] { kernel(args); }); });
    }
}

inline void join_all(std::vector<std::thread>* pool) {
  for (auto& t : *pool) t.join();
  pool->clear();
}

// Chaos mode: memory accesses of the emulated kernels now and then hand the CPU to another
// fiber, or put the whole CTA to sleep for a moment, so that ranks and CTAs drift apart
// and interleavings a quiet machine would never produce do occur. Deterministic per CTA.
inline bool g_chaos = false;
inline void chaos_point() {
  if (!g_chaos || g_cta == nullptr) return;
  static thread_local uint32_t state = 0;
  if (state == 0) state = 0x9E3779B9u ^ (g_cta->bid.x * 7919u + g_cta->bid.y * 104729u + 1u);
  state ^= state << 13; state ^= state >> 17; state ^= state << 5;
  if ((state & 0x3f) == 0) {
    spin_yield();
  } else if ((state & 0x7ff) == 1) {
    struct timespec ts = {0, (long)(20000 + (state >> 12) % 200000)};
    nanosleep(&ts, nullptr);
  }
}

inline uint64_t now_ns() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

}  // namespace sim

#define threadIdx (sim::self().tid)
#define blockIdx (sim::g_cta->bid)
#define blockDim (sim::g_cta->bdim)
#define gridDim (sim::g_cta->gdim)
#define __syncthreads() sim::syncthreads()
#define __syncthreads_or(p) sim::syncthreads_or(p)
#define __nanosleep(ns) sim::spin_yield()

inline void __threadfence() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
inline unsigned atomicInc(unsigned* p, unsigned limit) {
  unsigned old = __atomic_load_n(p, __ATOMIC_SEQ_CST);
  for (;;) {
    unsigned next = old >= limit ? 0u : old + 1u;
    if (__atomic_compare_exchange_n(p, &old, next, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST)) return old;
  }
}
