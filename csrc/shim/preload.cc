// LD_PRELOAD hook that routes an unmodified CUDA application's large device
// allocations to the service, so that its buffers can be used in collectives without
// calling mccsMalloc. The reference has no such hook: its applications must call
// `libmccs::cuda_malloc` themselves (src/libmccs/src/memory.rs:12-37).
//
//   LD_PRELOAD=libmccs_preload.so MCCS_PRELOAD_MIN_BYTES=1048576 ./app
//
// cudaMalloc / cudaFree (runtime API, dynamically linked libcudart) are interposed.
// Requests below the threshold, and every request made while the hook itself is
// running, go to the real functions.
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>

#include <mutex>
#include <set>

#include "../include/mccs.h"

namespace {
using MallocFn = int (*)(void**, size_t);
using FreeFn = int (*)(void*);
using GetDeviceFn = int (*)(int*);

std::mutex g_mu;
std::set<void*> g_ours;
thread_local bool g_inside = false;

size_t min_bytes() {
  static size_t v = [] {
    const char* s = getenv("MCCS_PRELOAD_MIN_BYTES");
    return s ? (size_t)strtoull(s, nullptr, 0) : (size_t)(1u << 20);
  }();
  return v;
}
template <typename F> F real(const char* name) { return reinterpret_cast<F>(dlsym(RTLD_NEXT, name)); }
}  // namespace

extern "C" int cudaMalloc(void** ptr, size_t size) {
  static MallocFn real_malloc = real<MallocFn>("cudaMalloc");
  static GetDeviceFn get_device = real<GetDeviceFn>("cudaGetDevice");
  if (!g_inside && size >= min_bytes() && get_device) {
    g_inside = true;
    int dev = 0;
    void* p = nullptr;
    if (get_device(&dev) == 0 && mccsMalloc(&p, dev, size) == mccsSuccess) {
      {
        std::lock_guard<std::mutex> g(g_mu);
        g_ours.insert(p);
      }
      *ptr = p;
      g_inside = false;
      return 0;
    }
    g_inside = false;
  }
  return real_malloc ? real_malloc(ptr, size) : 2 /* cudaErrorMemoryAllocation */;
}

extern "C" int cudaFree(void* ptr) {
  static FreeFn real_free = real<FreeFn>("cudaFree");
  if (ptr) {
    bool ours;
    {
      std::lock_guard<std::mutex> g(g_mu);
      ours = g_ours.erase(ptr) != 0;
    }
    if (ours) {
      g_inside = true;
      mccsFree(ptr);
      g_inside = false;
      return 0;
    }
  }
  return real_free ? real_free(ptr) : 0;
}
