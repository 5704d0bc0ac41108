// Host stand-ins for the PTX wrappers of kernels/dev_prims.cuh (included from there when
// MCCS_HOST_SIM is defined): system-scope flag accesses become host atomics, bulk
// loads/stores become memcpy, and a `multimem` address is looked up in a table of
// emulated multicast regions (one backing buffer per rank at the same offset).
#pragma once
#include <stdint.h>
#include <string.h>

#include <mutex>
#include <shared_mutex>
#include <vector>

namespace mccs {
namespace dev {

inline uint32_t ld_acquire_sys_u32(const uint32_t* p) { return __atomic_load_n(p, __ATOMIC_SEQ_CST); }
inline uint32_t ld_relaxed_sys_u32(const uint32_t* p) { return __atomic_load_n(p, __ATOMIC_SEQ_CST); }
inline void st_release_sys_u32(uint32_t* p, uint32_t v) { __atomic_store_n(p, v, __ATOMIC_SEQ_CST); }
inline void st_relaxed_sys_u32(uint32_t* p, uint32_t v) { __atomic_store_n(p, v, __ATOMIC_SEQ_CST); }
inline uint64_t ld_acquire_sys_u64(const uint64_t* p) { return __atomic_load_n(p, __ATOMIC_SEQ_CST); }
inline void st_release_sys_u64(uint64_t* p, uint64_t v) { __atomic_store_n(p, v, __ATOMIC_SEQ_CST); }
inline void st_relaxed_sys_u64(uint64_t* p, uint64_t v) { __atomic_store_n(p, v, __ATOMIC_SEQ_CST); }
inline uint64_t globaltimer_ns() { return sim::now_ns(); }
inline void fence_sys() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }

template <int BYTES> struct Raw;
template <> struct Raw<1> { uint8_t x; };
template <> struct Raw<2> { uint16_t x; };
template <> struct Raw<4> { uint32_t x; };
template <> struct Raw<8> { uint64_t x; };
template <> struct alignas(16) Raw<16> { uint32_t x, y, z, w; };
template <> struct alignas(32) Raw<32> { uint32_t a[8]; };

// A misaligned access is a fault on the GPU; here it ends the test.
inline void sim_check_aligned(const void* p, int bytes) {
  if (((uintptr_t)p & (uintptr_t)(bytes - 1)) != 0) {
    fprintf(stderr, "simulated kernel: %d-byte access at misaligned address %p\n", bytes, p);
    abort();
  }
}
template <int BYTES> inline Raw<BYTES> ld_data(const void* p) {
  sim::chaos_point();
  sim_check_aligned(p, BYTES);
  Raw<BYTES> r;
  memcpy(&r, p, BYTES);
  return r;
}
template <int BYTES> inline void st_data(void* p, Raw<BYTES> v) {
  sim::chaos_point();
  sim_check_aligned(p, BYTES);
  memcpy(p, &v, BYTES);
}

// Emulated multicast regions: [base, base + size) stands for the same offsets of every
// rank's backing buffer.
// The table may change while kernels of other communicators run (a service binds and
// drops regions at any time): every multimem access holds the shared lock while it uses
// an entry, sim_mc_add / sim_mc_remove take it exclusively.
struct SimMcRegion { uintptr_t base; size_t size; std::vector<char*> backing; };
inline std::vector<SimMcRegion>& sim_mc_regions() { static std::vector<SimMcRegion> v; return v; }
inline std::shared_mutex& sim_mc_mutex() { static std::shared_mutex m; return m; }
inline const SimMcRegion& sim_mc_find(const void* mc, size_t* off) {   // shared lock held by the caller
  const uintptr_t a = (uintptr_t)mc;
  for (const SimMcRegion& r : sim_mc_regions())
    if (a >= r.base && a + 16 <= r.base + r.size) { *off = a - r.base; return r; }
  fprintf(stderr, "simulated kernel: multimem access outside every multicast region (%p)\n", mc);
  abort();
}
inline void sim_mc_add(uintptr_t base, size_t size, const std::vector<char*>& backing) {
  std::unique_lock<std::shared_mutex> g(sim_mc_mutex());
  sim_mc_regions().push_back(SimMcRegion{base, size, backing});
}
inline void sim_mc_remove(uintptr_t base) {
  std::unique_lock<std::shared_mutex> g(sim_mc_mutex());
  auto& v = sim_mc_regions();
  for (size_t i = 0; i < v.size(); i++)
    if (v[i].base == base) { v.erase(v.begin() + (long)i); return; }
}

template <typename T> struct Multimem;
template <typename T> struct SimMultimem {
  static constexpr bool kSupported = true;
  static Raw<16> ld_reduce_add(const void* mc);
};
template <> struct Multimem<float> : SimMultimem<float> {};
template <> struct Multimem<__nv_bfloat16> : SimMultimem<__nv_bfloat16> {};
template <> struct Multimem<__half> : SimMultimem<__half> {};

inline float sim_to_float(float v) { return v; }
inline float sim_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
inline float sim_to_float(__half v) { return __half2float(v); }
inline void sim_from_float(float f, float* out) { *out = f; }
inline void sim_from_float(float f, __nv_bfloat16* out) { *out = __float2bfloat16_rn(f); }
inline void sim_from_float(float f, __half* out) { *out = __float2half_rn(f); }

template <typename T> Raw<16> SimMultimem<T>::ld_reduce_add(const void* mc) {
  sim::chaos_point();
  sim_check_aligned(mc, 16);
  size_t off = 0;
  std::shared_lock<std::shared_mutex> mc_guard(sim_mc_mutex());
  const SimMcRegion& r = sim_mc_find(mc, &off);
  constexpr int kN = 16 / (int)sizeof(T);
  float acc[kN];
  for (int e = 0; e < kN; e++) acc[e] = 0.0f;
  for (char* b : r.backing) {
    T in[kN];
    memcpy(in, b + off, 16);
    for (int e = 0; e < kN; e++) acc[e] += sim_to_float(in[e]);   // fp32 accumulation, as `.acc::f32`
  }
  T out[kN];
  for (int e = 0; e < kN; e++) sim_from_float(acc[e], &out[e]);
  Raw<16> raw;
  memcpy(&raw, out, 16);
  return raw;
}
inline void multimem_st16(void* mc, Raw<16> v) {
  sim::chaos_point();
  sim_check_aligned(mc, 16);
  size_t off = 0;
  std::shared_lock<std::shared_mutex> mc_guard(sim_mc_mutex());
  const SimMcRegion& r = sim_mc_find(mc, &off);
  for (char* b : r.backing) memcpy(b + off, &v, 16);
}

}  // namespace dev
}  // namespace mccs
