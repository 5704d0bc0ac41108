// Device-side building blocks of the sm_100a collective kernels: system-scope
// loads/stores, NVLS multimem instructions, bounded flag waits, the cross-rank CTA
// barrier, element packs and reduction functors.
//
// What this replaces in the reference: `Primitives<ProtoSimple>` with its
// waitPeer/postPeer spin loops (src/collectives/src/prims_simple.h:58-125), the
// 128-bit volatile load/store helpers (src/collectives/src/op128.h:10-66) and the
// reduction functors (src/collectives/src/reduce_kernel.h). Differences by design:
// every wait is bounded by a `globaltimer` deadline and reports through a status
// word instead of spinning forever on a lost peer; 16-bit floating sums accumulate
// in fp32 (the reference adds in the 16-bit type, reduce_kernel.h:236-286).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include <type_traits>

#include "dev_types.h"

namespace mccs {
namespace dev {

#ifdef MCCS_HOST_SIM
// CPU emulation of the kernels for tests: the PTX wrappers below are replaced by host
// code with the same names and meaning.
}  // namespace dev
}  // namespace mccs
#include "../tests/sim/sim_prims.h"
namespace mccs {
namespace dev {
#else
// ----------------------------------------------------------------------------
// Scalar system-scope flag accesses
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_sys_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u64(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_u64(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// ----------------------------------------------------------------------------
// Bulk data loads/stores. Peer memory is read with system-scope relaxed loads so
// that no stale L1 line can serve a location another GPU has rewritten.
// ----------------------------------------------------------------------------
template <int BYTES> struct Raw;
template <> struct Raw<1> { uint8_t x; };
template <> struct Raw<2> { uint16_t x; };
template <> struct Raw<4> { uint32_t x; };
template <> struct Raw<8> { uint64_t x; };
template <> struct alignas(16) Raw<16> { uint32_t x, y, z, w; };
template <> struct alignas(32) Raw<32> { uint32_t a[8]; };   // sm_100 has 256-bit global loads and stores

template <int BYTES> __device__ __forceinline__ Raw<BYTES> ld_data(const void* p);
template <int BYTES> __device__ __forceinline__ void st_data(void* p, Raw<BYTES> v);

template <> __device__ __forceinline__ Raw<1> ld_data<1>(const void* p) {
  uint32_t t;
  asm volatile("ld.relaxed.sys.global.u8 %0, [%1];" : "=r"(t) : "l"(p));
  Raw<1> r; r.x = (uint8_t)t; return r;
}
template <> __device__ __forceinline__ Raw<2> ld_data<2>(const void* p) {
  Raw<2> r;
  asm volatile("ld.relaxed.sys.global.u16 %0, [%1];" : "=h"(r.x) : "l"(p));
  return r;
}
template <> __device__ __forceinline__ Raw<4> ld_data<4>(const void* p) {
  Raw<4> r;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(r.x) : "l"(p));
  return r;
}
template <> __device__ __forceinline__ Raw<8> ld_data<8>(const void* p) {
  Raw<8> r;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(r.x) : "l"(p));
  return r;
}
template <> __device__ __forceinline__ Raw<16> ld_data<16>(const void* p) {
  Raw<16> r;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
template <> __device__ __forceinline__ Raw<32> ld_data<32>(const void* p) {
  Raw<32> r;
  asm volatile("ld.relaxed.sys.global.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r.a[0]), "=r"(r.a[1]), "=r"(r.a[2]), "=r"(r.a[3]), "=r"(r.a[4]), "=r"(r.a[5]), "=r"(r.a[6]), "=r"(r.a[7])
               : "l"(p));
  return r;
}
template <> __device__ __forceinline__ void st_data<32>(void* p, Raw<32> v) {
  asm volatile("st.relaxed.sys.global.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.a[0]), "r"(v.a[1]),
               "r"(v.a[2]), "r"(v.a[3]), "r"(v.a[4]), "r"(v.a[5]), "r"(v.a[6]), "r"(v.a[7]));
}
template <> __device__ __forceinline__ void st_data<1>(void* p, Raw<1> v) {
  asm volatile("st.relaxed.sys.global.u8 [%0], %1;" ::"l"(p), "r"((uint32_t)v.x));
}
template <> __device__ __forceinline__ void st_data<2>(void* p, Raw<2> v) {
  asm volatile("st.relaxed.sys.global.u16 [%0], %1;" ::"l"(p), "h"(v.x));
}
template <> __device__ __forceinline__ void st_data<4>(void* p, Raw<4> v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v.x));
}
template <> __device__ __forceinline__ void st_data<8>(void* p, Raw<8> v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v.x));
}
template <> __device__ __forceinline__ void st_data<16>(void* p, Raw<16> v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w));
}

// ----------------------------------------------------------------------------
// NVLS: one instruction addressed at a multicast mapping is executed by the
// NVSwitch against every GPU bound to it (sum in the switch / replicate a store).
// ----------------------------------------------------------------------------
template <typename T> struct Multimem;  // specialised for the float types with .v4 forms
template <> struct Multimem<float> {
  static constexpr bool kSupported = true;
  static __device__ __forceinline__ Raw<16> ld_reduce_add(const void* mc) {
    Raw<16> r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(mc)
                 : "memory");
    return r;
  }
};
template <> struct Multimem<__nv_bfloat16> {
  static constexpr bool kSupported = true;
  static __device__ __forceinline__ Raw<16> ld_reduce_add(const void* mc) {
    Raw<16> r;
    asm volatile(
        "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
        : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
        : "l"(mc)
        : "memory");
    return r;
  }
};
template <> struct Multimem<__half> {
  static constexpr bool kSupported = true;
  static __device__ __forceinline__ Raw<16> ld_reduce_add(const void* mc) {
    Raw<16> r;
    asm volatile(
        "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
        : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
        : "l"(mc)
        : "memory");
    return r;
  }
};
__device__ __forceinline__ void multimem_st16(void* mc, Raw<16> v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc),
               "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

#endif  // MCCS_HOST_SIM

// ----------------------------------------------------------------------------
// Bounded waits
// ----------------------------------------------------------------------------
// Spin until *p >= want (wrap-safe). Gives up when the deadline passes or the
// host raises `*abort_word`; returns a DevStatus (kDevOk on success). The clock is
// only read every 256 polls so the common case stays a tight load loop.
__device__ __forceinline__ uint32_t wait_ge_u32(const uint32_t* p, uint32_t want,
                                                uint64_t deadline, const uint32_t* abort_word,
                                                uint32_t timeout_code) {
  uint32_t spins = 0;
  while ((int32_t)(ld_acquire_sys_u32(p) - want) < 0) {
    if ((++spins & 0xffu) == 0) {
      if (ld_relaxed_sys_u32(abort_word) != 0) return kDevAborted;
      if (globaltimer_ns() > deadline) return timeout_code;
      __nanosleep(20);
    }
  }
  return kDevOk;
}
__device__ __forceinline__ uint32_t wait_ge_u64(const uint64_t* p, uint64_t want,
                                                uint64_t deadline, const uint32_t* abort_word,
                                                uint32_t timeout_code) {
  uint32_t spins = 0;
  while ((int64_t)(ld_acquire_sys_u64(p) - want) < 0) {
    if ((++spins & 0xffu) == 0) {
      if (ld_relaxed_sys_u32(abort_word) != 0) return kDevAborted;
      if (globaltimer_ns() > deadline) return timeout_code;
      __nanosleep(20);
    }
  }
  return kDevOk;
}

__device__ __forceinline__ void report_error(StatusBlock* st, uint32_t code, uint32_t detail) {
  // Plain system-scope stores: the block lives in host-mapped memory where device
  // atomics may be unavailable; concurrent writers store equivalent information.
  st_relaxed_sys_u32(&st->error_peer, detail);
  st_relaxed_sys_u32(&st->error, code);
}

// Barrier between the CTAs with the same blockIdx.x on every rank.
// kPublish: writes made by any thread of this CTA before the call are visible to
// every rank after it returns on that rank (needed when peers consume data this
// CTA stored remotely). Returns false when a wait was abandoned; the caller must
// then skip its remaining work and return.
template <bool kPublish>
__device__ __forceinline__ bool rank_barrier(const CollArgs& a, int rank, uint32_t value,
                                             uint32_t timeout_code) {
  __syncthreads();
  const int t = threadIdx.x;
  uint32_t err = kDevOk;
  if (t < a.nranks) {
    // The release store is cumulative over what the CTA wrote before the
    // __syncthreads above, so one release per peer publishes the whole CTA's data.
    if (kPublish) st_release_sys_u32(&a.pad[t]->barrier[blockIdx.x][rank], value);
    else st_relaxed_sys_u32(&a.pad[t]->barrier[blockIdx.x][rank], value);
    const uint64_t deadline = globaltimer_ns() + a.timeout_ns;
    err = wait_ge_u32(&a.pad[rank]->barrier[blockIdx.x][t], value, deadline,
                      &a.status[rank]->abort, timeout_code);
    if (err != kDevOk) report_error(a.status[rank], err, (uint32_t)t);
  }
  return __syncthreads_or(err != kDevOk) == 0;
}

// ----------------------------------------------------------------------------
// Element packs: BYTES of storage holding N elements of T, unpacked into an
// accumulator type (fp32 for 16-bit floats) for the reduction.
// ----------------------------------------------------------------------------
template <typename T> struct AccOf { using type = T; };
template <> struct AccOf<__half> { using type = float; };
template <> struct AccOf<__nv_bfloat16> { using type = float; };
template <> struct AccOf<int8_t> { using type = int32_t; };
template <> struct AccOf<uint8_t> { using type = uint32_t; };

template <typename T> __device__ __forceinline__ typename AccOf<T>::type to_acc(T v) {
  return (typename AccOf<T>::type)v;
}
template <> __device__ __forceinline__ float to_acc<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_acc<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_acc(typename AccOf<T>::type v) {
  return (T)v;
}
template <> __device__ __forceinline__ __half from_acc<__half>(float v) {
  return __float2half_rn(v);
}
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

template <typename T, int BYTES> struct Pack {
  static constexpr int kN = BYTES / (int)sizeof(T);
  using Acc = typename AccOf<T>::type;
  union U {
    Raw<BYTES> raw;
    T e[kN];
    __device__ U() {}
  };
  static __device__ __forceinline__ void unpack(Raw<BYTES> r, Acc (&out)[kN]) {
    U u; u.raw = r;
#pragma unroll
    for (int i = 0; i < kN; i++) out[i] = to_acc<T>(u.e[i]);
  }
  static __device__ __forceinline__ Raw<BYTES> pack(const Acc (&in)[kN]) {
    U u;
#pragma unroll
    for (int i = 0; i < kN; i++) u.e[i] = from_acc<T>(in[i]);
    return u.raw;
  }
};

// ----------------------------------------------------------------------------
// Reduction functors on accumulator values. `pre`/`post` implement PreMulSum and
// SumPostDiv (src/ipc/mccs/src/command.rs:33-42); they are the identity otherwise.
// ----------------------------------------------------------------------------
struct OpSum {
  template <typename A> static __device__ __forceinline__ A apply(A x, A y) { return x + y; }
};
struct OpProd {
  template <typename A> static __device__ __forceinline__ A apply(A x, A y) { return x * y; }
};
struct OpMax {
  template <typename A> static __device__ __forceinline__ A apply(A x, A y) { return x > y ? x : y; }
};
struct OpMin {
  template <typename A> static __device__ __forceinline__ A apply(A x, A y) { return x < y ? x : y; }
};

// Scaling applied to each input (PreMulSum) or to the final value (SumPostDiv).
// Floating accumulators multiply by `scale`; integer accumulators multiply for
// PreMulSum and divide by round(1/scale) for SumPostDiv.
template <typename A> struct Scaler {
  int mode;  // 0 none, 1 pre-multiply, 2 post-scale
  float scale;
  __device__ __forceinline__ A pre(A x) const { return mode == 1 ? mul(x) : x; }
  __device__ __forceinline__ A post(A x) const { return mode == 2 ? div(x) : x; }
  __device__ __forceinline__ A mul(A x) const {
    if constexpr (std::is_floating_point<A>::value)
      return (A)(x * (A)scale);
    else
      return (A)(x * (A)llrintf(scale));
  }
  __device__ __forceinline__ A div(A x) const {
    if constexpr (std::is_floating_point<A>::value) {
      return (A)(x * (A)scale);
    } else {
      A d = (A)llrintf(1.0f / scale);
      return d == 0 ? x : (A)(x / d);
    }
  }
};

__device__ __forceinline__ int scaler_mode(int op) {
  return op == kPreMulSum ? 1 : (op == kSumPostDiv ? 2 : 0);
}

}  // namespace dev
}  // namespace mccs
