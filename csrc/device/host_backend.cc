// Host backend: "device memory" is memfd shared memory, streams and events are
// no-ops (every launch completes before it returns) and collectives run as plain
// CPU loops over all ranks' buffers. It exists so that the daemon, the shim, the
// planner, QoS and reconfiguration can be exercised end to end without a GPU — the
// in-process multi-engine harness the reference only has as dead code
// (src/mccs/src/control.rs:358-1141).
#include <errno.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <unistd.h>

#include <atomic>
#include <type_traits>
#include <vector>

#include "../common/log.h"
#include "../ipc/uds.h"
#include <sched.h>
#include <mutex>
#include <map>

#include "backend.h"
#include "emulated_kernels.h"

namespace mccs {
namespace {

inline float bf16_to_float(uint16_t v) {
  uint32_t u = (uint32_t)v << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
inline uint16_t float_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // NaN
  u += 0x7fffu + ((u >> 16) & 1u);  // round to nearest even
  return (uint16_t)(u >> 16);
}
inline float half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) u = sign;
    else {
      int e = -1;
      do { man <<= 1; e++; } while (!(man & 0x400u));
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}
inline uint16_t float_to_half(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint32_t sign = (u >> 16) & 0x8000u;
  int32_t exp = (int32_t)((u >> 23) & 0xff) - 127 + 15;
  uint32_t man = u & 0x7fffffu;
  if (((u >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000u;
    uint32_t shift = (uint32_t)(14 - exp);
    uint32_t half_man = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_man & 1u))) half_man++;
    return (uint16_t)(sign | half_man);
  }
  uint32_t half_man = man >> 13;
  uint32_t rem = man & 0x1fffu;
  uint16_t out = (uint16_t)(sign | ((uint32_t)exp << 10) | half_man);
  if (rem > 0x1000u || (rem == 0x1000u && (half_man & 1u))) out++;
  return out;
}

template <typename T> struct Codec {
  using Acc = T;
  static Acc load(const void* p, uint64_t i) { return ((const T*)p)[i]; }
  static void store(void* p, uint64_t i, Acc v) { ((T*)p)[i] = v; }
};
struct HalfTag {}; struct Bf16Tag {};
template <> struct Codec<HalfTag> {
  using Acc = float;
  static Acc load(const void* p, uint64_t i) { return half_to_float(((const uint16_t*)p)[i]); }
  static void store(void* p, uint64_t i, Acc v) { ((uint16_t*)p)[i] = float_to_half(v); }
};
template <> struct Codec<Bf16Tag> {
  using Acc = float;
  static Acc load(const void* p, uint64_t i) { return bf16_to_float(((const uint16_t*)p)[i]); }
  static void store(void* p, uint64_t i, Acc v) { ((uint16_t*)p)[i] = float_to_bf16(v); }
};
template <> struct Codec<int8_t> {
  using Acc = int32_t;
  static Acc load(const void* p, uint64_t i) { return ((const int8_t*)p)[i]; }
  static void store(void* p, uint64_t i, Acc v) { ((int8_t*)p)[i] = (int8_t)v; }
};
template <> struct Codec<uint8_t> {
  using Acc = uint32_t;
  static Acc load(const void* p, uint64_t i) { return ((const uint8_t*)p)[i]; }
  static void store(void* p, uint64_t i, Acc v) { ((uint8_t*)p)[i] = (uint8_t)v; }
};

template <typename Tag, int ESZ>
void cpu_allreduce(const CollArgs& a) {
  using C = Codec<Tag>;
  using Acc = typename C::Acc;
  constexpr bool is_float = std::is_floating_point<Acc>::value;
  const int n = a.nranks;
  if (a.count == 0) return;
  // Results go through a temporary so that in-place calls (recv aliasing send) work.
  std::vector<uint8_t> tmp((size_t)a.count * ESZ);
  long long imul = llrintf(a.scale);
  long long idiv = a.scale != 0 ? llrintf(1.0f / a.scale) : 1;
  for (uint64_t i = 0; i < a.count; i++) {
    Acc acc = C::load(a.send[0], i);
    auto pre = [&](Acc x) -> Acc {
      if (a.op != kPreMulSum) return x;
      if (is_float) return (Acc)(x * (Acc)a.scale);
      return (Acc)(x * (Acc)imul);
    };
    acc = pre(acc);
    for (int r = 1; r < n; r++) {
      Acc x = pre(C::load(a.send[r], i));
      switch (a.op) {
        case kProd: acc = (Acc)(acc * x); break;
        case kMax: acc = acc > x ? acc : x; break;
        case kMin: acc = acc < x ? acc : x; break;
        default: acc = (Acc)(acc + x); break;
      }
    }
    if (a.op == kSumPostDiv) {
      if (is_float) acc = (Acc)(acc * (Acc)a.scale);
      else if (idiv != 0) acc = (Acc)(acc / (Acc)idiv);
    }
    C::store(tmp.data(), i, acc);
  }
  for (int r = 0; r < n; r++) memcpy(a.recv[r], tmp.data(), tmp.size());
}

void cpu_allgather(const CollArgs& a) {
  const int n = a.nranks;
  if (a.count == 0) return;
  std::vector<uint8_t> tmp((size_t)a.count * n);
  for (int r = 0; r < n; r++) memcpy(tmp.data() + (size_t)r * a.count, a.send[r], a.count);
  for (int r = 0; r < n; r++) memcpy(a.recv[r], tmp.data(), tmp.size());
}

class HostBackend : public Backend {
 public:
  explicit HostBackend(const BackendOptions& opt)
      : ndev_(opt.host_devices > 0 ? opt.host_devices : 1), emulate_(opt.emulate_kernels), memops_(opt.host_memops),
        no_peer_(opt.host_no_peer_access) {}
  uint32_t kind() const override { return proto::kBackendHost; }
  int device_count() const override { return ndev_; }
  bool nvls_supported() const override { return emulate_; }   // emulated multicast regions (see mc_create)
  bool peer_access(int a, int b) const override {
    for (const auto& p : no_peer_)
      if ((p.first == a && p.second == b) || (p.first == b && p.second == a)) return false;
    return true;
  }
  std::string describe() const override {
    return "host backend (" + std::to_string(ndev_) + " emulated devices" + (emulate_ ? ", kernels on the SIMT emulator)" : ")");
  }
  std::string cpu_affinity(int) const override { return ""; }
  int set_device(int dev) override { return dev >= 0 && dev < ndev_ ? proto::kOk : proto::kErrInvalidArgument; }

  int alloc(int dev, size_t bytes, Allocation* out) override {
    if (dev < 0 || dev >= ndev_ || bytes == 0) return proto::kErrInvalidArgument;
    size_t page = (size_t)sysconf(_SC_PAGESIZE);
    size_t size = (bytes + page - 1) / page * page;
    int fd = ipc::memfd_make("mccs-hostmem", size);
    if (fd < 0) return proto::kErrOutOfMemory;
    void* p = ipc::map_shared(fd, size);
    if (!p) { close(fd); return proto::kErrOutOfMemory; }
    out->device = dev;
    out->va = (uint64_t)p;
    out->size = size;
    out->requested = bytes;
    out->share_kind = proto::kShareHostFd;
    out->share_fd = fd;
    out->vmm_handle = 0;
    return proto::kOk;
  }
  int release(Allocation* a) override {
    if (a->va) ipc::unmap_shared((void*)a->va, a->size);
    if (a->share_fd >= 0) close(a->share_fd);
    a->va = 0; a->share_fd = -1;
    return proto::kOk;
  }
  // Scratch lives in anonymous shared memory so that a client process can map it too
  // (client-side launch: its kernels address every rank's pads, status blocks and FIFOs).
  int scratch_alloc(int, size_t bytes, bool, bool, void** out) override {
    const size_t page = (size_t)sysconf(_SC_PAGESIZE);
    const size_t size = (bytes + page - 1) / page * page;
    int fd = ipc::memfd_make("mccs-scratch", size);
    if (fd < 0) return proto::kErrOutOfMemory;
    void* p = ipc::map_shared(fd, size);
    if (!p) { close(fd); return proto::kErrOutOfMemory; }
    memset(p, 0, size);
    {
      std::lock_guard<std::mutex> g(scratch_mu_);
      scratch_[p] = {fd, size};
    }
    *out = p;
    return proto::kOk;
  }
  int scratch_free(int, void* p, size_t, bool) override {
    std::pair<int, size_t> e{-1, 0};
    {
      std::lock_guard<std::mutex> g(scratch_mu_);
      auto it = scratch_.find(p);
      if (it == scratch_.end()) return proto::kErrNotFound;
      e = it->second;
      scratch_.erase(it);
    }
    ipc::unmap_shared(p, e.second);
    close(e.first);
    return proto::kOk;
  }
  int hostmem_alloc(size_t bytes, bool, void** out) override { return scratch_alloc(0, bytes, true, true, out); }
  int hostmem_free(void* p) override { return scratch_free(0, p, 0, true); }
  bool client_launch_supported() const override { return true; }
  int scratch_export(void* p, int* fd, size_t* bytes, uint32_t* share_kind) override {
    std::lock_guard<std::mutex> g(scratch_mu_);
    auto it = scratch_.find(p);
    if (it == scratch_.end()) return proto::kErrNotFound;
    *fd = it->second.first;
    *bytes = it->second.second;
    *share_kind = proto::kShareHostFd;
    return proto::kOk;
  }

  int stream_create(int, int, void** s) override { *s = (void*)(uintptr_t)(++next_handle_); return proto::kOk; }
  int stream_destroy(int, void*) override { return proto::kOk; }
  int stream_query(int, void*) override { return 0; }
  int stream_sync(int, void*) override { return proto::kOk; }
  int event_create(int, void** ev, uint8_t handle[proto::kIpcHandleBytes]) override {
    *ev = (void*)(uintptr_t)(++next_handle_);
    memset(handle, 0, proto::kIpcHandleBytes);
    return proto::kOk;
  }
  int event_open(int, const uint8_t*, void** ev) override { *ev = (void*)(uintptr_t)(++next_handle_); return proto::kOk; }
  int event_destroy(int, void*) override { return proto::kOk; }
  int stream_wait_event(int, void*, void*) override { return proto::kOk; }
  int event_record(int, void*, void*) override { return proto::kOk; }
  // Stream memory operations, done by the CPU at once (a host "stream" has nothing queued
  // when a call returns): the mem-op protocol between client library and proxies runs
  // unchanged, which is what lets it be tested without a GPU.
  bool memops_supported() const override { return memops_; }
  int stream_wait_value64(int, void*, uint64_t addr, uint64_t value) override {
    while ((int64_t)(__atomic_load_n((uint64_t*)addr, __ATOMIC_ACQUIRE) - value) < 0) sched_yield();
    return proto::kOk;
  }
  int stream_write_value64(int, void*, uint64_t addr, uint64_t value) override {
    __atomic_store_n((uint64_t*)addr, value, __ATOMIC_RELEASE);
    return proto::kOk;
  }
  int zero_memory(int, uint64_t addr, size_t bytes) override { memset((void*)addr, 0, bytes); return proto::kOk; }
  int sync_page_create(int, SyncPage* out) override {
    if (!memops_) return proto::kErrUnsupported;
    const size_t bytes = 4096;
    int fd = ipc::memfd_make("mccs-sync", bytes);
    if (fd < 0) return proto::kErrOutOfMemory;
    void* p = ipc::map_shared(fd, bytes);
    if (!p) { close(fd); return proto::kErrOutOfMemory; }
    memset(p, 0, bytes);
    out->fd = fd;
    out->host = p;
    out->dev_addr = (uint64_t)p;
    out->bytes = bytes;
    return proto::kOk;
  }
  int sync_page_destroy(int, SyncPage* p) override {
    if (!p->host) return proto::kOk;
    ipc::unmap_shared(p->host, p->bytes);
    close(p->fd);
    p->host = nullptr;
    p->fd = -1;
    return proto::kOk;
  }
  // With the emulated kernels a multicast region is an address range that is reserved but
  // never accessible; the emulator turns accesses to it into accesses to every rank's
  // buffer at the same offset.
  int mc_create(const std::vector<const Allocation*>& per_rank, McRegion* out, bool) override {
    if (!emulate_) return proto::kErrUnsupported;
    const int n = (int)per_rank.size();
    if (n < 2 || n > kMaxRanks) return proto::kErrInvalidArgument;
    size_t size = (size_t)-1;
    std::vector<void*> backing;
    for (const Allocation* a : per_rank) {
      if (!a || !a->va) return proto::kErrUnsupported;
      size = a->size < size ? a->size : size;
      backing.push_back((void*)a->va);
    }
    const size_t page = (size_t)sysconf(_SC_PAGESIZE);
    size = size / page * page;
    if (size == 0) return proto::kErrUnsupported;
    void* base = mmap(nullptr, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
    if (base == MAP_FAILED) return proto::kErrOutOfMemory;
    emulated_mc_add((uint64_t)base, size, backing);
    McRegion reg;
    reg.handle = (uint64_t)base;
    reg.size = size;
    reg.gran = page;
    reg.nranks = n;
    for (int r = 0; r < n; r++) { reg.va[r] = (uint64_t)base; reg.devices[r] = per_rank[r]->device; }
    *out = reg;
    return proto::kOk;
  }
  int mc_destroy(McRegion* reg) override {
    if (!reg->handle) return proto::kOk;
    emulated_mc_remove(reg->handle);
    munmap((void*)reg->handle, reg->size);
    reg->handle = 0;
    return proto::kOk;
  }

  bool variant_supported(int variant, int dtype, int op) const override {
    if (!variant_is_nvls(variant)) return true;
    if (!emulate_) return false;
    if (variant == kAgNvls) return true;   // (kRsNvls reduces: the type rule below applies)
    return (dtype == kFloat32 || dtype == kFloat16 || dtype == kBfloat16) && (op == kSum || op == kPreMulSum || op == kSumPostDiv);
  }
  int max_group_ctas(int, int, int, int, int) const override { return kMaxCtas; }

  bool batch_supported(int variant, int dtype, int op) const override {
    return variant == kArTwoShot || (variant == kArNvlsTwo && variant_supported(variant, dtype, op));
  }
  int max_group_batch_ctas(int, int, int, int, int) const override { return kMaxCtas; }
  int launch_batch(int dev, const BatchArgs& b, LaunchDims dims, void* stream) override {
    if (b.nops < 1 || b.nops > kMaxBatch) return proto::kErrInvalidArgument;
    if (emulate_) return emulated_launch_batch(b, dims) ? proto::kOk : proto::kErrUnsupported;
    for (int k = 0; k < b.nops; k++) {
      CollArgs a = b.base;
      a.count = b.count[k];
      for (int r = 0; r < a.nranks; r++) { a.send[r] = b.send[k][r]; a.recv[r] = b.recv[k][r]; }
      int rc = launch(dev, kAllReduce, a, dims, stream);
      if (rc != proto::kOk) return rc;
    }
    return proto::kOk;
  }

  int launch(int, int kind, const CollArgs& a, LaunchDims dims_, void*) override {
    if (!a.emulated && a.nranks > 1) return proto::kErrUnsupported;
    // The real kernels on the SIMT emulator: they do their own abort and status handling.
    if (emulate_) return emulated_launch(kind, a, dims_) ? proto::kOk : proto::kErrUnsupported;
    if (a.status[0] && __atomic_load_n(&a.status[0]->abort, __ATOMIC_ACQUIRE)) {
      for (int r = 0; r < a.nranks; r++) if (a.status[r]) __atomic_store_n(&a.status[r]->error, (uint32_t)kDevAborted, __ATOMIC_RELEASE);
      return proto::kOk;
    }
    if (kind == kAllGather) {
      cpu_allgather(a);
    } else if (kind == kReduceScatter && a.nranks > 1) {
      // Block q of every rank's input, reduced, is rank q's output: nranks small all-reduces
      // whose every "rank" stores to the one destination.
      const uint64_t block = a.count * (uint64_t)dtype_size(a.dtype);
      for (int q = 0; q < a.nranks; q++) {
        CollArgs b = a;
        for (int r = 0; r < a.nranks; r++) {
          b.send[r] = (const char*)a.send[r] + (uint64_t)q * block;
          b.recv[r] = a.recv[q];
        }
        int rc = launch_allreduce_loops(b);
        if (rc != proto::kOk) return rc;
      }
    } else {
      int rc = launch_allreduce_loops(a);
      if (rc != proto::kOk) return rc;
    }
    for (int r = 0; r < a.nranks; r++)
      if (a.status[r]) __atomic_store_n(&a.status[r]->done_seq, a.seq, __ATOMIC_RELEASE);
    return proto::kOk;
  }

 private:
  static int launch_allreduce_loops(const CollArgs& a) {
    {
      switch (a.dtype) {
        case kInt8: cpu_allreduce<int8_t, 1>(a); break;
        case kUint8: cpu_allreduce<uint8_t, 1>(a); break;
        case kInt32: cpu_allreduce<int32_t, 4>(a); break;
        case kUint32: cpu_allreduce<uint32_t, 4>(a); break;
        case kInt64: cpu_allreduce<int64_t, 8>(a); break;
        case kUint64: cpu_allreduce<uint64_t, 8>(a); break;
        case kFloat16: cpu_allreduce<HalfTag, 2>(a); break;
        case kFloat32: cpu_allreduce<float, 4>(a); break;
        case kFloat64: cpu_allreduce<double, 8>(a); break;
        case kBfloat16: cpu_allreduce<Bf16Tag, 2>(a); break;
        default: return proto::kErrInvalidArgument;
      }
    }
    return proto::kOk;
  }

  std::mutex scratch_mu_;
  std::map<void*, std::pair<int, size_t>> scratch_;
  int ndev_;
  bool emulate_;
  bool memops_;
  std::vector<std::pair<int, int>> no_peer_;
  std::atomic<uint64_t> next_handle_{0x1000};
};

}  // namespace

Backend* make_host_backend(const BackendOptions& opt) { return new HostBackend(opt); }

Backend* make_backend(const BackendOptions& opt) {
  if (!opt.force_host) {
    std::string why;
    Backend* b = make_cuda_backend(opt, &why);
    if (b) return b;
    LOG_INFO("CUDA backend unavailable (%s); using the host backend", why.c_str());
  }
  return make_host_backend(opt);
}

}  // namespace mccs
