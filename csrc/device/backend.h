// Device backend seam of the service: everything the daemon needs from "the
// devices" — client-mappable allocations, communicator scratch memory, streams,
// interprocess events, NVLS multicast bindings and kernel launches. Two
// implementations: CUDA (B200 boxes) and a host one (shared memory + CPU
// collectives) that lets the whole control path run where no GPU exists.
//
// Reference counterparts: daemon-side cudaMalloc + cudaIpcGetMemHandle
// (src/mccs/src/daemon/engine.rs:83-126), DeviceAlloc/DeviceHostMapped
// (src/mccs/src/cuda/alloc.rs:28-99,171-183), backend stream and interprocess event
// creation (src/mccs/src/proxy/init.rs:167-175), cudaLaunchKernel of the collective
// (src/mccs/src/proxy/plan.rs:637-669).
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

#include "../common/protocol.h"
#include "../kernels/dev_types.h"

namespace mccs {

struct Allocation {
  uint64_t id = 0;
  int device = -1;
  uint64_t va = 0;           // address in the daemon's address space
  size_t size = 0;           // mapped size
  size_t requested = 0;
  uint32_t share_kind = 0;   // proto::ShareKind for out-of-process clients
  int share_fd = -1;         // memfd or exported VMM handle (daemon keeps it open)
  uint8_t ipc_handle[proto::kIpcHandleBytes] = {0};
  uint64_t vmm_handle = 0;   // CUmemGenericAllocationHandle (0 when not VMM)
  uint64_t owner_session = 0;
};

// One multicast object with the same-offset allocation of every rank bound to it.
struct McRegion {
  uint64_t handle = 0;
  uint64_t id = 0;                // name of the region in plans handed to clients
  size_t size = 0;
  size_t gran = 0;                // alignment a mapping of the object needs
  int share_fd = -1;              // exported object (client-side launch), kept open until destroyed
  uint64_t mems[kMaxRanks] = {0}; // the allocation bound per rank
  uint64_t va[kMaxRanks] = {0};   // mapping used by rank r's kernels
  int nranks = 0;
  int devices[kMaxRanks] = {0};
  uint64_t bound[kMaxRanks] = {0};  // allocation handle bound per rank (for unbinding)
};

// A small page of 64-bit semaphores that the daemon (CPU and GPU), the client's CPU
// and the client's GPU streams can all address: shared host memory (memfd), registered
// with CUDA on both sides so that stream memory operations can target it.
struct SyncPage {
  int fd = -1;
  void* host = nullptr;      // CPU address in the daemon
  uint64_t dev_addr = 0;     // address for stream memory operations issued by the daemon
  size_t bytes = 0;
};

struct BackendOptions {
  int host_devices = 8;        // device count the host backend pretends to have
  bool allow_vmm = true;
  bool allow_nvls = true;
  bool force_host = false;
  bool allow_memops = true;
  bool host_memops = false;     // host backend: offer semaphore pages, "stream memory operations" done by the CPU
  bool emulate_kernels = false; // host backend: run the real kernels on the SIMT emulator instead of plain loops
  std::vector<std::pair<int, int>> host_no_peer_access;   // host backend: device pairs that report no peer access (to exercise transport selection)
};

class Backend {
 public:
  virtual ~Backend() {}
  virtual uint32_t kind() const = 0;   // proto::Backend
  virtual int device_count() const = 0;
  virtual bool nvls_supported() const = 0;
  virtual bool peer_access(int dev_a, int dev_b) const = 0;
  virtual std::string describe() const = 0;
  // Comma separated CPU list local to the device ("" when unknown); used to pin the
  // proxy thread the way the reference pins by NVML affinity
  // (src/mccs/src/runtime/affinity.rs:59-76).
  virtual std::string cpu_affinity(int dev) const = 0;

  // Makes `dev` current for the calling thread (proxy threads call this once).
  virtual int set_device(int dev) = 0;

  // All int-returning functions give a proto::Status.
  virtual int alloc(int dev, size_t bytes, Allocation* out) = 0;
  virtual int release(Allocation* a) = 0;

  // Zero-filled scratch readable and writable from every device. host_staged places
  // it in pinned host memory (the host-staged transport). `shareable` asks for a block
  // that scratch_export can hand to another process (client-side launch).
  virtual int scratch_alloc(int dev, size_t bytes, bool host_staged, bool shareable, void** out) = 0;
  virtual int scratch_free(int dev, void* p, size_t bytes, bool host_staged) = 0;
  // Host-visible memory the device writes (status blocks).
  virtual int hostmem_alloc(size_t bytes, bool shareable, void** out) = 0;
  virtual int hostmem_free(void* p) = 0;
  // Client-side launch: whether blocks made with `shareable` can be mapped by the
  // clients' processes at all, and a file descriptor plus its proto::ShareKind through
  // which one is mapped (the backend keeps the descriptor open until the block is freed).
  virtual bool client_launch_supported() const = 0;
  virtual int scratch_export(void* p, int* fd, size_t* bytes, uint32_t* share_kind) = 0;

  virtual int stream_create(int dev, int priority, void** stream) = 0;
  virtual int stream_destroy(int dev, void* stream) = 0;
  virtual int stream_query(int dev, void* stream) = 0;   // 0 idle, 1 busy, <0 Status
  virtual int stream_sync(int dev, void* stream) = 0;
  virtual int event_create(int dev, void** ev, uint8_t handle[proto::kIpcHandleBytes]) = 0;
  virtual int event_open(int dev, const uint8_t handle[proto::kIpcHandleBytes], void** ev) = 0;
  virtual int event_destroy(int dev, void* ev) = 0;
  virtual int stream_wait_event(int dev, void* stream, void* ev) = 0;
  virtual int event_record(int dev, void* ev, void* stream) = 0;

  // Stream memory operations on 64-bit words in device memory (mem-op sync mode).
  virtual bool memops_supported() const = 0;
  virtual int stream_wait_value64(int dev, void* stream, uint64_t addr, uint64_t value) = 0;   // waits *addr >= value
  virtual int stream_write_value64(int dev, void* stream, uint64_t addr, uint64_t value) = 0;
  virtual int zero_memory(int dev, uint64_t addr, size_t bytes) = 0;
  virtual int sync_page_create(int dev, SyncPage* out) = 0;
  virtual int sync_page_destroy(int dev, SyncPage* p) = 0;

  // `shareable`: the object can be handed to the clients' processes (client-side launch).
  virtual int mc_create(const std::vector<const Allocation*>& per_rank, McRegion* out, bool shareable) = 0;
  virtual int mc_destroy(McRegion* r) = 0;

  // Launches one collective kernel on `stream` of `dev`. With a.emulated the grid
  // covers every rank (cooperative launch on one device, or a CPU loop).
  virtual int launch(int dev, int kind, const CollArgs& a, LaunchDims dims, void* stream) = 0;
  virtual bool variant_supported(int variant, int dtype, int op) const = 0;
  // CTAs per rank that fit when one cooperative launch carries all `nranks` ranks.
  virtual int max_group_ctas(int variant, int dtype, int op, int threads, int nranks) const = 0;

  // Fused AllReduce: several consecutive collectives of one communicator in one launch
  // (kernels/batch.cuh; the reference's fused work elements, src/mccs/src/proxy/plan.rs:122-141).
  virtual bool batch_supported(int variant, int dtype, int op) const = 0;
  virtual int max_group_batch_ctas(int variant, int dtype, int op, int threads, int nranks) const = 0;
  virtual int launch_batch(int dev, const BatchArgs& b, LaunchDims dims, void* stream) = 0;
};

// Returns nullptr (and a reason) when no usable CUDA device exists.
Backend* make_cuda_backend(const BackendOptions& opt, std::string* why);
Backend* make_host_backend(const BackendOptions& opt);
// CUDA when available and not forced off, else host.
Backend* make_backend(const BackendOptions& opt);

}  // namespace mccs
