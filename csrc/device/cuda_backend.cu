// CUDA backend for one NVSwitch box. One daemon process owns every GPU, so peer
// memory needs no handle exchange: client allocations are CUDA VMM allocations
// mapped with read/write access for all GPUs (and exported to the client as a POSIX
// file descriptor), and NVLS multicast objects are created, bound and mapped right
// here. When VMM export is not available the backend falls back to cudaMalloc +
// cudaIpcGetMemHandle (what the reference does, src/mccs/src/daemon/engine.rs:83-126)
// with cudaDeviceEnablePeerAccess between the GPUs; NVLS is then off.
//
// The driver API is reached through cudaGetDriverEntryPoint, so the library carries
// no link-time dependency on libcuda and loads on machines without a GPU.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <mutex>
#include <vector>

#include "../common/log.h"
#include "../ipc/uds.h"
#include "../kernels/launch.h"
#include "backend.h"

namespace mccs {
namespace {

#define DRV_FN(name) decltype(&name) name##_ = nullptr

struct Driver {
  DRV_FN(cuGetErrorString);
  DRV_FN(cuDeviceGet);
  DRV_FN(cuDeviceGetAttribute);
  DRV_FN(cuMemGetAllocationGranularity);
  DRV_FN(cuMemCreate);
  DRV_FN(cuMemRelease);
  DRV_FN(cuMemAddressReserve);
  DRV_FN(cuMemAddressFree);
  DRV_FN(cuMemMap);
  DRV_FN(cuMemUnmap);
  DRV_FN(cuMemSetAccess);
  DRV_FN(cuMemExportToShareableHandle);
  DRV_FN(cuMulticastCreate);
  DRV_FN(cuMulticastAddDevice);
  DRV_FN(cuMulticastBindMem);
  DRV_FN(cuMulticastUnbind);
  DRV_FN(cuMulticastGetGranularity);
  DRV_FN(cuStreamWaitValue64);
  DRV_FN(cuStreamWriteValue64);
  bool memops_ok = false;
  bool ok = false;
  bool mc_ok = false;
};

template <typename Fn>
bool load_sym(const char* name, Fn* out) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult res;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &res);
  if (e != cudaSuccess || res != cudaDriverEntryPointSuccess || !p) {
    cudaGetLastError();
    return false;
  }
  *out = reinterpret_cast<Fn>(p);
  return true;
}

#define LOAD(name) load_sym(#name, &d.name##_)

void load_driver(Driver& d) {
  d.ok = LOAD(cuGetErrorString) && LOAD(cuDeviceGet) && LOAD(cuDeviceGetAttribute) &&
         LOAD(cuMemGetAllocationGranularity) && LOAD(cuMemCreate) && LOAD(cuMemRelease) &&
         LOAD(cuMemAddressReserve) && LOAD(cuMemAddressFree) && LOAD(cuMemMap) &&
         LOAD(cuMemUnmap) && LOAD(cuMemSetAccess) && LOAD(cuMemExportToShareableHandle);
  d.mc_ok = d.ok && LOAD(cuMulticastCreate) && LOAD(cuMulticastAddDevice) &&
            LOAD(cuMulticastBindMem) && LOAD(cuMulticastUnbind) && LOAD(cuMulticastGetGranularity);
  d.memops_ok = d.ok && LOAD(cuStreamWaitValue64) && LOAD(cuStreamWriteValue64);
}

#define RT_CHECK(expr, status)                                                          \
  do {                                                                                  \
    cudaError_t e__ = (expr);                                                           \
    if (e__ != cudaSuccess) {                                                           \
      LOG_ERROR("%s failed: %s", #expr, cudaGetErrorString(e__));                       \
      cudaGetLastError();                                                               \
      return (status);                                                                  \
    }                                                                                   \
  } while (0)

// Restores the calling thread's current device on scope exit. Proxy threads keep
// their own GPU current; helpers that must touch another device use this.
struct DeviceGuard {
  int saved = -1;
  DeviceGuard() { if (cudaGetDevice(&saved) != cudaSuccess) { saved = -1; cudaGetLastError(); } }
  ~DeviceGuard() { if (saved >= 0) cudaSetDevice(saved); }
};

class CudaBackend : public Backend {
 public:
  bool init(const BackendOptions& opt, std::string* why) {
    // One hardware queue per stream as far as the GPU allows: a backend stream that waits
    // for one tenant's "submitted" mark must not hold up another tenant's stream.
    setenv("CUDA_DEVICE_MAX_CONNECTIONS", "32", 0);
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
      *why = e != cudaSuccess ? cudaGetErrorString(e) : "no CUDA device";
      cudaGetLastError();
      return false;
    }
    ndev_ = n > kMaxRanks ? kMaxRanks : n;
    for (int d = 0; d < ndev_; d++) {
      if (cudaSetDevice(d) != cudaSuccess || cudaFree(0) != cudaSuccess) {
        *why = "cannot initialise device " + std::to_string(d);
        cudaGetLastError();
        return false;
      }
    }
    load_driver(drv_);
    // Peer topology.
    for (int a = 0; a < ndev_; a++)
      for (int b = 0; b < ndev_; b++) {
        int can = a == b;
        if (a != b) cudaDeviceCanAccessPeer(&can, a, b);
        peer_[a][b] = can != 0;
      }
    vmm_ = opt.allow_vmm && drv_.ok && probe_vmm();
    if (!vmm_) enable_runtime_peer_access();
    nvls_ = vmm_ && opt.allow_nvls && drv_.mc_ok && ndev_ >= 2 && probe_multicast();
    memops_ = drv_.memops_ok && opt.allow_memops;
    for (int d = 0; d < ndev_ && memops_; d++) {
      CUdevice dev;
      int ok64 = 0;
      if (drv_.cuDeviceGet_(&dev, d) != CUDA_SUCCESS) { memops_ = false; break; }
      drv_.cuDeviceGetAttribute_(&ok64, CU_DEVICE_ATTRIBUTE_CAN_USE_64_BIT_STREAM_MEM_OPS, dev);
      if (!ok64) memops_ = false;
    }
    host_ptr_is_dev_ptr_ = true;
    for (int d = 0; d < ndev_; d++) {
      int same = 0;
      if (cudaDeviceGetAttribute(&same, cudaDevAttrCanUseHostPointerForRegisteredMem, d) != cudaSuccess) { cudaGetLastError(); same = 0; }
      if (!same) host_ptr_is_dev_ptr_ = false;
    }
    cudaSetDevice(0);
    LOG_INFO("%s", describe().c_str());
    return true;
  }

  uint32_t kind() const override { return proto::kBackendCuda; }
  int device_count() const override { return ndev_; }
  bool nvls_supported() const override { return nvls_; }
  bool peer_access(int a, int b) const override {
    return a >= 0 && b >= 0 && a < ndev_ && b < ndev_ && peer_[a][b];
  }
  std::string describe() const override {
    char buf[256];
    snprintf(buf, sizeof buf, "cuda backend: %d device(s), alloc=%s, nvls=%s, sync=%s, gran=%zu", ndev_,
             vmm_ ? "vmm+fd" : "cudaMalloc+ipc", nvls_ ? "on" : "off", memops_ ? "memops" : "events", gran_);
    return buf;
  }
  std::string cpu_affinity(int dev) const override {
    char bus[32] = {0};
    if (cudaDeviceGetPCIBusId(bus, sizeof bus, dev) != cudaSuccess) { cudaGetLastError(); return ""; }
    for (char* c = bus; *c; c++) if (*c >= 'A' && *c <= 'Z') *c = (char)(*c - 'A' + 'a');
    std::string path = std::string("/sys/bus/pci/devices/") + bus + "/local_cpulist";
    FILE* f = fopen(path.c_str(), "r");
    if (!f) return "";
    char line[512] = {0};
    if (!fgets(line, sizeof line, f)) line[0] = 0;
    fclose(f);
    size_t len = strlen(line);
    while (len && (line[len - 1] == '\n' || line[len - 1] == ' ')) line[--len] = 0;
    return line;
  }
  int set_device(int dev) override {
    RT_CHECK(cudaSetDevice(dev), proto::kErrDevice);
    return proto::kOk;
  }

  // ------------------------------------------------------------------ allocation
  int alloc(int dev, size_t bytes, Allocation* out) override {
    DeviceGuard guard;
    if (dev < 0 || dev >= ndev_ || bytes == 0) return proto::kErrInvalidArgument;
    out->device = dev;
    out->requested = bytes;
    if (vmm_) {
      size_t size = (bytes + gran_ - 1) / gran_ * gran_;
      CUmemGenericAllocationHandle h = 0;
      CUdeviceptr va = 0;
      int rc = vmm_create_mapped(dev, size, true, &h, &va);
      if (rc != proto::kOk) return rc;
      int fd = -1;
      CUresult r = drv_.cuMemExportToShareableHandle_(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
      if (r != CUDA_SUCCESS) {
        log_cu("cuMemExportToShareableHandle", r);
        vmm_destroy(h, va, size);
        return proto::kErrDevice;
      }
      out->va = (uint64_t)va;
      out->size = size;
      out->share_kind = proto::kShareVmmFd;
      out->share_fd = fd;
      out->vmm_handle = (uint64_t)h;
      return proto::kOk;
    }
    RT_CHECK(cudaSetDevice(dev), proto::kErrDevice);
    void* p = nullptr;
    size_t size = (bytes + 511) / 512 * 512;
    cudaError_t e = cudaMalloc(&p, size);
    if (e != cudaSuccess) { cudaGetLastError(); return proto::kErrOutOfMemory; }
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
      LOG_ERROR("cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
      cudaGetLastError();
      cudaFree(p);
      return proto::kErrDevice;
    }
    static_assert(sizeof(h) == proto::kIpcHandleBytes, "CUDA IPC handle size");
    memcpy(out->ipc_handle, &h, sizeof h);
    out->va = (uint64_t)p;
    out->size = size;
    out->share_kind = proto::kShareCudaIpc;
    out->share_fd = -1;
    out->vmm_handle = 0;
    return proto::kOk;
  }

  int release(Allocation* a) override {
    DeviceGuard guard;
    if (!a->va) return proto::kOk;
    if (a->vmm_handle) {
      vmm_destroy((CUmemGenericAllocationHandle)a->vmm_handle, (CUdeviceptr)a->va, a->size);
      if (a->share_fd >= 0) close(a->share_fd);
    } else {
      cudaSetDevice(a->device);
      cudaFree((void*)a->va);
    }
    a->va = 0; a->share_fd = -1; a->vmm_handle = 0;
    return proto::kOk;
  }

  int scratch_alloc(int dev, size_t bytes, bool host_staged, bool shareable, void** out) override {
    DeviceGuard guard;
    if (shareable && (host_staged || !vmm_)) return proto::kErrUnsupported;
    if (host_staged) {
      void* p = nullptr;
      RT_CHECK(cudaHostAlloc(&p, bytes, cudaHostAllocPortable | cudaHostAllocMapped), proto::kErrOutOfMemory);
      memset(p, 0, bytes);
      *out = p;
      return proto::kOk;
    }
    RT_CHECK(cudaSetDevice(dev), proto::kErrDevice);
    if (vmm_) {
      size_t size = (bytes + gran_ - 1) / gran_ * gran_;
      CUmemGenericAllocationHandle h = 0;
      CUdeviceptr va = 0;
      int rc = vmm_create_mapped(dev, size, shareable, &h, &va);
      if (rc != proto::kOk) return rc;
      int fd = -1;
      if (shareable) {
        // Exported once; every client that maps the block gets a duplicate of this descriptor.
        CUresult r = drv_.cuMemExportToShareableHandle_(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
        if (r != CUDA_SUCCESS) {
          log_cu("cuMemExportToShareableHandle(scratch)", r);
          vmm_destroy(h, va, size);
          return proto::kErrDevice;
        }
      }
      cudaError_t e = cudaMemset((void*)va, 0, size);
      if (e == cudaSuccess) e = cudaDeviceSynchronize();
      if (e != cudaSuccess) {
        LOG_ERROR("clearing scratch memory failed: %s", cudaGetErrorString(e));
        cudaGetLastError();
        if (fd >= 0) close(fd);
        vmm_destroy(h, va, size);
        return proto::kErrDevice;
      }
      std::lock_guard<std::mutex> g(mu_);
      scratch_.push_back({(uint64_t)va, (uint64_t)h, size, fd});
      *out = (void*)va;
      return proto::kOk;
    }
    void* p = nullptr;
    RT_CHECK(cudaMalloc(&p, bytes), proto::kErrOutOfMemory);
    RT_CHECK(cudaMemset(p, 0, bytes), proto::kErrDevice);
    RT_CHECK(cudaDeviceSynchronize(), proto::kErrDevice);
    *out = p;
    return proto::kOk;
  }
  int scratch_free(int dev, void* p, size_t, bool host_staged) override {
    DeviceGuard guard;
    if (!p) return proto::kOk;
    if (host_staged) { cudaFreeHost(p); return proto::kOk; }
    if (vmm_) {
      std::lock_guard<std::mutex> g(mu_);
      for (size_t i = 0; i < scratch_.size(); i++) {
        if (scratch_[i].va == (uint64_t)p) {
          vmm_destroy((CUmemGenericAllocationHandle)scratch_[i].handle, (CUdeviceptr)scratch_[i].va, scratch_[i].size);
          if (scratch_[i].fd >= 0) close(scratch_[i].fd);
          scratch_.erase(scratch_.begin() + (long)i);
          return proto::kOk;
        }
      }
      return proto::kErrNotFound;
    }
    cudaSetDevice(dev);
    cudaFree(p);
    return proto::kOk;
  }
  int hostmem_alloc(size_t bytes, bool shareable, void** out) override {
    void* p = nullptr;
    if (shareable) {
      // Shared host memory that this process and the clients both register with CUDA, the
      // way the semaphore pages are made. Kernels get the host address, which is only a
      // valid device address where the platform says so.
      if (!host_ptr_is_dev_ptr_) return proto::kErrUnsupported;
      const size_t page = (size_t)sysconf(_SC_PAGESIZE);
      const size_t size = (bytes + page - 1) / page * page;
      int fd = ipc::memfd_make("mccs-status", size);
      if (fd < 0) return proto::kErrOutOfMemory;
      p = ipc::map_shared(fd, size);
      if (!p) { close(fd); return proto::kErrOutOfMemory; }
      memset(p, 0, size);
      cudaError_t e = cudaHostRegister(p, size, cudaHostRegisterPortable | cudaHostRegisterMapped);
      void* d = nullptr;
      if (e == cudaSuccess) e = cudaHostGetDevicePointer(&d, p, 0);
      if (e != cudaSuccess || d != p) {
        LOG_ERROR("registering a shared status block failed: %s", e != cudaSuccess ? cudaGetErrorString(e) : "device address differs from host address");
        if (e == cudaSuccess) cudaHostUnregister(p);
        cudaGetLastError();
        ipc::unmap_shared(p, size);
        close(fd);
        return proto::kErrDevice;
      }
      std::lock_guard<std::mutex> g(mu_);
      shared_host_.push_back({p, size, fd});
      *out = p;
      return proto::kOk;
    }
    RT_CHECK(cudaHostAlloc(&p, bytes, cudaHostAllocPortable | cudaHostAllocMapped), proto::kErrOutOfMemory);
    memset(p, 0, bytes);
    *out = p;
    return proto::kOk;
  }
  int hostmem_free(void* p) override {
    if (!p) return proto::kOk;
    {
      std::lock_guard<std::mutex> g(mu_);
      for (size_t i = 0; i < shared_host_.size(); i++) {
        if (shared_host_[i].p != p) continue;
        cudaHostUnregister(p);
        cudaGetLastError();
        ipc::unmap_shared(p, shared_host_[i].size);
        close(shared_host_[i].fd);
        shared_host_.erase(shared_host_.begin() + (long)i);
        return proto::kOk;
      }
    }
    cudaFreeHost(p);
    return proto::kOk;
  }

  // ------------------------------------------------------------ streams and events
  int stream_create(int dev, int priority, void** stream) override {
    DeviceGuard guard;
    RT_CHECK(cudaSetDevice(dev), proto::kErrDevice);
    cudaStream_t s;
    RT_CHECK(cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, priority), proto::kErrDevice);
    *stream = (void*)s;
    return proto::kOk;
  }
  int stream_destroy(int dev, void* stream) override {
    DeviceGuard guard;
    cudaSetDevice(dev);
    cudaStreamDestroy((cudaStream_t)stream);
    return proto::kOk;
  }
  int stream_query(int, void* stream) override {
    cudaError_t e = cudaStreamQuery((cudaStream_t)stream);
    if (e == cudaSuccess) return 0;
    if (e == cudaErrorNotReady) { cudaGetLastError(); return 1; }
    LOG_ERROR("cudaStreamQuery: %s", cudaGetErrorString(e));
    return proto::kErrDevice;
  }
  int stream_sync(int, void* stream) override {
    RT_CHECK(cudaStreamSynchronize((cudaStream_t)stream), proto::kErrDevice);
    return proto::kOk;
  }
  int event_create(int dev, void** ev, uint8_t handle[proto::kIpcHandleBytes]) override {
    DeviceGuard guard;
    RT_CHECK(cudaSetDevice(dev), proto::kErrDevice);
    cudaEvent_t e;
    RT_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming | cudaEventInterprocess), proto::kErrDevice);
    cudaIpcEventHandle_t h;
    memset(&h, 0, sizeof h);
    cudaError_t rc = cudaIpcGetEventHandle(&h, e);
    if (rc != cudaSuccess) {
      // Still usable by clients living in the daemon's own process.
      LOG_WARN("cudaIpcGetEventHandle: %s", cudaGetErrorString(rc));
      cudaGetLastError();
    }
    static_assert(sizeof(h) == proto::kIpcHandleBytes, "CUDA IPC event handle size");
    memcpy(handle, &h, sizeof h);
    *ev = (void*)e;
    return proto::kOk;
  }
  int event_open(int dev, const uint8_t handle[proto::kIpcHandleBytes], void** ev) override {
    DeviceGuard guard;
    RT_CHECK(cudaSetDevice(dev), proto::kErrDevice);
    cudaIpcEventHandle_t h;
    memcpy(&h, handle, sizeof h);
    cudaEvent_t e;
    RT_CHECK(cudaIpcOpenEventHandle(&e, h), proto::kErrDevice);
    *ev = (void*)e;
    return proto::kOk;
  }
  int event_destroy(int dev, void* ev) override {
    DeviceGuard guard;
    cudaSetDevice(dev);
    cudaEventDestroy((cudaEvent_t)ev);
    return proto::kOk;
  }
  int stream_wait_event(int, void* stream, void* ev) override {
    RT_CHECK(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)ev, 0), proto::kErrDevice);
    return proto::kOk;
  }
  int event_record(int, void* ev, void* stream) override {
    RT_CHECK(cudaEventRecord((cudaEvent_t)ev, (cudaStream_t)stream), proto::kErrDevice);
    return proto::kOk;
  }

  bool memops_supported() const override { return memops_; }
  int stream_wait_value64(int, void* stream, uint64_t addr, uint64_t value) override {
    CUresult r = drv_.cuStreamWaitValue64_((CUstream)stream, (CUdeviceptr)addr, value, CU_STREAM_WAIT_VALUE_GEQ);
    if (r != CUDA_SUCCESS) { log_cu("cuStreamWaitValue64", r); return proto::kErrDevice; }
    return proto::kOk;
  }
  int stream_write_value64(int, void* stream, uint64_t addr, uint64_t value) override {
    CUresult r = drv_.cuStreamWriteValue64_((CUstream)stream, (CUdeviceptr)addr, value, CU_STREAM_WRITE_VALUE_DEFAULT);
    if (r != CUDA_SUCCESS) { log_cu("cuStreamWriteValue64", r); return proto::kErrDevice; }
    return proto::kOk;
  }
  int zero_memory(int dev, uint64_t addr, size_t bytes) override {
    DeviceGuard guard;
    RT_CHECK(cudaSetDevice(dev), proto::kErrDevice);
    RT_CHECK(cudaMemset((void*)addr, 0, bytes), proto::kErrDevice);
    RT_CHECK(cudaDeviceSynchronize(), proto::kErrDevice);
    return proto::kOk;
  }

  int sync_page_create(int dev, SyncPage* out) override {
    DeviceGuard guard;
    RT_CHECK(cudaSetDevice(dev), proto::kErrDevice);
    const size_t bytes = 4096;
    int fd = ipc::memfd_make("mccs-sync", bytes);
    if (fd < 0) return proto::kErrOutOfMemory;
    void* p = ipc::map_shared(fd, bytes);
    if (!p) { close(fd); return proto::kErrOutOfMemory; }
    memset(p, 0, bytes);
    cudaError_t e = cudaHostRegister(p, bytes, cudaHostRegisterPortable | cudaHostRegisterMapped);
    void* d = nullptr;
    if (e == cudaSuccess) e = cudaHostGetDevicePointer(&d, p, 0);
    if (e != cudaSuccess) {
      LOG_ERROR("registering the semaphore page failed: %s", cudaGetErrorString(e));
      cudaGetLastError();
      ipc::unmap_shared(p, bytes);
      close(fd);
      return proto::kErrDevice;
    }
    out->fd = fd;
    out->host = p;
    out->dev_addr = (uint64_t)d;
    out->bytes = bytes;
    return proto::kOk;
  }
  int sync_page_destroy(int dev, SyncPage* p) override {
    if (!p->host) return proto::kOk;
    DeviceGuard guard;
    cudaSetDevice(dev);
    cudaHostUnregister(p->host);
    cudaGetLastError();
    ipc::unmap_shared(p->host, p->bytes);
    if (p->fd >= 0) close(p->fd);
    *p = SyncPage();
    return proto::kOk;
  }

  // ------------------------------------------------------------------- multicast
  int mc_create(const std::vector<const Allocation*>& per_rank, McRegion* out, bool shareable) override {
    DeviceGuard guard;
    if (!nvls_) return proto::kErrUnsupported;
    const int n = (int)per_rank.size();
    if (n < 2 || n > kMaxRanks) return proto::kErrInvalidArgument;
    size_t size = (size_t)-1;
    for (int r = 0; r < n; r++) {
      if (!per_rank[r] || !per_rank[r]->vmm_handle) return proto::kErrUnsupported;
      for (int q = 0; q < r; q++)
        if (per_rank[q]->device == per_rank[r]->device) return proto::kErrUnsupported;
      if (per_rank[r]->size < size) size = per_rank[r]->size;
    }
    CUmulticastObjectProp prop;
    memset(&prop, 0, sizeof prop);
    prop.numDevices = (unsigned)n;
    prop.size = size;
    prop.handleTypes = shareable ? CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR : 0;
    size_t mc_gran = 0;
    CUresult r = drv_.cuMulticastGetGranularity_(&mc_gran, &prop, CU_MULTICAST_GRANULARITY_MINIMUM);
    if (r != CUDA_SUCCESS || mc_gran == 0) { log_cu("cuMulticastGetGranularity", r); return proto::kErrDevice; }
    size = size / mc_gran * mc_gran;
    if (size == 0) return proto::kErrUnsupported;
    prop.size = size;
    CUmemGenericAllocationHandle mc = 0;
    r = drv_.cuMulticastCreate_(&mc, &prop);
    if (r != CUDA_SUCCESS) { log_cu("cuMulticastCreate", r); return proto::kErrDevice; }
    McRegion reg;
    reg.handle = (uint64_t)mc;
    reg.size = size;
    reg.gran = mc_gran;
    reg.nranks = n;
    if (shareable) {
      int fd = -1;
      r = drv_.cuMemExportToShareableHandle_(&fd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
      if (r != CUDA_SUCCESS) { log_cu("cuMemExportToShareableHandle(multicast)", r); drv_.cuMemRelease_(mc); return proto::kErrDevice; }
      reg.share_fd = fd;
    }
    for (int i = 0; i < n; i++) {
      CUdevice dev;
      drv_.cuDeviceGet_(&dev, per_rank[i]->device);
      r = drv_.cuMulticastAddDevice_(mc, dev);
      if (r != CUDA_SUCCESS) { log_cu("cuMulticastAddDevice", r); mc_destroy(&reg); return proto::kErrDevice; }
      reg.devices[i] = per_rank[i]->device;
    }
    for (int i = 0; i < n; i++) {
      cudaSetDevice(per_rank[i]->device);
      r = drv_.cuMulticastBindMem_(mc, 0, (CUmemGenericAllocationHandle)per_rank[i]->vmm_handle, 0, size, 0);
      if (r != CUDA_SUCCESS) { log_cu("cuMulticastBindMem", r); mc_destroy(&reg); return proto::kErrDevice; }
      reg.bound[i] = per_rank[i]->vmm_handle;
    }
    // One mapping per rank, accessible from that rank's device.
    for (int i = 0; i < n; i++) {
      cudaSetDevice(per_rank[i]->device);
      CUdeviceptr va = 0;
      r = drv_.cuMemAddressReserve_(&va, size, mc_gran, 0, 0);
      if (r != CUDA_SUCCESS) { log_cu("cuMemAddressReserve(mc)", r); mc_destroy(&reg); return proto::kErrDevice; }
      reg.va[i] = (uint64_t)va;
      r = drv_.cuMemMap_(va, size, 0, mc, 0);
      if (r != CUDA_SUCCESS) { log_cu("cuMemMap(mc)", r); mc_destroy(&reg); return proto::kErrDevice; }
      CUmemAccessDesc desc;
      memset(&desc, 0, sizeof desc);
      desc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
      desc.location.id = per_rank[i]->device;
      desc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
      r = drv_.cuMemSetAccess_(va, size, &desc, 1);
      if (r != CUDA_SUCCESS) { log_cu("cuMemSetAccess(mc)", r); mc_destroy(&reg); return proto::kErrDevice; }
    }
    *out = reg;
    return proto::kOk;
  }

  int mc_destroy(McRegion* reg) override {
    DeviceGuard guard;
    if (!reg->handle) return proto::kOk;
    for (int i = 0; i < reg->nranks; i++) {
      if (reg->va[i]) {
        drv_.cuMemUnmap_((CUdeviceptr)reg->va[i], reg->size);
        drv_.cuMemAddressFree_((CUdeviceptr)reg->va[i], reg->size);
        reg->va[i] = 0;
      }
    }
    for (int i = 0; i < reg->nranks; i++) {
      if (reg->bound[i]) {
        CUdevice dev;
        drv_.cuDeviceGet_(&dev, reg->devices[i]);
        drv_.cuMulticastUnbind_((CUmemGenericAllocationHandle)reg->handle, dev, 0, reg->size);
        reg->bound[i] = 0;
      }
    }
    drv_.cuMemRelease_((CUmemGenericAllocationHandle)reg->handle);
    if (reg->share_fd >= 0) close(reg->share_fd);
    reg->share_fd = -1;
    reg->handle = 0;
    return proto::kOk;
  }

  // ---------------------------------------------------------------------- launch
  bool variant_supported(int variant, int dtype, int op) const override {
    if (variant_is_nvls(variant) && !nvls_) return false;
    return kernel_function(variant, dtype, op) != nullptr;
  }

  int max_group_ctas(int variant, int dtype, int op, int threads, int nranks) const override {
    return max_cooperative_ctas(variant, dtype, op, threads, nranks);
  }

  // Client-side launch needs pads and FIFOs that other processes can import (VMM with
  // descriptor export) and status blocks whose host address is also their device address.
  bool client_launch_supported() const override { return vmm_ && host_ptr_is_dev_ptr_; }
  int scratch_export(void* p, int* fd, size_t* bytes, uint32_t* share_kind) override {
    std::lock_guard<std::mutex> g(mu_);
    for (const Scratch& sc : scratch_)
      if (sc.va == (uint64_t)p && sc.fd >= 0) {
        *fd = sc.fd; *bytes = sc.size; *share_kind = proto::kShareVmmFd;
        return proto::kOk;
      }
    for (const SharedHost& sh : shared_host_)
      if (sh.p == p) {
        *fd = sh.fd; *bytes = sh.size; *share_kind = proto::kShareHostFd;
        return proto::kOk;
      }
    return proto::kErrNotFound;
  }

  bool batch_supported(int variant, int dtype, int op) const override {
    if (variant_is_nvls(variant) && !nvls_) return false;
    return batch_kernel_function(variant, dtype, op) != nullptr;
  }
  int max_group_batch_ctas(int variant, int dtype, int op, int threads, int nranks) const override {
    return max_cooperative_batch_ctas(variant, dtype, op, threads, nranks);
  }
  int launch_batch(int dev, const BatchArgs& b, LaunchDims dims, void* stream) override {
    (void)dev;
    cudaError_t e = mccs::launch_batch(b, dims, stream);
    if (e != cudaSuccess) {
      LOG_ERROR("fused launch of %d x %s failed: %s", b.nops, variant_name(b.base.variant), cudaGetErrorString(e));
      cudaGetLastError();
      return proto::kErrDevice;
    }
    return proto::kOk;
  }

  int launch(int dev, int kind, const CollArgs& a, LaunchDims dims, void* stream) override {
    (void)dev;
    cudaError_t e = launch_collective(kind, a, dims, stream);
    if (e != cudaSuccess) {
      LOG_ERROR("launch %s failed: %s", variant_name(a.variant), cudaGetErrorString(e));
      cudaGetLastError();
      return proto::kErrDevice;
    }
    return proto::kOk;
  }

 private:
  struct Scratch { uint64_t va, handle; size_t size; int fd; };   // fd: exported handle, -1 when not shareable
  struct SharedHost { void* p; size_t size; int fd; };

  void log_cu(const char* what, CUresult r) {
    const char* s = nullptr;
    if (drv_.cuGetErrorString_) drv_.cuGetErrorString_(r, &s);
    LOG_ERROR("%s failed: %s (%d)", what, s ? s : "?", (int)r);
  }

  CUmemAllocationProp alloc_prop(int dev, bool shareable) {
    CUmemAllocationProp prop;
    memset(&prop, 0, sizeof prop);
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = dev;
    prop.requestedHandleTypes = shareable ? CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR : CU_MEM_HANDLE_TYPE_NONE;
    return prop;
  }

  // Physical allocation on `dev`, mapped once, readable/writable from every GPU that
  // has peer access to `dev`.
  int vmm_create_mapped(int dev, size_t size, bool shareable, CUmemGenericAllocationHandle* h_out,
                        CUdeviceptr* va_out) {
    cudaSetDevice(dev);
    CUmemAllocationProp prop = alloc_prop(dev, shareable);
    CUmemGenericAllocationHandle h = 0;
    CUresult r = drv_.cuMemCreate_(&h, size, &prop, 0);
    if (r != CUDA_SUCCESS) {
      log_cu("cuMemCreate", r);
      return r == CUDA_ERROR_OUT_OF_MEMORY ? proto::kErrOutOfMemory : proto::kErrDevice;
    }
    CUdeviceptr va = 0;
    r = drv_.cuMemAddressReserve_(&va, size, gran_, 0, 0);
    if (r != CUDA_SUCCESS) { log_cu("cuMemAddressReserve", r); drv_.cuMemRelease_(h); return proto::kErrDevice; }
    r = drv_.cuMemMap_(va, size, 0, h, 0);
    if (r != CUDA_SUCCESS) {
      log_cu("cuMemMap", r);
      drv_.cuMemAddressFree_(va, size);
      drv_.cuMemRelease_(h);
      return proto::kErrDevice;
    }
    std::vector<CUmemAccessDesc> descs;
    for (int d = 0; d < ndev_; d++) {
      if (!peer_[d][dev]) continue;
      CUmemAccessDesc desc;
      memset(&desc, 0, sizeof desc);
      desc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
      desc.location.id = d;
      desc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
      descs.push_back(desc);
    }
    r = drv_.cuMemSetAccess_(va, size, descs.data(), descs.size());
    if (r != CUDA_SUCCESS) {
      log_cu("cuMemSetAccess", r);
      vmm_destroy(h, va, size);
      return proto::kErrDevice;
    }
    *h_out = h;
    *va_out = va;
    return proto::kOk;
  }

  void vmm_destroy(CUmemGenericAllocationHandle h, CUdeviceptr va, size_t size) {
    drv_.cuMemUnmap_(va, size);
    drv_.cuMemAddressFree_(va, size);
    drv_.cuMemRelease_(h);
  }

  bool probe_vmm() {
    for (int d = 0; d < ndev_; d++) {
      CUdevice dev;
      if (drv_.cuDeviceGet_(&dev, d) != CUDA_SUCCESS) return false;
      int vmm = 0, fd_ok = 0;
      drv_.cuDeviceGetAttribute_(&vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev);
      drv_.cuDeviceGetAttribute_(&fd_ok, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev);
      if (!vmm || !fd_ok) return false;
    }
    CUmemAllocationProp prop = alloc_prop(0, true);
    size_t g = 0;
    if (drv_.cuMemGetAllocationGranularity_(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || g == 0)
      return false;
    gran_ = g;
    // One trial allocation with export, so that a container that forbids the export
    // is detected now and not at the first client malloc.
    CUmemGenericAllocationHandle h = 0;
    CUdeviceptr va = 0;
    if (vmm_create_mapped(0, gran_, true, &h, &va) != proto::kOk) return false;
    int fd = -1;
    CUresult r = drv_.cuMemExportToShareableHandle_(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    vmm_destroy(h, va, gran_);
    if (r != CUDA_SUCCESS) { log_cu("cuMemExportToShareableHandle(probe)", r); return false; }
    if (fd >= 0) close(fd);
    return true;
  }

  bool probe_multicast() {
    for (int d = 0; d < ndev_; d++) {
      CUdevice dev;
      if (drv_.cuDeviceGet_(&dev, d) != CUDA_SUCCESS) return false;
      int mc = 0;
      drv_.cuDeviceGetAttribute_(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev);
      if (!mc) return false;
    }
    CUmulticastObjectProp prop;
    memset(&prop, 0, sizeof prop);
    prop.numDevices = (unsigned)ndev_;
    prop.size = gran_;
    size_t g = 0;
    if (drv_.cuMulticastGetGranularity_(&g, &prop, CU_MULTICAST_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || g == 0)
      return false;
    // Client allocations are rounded so that whole allocations can be bound.
    if (g > gran_) gran_ = g;
    return true;
  }

  void enable_runtime_peer_access() {
    for (int a = 0; a < ndev_; a++) {
      cudaSetDevice(a);
      for (int b = 0; b < ndev_; b++) {
        if (a == b || !peer_[a][b]) continue;
        cudaError_t e = cudaDeviceEnablePeerAccess(b, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
          LOG_WARN("cudaDeviceEnablePeerAccess(%d->%d): %s", a, b, cudaGetErrorString(e));
        cudaGetLastError();
      }
    }
  }

  int ndev_ = 0;
  bool vmm_ = false;
  bool nvls_ = false;
  bool memops_ = false;
  size_t gran_ = 2u << 20;
  bool peer_[kMaxRanks][kMaxRanks] = {{false}};
  Driver drv_;
  std::mutex mu_;
  std::vector<Scratch> scratch_;
  std::vector<SharedHost> shared_host_;
  bool host_ptr_is_dev_ptr_ = false;
};

}  // namespace

Backend* make_cuda_backend(const BackendOptions& opt, std::string* why) {
  CudaBackend* b = new CudaBackend();
  if (!b->init(opt, why)) { delete b; return nullptr; }
  return b;
}

}  // namespace mccs

// Self-test of the bounded device-side waits: launches rank 0 of a two-rank
// all-reduce whose peer is never launched, so the start barrier waits for a flag that
// nothing sets, gives up after `timeout_ms`, reports through the status block and
// returns. The context stays usable. Returns 0 when the launch and the
// synchronisation succeeded; *error_out receives the DevStatus the kernel reported.
extern "C" int mccs_selftest_bounded_wait(int device, int timeout_ms, unsigned* error_out, double* elapsed_ms) {
  using namespace mccs;
  if (cudaSetDevice(device) != cudaSuccess) { cudaGetLastError(); return -1; }
  SignalPad* pads[2] = {nullptr, nullptr};
  StatusBlock* status[2] = {nullptr, nullptr};
  float* data = nullptr;
  int rc = -1;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  do {
    if (cudaMalloc(&data, 4 * 4096) != cudaSuccess) break;
    if (cudaMemset(data, 0, 4 * 4096) != cudaSuccess) break;
    bool ok = true;
    for (int r = 0; r < 2 && ok; r++) {
      ok = cudaMalloc(&pads[r], sizeof(SignalPad)) == cudaSuccess &&
           cudaMemset(pads[r], 0, sizeof(SignalPad)) == cudaSuccess &&
           cudaHostAlloc(&status[r], sizeof(StatusBlock), cudaHostAllocPortable | cudaHostAllocMapped) == cudaSuccess;
      if (ok) memset(status[r], 0, sizeof(StatusBlock));
    }
    if (!ok) break;
    CollArgs a;
    memset(&a, 0, sizeof a);
    a.rank = 0;
    a.nranks = 2;
    a.dtype = kFloat32;
    a.op = kSum;
    a.variant = kArTwoShot;
    a.count = 1024;
    a.seq = 1;
    a.scale = 1.0f;
    a.epoch = 1;
    a.timeout_ns = (uint64_t)timeout_ms * 1000000ull;
    for (int r = 0; r < 2; r++) {
      a.send[r] = data + r * 1024;
      a.recv[r] = data + 2048 + r * 1024;
      a.pad[r] = pads[r];
      a.status[r] = status[r];
    }
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) break;
    cudaEventRecord(e0, 0);
    if (launch_collective(kAllReduce, a, LaunchDims{1, 128}, nullptr) != cudaSuccess) break;
    cudaEventRecord(e1, 0);
    if (cudaDeviceSynchronize() != cudaSuccess) break;
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    if (elapsed_ms) *elapsed_ms = ms;
    if (error_out) *error_out = status[0]->error;
    rc = 0;
  } while (0);
  cudaGetLastError();
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  for (int r = 0; r < 2; r++) {
    if (pads[r]) cudaFree(pads[r]);
    if (status[r]) cudaFreeHost(status[r]);
  }
  if (data) cudaFree(data);
  return rc;
}
