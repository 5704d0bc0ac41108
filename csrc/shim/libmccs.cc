// libmccs: the client shim. See csrc/include/mccs.h for the API and its map to the
// reference's Rust crate (src/libmccs/src/{lib,memory,communicator,collectives}.rs).
//
// The library uses the CUDA *driver* API only, loaded with dlopen at first need, so
// it has no link-time CUDA dependency, loads on machines without a GPU (the daemon's
// host backend) and never creates a second CUDA runtime inside a PyTorch process.
#include "../include/mccs.h"

#include <arpa/inet.h>
#include <cuda.h>
#include <dlfcn.h>
#include <errno.h>
#include <execinfo.h>
#include <signal.h>
#include <netdb.h>
#include <poll.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <time.h>
#include <unistd.h>

#include <chrono>
#include <condition_variable>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../common/log.h"
#include "../common/protocol.h"
#include "../common/value.h"
#include "../ipc/shm_ring.h"
#include "../ipc/uds.h"
#include "../device/emulated_kernels.h"
#include "../kernels/dev_types.h"

using namespace mccs;

namespace {

// ------------------------------------------------------------------ driver API
#define DRV_FN(name) decltype(&name) name##_ = nullptr
struct Driver {
  void* lib = nullptr;
  bool tried = false, ok = false;
  DRV_FN(cuInit);
  DRV_FN(cuDeviceGet);
  DRV_FN(cuCtxGetCurrent);
  DRV_FN(cuCtxSetCurrent);
  DRV_FN(cuCtxGetDevice);
  DRV_FN(cuDevicePrimaryCtxRetain);
  DRV_FN(cuEventCreate);
  DRV_FN(cuEventDestroy);
  DRV_FN(cuEventRecord);
  DRV_FN(cuStreamWaitEvent);
  DRV_FN(cuIpcGetEventHandle);
  DRV_FN(cuIpcOpenEventHandle);
  DRV_FN(cuIpcOpenMemHandle);
  DRV_FN(cuIpcCloseMemHandle);
  DRV_FN(cuMemImportFromShareableHandle);
  DRV_FN(cuMemAddressReserve);
  DRV_FN(cuMemAddressFree);
  DRV_FN(cuMemMap);
  DRV_FN(cuMemUnmap);
  DRV_FN(cuMemSetAccess);
  DRV_FN(cuMemRelease);
  DRV_FN(cuGetErrorString);
  DRV_FN(cuStreamWaitValue64);
  DRV_FN(cuStreamWriteValue64);
  DRV_FN(cuMemHostRegister);
  DRV_FN(cuMemHostUnregister);
  DRV_FN(cuMemHostGetDevicePointer);
  DRV_FN(cuCtxSynchronize);
  bool memops = false;
};
Driver g_drv;

template <typename Fn> bool sym(void* lib, const char* name, Fn* out) {
  void* p = dlsym(lib, name);
  if (!p) return false;
  *out = reinterpret_cast<Fn>(p);
  return true;
}

bool load_driver() {
  if (g_drv.tried) return g_drv.ok;
  g_drv.tried = true;
  g_drv.lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_LOCAL);
  if (!g_drv.lib) return false;
  void* l = g_drv.lib;
  // Versioned names are what cuda.h's macros map the plain names to.
  g_drv.ok = sym(l, "cuInit", &g_drv.cuInit_) && sym(l, "cuDeviceGet", &g_drv.cuDeviceGet_) &&
             sym(l, "cuCtxGetCurrent", &g_drv.cuCtxGetCurrent_) && sym(l, "cuCtxSetCurrent", &g_drv.cuCtxSetCurrent_) &&
             sym(l, "cuCtxGetDevice", &g_drv.cuCtxGetDevice_) &&
             sym(l, "cuDevicePrimaryCtxRetain", &g_drv.cuDevicePrimaryCtxRetain_) &&
             sym(l, "cuEventCreate", &g_drv.cuEventCreate_) && sym(l, "cuEventDestroy_v2", &g_drv.cuEventDestroy_) &&
             sym(l, "cuEventRecord", &g_drv.cuEventRecord_) && sym(l, "cuStreamWaitEvent", &g_drv.cuStreamWaitEvent_) &&
             sym(l, "cuIpcGetEventHandle", &g_drv.cuIpcGetEventHandle_) &&
             sym(l, "cuIpcOpenEventHandle", &g_drv.cuIpcOpenEventHandle_) &&
             sym(l, "cuIpcOpenMemHandle_v2", &g_drv.cuIpcOpenMemHandle_) &&
             sym(l, "cuIpcCloseMemHandle", &g_drv.cuIpcCloseMemHandle_) &&
             sym(l, "cuMemImportFromShareableHandle", &g_drv.cuMemImportFromShareableHandle_) &&
             sym(l, "cuMemAddressReserve", &g_drv.cuMemAddressReserve_) &&
             sym(l, "cuMemAddressFree", &g_drv.cuMemAddressFree_) && sym(l, "cuMemMap", &g_drv.cuMemMap_) &&
             sym(l, "cuMemUnmap", &g_drv.cuMemUnmap_) && sym(l, "cuMemSetAccess", &g_drv.cuMemSetAccess_) &&
             sym(l, "cuMemRelease", &g_drv.cuMemRelease_) && sym(l, "cuGetErrorString", &g_drv.cuGetErrorString_);
  g_drv.memops = sym(l, "cuStreamWaitValue64_v2", &g_drv.cuStreamWaitValue64_) &&
                 sym(l, "cuStreamWriteValue64_v2", &g_drv.cuStreamWriteValue64_) &&
                 sym(l, "cuMemHostRegister_v2", &g_drv.cuMemHostRegister_) &&
                 sym(l, "cuMemHostUnregister", &g_drv.cuMemHostUnregister_) &&
                 sym(l, "cuMemHostGetDevicePointer_v2", &g_drv.cuMemHostGetDevicePointer_);
  sym(l, "cuCtxSynchronize", &g_drv.cuCtxSynchronize_);
  if (g_drv.ok && g_drv.cuInit_(0) != CUDA_SUCCESS) g_drv.ok = false;
  return g_drv.ok;
}

const char* cu_err(CUresult r) {
  const char* s = nullptr;
  if (g_drv.cuGetErrorString_) g_drv.cuGetErrorString_(r, &s);
  return s ? s : "unknown CUDA error";
}

// Makes the primary context of `device` current for the scope (and restores what
// was current), so that the shim works from threads that have not touched CUDA yet
// and never disturbs the caller's current device.
struct CtxScope {
  CUcontext saved = nullptr;
  bool switched = false;
  bool ok = false;
  explicit CtxScope(int device) {
    if (device < 0) { ok = true; return; }   // nothing to make current (host backend)
    if (!load_driver()) return;
    CUcontext cur = nullptr;
    g_drv.cuCtxGetCurrent_(&cur);
    if (cur) {
      CUdevice d;
      if (g_drv.cuCtxGetDevice_(&d) == CUDA_SUCCESS && (int)d == device) { ok = true; return; }
    }
    CUdevice dev;
    if (g_drv.cuDeviceGet_(&dev, device) != CUDA_SUCCESS) return;
    CUcontext primary = nullptr;
    if (g_drv.cuDevicePrimaryCtxRetain_(&primary, dev) != CUDA_SUCCESS) return;
    saved = cur;
    if (g_drv.cuCtxSetCurrent_(primary) != CUDA_SUCCESS) return;
    switched = true;
    ok = true;
  }
  ~CtxScope() { if (switched) g_drv.cuCtxSetCurrent_(saved); }
};

// ------------------------------------------------------------------ state
struct MemRec {
  uint64_t mem_id = 0;
  uint64_t base = 0;
  size_t size = 0;
  int device = 0;
  uint32_t share_kind = 0;
  uint64_t vmm_handle = 0;
};

// A block of another owner (a peer's buffer, a rank's signal pad, status block or FIFOs)
// mapped into this process for client-side launch.
struct Mapped {
  uint64_t addr = 0;        // the address kernels launched here use
  void* host = nullptr;     // CPU-readable address, null for device memory
  size_t bytes = 0;
  uint32_t share_kind = 0;
  uint64_t vmm_handle = 0;
  bool registered = false;  // host memory registered with CUDA here
  bool emulated_mc = false; // an emulated multicast region (host backend): an inaccessible range known to the emulator
};

struct StreamRec {
  uint64_t stream_id = 0;
  CUevent event = nullptr;   // "submitted" marker recorded on the user's stream
  int device = 0;
};

struct Reply {
  proto::AnyMsg msg;
  std::vector<int> fds;
};

struct Context {
  std::mutex mu;
  int fd = -1;
  bool connected = false;
  uint32_t backend = 0;
  int daemon_pid = 0;
  bool same_process = false;
  int num_devices = 0;
  uint64_t session_id = 0;
  uint32_t sync_mode = 0;
  uint32_t next_req = 1;
  std::map<uint64_t, MemRec> mem;                       // base -> record
  std::map<uint64_t, uint64_t> mem_base_by_id;          // allocation id -> base (plans name allocations by id)
  std::map<std::pair<int, uint64_t>, StreamRec> streams;   // (device, stream) -> record
  uint64_t wc_timeout_ms = 300000;
  // reply demultiplexing (see roundtrip)
  bool reader_active = false;
  std::condition_variable reply_cv;
  std::map<uint32_t, struct Reply> replies;
  std::vector<struct mccsComm*> comms;   // live communicators (flushed before memory is freed)
};
Context g_ctx;

thread_local int g_group_depth = 0;
struct GroupItem { struct mccsComm* comm; mccsStream_t stream; };
thread_local std::vector<GroupItem> g_group_items;

}  // namespace

struct mccsComm {
  uint64_t handle = 0;
  uint32_t id = 0;
  int rank = 0, nranks = 0, device = 0;
  void* dp_mem = nullptr;
  size_t dp_bytes = 0;
  ipc::Ring wq, cq;
  proto::DpStatus* dp_status = nullptr;
  uint64_t memop_posted = 0;     // mem-op requests posted (their completions are counted, not queued)
  CUevent backend_event = nullptr;
  bool event_owned = false;
  uint64_t next_user_seq = 1;
  uint64_t outstanding = 0;      // requests posted whose completion was not read yet
  uint32_t last_variant = 0, last_ctas = 0;
  int sticky_error = 0;
  bool deferred_wait = false;         // collectives do not queue "wait done"; mccsCommWait does
  uint64_t last_posted_seq = 0;       // user_seq of the newest request posted
  pthread_t owner = pthread_self();   // the thread that created (and uses) the communicator
  // mem-op synchronisation (proto::kSyncMemOps): semaphore page shared with the daemon
  // (host memory mapped here and registered for device access)
  void* sync_host = nullptr;
  size_t sync_bytes = 0;
  uint64_t sync_base = 0;     // device address of the page for stream memory operations
  bool sync_emulated = false; // host backend: the CPU writes and awaits the semaphores itself
  std::map<uint64_t, uint32_t> stream_slot;            // stream handle -> semaphore index
  uint64_t slot_value[proto::kSyncMaxStreams] = {0};   // last value written per semaphore
  // client-side launch (proto::kLaunchClient): plans come back through `pq`, the kernels
  // are launched here and address every rank's pads, status blocks, FIFOs and buffers
  bool client_launch = false;
  bool group_defer = false;      // inside a group, requests are only posted; the plans are taken at the end (fused launches)
  ipc::Ring pq;
  Mapped pad_map[kMaxRanks], status_map[kMaxRanks], fifo_map[kMaxRanks];
  uint64_t fifo_slot_bytes = 0;
  std::map<uint64_t, Mapped> peer_mem;                 // allocations of other ranks, mapped on first use
  std::map<uint64_t, Mapped> mc_map;                   // multicast regions named in plans, mapped on first use
  bool launched_here = false;                          // a kernel of this communicator may still be running on a caller's stream
  CUevent launch_event = nullptr;                      // deferred waiting: recorded behind the newest kernel launched here
  bool launch_event_set = false;
};

namespace {

// The daemon is gone (its end of the control socket closed). In stream-memory-operation
// mode a caller's stream may already hold a "wait until done >= n" that only the daemon
// would have satisfied; left alone, that stream and everything queued behind it would sit
// there until the process is killed. The semaphore page is host memory mapped in this
// process too, so the library satisfies every such wait itself with a value above any
// sequence number (the comparison is cyclic, hence 2^62 and not all ones) and marks the
// communicators failed: the waits fall through, the results are undefined, and the next
// call on each communicator reports mccsNotConnected.
void on_daemon_lost_locked() {
  Context& c = g_ctx;
  c.connected = false;
  for (mccsComm* comm : c.comms) {
    if (!comm->sticky_error) comm->sticky_error = mccsNotConnected;
    if (comm->sync_host)
      __atomic_store_n((uint64_t*)comm->sync_host + proto::kSyncDoneSlot, 1ull << 62, __ATOMIC_RELEASE);
  }
  c.reply_cv.notify_all();
}

// For the places that notice the closed socket themselves, without the lock held.
mccsResult_t daemon_lost() {
  std::unique_lock<std::mutex> g(g_ctx.mu);
  if (g_ctx.connected) on_daemon_lost_locked();
  return mccsNotConnected;
}

// Watches the control socket for the daemon's death, because a process whose threads all
// sit in a stream synchronisation makes no call that would notice it.
std::atomic<bool> g_watch_stop{false};
std::atomic<int> g_watch_generation{0};
struct WatchStopAtExit { ~WatchStopAtExit() { g_watch_stop.store(true); } } g_watch_stop_at_exit;

void* watch_daemon(void* arg) {
  const int my_generation = (int)(intptr_t)arg;
  for (;;) {
    if (g_watch_stop.load() || g_watch_generation.load() != my_generation) return nullptr;
    int fd;
    {
      std::unique_lock<std::mutex> g(g_ctx.mu);
      if (!g_ctx.connected || g_ctx.fd < 0) return nullptr;
      fd = g_ctx.fd;
    }
    struct pollfd pf = {fd, 0, 0};
    const int rc = poll(&pf, 1, 100);
    if (g_watch_stop.load() || g_watch_generation.load() != my_generation) return nullptr;
    if (rc > 0 && (pf.revents & (POLLHUP | POLLERR | POLLNVAL))) {
      std::unique_lock<std::mutex> g(g_ctx.mu);
      if (g_ctx.connected && g_ctx.fd == fd && g_watch_generation.load() == my_generation) {
        LOG_ERROR("the mccs daemon closed the connection: pending stream waits are released, communicators fail");
        on_daemon_lost_locked();
      }
      return nullptr;
    }
  }
}

void start_daemon_watch() {
  pthread_t t;
  pthread_attr_t attr;
  pthread_attr_init(&attr);
  pthread_attr_setdetachstate(&attr, PTHREAD_CREATE_DETACHED);
  const int generation = g_watch_generation.fetch_add(1) + 1;
  if (pthread_create(&t, &attr, watch_daemon, (void*)(intptr_t)generation) != 0)
    LOG_WARN("could not start the daemon watch thread: a daemon that dies will only be noticed by the next call");
  pthread_attr_destroy(&attr);
}

std::string default_control_path() {
  const char* direct = getenv("MCCS_CONTROL");
  if (direct && direct[0] == '/') return direct;
  const char* prefix = getenv("MCCS_PREFIX");
  std::string p = prefix ? prefix : "/tmp/mccs-${USER}";
  p = expand_env(p);
  if (!p.empty() && p.back() == '/') p.pop_back();
  return p + "/" + (direct ? direct : "control.sock");
}

// Request/reply on the control connection. The caller holds g_ctx.mu through `lk`;
// the lock is released while waiting so that several threads can have requests in
// flight (communicator creation blocks until all ranks have joined, and those ranks
// may be threads of this very process). Whichever waiting thread finds the socket
// free reads it and files replies by request id for the others.
mccsResult_t roundtrip(std::unique_lock<std::mutex>& lk, proto::AnyMsg& m, size_t len, uint32_t expect_type,
                       std::vector<int>* fds, int timeout_ms) {
  Context& c = g_ctx;
  m.h.magic = proto::kMagic;
  m.h.req_id = c.next_req++;
  const uint32_t req = m.h.req_id;
  ssize_t n = ipc::uds_send(c.fd, &m, len);
  if (n < 0) return mccsProtocolError;
  struct timespec t0;
  clock_gettime(CLOCK_MONOTONIC, &t0);
  for (;;) {
    auto it = c.replies.find(req);
    if (it != c.replies.end()) {
      m = it->second.msg;
      if (fds) *fds = it->second.fds;
      else for (int f : it->second.fds) close(f);
      c.replies.erase(it);
      if (m.h.type != expect_type) return mccsProtocolError;
      return (mccsResult_t)m.h.status;
    }
    if (!c.connected && c.session_id != 0) return mccsNotConnected;
    struct timespec t1;
    clock_gettime(CLOCK_MONOTONIC, &t1);
    int64_t ms = (int64_t)(t1.tv_sec - t0.tv_sec) * 1000 + (t1.tv_nsec - t0.tv_nsec) / 1000000;
    if (ms > timeout_ms) return mccsTimeout;
    if (c.reader_active) {
      c.reply_cv.wait_for(lk, std::chrono::milliseconds(20));
      continue;
    }
    c.reader_active = true;
    const int fd = c.fd;
    lk.unlock();
    Reply rep;
    ssize_t got = -EAGAIN;
    int rc = ipc::wait_readable(fd, 20);
    if (rc > 0) got = ipc::uds_recv(fd, &rep.msg, sizeof rep.msg, &rep.fds);
    lk.lock();
    c.reader_active = false;
    if (rc > 0) {
      if (got <= 0 && got != -EAGAIN) { on_daemon_lost_locked(); return mccsNotConnected; }
      if (got >= (ssize_t)sizeof(proto::Header) && rep.msg.h.magic == proto::kMagic)
        c.replies[rep.msg.h.req_id] = rep;
    } else if (rc < 0) {
      c.reply_cv.notify_all();
      return mccsProtocolError;
    }
    c.reply_cv.notify_all();
  }
}

mccsResult_t ensure_connected_locked(std::unique_lock<std::mutex>& lk, const char* path) {
  Context& c = g_ctx;
  if (c.connected) return mccsSuccess;
  std::string p = path && path[0] ? path : default_control_path();
  int fd = -1;
  // The daemon may still be starting: retry briefly.
  for (int i = 0; i < 100; i++) {
    fd = ipc::uds_connect(p);
    if (fd >= 0) break;
    usleep(50000);
  }
  if (fd < 0) {
    LOG_ERROR("cannot connect to the mccs daemon at %s: %s", p.c_str(), strerror(-fd));
    return mccsNotConnected;
  }
  c.fd = fd;
  proto::AnyMsg m;
  memset(&m, 0, sizeof m);
  m.h.type = proto::kHello;
  m.hello.version = proto::kVersion;
  m.hello.pid = (int)getpid();
  const char* aff = getenv("MCCS_DEVICE_AFFINITY");
  m.hello.device_affinity = aff ? atoi(aff) : -1;
  const char* app = getenv("MCCS_APP_NAME");
  snprintf(m.hello.app_name, sizeof m.hello.app_name, "%s", app ? app : program_invocation_short_name);
  mccsResult_t r = roundtrip(lk, m, sizeof(proto::Hello), proto::kWelcome, nullptr, 10000);
  if (r != mccsSuccess) { close(fd); c.fd = -1; return r; }
  c.backend = m.welcome.backend;
  c.daemon_pid = m.welcome.daemon_pid;
  c.same_process = c.daemon_pid == (int)getpid();
  c.num_devices = (int)m.welcome.num_devices;
  c.session_id = m.welcome.session_id;
  c.sync_mode = m.welcome.sync_mode;
  const char* to = getenv("MCCS_WC_TIMEOUT_MS");
  if (to) c.wc_timeout_ms = strtoull(to, nullptr, 10);
  c.connected = true;
  if (!c.same_process) start_daemon_watch();   // an embedded daemon cannot die on its own
  if (c.backend == proto::kBackendCuda && !load_driver()) {
    LOG_ERROR("the daemon runs on CUDA but libcuda.so.1 cannot be loaded here");
    return mccsDeviceError;
  }
  return mccsSuccess;
}

const MemRec* find_mem_locked(const void* ptr) {
  const uint64_t a = (uint64_t)ptr;
  auto it = g_ctx.mem.upper_bound(a);
  if (it == g_ctx.mem.begin()) return nullptr;
  --it;
  if (a >= it->second.base + it->second.size) return nullptr;
  return &it->second;
}

mccsResult_t register_stream_locked(std::unique_lock<std::mutex>& lk, int device, mccsStream_t stream, StreamRec** out) {
  Context& c = g_ctx;
  auto key = std::make_pair(device, (uint64_t)stream);
  auto it = c.streams.find(key);
  if (it != c.streams.end()) { *out = &it->second; return mccsSuccess; }
  StreamRec rec;
  rec.device = device;
  proto::AnyMsg m;
  memset(&m, 0, sizeof m);
  m.h.type = proto::kRegisterStream;
  m.reg_stream.device = device;
  m.reg_stream.stream = (uint64_t)stream;
  if (c.backend == proto::kBackendCuda) {
    CtxScope scope(device);
    if (!scope.ok) return mccsDeviceError;
    unsigned flags = CU_EVENT_DISABLE_TIMING | (c.same_process ? 0u : (unsigned)CU_EVENT_INTERPROCESS);
    CUresult r = g_drv.cuEventCreate_(&rec.event, flags);
    if (r != CUDA_SUCCESS) { LOG_ERROR("cuEventCreate: %s", cu_err(r)); return mccsDeviceError; }
    if (c.same_process) {
      m.reg_stream.event_raw = (uint64_t)rec.event;
    } else {
      CUipcEventHandle h;
      r = g_drv.cuIpcGetEventHandle_(&h, rec.event);
      if (r != CUDA_SUCCESS) { LOG_ERROR("cuIpcGetEventHandle: %s", cu_err(r)); return mccsDeviceError; }
      static_assert(sizeof h == proto::kIpcHandleBytes, "IPC event handle size");
      memcpy(m.reg_stream.event_handle, &h, sizeof h);
    }
  }
  mccsResult_t r = roundtrip(lk, m, sizeof(proto::RegisterStreamReq), proto::kRegisterStreamReply, nullptr, 30000);
  if (r != mccsSuccess) return r;
  rec.stream_id = m.reg_stream_reply.stream_id;
  auto ins = c.streams.emplace(key, rec);
  *out = &ins.first->second;
  return mccsSuccess;
}

// Maps an allocation the daemon made (rec.share_kind/size/device filled in) into
// this process; `fd` is the descriptor that came with the reply (-1 if none).
mccsResult_t map_allocation(MemRec& rec, int fd, const uint8_t* ipc_handle, uint64_t daemon_va) {
  switch (rec.share_kind) {
    case proto::kShareSameProcess:
      rec.base = daemon_va;
      return mccsSuccess;
    case proto::kShareHostFd: {
      if (fd < 0) return mccsProtocolError;
      void* p = mmap(nullptr, rec.size, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
      if (p == MAP_FAILED) return mccsOutOfMemory;
      rec.base = (uint64_t)p;
      return mccsSuccess;
    }
    case proto::kShareVmmFd: {
      if (fd < 0) return mccsProtocolError;
      CtxScope scope(rec.device);
      if (!scope.ok) return mccsDeviceError;
      CUmemGenericAllocationHandle h = 0;
      CUresult cr = g_drv.cuMemImportFromShareableHandle_(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      if (cr != CUDA_SUCCESS) { LOG_ERROR("cuMemImportFromShareableHandle: %s", cu_err(cr)); return mccsDeviceError; }
      CUdeviceptr va = 0;
      cr = g_drv.cuMemAddressReserve_(&va, rec.size, 0, 0, 0);
      if (cr != CUDA_SUCCESS) { g_drv.cuMemRelease_(h); return mccsOutOfMemory; }
      cr = g_drv.cuMemMap_(va, rec.size, 0, h, 0);
      if (cr != CUDA_SUCCESS) {
        LOG_ERROR("cuMemMap: %s", cu_err(cr));
        g_drv.cuMemAddressFree_(va, rec.size);
        g_drv.cuMemRelease_(h);
        return mccsDeviceError;
      }
      CUmemAccessDesc desc;
      memset(&desc, 0, sizeof desc);
      desc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
      desc.location.id = rec.device;
      desc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
      cr = g_drv.cuMemSetAccess_(va, rec.size, &desc, 1);
      if (cr != CUDA_SUCCESS) {
        LOG_ERROR("cuMemSetAccess: %s", cu_err(cr));
        g_drv.cuMemUnmap_(va, rec.size);
        g_drv.cuMemAddressFree_(va, rec.size);
        g_drv.cuMemRelease_(h);
        return mccsDeviceError;
      }
      rec.base = (uint64_t)va;
      rec.vmm_handle = (uint64_t)h;
      return mccsSuccess;
    }
    case proto::kShareCudaIpc: {
      CtxScope scope(rec.device);
      if (!scope.ok) return mccsDeviceError;
      CUipcMemHandle h;
      memcpy(&h, ipc_handle, sizeof h);
      CUdeviceptr p = 0;
      CUresult cr = g_drv.cuIpcOpenMemHandle_(&p, h, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS);
      if (cr != CUDA_SUCCESS) { LOG_ERROR("cuIpcOpenMemHandle: %s", cu_err(cr)); return mccsDeviceError; }
      rec.base = (uint64_t)p;
      return mccsSuccess;
    }
  }
  return mccsProtocolError;
}

void unmap_allocation(const MemRec& rec) {
  if (!rec.base) return;
  if (rec.share_kind == proto::kShareHostFd) {
    munmap((void*)rec.base, rec.size);
  } else if (rec.share_kind == proto::kShareVmmFd && g_drv.ok) {
    CtxScope scope(rec.device);
    g_drv.cuMemUnmap_((CUdeviceptr)rec.base, rec.size);
    g_drv.cuMemAddressFree_((CUdeviceptr)rec.base, rec.size);
    g_drv.cuMemRelease_((CUmemGenericAllocationHandle)rec.vmm_handle);
  } else if (rec.share_kind == proto::kShareCudaIpc && g_drv.ok) {
    CtxScope scope(rec.device);
    g_drv.cuIpcCloseMemHandle_((CUdeviceptr)rec.base);
  }
}

// The collective kernels for client-side launch on a GPU live in a library of their own
// next to this one (it carries the device code and a static CUDA runtime), loaded when the
// first communicator in that mode is created.
typedef unsigned long long (*KernelsAbiFn)(void);
typedef int (*KernelsLaunchFn)(int, const CollArgs*, int, int, void*, const char**);
typedef int (*KernelsLaunchBatchFn)(const BatchArgs*, int, int, void*, const char**);
struct KernelsLib {
  bool tried = false;
  void* lib = nullptr;
  KernelsLaunchFn launch = nullptr;
  KernelsLaunchBatchFn launch_batch = nullptr;
};
KernelsLib g_klib;

bool load_kernels_lib() {   // g_ctx.mu held
  if (g_klib.tried) return g_klib.launch != nullptr;
  g_klib.tried = true;
  std::string path = "libmccs_kernels.so";
  Dl_info info;
  if (dladdr((void*)&load_kernels_lib, &info) && info.dli_fname) {
    std::string self = info.dli_fname;
    size_t slash = self.rfind('/');
    if (slash != std::string::npos) path = self.substr(0, slash + 1) + path;
  }
  const char* over = getenv("MCCS_KERNELS_LIB");
  if (over && over[0]) path = over;
  g_klib.lib = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
  if (!g_klib.lib) { LOG_ERROR("client-side launch: cannot load %s: %s", path.c_str(), dlerror()); return false; }
  KernelsAbiFn abi = (KernelsAbiFn)dlsym(g_klib.lib, "mccs_kernels_abi");
  KernelsLaunchFn fn = (KernelsLaunchFn)dlsym(g_klib.lib, "mccs_kernels_launch");
  g_klib.launch_batch = (KernelsLaunchBatchFn)dlsym(g_klib.lib, "mccs_kernels_launch_batch");
  if (!abi || !fn || abi() != (sizeof(CollArgs) | ((unsigned long long)sizeof(BatchArgs) << 32))) {
    LOG_ERROR("client-side launch: %s does not match this library", path.c_str());
    return false;
  }
  g_klib.launch = fn;
  return true;
}

// Client-side launch: maps a block described by a kMapScratch / kMapMem reply for the
// kernels this process launches on `device` (-1: host backend). The descriptor stays the
// caller's to close.
mccsResult_t map_block(int fd, size_t bytes, uint32_t share_kind, uint64_t daemon_va, int device, Mapped* out) {
  *out = Mapped();
  out->bytes = bytes;
  out->share_kind = share_kind;
  if (share_kind == proto::kShareSameProcess) {
    out->addr = daemon_va;
    return daemon_va ? mccsSuccess : mccsProtocolError;
  }
  if (share_kind == proto::kShareVmmFd) {
    // Device memory of any GPU of the box: imported and made accessible to `device`.
    MemRec rec;
    rec.size = bytes;
    rec.device = device;
    rec.share_kind = share_kind;
    mccsResult_t r = map_allocation(rec, fd, nullptr, 0);
    if (r != mccsSuccess) return r;
    out->addr = rec.base;
    out->vmm_handle = rec.vmm_handle;
    return mccsSuccess;
  }
  if (share_kind != proto::kShareHostFd || fd < 0) return mccsUnsupported;
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (p == MAP_FAILED) return mccsOutOfMemory;
  out->host = p;
  out->addr = (uint64_t)p;
  if (device >= 0) {
    // Shared host memory that kernels address: pinned and mapped into the device's
    // address space here, as the daemon did on its side.
    CtxScope scope(device);
    if (!scope.ok || !g_drv.memops) { munmap(p, bytes); return mccsDeviceError; }
    CUresult cr = g_drv.cuMemHostRegister_(p, bytes, CU_MEMHOSTREGISTER_PORTABLE | CU_MEMHOSTREGISTER_DEVICEMAP);
    CUdeviceptr d = 0;
    if (cr == CUDA_SUCCESS) {
      out->registered = true;
      cr = g_drv.cuMemHostGetDevicePointer_(&d, p, 0);
    }
    if (cr != CUDA_SUCCESS) {
      LOG_ERROR("registering shared host memory for client-side launch: %s", cu_err(cr));
      if (out->registered) g_drv.cuMemHostUnregister_(p);
      munmap(p, bytes);
      *out = Mapped();
      return mccsDeviceError;
    }
    out->addr = (uint64_t)d;
  }
  return mccsSuccess;
}

void unmap_block(Mapped& m, int device) {
  if (!m.addr) return;
  if (m.emulated_mc) {
    emulated_mc_remove(m.addr);
    munmap((void*)m.addr, m.bytes);
    m = Mapped();
    return;
  }
  if (m.share_kind == proto::kShareVmmFd) {
    MemRec rec;
    rec.base = m.addr; rec.size = m.bytes; rec.device = device; rec.share_kind = m.share_kind; rec.vmm_handle = m.vmm_handle;
    unmap_allocation(rec);
  } else if (m.share_kind == proto::kShareHostFd && m.host) {
    if (m.registered && g_drv.ok) {
      CtxScope scope(device);
      if (scope.ok) g_drv.cuMemHostUnregister_(m.host);
    }
    munmap(m.host, m.bytes);
  }
  m = Mapped();
}

// Spins for the completion of the oldest outstanding request of `comm`.
mccsResult_t wait_completion(mccsComm* comm, proto::WorkCompletion* wc) {
  struct timespec t0;
  clock_gettime(CLOCK_MONOTONIC, &t0);
  uint64_t spins = 0;
  while (!comm->cq.try_pop(wc)) {
    if ((++spins & 0xfff) == 0) {
      struct timespec t1;
      clock_gettime(CLOCK_MONOTONIC, &t1);
      uint64_t ms = (uint64_t)(t1.tv_sec - t0.tv_sec) * 1000 + (uint64_t)((t1.tv_nsec - t0.tv_nsec) / 1000000);
      if (ms > g_ctx.wc_timeout_ms) return mccsTimeout;
      // A dead daemon never completes anything: notice the closed control connection.
      struct pollfd pf = {g_ctx.fd, 0, 0};
      if (poll(&pf, 1, 0) > 0 && (pf.revents & (POLLHUP | POLLERR))) return daemon_lost();
      if (spins > (1u << 22)) usleep(50);
    }
  }
  comm->outstanding--;
  comm->last_variant = wc->variant;
  comm->last_ctas = wc->ctas;
  if (wc->status != 0 && comm->sticky_error == 0) comm->sticky_error = wc->status;
  return (mccsResult_t)wc->status;
}

mccsResult_t finish_on_stream(mccsComm* comm, mccsStream_t stream) {
  if (g_ctx.backend != proto::kBackendCuda || !comm->backend_event) return mccsSuccess;
  CtxScope scope(comm->device);
  if (!scope.ok) return mccsDeviceError;
  CUresult r = g_drv.cuStreamWaitEvent_((CUstream)stream, comm->backend_event, 0);
  if (r != CUDA_SUCCESS) { LOG_ERROR("cuStreamWaitEvent: %s", cu_err(r)); return mccsDeviceError; }
  return mccsSuccess;
}

// Takes whatever completions have arrived, without waiting.
void reap_completions(mccsComm* comm) {
  if (comm->dp_status && comm->memop_posted) {
    const uint64_t done = __atomic_load_n(&comm->dp_status->completed, __ATOMIC_ACQUIRE);
    if (done) {
      comm->last_variant = comm->dp_status->last_variant;
      comm->last_ctas = comm->dp_status->last_ctas;
    }
    if (comm->dp_status->first_error != 0 && comm->sticky_error == 0) comm->sticky_error = comm->dp_status->first_error;
  }
  proto::WorkCompletion wc;
  while (comm->outstanding > 0 && comm->cq.try_pop(&wc)) {
    comm->outstanding--;
    comm->last_variant = wc.variant;
    comm->last_ctas = wc.ctas;
    if (wc.status != 0 && comm->sticky_error == 0) comm->sticky_error = wc.status;
  }
}

// The two stream memory operations of the mem-op mode. On the host backend there is no
// stream: the write happens now and the wait blocks the caller (host collectives are
// complete when a call returns anyway), which keeps the protocol with the daemon the same.
mccsResult_t sem_write(mccsComm* comm, mccsStream_t stream, uint64_t addr, uint64_t value) {
  if (comm->sync_emulated) {
    __atomic_store_n((uint64_t*)addr, value, __ATOMIC_RELEASE);
    return mccsSuccess;
  }
  CUresult r = g_drv.cuStreamWriteValue64_((CUstream)stream, (CUdeviceptr)addr, value, CU_STREAM_WRITE_VALUE_DEFAULT);
  if (r != CUDA_SUCCESS) { LOG_ERROR("cuStreamWriteValue64: %s", cu_err(r)); return mccsDeviceError; }
  return mccsSuccess;
}

mccsResult_t sem_wait_geq(mccsComm* comm, mccsStream_t stream, uint64_t addr, uint64_t value) {
  if (comm->sync_emulated) {
    struct timespec t0;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    uint64_t spins = 0;
    while ((int64_t)(__atomic_load_n((uint64_t*)addr, __ATOMIC_ACQUIRE) - value) < 0) {
      if ((++spins & 0xfff) == 0) {
        struct timespec t1;
        clock_gettime(CLOCK_MONOTONIC, &t1);
        uint64_t ms = (uint64_t)(t1.tv_sec - t0.tv_sec) * 1000 + (uint64_t)((t1.tv_nsec - t0.tv_nsec) / 1000000);
        if (ms > g_ctx.wc_timeout_ms) return mccsTimeout;
        struct pollfd pf = {g_ctx.fd, 0, 0};
        if (poll(&pf, 1, 0) > 0 && (pf.revents & (POLLHUP | POLLERR))) return daemon_lost();
        if (spins > (1u << 20)) usleep(50);
      }
    }
    return mccsSuccess;
  }
  CUresult r = g_drv.cuStreamWaitValue64_((CUstream)stream, (CUdeviceptr)addr, value, CU_STREAM_WAIT_VALUE_GEQ);
  if (r != CUDA_SUCCESS) { LOG_ERROR("cuStreamWaitValue64: %s", cu_err(r)); return mccsDeviceError; }
  return mccsSuccess;
}

// Mem-op mode: nothing blocks. The caller's stream publishes "submitted", the request
// is posted, and the stream is told to wait for the request's "done" value, which the
// daemon's stream writes after the kernel. Errors surface on a later call.
mccsResult_t submit_memops(mccsComm* comm, proto::WorkRequest& wr, mccsStream_t stream) {
  reap_completions(comm);
  if (comm->sticky_error) return (mccsResult_t)comm->sticky_error;
  uint32_t slot;
  auto it = comm->stream_slot.find((uint64_t)stream);
  if (it == comm->stream_slot.end()) {
    // Two ranks of one communicator on the same stream can never finish: the second
    // rank's "submitted" mark would sit behind the first rank's "wait until done".
    std::unique_lock<std::mutex> g(g_ctx.mu);   // stream tables are only changed under this lock
    for (mccsComm* other : g_ctx.comms)
      if (!comm->sync_emulated && other != comm && other->id == comm->id && other->stream_slot.count((uint64_t)stream)) {
        LOG_ERROR("communicator %u: ranks %d and %d of this process use the same CUDA stream; give each rank "
                  "its own stream (or run the daemon with [b200] sync = \"events\")", comm->id, other->rank, comm->rank);
        return mccsInvalidArgument;
      }
    slot = (uint32_t)comm->stream_slot.size();
    if (slot >= proto::kSyncMaxStreams) return mccsUnsupported;
    comm->stream_slot[(uint64_t)stream] = slot;
  } else {
    slot = it->second;
  }
  wr.comm_handle = comm->handle;
  wr.user_seq = comm->next_user_seq++;
  wr.sync_slot = slot + 1;
  wr.sync_value = ++comm->slot_value[slot];
  CtxScope scope(comm->sync_emulated ? -1 : comm->device);
  if (!scope.ok) return mccsDeviceError;
  mccsResult_t sr = sem_write(comm, stream, comm->sync_base + 8 * (proto::kSyncFirstStreamSlot + slot), wr.sync_value);
  if (sr != mccsSuccess) return sr;
  uint64_t spins = 0;
  while (!comm->wq.try_push(&wr)) {
    reap_completions(comm);
    if ((++spins & 0xffff) == 0) {
      struct pollfd pf = {g_ctx.fd, 0, 0};
      if (poll(&pf, 1, 0) > 0 && (pf.revents & (POLLHUP | POLLERR))) return daemon_lost();
    }
  }
  comm->memop_posted++;
  comm->last_posted_seq = wr.user_seq;
  if (comm->deferred_wait) return mccsSuccess;
  if (g_group_depth > 0) {
    // Inside a group the stream is not made to wait after every collective: the daemon
    // sees all of them submitted at once and queues their kernels back to back;
    // mccsGroupEnd orders the stream after the last one.
    g_group_items.push_back({comm, stream});
    return mccsSuccess;
  }
  sr = sem_wait_geq(comm, stream, comm->sync_base + 8 * proto::kSyncDoneSlot, wr.user_seq);
  if (sr != mccsSuccess) return sr;
  if (comm->sync_emulated) {
    // the call is synchronous here: report this request's own error, as the event mode does
    reap_completions(comm);
    if (comm->sticky_error) return (mccsResult_t)comm->sticky_error;
  }
  return mccsSuccess;
}

// Address, in this process, of byte `off` of allocation `mem_id`: one of the caller's own
// allocations, or a peer's, mapped on first use (client-side launch only).
mccsResult_t resolve_mem(std::unique_lock<std::mutex>& g, mccsComm* comm, uint64_t mem_id, uint64_t off, uint64_t* out) {
  auto own = g_ctx.mem_base_by_id.find(mem_id);
  if (own != g_ctx.mem_base_by_id.end()) { *out = own->second + off; return mccsSuccess; }
  auto it = comm->peer_mem.find(mem_id);
  if (it == comm->peer_mem.end()) {
    proto::AnyMsg m;
    memset(&m, 0, sizeof m);
    m.h.type = proto::kMapMem;
    m.map_mem.comm_handle = comm->handle;
    m.map_mem.mem_id = mem_id;
    std::vector<int> fds;
    mccsResult_t r = roundtrip(g, m, sizeof(proto::MapMemReq), proto::kMapMemReply, &fds, 30000);
    if (r != mccsSuccess) return r;
    Mapped mp;
    r = map_block(fds.empty() ? -1 : fds[0], (size_t)m.map_mem_reply.bytes, m.map_mem_reply.share_kind, m.map_mem_reply.daemon_va,
                  g_ctx.backend == proto::kBackendCuda ? comm->device : -1, &mp);
    for (int f : fds) close(f);
    if (r != mccsSuccess) return r;
    it = comm->peer_mem.emplace(mem_id, mp).first;
  }
  if (off > it->second.bytes) return mccsInvalidArgument;
  *out = it->second.addr + off;
  return mccsSuccess;
}

// Multicast address of byte `off` of region `mc_id` for this rank's kernels; the region is
// mapped on first use: the exported multicast object on a GPU, an emulated region over this
// process's own mappings of the ranks' buffers on the host backend.
mccsResult_t resolve_mc(std::unique_lock<std::mutex>& g, mccsComm* comm, uint64_t mc_id, uint64_t off, uint64_t* out) {
  auto it = comm->mc_map.find(mc_id);
  if (it == comm->mc_map.end()) {
    proto::AnyMsg m;
    memset(&m, 0, sizeof m);
    m.h.type = proto::kMapMc;
    m.map_mc.comm_handle = comm->handle;
    m.map_mc.mc_id = mc_id;
    std::vector<int> fds;
    mccsResult_t rt = roundtrip(g, m, sizeof(proto::MapMcReq), proto::kMapMcReply, &fds, 30000);
    if (rt != mccsSuccess) return rt;
    const proto::MapMcReply& rep = m.map_mc_reply;
    Mapped mp;
    mp.bytes = (size_t)rep.bytes;
    mp.share_kind = rep.share_kind;
    mccsResult_t r = mccsSuccess;
    if (rep.share_kind == proto::kShareSameProcess) {
      mp.addr = rep.daemon_va;
      if (!mp.addr) r = mccsProtocolError;
    } else if (rep.share_kind == proto::kShareVmmFd && !fds.empty()) {
      CtxScope scope(comm->device);
      CUmemGenericAllocationHandle h = 0;
      CUdeviceptr va = 0;
      CUresult cr = scope.ok ? g_drv.cuMemImportFromShareableHandle_(&h, (void*)(uintptr_t)fds[0], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR)
                             : CUDA_ERROR_INVALID_CONTEXT;
      if (cr == CUDA_SUCCESS) {
        cr = g_drv.cuMemAddressReserve_(&va, mp.bytes, (size_t)rep.align, 0, 0);
        if (cr == CUDA_SUCCESS) {
          cr = g_drv.cuMemMap_(va, mp.bytes, 0, h, 0);
          if (cr == CUDA_SUCCESS) {
            CUmemAccessDesc desc;
            memset(&desc, 0, sizeof desc);
            desc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
            desc.location.id = comm->device;
            desc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
            cr = g_drv.cuMemSetAccess_(va, mp.bytes, &desc, 1);
            if (cr != CUDA_SUCCESS) g_drv.cuMemUnmap_(va, mp.bytes);
          }
          if (cr != CUDA_SUCCESS) g_drv.cuMemAddressFree_(va, mp.bytes);
        }
        if (cr != CUDA_SUCCESS) g_drv.cuMemRelease_(h);
      }
      if (cr != CUDA_SUCCESS) {
        LOG_ERROR("mapping multicast region %llu: %s", (unsigned long long)mc_id, cu_err(cr));
        r = mccsDeviceError;
      } else {
        mp.addr = (uint64_t)va;
        mp.vmm_handle = (uint64_t)h;
      }
    } else if (rep.share_kind == proto::kShareHostFd && g_ctx.backend == proto::kBackendHost) {
      std::vector<void*> backing;
      for (uint32_t q = 0; q < rep.nranks && q < 8 && r == mccsSuccess; q++) {
        uint64_t p = 0;
        r = resolve_mem(g, comm, rep.mems[q], 0, &p);
        backing.push_back((void*)p);
      }
      if (r == mccsSuccess) {
        void* base = mmap(nullptr, mp.bytes, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
        if (base == MAP_FAILED) r = mccsOutOfMemory;
        else {
          emulated_mc_add((uint64_t)base, mp.bytes, backing);
          mp.addr = (uint64_t)base;
          mp.emulated_mc = true;
        }
      }
    } else {
      r = mccsUnsupported;
    }
    for (int f : fds) close(f);
    if (r != mccsSuccess) return r;
    it = comm->mc_map.emplace(mc_id, mp).first;
  }
  if (off > it->second.bytes) return mccsInvalidArgument;
  *out = it->second.addr + off;
  return mccsSuccess;
}

// Waits for the next message of the plan ring, which must answer request `user_seq`.
mccsResult_t wait_plan(mccsComm* comm, uint64_t user_seq, proto::PlanMsg* plan) {
  uint64_t spins = 0;
  struct timespec t0;
  clock_gettime(CLOCK_MONOTONIC, &t0);
  while (!comm->pq.try_pop(plan)) {
    if ((++spins & 0xfff) == 0) {
      struct timespec t1;
      clock_gettime(CLOCK_MONOTONIC, &t1);
      uint64_t ms = (uint64_t)(t1.tv_sec - t0.tv_sec) * 1000 + (uint64_t)((t1.tv_nsec - t0.tv_nsec) / 1000000);
      if (ms > g_ctx.wc_timeout_ms) return mccsTimeout;
      struct pollfd pf = {g_ctx.fd, 0, 0};
      if (poll(&pf, 1, 0) > 0 && (pf.revents & (POLLHUP | POLLERR))) return daemon_lost();
      if (spins > (1u << 20)) usleep(50);
    }
  }
  if (plan->user_seq != user_seq) return mccsProtocolError;
  if (plan->status != 0) {
    if (comm->sticky_error == 0) comm->sticky_error = plan->status;
    return (mccsResult_t)plan->status;
  }
  if (plan->nranks != comm->nranks) return mccsProtocolError;
  return mccsSuccess;
}

// The kernel arguments a plan describes, with every address resolved in this process: the
// caller's own allocations by id, peers' buffers and multicast regions from this
// communicator's maps (filled on first use).
mccsResult_t args_from_plan(mccsComm* comm, const proto::PlanMsg& plan, CollArgs* out) {
  CollArgs& a = *out;
  memset(&a, 0, sizeof a);
  a.rank = comm->rank;
  a.nranks = comm->nranks;
  a.dtype = plan.dtype;
  a.op = plan.op;
  a.variant = plan.variant;
  a.count = plan.count;
  a.seq = plan.ticket;
  a.scale = plan.scale;
  a.epoch = plan.epoch;
  a.timeout_ns = plan.timeout_ns;
  a.trace = plan.trace;
  a.unroll_hint = plan.variant_hint;
  std::unique_lock<std::mutex> g(g_ctx.mu);
  for (int r = 0; r < comm->nranks; r++) {
    uint64_t s = 0, d = 0;
    mccsResult_t rr = resolve_mem(g, comm, plan.rank[r].send_mem, plan.rank[r].send_off, &s);
    if (rr == mccsSuccess) rr = resolve_mem(g, comm, plan.rank[r].recv_mem, plan.rank[r].recv_off, &d);
    if (rr != mccsSuccess) return rr;
    a.send[r] = (const void*)s;
    a.recv[r] = (void*)d;
    a.pad[r] = (SignalPad*)comm->pad_map[r].addr;
    a.status[r] = (StatusBlock*)comm->status_map[r].addr;
    a.fifo[r] = (char*)comm->fifo_map[r].addr;
  }
  if (plan.mc_send_id) {
    uint64_t p = 0;
    mccsResult_t rr = resolve_mc(g, comm, plan.mc_send_id, plan.mc_send_off, &p);
    if (rr != mccsSuccess) return rr;
    a.mc_send = (const void*)p;
  }
  if (plan.mc_recv_id) {
    uint64_t p = 0;
    mccsResult_t rr = resolve_mc(g, comm, plan.mc_recv_id, plan.mc_recv_off, &p);
    if (rr != mccsSuccess) return rr;
    a.mc_recv = (void*)p;
  }
  g.unlock();
  a.fifo_slot_bytes = comm->fifo_slot_bytes;
  memcpy(a.ring, plan.ring, sizeof a.ring);
  for (int ch = 0; ch < kMaxRingChannels; ch++) a.ring_step_base[ch] = plan.ring_step_base[ch];
  return mccsSuccess;
}

// Launches one kernel of this rank on `stream`: a single collective (`batch` null) or a fused
// launch of several. On the caller's stream, in the caller's context: ordered against the
// caller's other work like any kernel of its own. An error a previous kernel left behind (a
// wait that ran out, an abort raised by the daemon) ends the communicator before the launch.
mccsResult_t launch_here(mccsComm* comm, int kind, const CollArgs& a, const BatchArgs* batch, LaunchDims dims, mccsStream_t stream) {
  const StatusBlock* mine = (const StatusBlock*)comm->status_map[comm->rank].host;
  if (g_ctx.backend == proto::kBackendCuda) {
    uint32_t before = __atomic_load_n(&mine->error, __ATOMIC_ACQUIRE);
    if (before != 0) {
      comm->sticky_error = before == kDevAborted ? mccsAborted : mccsTimeout;
      return (mccsResult_t)comm->sticky_error;
    }
    if (!g_klib.launch || (batch && !g_klib.launch_batch)) return mccsUnsupported;
    CtxScope scope(comm->device);
    if (!scope.ok) return mccsDeviceError;
    const char* what = nullptr;
    int e = batch ? g_klib.launch_batch(batch, dims.ctas, dims.threads, (void*)stream, &what)
                  : g_klib.launch(kind, &a, dims.ctas, dims.threads, (void*)stream, &what);
    if (e != 0) {
      LOG_ERROR("client-side launch of %s failed: %s", variant_name(a.variant), what ? what : "?");
      comm->sticky_error = mccsDeviceError;
      return mccsDeviceError;
    }
    comm->launched_here = true;
    if (comm->deferred_wait) {
      // The caller will name the stream that needs the results later (mccsCommWait).
      if (!comm->launch_event && g_drv.cuEventCreate_(&comm->launch_event, CU_EVENT_DISABLE_TIMING) != CUDA_SUCCESS) {
        comm->launch_event = nullptr;
        return mccsDeviceError;
      }
      if (g_drv.cuEventRecord_(comm->launch_event, (CUstream)stream) != CUDA_SUCCESS) return mccsDeviceError;
      comm->launch_event_set = true;
    }
    return mccsSuccess;
  }
  if (!(batch ? emulated_launch_batch_rank(*batch, dims) : emulated_launch_rank(kind, a, dims))) return mccsUnsupported;
  const uint32_t err = __atomic_load_n(&mine->error, __ATOMIC_ACQUIRE);
  if (err != 0) {
    comm->sticky_error = err == kDevAborted ? mccsAborted : mccsTimeout;
    return (mccsResult_t)comm->sticky_error;
  }
  return mccsSuccess;
}

// Takes the answer(s) to request `user_seq` from the plan ring and launches what they
// describe: one kernel, or one kernel per time slice (the daemon hands each slice's plan out
// once that slice is admitted). `plan` is the first answer, already taken.
mccsResult_t run_planned(mccsComm* comm, uint64_t user_seq, proto::PlanMsg& plan, mccsStream_t stream) {
  for (;;) {
    comm->last_variant = (uint32_t)plan.variant;
    comm->last_ctas = (uint32_t)plan.ctas;
    CollArgs a;
    mccsResult_t r = args_from_plan(comm, plan, &a);
    if (r != mccsSuccess) return r;
    r = launch_here(comm, plan.kind, a, nullptr, LaunchDims{plan.ctas, plan.threads}, stream);
    if (r != mccsSuccess) return r;
    if (plan.slice + 1 >= (plan.nslices > 0 ? plan.nslices : 1)) return mccsSuccess;
    r = wait_plan(comm, user_seq, &plan);
    if (r != mccsSuccess) return r;
  }
}

// Requests posted inside a group whose plans have not been taken yet (client-side launch with
// fused launches enabled in the daemon): posting all of them before the first plan is read
// is what lets the daemon see them together and carry several in one kernel.
struct DeferredLaunch { mccsComm* comm; uint64_t user_seq; mccsStream_t stream; };
thread_local std::vector<DeferredLaunch> g_deferred;

bool names_deferred(const mccsComm* comm) {
  for (const DeferredLaunch& d : g_deferred)
    if (d.comm == comm) return true;
  return false;
}

bool ring_out_of_step(mccsResult_t r) { return r == mccsTimeout || r == mccsNotConnected || r == mccsProtocolError; }

// A fused launch: `head` (the answer to items[i]) carries the launch shape, the barrier epoch
// and the ticket; the answers to the next batch_len - 1 requests of the same communicator
// carry the other members' buffers. Every answer is taken off the ring even when one member
// cannot run here (the launch then does not happen), so the ring stays in step.
mccsResult_t launch_fused(const std::vector<DeferredLaunch>& items, size_t i, const proto::PlanMsg& head) {
  mccsComm* comm = items[i].comm;
  const int len = head.batch_len;
  if (len > kMaxBatch || i + (size_t)len > items.size()) return mccsProtocolError;
  for (int k = 1; k < len; k++)
    if (items[i + (size_t)k].comm != comm) return mccsProtocolError;
  comm->last_variant = (uint32_t)head.variant;
  comm->last_ctas = (uint32_t)head.ctas;
  BatchArgs b;
  memset(&b, 0, sizeof b);
  b.nops = len;
  mccsResult_t result = args_from_plan(comm, head, &b.base);
  for (int k = 0; k < len; k++) {
    proto::PlanMsg member = head;
    if (k > 0) {
      mccsResult_t r = wait_plan(comm, items[i + (size_t)k].user_seq, &member);
      if (ring_out_of_step(r)) return r;
      if (r == mccsSuccess && member.batch_len != -1) return mccsProtocolError;
      if (r != mccsSuccess) {
        if (result == mccsSuccess) result = r;
        continue;
      }
    }
    if (result != mccsSuccess) continue;
    CollArgs ma;
    result = args_from_plan(comm, member, &ma);
    if (result != mccsSuccess) continue;
    b.count[k] = member.count;
    for (int q = 0; q < comm->nranks; q++) { b.send[k][q] = ma.send[q]; b.recv[k][q] = ma.recv[q]; }
    b.mc_send[k] = ma.mc_send;
    b.mc_recv[k] = ma.mc_recv;
  }
  if (result != mccsSuccess) return result;
  return launch_here(comm, kAllReduce, b.base, &b, LaunchDims{head.ctas, head.threads}, items[i].stream);
}

mccsResult_t flush_deferred() {
  std::vector<DeferredLaunch> items;
  items.swap(g_deferred);
  mccsResult_t result = mccsSuccess;
  for (size_t i = 0; i < items.size(); i++) {
    mccsComm* comm = items[i].comm;
    proto::PlanMsg plan;
    mccsResult_t r = wait_plan(comm, items[i].user_seq, &plan);
    if (r == mccsSuccess && plan.batch_len >= 2) {
      r = launch_fused(items, i, plan);
      i += (size_t)plan.batch_len - 1;
    } else if (r == mccsSuccess) {
      r = run_planned(comm, items[i].user_seq, plan, items[i].stream);
    }
    if (r != mccsSuccess) {
      if (result == mccsSuccess) result = r;
      if (ring_out_of_step(r)) return r;
    }
  }
  return result;
}

// Client-side launch: post the request, wait for the plan the daemon makes for all ranks
// (variant, launch shape, barrier epoch, ticket, ring order, everybody's buffers), and
// launch this rank's kernel here. The daemon never touches a stream for this collective.
mccsResult_t submit_client_launch(mccsComm* comm, proto::WorkRequest& wr, mccsStream_t stream) {
  if (comm->sticky_error) return (mccsResult_t)comm->sticky_error;
  wr.comm_handle = comm->handle;
  wr.user_seq = comm->next_user_seq++;
  uint64_t spins = 0;
  while (!comm->wq.try_push(&wr)) {
    if ((++spins & 0xffff) == 0) {
      struct pollfd pf = {g_ctx.fd, 0, 0};
      if (poll(&pf, 1, 0) > 0 && (pf.revents & (POLLHUP | POLLERR))) return daemon_lost();
    }
  }
  comm->last_posted_seq = wr.user_seq;
  if (g_group_depth > 0 && comm->group_defer) {
    // Inside a group: only posted here; mccsGroupEnd (or a group that outgrows the plan
    // ring) takes the plans and launches.
    g_deferred.push_back({comm, wr.user_seq, stream});
    if (g_deferred.size() >= proto::kPqDepth - 1) return flush_deferred();
    return mccsSuccess;
  }
  proto::PlanMsg plan;
  mccsResult_t r = wait_plan(comm, wr.user_seq, &plan);
  if (r != mccsSuccess) return r;
  return run_planned(comm, wr.user_seq, plan, stream);
}

mccsResult_t submit(mccsComm* comm, proto::WorkRequest& wr, const void* send, void* recv, uint64_t send_bytes,
                    uint64_t recv_bytes, mccsStream_t stream) {
  if (!comm) return mccsInvalidArgument;
  StreamRec* srec = nullptr;
  {
    std::unique_lock<std::mutex> g(g_ctx.mu);
    if (!g_ctx.connected) return mccsNotConnected;
    const MemRec* sm = find_mem_locked(send);
    const MemRec* rm = find_mem_locked(recv);
    if (!sm || !rm) {
      LOG_ERROR("collective buffers must come from mccsMalloc (send %p, recv %p)", send, recv);
      return mccsInvalidArgument;
    }
    wr.send_mem = sm->mem_id; wr.send_off = (uint64_t)send - sm->base;
    wr.recv_mem = rm->mem_id; wr.recv_off = (uint64_t)recv - rm->base;
    if (wr.send_off + send_bytes > sm->size || wr.recv_off + recv_bytes > rm->size) return mccsInvalidArgument;
    if (!comm->sync_base && !comm->client_launch) {
      mccsResult_t r = register_stream_locked(g, comm->device, stream, &srec);
      if (r != mccsSuccess) return r;
    }
  }
  if (comm->client_launch) return submit_client_launch(comm, wr, stream);
  if (comm->sync_base) return submit_memops(comm, wr, stream);
  wr.comm_handle = comm->handle;
  wr.stream_id = srec->stream_id;
  wr.user_seq = comm->next_user_seq++;
  if (g_group_depth > 0) wr.flags |= proto::kWrGroupMore;
  if (g_ctx.backend == proto::kBackendCuda) {
    CtxScope scope(comm->device);
    if (!scope.ok) return mccsDeviceError;
    CUresult r = g_drv.cuEventRecord_(srec->event, (CUstream)stream);
    if (r != CUDA_SUCCESS) { LOG_ERROR("cuEventRecord: %s", cu_err(r)); return mccsDeviceError; }
  }
  // Post. A full ring means completions are waiting to be read (grouped calls).
  while (!comm->wq.try_push(&wr)) {
    proto::WorkCompletion wc;
    if (comm->outstanding > 0 && comm->cq.try_pop(&wc)) {
      comm->outstanding--;
      if (wc.status != 0 && comm->sticky_error == 0) comm->sticky_error = wc.status;
    }
  }
  comm->outstanding++;
  if (g_group_depth > 0) {
    g_group_items.push_back({comm, stream});
    return mccsSuccess;
  }
  proto::WorkCompletion wc;
  mccsResult_t r = mccsSuccess;
  while (comm->outstanding > 0) {
    mccsResult_t one = wait_completion(comm, &wc);
    if (one == mccsTimeout || one == mccsNotConnected) return one;
    if (one != mccsSuccess) r = one;
  }
  if (r != mccsSuccess) return r;
  if (comm->deferred_wait) return mccsSuccess;
  return finish_on_stream(comm, stream);
}

}  // namespace

// Optional native backtrace on a crash (MCCS_BACKTRACE=1): prints the C/C++ frames to
// stderr, then hands over to whatever handler was installed before (Python's
// faulthandler, the default action).
namespace {
struct sigaction g_prev_segv;
void on_segv(int sig, siginfo_t* info, void* uctx) {
  void* frames[64];
  int n = backtrace(frames, 64);
  const char msg[] = "\n[libmccs] fatal signal, native backtrace:\n";
  if (write(2, msg, sizeof msg - 1) < 0) {}
  backtrace_symbols_fd(frames, n, 2);
  if (g_prev_segv.sa_flags & SA_SIGINFO) {
    if (g_prev_segv.sa_sigaction) g_prev_segv.sa_sigaction(sig, info, uctx);
  } else if (g_prev_segv.sa_handler && g_prev_segv.sa_handler != SIG_DFL && g_prev_segv.sa_handler != SIG_IGN) {
    g_prev_segv.sa_handler(sig);
  }
  signal(sig, SIG_DFL);
  raise(sig);
}
__attribute__((constructor)) void install_backtrace_handler() {
  const char* e = getenv("MCCS_BACKTRACE");
  if (!e || e[0] == '0') return;
  struct sigaction sa;
  memset(&sa, 0, sizeof sa);
  sa.sa_sigaction = on_segv;
  sa.sa_flags = SA_SIGINFO | SA_ONSTACK;
  sigaction(SIGSEGV, &sa, &g_prev_segv);
}
}  // namespace

// ---------------------------------------------------------------------------
// Public API
// ---------------------------------------------------------------------------
extern "C" {

mccsResult_t mccsInit(const char* control_socket_path) {
  std::unique_lock<std::mutex> g(g_ctx.mu);
  return ensure_connected_locked(g, control_socket_path);
}

mccsResult_t mccsFinalize(void) {
  std::unique_lock<std::mutex> g(g_ctx.mu);
  Context& c = g_ctx;
  if (!c.connected) return mccsSuccess;
  proto::AnyMsg m;
  memset(&m, 0, sizeof m);
  m.h.magic = proto::kMagic;
  m.h.type = proto::kGoodbye;
  ipc::uds_send(c.fd, &m, sizeof(proto::Header));
  g_watch_generation.fetch_add(1);   // retires the watch thread of this connection
  close(c.fd);
  c.fd = -1;
  c.connected = false;
  for (auto& kv : c.mem) unmap_allocation(kv.second);
  c.mem.clear();
  c.mem_base_by_id.clear();
  if (g_drv.ok)
    for (auto& kv : c.streams)
      if (kv.second.event) { CtxScope scope(kv.second.device); g_drv.cuEventDestroy_(kv.second.event); }
  c.streams.clear();
  return mccsSuccess;
}

int mccsBackendKind(void) {
  std::unique_lock<std::mutex> g(g_ctx.mu);
  if (ensure_connected_locked(g, nullptr) != mccsSuccess) return -1;
  return (int)g_ctx.backend;
}

int mccsDeviceCount(void) {
  std::unique_lock<std::mutex> g(g_ctx.mu);
  if (ensure_connected_locked(g, nullptr) != mccsSuccess) return -1;
  return g_ctx.num_devices;
}

mccsResult_t mccsMalloc(void** ptr, int device, size_t size) {
  if (!ptr || size == 0) return mccsInvalidArgument;
  std::unique_lock<std::mutex> g(g_ctx.mu);
  mccsResult_t r = ensure_connected_locked(g, nullptr);
  if (r != mccsSuccess) return r;
  proto::AnyMsg m;
  memset(&m, 0, sizeof m);
  m.h.type = proto::kMalloc;
  m.malloc_req.device = device;
  m.malloc_req.size = size;
  std::vector<int> fds;
  r = roundtrip(g, m, sizeof(proto::MallocReq), proto::kMallocReply, &fds, 60000);
  auto close_fds = [&]() { for (int f : fds) close(f); };
  if (r != mccsSuccess) { close_fds(); return r; }
  MemRec rec;
  rec.mem_id = m.malloc_reply.mem_id;
  rec.size = m.malloc_reply.size;
  rec.device = m.malloc_reply.device;
  rec.share_kind = m.malloc_reply.share_kind;
  mccsResult_t fail = map_allocation(rec, fds.empty() ? -1 : fds[0], m.malloc_reply.ipc_handle, m.malloc_reply.daemon_va);
  close_fds();
  if (fail != mccsSuccess) {
    proto::AnyMsg f;
    memset(&f, 0, sizeof f);
    f.h.type = proto::kFree;
    f.free_req.mem_id = rec.mem_id;
    roundtrip(g, f, sizeof(proto::FreeReq), proto::kFreeReply, nullptr, 30000);
    return fail;
  }
  g_ctx.mem[rec.base] = rec;
  g_ctx.mem_base_by_id[rec.mem_id] = rec.base;
  *ptr = (void*)rec.base;
  return mccsSuccess;
}

mccsResult_t mccsFree(void* ptr) {
  if (!ptr) return mccsSuccess;
  {
    // Requests that name this memory may still sit in a request ring (calls return
    // before the daemon takes them): let the daemon take them first.
    // Only this thread's communicators: completions of another thread's requests are
    // that thread's to read, and another thread may destroy its communicator at any
    // time, so those are looked at under the lock only.
    std::vector<mccsComm*> mine;
    {
      std::unique_lock<std::mutex> g(g_ctx.mu);
      for (mccsComm* c : g_ctx.comms)
        if (pthread_equal(c->owner, pthread_self())) mine.push_back(c);
    }
    if (g_ctx.connected)
      for (mccsComm* c : mine)
        if (c->outstanding || c->memop_posted || names_deferred(c)) mccsCommFlush(c);
    // Kernels launched from here (client-side launch) run on the caller's streams: the
    // daemon cannot wait for them, so this call does, before the memory and the multicast
    // bindings that name it go away.
    if (g_ctx.backend == proto::kBackendCuda && g_drv.cuCtxSynchronize_)
      for (mccsComm* c : mine)
        if (c->launched_here) {
          CtxScope scope(c->device);
          if (scope.ok) g_drv.cuCtxSynchronize_();
        }
  }
  std::unique_lock<std::mutex> g(g_ctx.mu);
  auto it = g_ctx.mem.find((uint64_t)ptr);
  if (it == g_ctx.mem.end()) return mccsNotFound;
  MemRec rec = it->second;
  mccsResult_t res = mccsSuccess;
  if (g_ctx.connected) {
    // The daemon refuses to release memory that a collective still names which has not
    // been launched on every rank (a peer's kernel may be about to store into it). After
    // the flush above that can only be a matter of the other ranks' proxies catching up,
    // so the request is repeated for a bounded time before the error is handed on.
    for (int attempt = 0;; attempt++) {
      proto::AnyMsg m;
      memset(&m, 0, sizeof m);
      m.h.type = proto::kFree;
      m.free_req.mem_id = rec.mem_id;
      res = roundtrip(g, m, sizeof(proto::FreeReq), proto::kFreeReply, nullptr, 60000);
      if (res != mccsBusy || attempt >= 2000) break;
      g.unlock();
      usleep(1000);
      g.lock();
      it = g_ctx.mem.find((uint64_t)ptr);
      if (it == g_ctx.mem.end()) return mccsNotFound;   // freed by another thread meanwhile
    }
    if (res == mccsBusy) return res;   // still mapped and still owned: the caller may retry
  }
  unmap_allocation(rec);
  g_ctx.mem.erase(it);
  g_ctx.mem_base_by_id.erase(rec.mem_id);
  return res;
}

mccsResult_t mccsMemInfo(const void* ptr, uint64_t* mem_id, uint64_t* offset, uint64_t* alloc_size) {
  std::unique_lock<std::mutex> g(g_ctx.mu);
  const MemRec* r = find_mem_locked(ptr);
  if (!r) return mccsNotFound;
  if (mem_id) *mem_id = r->mem_id;
  if (offset) *offset = (uint64_t)ptr - r->base;
  if (alloc_size) *alloc_size = r->size;
  return mccsSuccess;
}

mccsResult_t mccsCommInitRank(mccsComm_t* comm, uint32_t unique_id, int rank, int nranks, int device,
                              const char* root_addr) {
  if (!comm) return mccsInvalidArgument;
  std::unique_lock<std::mutex> g(g_ctx.mu);
  mccsResult_t r = ensure_connected_locked(g, nullptr);
  if (r != mccsSuccess) return r;
  proto::AnyMsg m;
  memset(&m, 0, sizeof m);
  m.h.type = proto::kCommInit;
  m.comm_init.comm_id = unique_id;
  m.comm_init.rank = rank;
  m.comm_init.nranks = nranks;
  m.comm_init.device = device;
  if (root_addr) snprintf(m.comm_init.root_addr, sizeof m.comm_init.root_addr, "%s", root_addr);
  std::vector<int> fds;
  // Blocks until every rank has joined (the daemon bounds the wait).
  r = roundtrip(g, m, sizeof(proto::CommInitReq), proto::kCommInitReply, &fds, 600000);
  if (r != mccsSuccess) { for (int f : fds) close(f); return r; }
  if (fds.empty()) return mccsProtocolError;
  mccsComm* c = new mccsComm();
  c->handle = m.comm_init_reply.comm_handle;
  c->id = unique_id;
  c->rank = rank;
  c->nranks = nranks;
  c->device = device;
  c->dp_bytes = m.comm_init_reply.dp_bytes;
  c->dp_mem = mmap(nullptr, c->dp_bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fds[0], 0);
  if (c->dp_mem == MAP_FAILED) { for (int f : fds) close(f); delete c; return mccsOutOfMemory; }
  const size_t wq_bytes = proto::dp_wq_bytes();
  c->wq.attach(c->dp_mem);
  c->cq.attach((char*)c->dp_mem + wq_bytes);
  if (c->dp_bytes >= proto::dp_segment_bytes())
    c->dp_status = (proto::DpStatus*)((char*)c->dp_mem + wq_bytes + proto::dp_cq_bytes());
  if (g_ctx.backend == proto::kBackendCuda && m.comm_init_reply.sync_size && g_drv.memops && fds.size() > 1) {
    CtxScope scope(device);
    const size_t bytes = m.comm_init_reply.sync_size;
    void* p = scope.ok ? mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fds[1], 0) : MAP_FAILED;
    if (p != MAP_FAILED) {
      CUdeviceptr d = 0;
      CUresult cr = g_drv.cuMemHostRegister_(p, bytes, CU_MEMHOSTREGISTER_PORTABLE | CU_MEMHOSTREGISTER_DEVICEMAP);
      if (cr == CUDA_SUCCESS) cr = g_drv.cuMemHostGetDevicePointer_(&d, p, 0);
      if (cr == CUDA_SUCCESS) {
        c->sync_host = p;
        c->sync_bytes = bytes;
        c->sync_base = (uint64_t)d;
      } else {
        LOG_WARN("cannot register the semaphore page (%s); falling back to event synchronisation", cu_err(cr));
        munmap(p, bytes);
      }
    }
  }
  if (c->dp_bytes >= proto::dp_segment_bytes()) c->pq.attach((char*)c->dp_mem + proto::dp_pq_offset());
  c->client_launch = m.comm_init_reply.launch_mode == proto::kLaunchClient;
  c->group_defer = c->client_launch && m.comm_init_reply.group_defer != 0;
  c->fifo_slot_bytes = m.comm_init_reply.fifo_slot_bytes;
  if (g_ctx.backend == proto::kBackendHost && m.comm_init_reply.sync_size && fds.size() > 1) {
    const size_t bytes = m.comm_init_reply.sync_size;
    void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fds[1], 0);
    if (p != MAP_FAILED) {
      c->sync_host = p;
      c->sync_bytes = bytes;
      c->sync_base = (uint64_t)p;
      c->sync_emulated = true;
    }
  }
  for (int f : fds) close(f);
  fds.clear();
  if (g_ctx.backend == proto::kBackendCuda) {
    if (g_ctx.same_process) {
      c->backend_event = (CUevent)m.comm_init_reply.event_raw;
    } else {
      CtxScope scope(device);
      if (!scope.ok) { munmap(c->dp_mem, c->dp_bytes); delete c; return mccsDeviceError; }
      CUipcEventHandle h;
      memcpy(&h, m.comm_init_reply.event_handle, sizeof h);
      CUresult cr = g_drv.cuIpcOpenEventHandle_(&c->backend_event, h);
      if (cr != CUDA_SUCCESS) {
        LOG_ERROR("cuIpcOpenEventHandle: %s", cu_err(cr));
        munmap(c->dp_mem, c->dp_bytes);
        delete c;
        return mccsDeviceError;
      }
      c->event_owned = true;
    }
  }
  if (c->client_launch) {
    // Everything this rank's kernels address besides the buffers: every rank's signal pad
    // and status block, and (for the ring variants) every rank's FIFOs.
    for (int peer = 0; peer < nranks; peer++) {
      for (uint32_t kind : {(uint32_t)proto::kScratchPad, (uint32_t)proto::kScratchStatus, (uint32_t)proto::kScratchFifo}) {
        if (kind == proto::kScratchFifo && nranks == 1) continue;
        proto::AnyMsg q;
        memset(&q, 0, sizeof q);
        q.h.type = proto::kMapScratch;
        q.map_scratch.comm_handle = c->handle;
        q.map_scratch.rank = peer;
        q.map_scratch.kind = kind;
        std::vector<int> sfds;
        mccsResult_t mr = roundtrip(g, q, sizeof(proto::MapScratchReq), proto::kMapScratchReply, &sfds, 30000);
        Mapped mp;
        if (mr == mccsSuccess)
          mr = map_block(sfds.empty() ? -1 : sfds[0], (size_t)q.map_scratch_reply.bytes, q.map_scratch_reply.share_kind,
                         q.map_scratch_reply.daemon_va, g_ctx.backend == proto::kBackendCuda ? device : -1, &mp);
        for (int f : sfds) close(f);
        if (mr != mccsSuccess) {
          LOG_ERROR("cannot map rank %d's %s of communicator %u", peer, kind == proto::kScratchPad ? "signal pad" : kind == proto::kScratchStatus ? "status block" : "FIFOs", c->id);
          g_ctx.comms.push_back(c);      // mccsCommDestroy below undoes what exists so far
          g.unlock();
          mccsCommDestroy(c);
          return mr;
        }
        // inside the daemon's process the status block is the daemon's own (registered) host memory
        if (kind == proto::kScratchStatus && mp.share_kind == proto::kShareSameProcess) mp.host = (void*)mp.addr;
        if (kind == proto::kScratchPad) c->pad_map[peer] = mp;
        else if (kind == proto::kScratchStatus) c->status_map[peer] = mp;
        else c->fifo_map[peer] = mp;
      }
    }
    // The status block of this rank is read by the CPU here (device errors, the abort word).
    if (!c->status_map[rank].host) {
      LOG_ERROR("communicator %u: this rank's status block is not readable by the CPU", c->id);
      g_ctx.comms.push_back(c);
      g.unlock();
      mccsCommDestroy(c);
      return mccsProtocolError;
    }
    if (g_ctx.backend == proto::kBackendCuda && !load_kernels_lib()) {
      g_ctx.comms.push_back(c);
      g.unlock();
      mccsCommDestroy(c);
      return mccsUnsupported;
    }
  }
  g_ctx.comms.push_back(c);
  *comm = c;
  return mccsSuccess;
}

mccsResult_t mccsCommFlush(mccsComm_t comm) {
  if (!comm) return mccsInvalidArgument;
  // Requests of an open group whose plans have not been taken yet are launched now: nothing
  // that the caller does after a flush (free, destroy, reading the last plan) may find them
  // half way.
  if (names_deferred(comm)) {
    mccsResult_t r = flush_deferred();
    if (r == mccsTimeout || r == mccsNotConnected) return r;
  }
  proto::WorkCompletion wc;
  while (comm->outstanding > 0) {
    mccsResult_t r = wait_completion(comm, &wc);
    if (r == mccsTimeout || r == mccsNotConnected) return r;
  }
  if (comm->dp_status && comm->memop_posted) {
    struct timespec t0;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    uint64_t spins = 0;
    while (__atomic_load_n(&comm->dp_status->completed, __ATOMIC_ACQUIRE) < comm->memop_posted) {
      if ((++spins & 0xfff) == 0) {
        struct timespec t1;
        clock_gettime(CLOCK_MONOTONIC, &t1);
        uint64_t ms = (uint64_t)(t1.tv_sec - t0.tv_sec) * 1000 + (uint64_t)((t1.tv_nsec - t0.tv_nsec) / 1000000);
        if (ms > g_ctx.wc_timeout_ms) return mccsTimeout;
        struct pollfd pf = {g_ctx.fd, 0, 0};
        if (poll(&pf, 1, 0) > 0 && (pf.revents & (POLLHUP | POLLERR))) return daemon_lost();
        if (spins > (1u << 20)) usleep(50);
      }
    }
    reap_completions(comm);
  }
  return (mccsResult_t)comm->sticky_error;
}

mccsResult_t mccsCommDestroy(mccsComm_t comm) {
  if (!comm) return mccsSuccess;
  if (g_ctx.connected) mccsCommFlush(comm);   // every posted request has been taken by the daemon
  // A handle destroyed inside an open group must not be looked at again when the group ends.
  for (size_t i = g_group_items.size(); i-- > 0;)
    if (g_group_items[i].comm == comm) g_group_items.erase(g_group_items.begin() + (long)i);
  for (size_t i = g_deferred.size(); i-- > 0;)
    if (g_deferred[i].comm == comm) g_deferred.erase(g_deferred.begin() + (long)i);
  if (comm->launched_here && g_ctx.backend == proto::kBackendCuda && g_drv.cuCtxSynchronize_) {
    // Kernels of this communicator run on the caller's streams: they must be through
    // before the daemon takes the pads and FIFOs away. Their waits are bounded.
    CtxScope scope(comm->device);
    if (scope.ok) g_drv.cuCtxSynchronize_();
  }
  std::unique_lock<std::mutex> g(g_ctx.mu);
  mccsResult_t r = mccsSuccess;
  if (g_ctx.connected) {
    proto::AnyMsg m;
    memset(&m, 0, sizeof m);
    m.h.type = proto::kCommDestroy;
    m.comm_destroy.comm_handle = comm->handle;
    r = roundtrip(g, m, sizeof(proto::CommDestroyReq), proto::kCommDestroyReply, nullptr, 60000);
  }
  if (comm->event_owned && comm->backend_event && g_drv.ok) {
    CtxScope scope(comm->device);
    g_drv.cuEventDestroy_(comm->backend_event);
  }
  if (comm->launch_event && g_drv.ok) {
    CtxScope scope(comm->device);
    g_drv.cuEventDestroy_(comm->launch_event);
  }
  for (size_t i = 0; i < g_ctx.comms.size(); i++)
    if (g_ctx.comms[i] == comm) { g_ctx.comms.erase(g_ctx.comms.begin() + (long)i); break; }
  if (comm->dp_mem) munmap(comm->dp_mem, comm->dp_bytes);
  const int map_dev = g_ctx.backend == proto::kBackendCuda ? comm->device : -1;
  for (int k = 0; k < kMaxRanks; k++) {
    unmap_block(comm->pad_map[k], map_dev);
    unmap_block(comm->status_map[k], map_dev);
    unmap_block(comm->fifo_map[k], map_dev);
  }
  for (auto& kv : comm->mc_map) unmap_block(kv.second, map_dev);
  for (auto& kv : comm->peer_mem) unmap_block(kv.second, map_dev);
  if (comm->sync_host) {
    if (!comm->sync_emulated) {
      CtxScope scope(comm->device);
      if (scope.ok) g_drv.cuMemHostUnregister_(comm->sync_host);
    }
    munmap(comm->sync_host, comm->sync_bytes);
  }
  delete comm;
  return r;
}

mccsResult_t mccsCommRank(mccsComm_t comm, int* rank) { if (!comm || !rank) return mccsInvalidArgument; *rank = comm->rank; return mccsSuccess; }
mccsResult_t mccsCommSize(mccsComm_t comm, int* n) { if (!comm || !n) return mccsInvalidArgument; *n = comm->nranks; return mccsSuccess; }
uint64_t mccsCommHandle(mccsComm_t comm) { return comm ? comm->handle : 0; }

mccsResult_t mccsRegisterStream(int device, mccsStream_t stream) {
  std::unique_lock<std::mutex> g(g_ctx.mu);
  mccsResult_t r = ensure_connected_locked(g, nullptr);
  if (r != mccsSuccess) return r;
  StreamRec* rec = nullptr;
  return register_stream_locked(g, device, stream, &rec);
}

mccsResult_t mccsAllReduceEx(mccsComm_t comm, const void* send, void* recv, size_t count, mccsDataType_t dtype,
                             mccsRedOp_t op, float scale, mccsAlgo_t algo, mccsStream_t stream) {
  if (!comm || (int)dtype < 0 || (int)dtype >= kNumDataTypes || (int)op < 0 || (int)op >= kNumRedOps)
    return mccsInvalidArgument;
  const uint64_t esz = (uint64_t)dtype_size((int)dtype);
  if ((((uint64_t)send | (uint64_t)recv) & (esz - 1)) != 0 || count > (1ull << 44)) {
    LOG_ERROR("all-reduce buffers must be aligned to the element size (send %p, recv %p, %llu-byte elements)", send, recv,
              (unsigned long long)esz);
    return mccsInvalidArgument;
  }
  proto::WorkRequest wr;
  memset(&wr, 0, sizeof wr);
  wr.kind = kAllReduce;
  wr.dtype = (uint32_t)dtype;
  wr.op = (uint32_t)op;
  wr.count = count;
  wr.scale = scale;
  wr.variant = (uint32_t)algo;
  const uint64_t bytes = (uint64_t)count * esz;
  return submit(comm, wr, send, recv, bytes, bytes, stream);
}

mccsResult_t mccsAllReduce(mccsComm_t comm, const void* send, void* recv, size_t count, mccsDataType_t dtype,
                           mccsRedOp_t op, mccsStream_t stream) {
  return mccsAllReduceEx(comm, send, recv, count, dtype, op, 1.0f, mccsAlgoAuto, stream);
}

mccsResult_t mccsReduceScatterEx(mccsComm_t comm, const void* send, void* recv, size_t count, mccsDataType_t dtype,
                                 mccsRedOp_t op, float scale, mccsAlgo_t algo, mccsStream_t stream) {
  if (!comm || (int)dtype < 0 || (int)dtype >= kNumDataTypes || (int)op < 0 || (int)op >= kNumRedOps)
    return mccsInvalidArgument;
  const uint64_t esz = (uint64_t)dtype_size((int)dtype);
  if ((((uint64_t)send | (uint64_t)recv) & (esz - 1)) != 0 || count > (1ull << 44)) {
    LOG_ERROR("reduce-scatter buffers must be aligned to the element size (send %p, recv %p, %llu-byte elements)", send, recv,
              (unsigned long long)esz);
    return mccsInvalidArgument;
  }
  proto::WorkRequest wr;
  memset(&wr, 0, sizeof wr);
  wr.kind = kReduceScatter;
  wr.dtype = (uint32_t)dtype;
  wr.op = (uint32_t)op;
  wr.count = count;
  wr.scale = scale;
  wr.variant = (uint32_t)algo;
  const uint64_t bytes = (uint64_t)count * esz;
  return submit(comm, wr, send, recv, bytes * (uint64_t)comm->nranks, bytes, stream);
}

mccsResult_t mccsReduceScatter(mccsComm_t comm, const void* send, void* recv, size_t count, mccsDataType_t dtype,
                               mccsRedOp_t op, mccsStream_t stream) {
  return mccsReduceScatterEx(comm, send, recv, count, dtype, op, 1.0f, mccsAlgoAuto, stream);
}

mccsResult_t mccsAllGatherEx(mccsComm_t comm, const void* send, void* recv, size_t bytes, mccsAlgo_t algo,
                             mccsStream_t stream) {
  if (!comm) return mccsInvalidArgument;
  proto::WorkRequest wr;
  memset(&wr, 0, sizeof wr);
  wr.kind = kAllGather;
  wr.dtype = kUint8;
  wr.count = bytes;
  wr.scale = 1.0f;
  wr.variant = (uint32_t)algo;
  return submit(comm, wr, send, recv, bytes, (uint64_t)bytes * (uint64_t)comm->nranks, stream);
}

mccsResult_t mccsAllGather(mccsComm_t comm, const void* send, void* recv, size_t bytes, mccsStream_t stream) {
  return mccsAllGatherEx(comm, send, recv, bytes, mccsAlgoAuto, stream);
}

mccsResult_t mccsCommSetDeferredWait(mccsComm_t comm, int on) {
  if (!comm) return mccsInvalidArgument;
  comm->deferred_wait = on != 0;
  return mccsSuccess;
}

mccsResult_t mccsCommWait(mccsComm_t comm, mccsStream_t stream) {
  if (!comm) return mccsInvalidArgument;
  if (comm->sync_emulated) {
    if (!comm->last_posted_seq) return mccsSuccess;
    mccsResult_t r = sem_wait_geq(comm, stream, comm->sync_base + 8 * proto::kSyncDoneSlot, comm->last_posted_seq);
    if (r != mccsSuccess) return r;
    reap_completions(comm);
    return (mccsResult_t)comm->sticky_error;
  }
  if (g_ctx.backend != proto::kBackendCuda) return mccsSuccess;
  if (comm->client_launch) {
    // The kernels ran on the streams the collectives were given; `stream` waits for the
    // newest of them (launches of one communicator are made in order).
    if (comm->sticky_error) return (mccsResult_t)comm->sticky_error;
    if (!comm->launch_event_set) return mccsSuccess;
    CtxScope scope(comm->device);
    if (!scope.ok) return mccsDeviceError;
    CUresult cr = g_drv.cuStreamWaitEvent_((CUstream)stream, comm->launch_event, 0);
    if (cr != CUDA_SUCCESS) { LOG_ERROR("cuStreamWaitEvent: %s", cu_err(cr)); return mccsDeviceError; }
    return mccsSuccess;
  }
  if (comm->sync_base) {
    if (!comm->last_posted_seq) return mccsSuccess;
    CtxScope scope(comm->device);
    if (!scope.ok) return mccsDeviceError;
    // "done" only grows and is written in submission order: the newest value covers all.
    return sem_wait_geq(comm, stream, comm->sync_base + 8 * proto::kSyncDoneSlot, comm->last_posted_seq);
  }
  return finish_on_stream(comm, stream);
}

mccsResult_t mccsGroupStart(void) { g_group_depth++; return mccsSuccess; }

mccsResult_t mccsGroupEnd(void) {
  if (g_group_depth <= 0) return mccsInvalidArgument;
  if (--g_group_depth > 0) return mccsSuccess;
  mccsResult_t result = g_deferred.empty() ? mccsSuccess : flush_deferred();
  std::vector<GroupItem> items;
  items.swap(g_group_items);
  // Collect every completion, then order each (communicator, stream) pair once.
  for (const GroupItem& it : items) {
    proto::WorkCompletion wc;
    while (it.comm->outstanding > 0) {
      mccsResult_t r = wait_completion(it.comm, &wc);
      if (r == mccsTimeout || r == mccsNotConnected) return r;
      if (r != mccsSuccess) result = r;
    }
  }
  std::vector<GroupItem> seen;
  for (const GroupItem& it : items) {
    bool dup = false;
    for (const GroupItem& s : seen) dup |= s.comm == it.comm && s.stream == it.stream;
    if (dup) continue;
    seen.push_back(it);
    if (it.comm->sticky_error && result == mccsSuccess) result = (mccsResult_t)it.comm->sticky_error;
    // Event mode: wait for the daemon's "done" event. Mem-op mode: wait for the "done"
    // value of the newest request (values grow in submission order).
    mccsResult_t r = it.comm->sync_base ? (it.comm->deferred_wait ? mccsSuccess : mccsCommWait(it.comm, it.stream))
                                        : finish_on_stream(it.comm, it.stream);
    if (r != mccsSuccess) result = r;
  }
  return result;
}

mccsResult_t mccsCommQuery(mccsComm_t comm, mccsCommInfo_t* info) {
  if (!comm || !info) return mccsInvalidArgument;
  std::unique_lock<std::mutex> g(g_ctx.mu);
  if (!g_ctx.connected) return mccsNotConnected;
  proto::AnyMsg m;
  memset(&m, 0, sizeof m);
  m.h.type = proto::kCommQuery;
  m.comm_query.comm_handle = comm->handle;
  mccsResult_t r = roundtrip(g, m, sizeof(proto::CommQueryReq), proto::kCommQueryReply, nullptr, 30000);
  if (r != mccsSuccess) return r;
  info->async_error = m.comm_query_reply.async_error;
  info->device_error = m.comm_query_reply.device_error;
  info->launched = m.comm_query_reply.launched;
  info->completed = m.comm_query_reply.completed;
  info->last_variant = m.comm_query_reply.last_variant;
  info->last_ctas = m.comm_query_reply.last_ctas;
  info->config_epoch = m.comm_query_reply.config_epoch;
  return mccsSuccess;
}

mccsResult_t mccsCommGetAsyncError(mccsComm_t comm, mccsResult_t* async_error) {
  mccsCommInfo_t info;
  mccsResult_t r = mccsCommQuery(comm, &info);
  if (r != mccsSuccess) return r;
  if (async_error) *async_error = (mccsResult_t)info.async_error;
  return mccsSuccess;
}

mccsResult_t mccsCommLastPlan(mccsComm_t comm, uint32_t* variant, uint32_t* ctas) {
  if (!comm) return mccsInvalidArgument;
  mccsCommFlush(comm);
  if (variant) *variant = comm->last_variant;
  if (ctas) *ctas = comm->last_ctas;
  return mccsSuccess;
}

int mccsCommLaunchMode(mccsComm_t comm) { return comm && comm->client_launch ? 1 : 0; }

const char* mccsGetErrorString(mccsResult_t r) {
  switch (r) {
    case mccsSuccess: return "success";
    case mccsInvalidArgument: return "invalid argument";
    case mccsOutOfMemory: return "out of memory";
    case mccsDeviceError: return "a CUDA call failed";
    case mccsProtocolError: return "protocol error";
    case mccsNotFound: return "not found";
    case mccsTimeout: return "timed out";
    case mccsAborted: return "aborted";
    case mccsMismatch: return "ranks disagree on the collective";
    case mccsUnsupported: return "unsupported";
    case mccsPeerLost: return "a peer rank went away";
    case mccsInternalError: return "internal error";
    case mccsNotConnected: return "not connected to the daemon";
    case mccsBusy: return "memory is still named by a queued collective";
  }
  return "unknown error";
}

const char* mccsAlgoName(int algo) { return variant_name(algo); }

mccsResult_t mccsAdminRequest(const char* host, int port, int type, const char* json_body, char* reply,
                              size_t reply_cap) {
  if (!host || port <= 0) return mccsInvalidArgument;
  struct addrinfo hints, *res = nullptr;
  memset(&hints, 0, sizeof hints);
  hints.ai_family = AF_INET;
  hints.ai_socktype = SOCK_STREAM;
  char portstr[16];
  snprintf(portstr, sizeof portstr, "%d", port);
  if (getaddrinfo(host, portstr, &hints, &res) != 0 || !res) return mccsNotConnected;
  int fd = socket(res->ai_family, res->ai_socktype | SOCK_CLOEXEC, res->ai_protocol);
  if (fd < 0) { freeaddrinfo(res); return mccsNotConnected; }
  if (connect(fd, res->ai_addr, res->ai_addrlen) < 0) { freeaddrinfo(res); close(fd); return mccsNotConnected; }
  freeaddrinfo(res);
  const std::string body = json_body ? json_body : "{}";
  uint8_t hdr[13];
  memcpy(hdr, &proto::kAdminMagic, 8);
  hdr[8] = (uint8_t)type;
  uint32_t len = (uint32_t)body.size();
  memcpy(hdr + 9, &len, 4);
  auto write_all = [&](const void* p, size_t n) {
    const char* c = (const char*)p;
    while (n) { ssize_t k = send(fd, c, n, MSG_NOSIGNAL); if (k <= 0) return false; c += k; n -= (size_t)k; }
    return true;
  };
  auto read_all = [&](void* p, size_t n) {
    char* c = (char*)p;
    while (n) {
      struct pollfd pf = {fd, POLLIN, 0};
      if (poll(&pf, 1, 30000) <= 0) return false;
      ssize_t k = read(fd, c, n);
      if (k <= 0) return false;
      c += k; n -= (size_t)k;
    }
    return true;
  };
  mccsResult_t result = mccsProtocolError;
  if (write_all(hdr, sizeof hdr) && write_all(body.data(), body.size()) && read_all(hdr, sizeof hdr)) {
    uint64_t magic;
    memcpy(&magic, hdr, 8);
    memcpy(&len, hdr + 9, 4);
    if (magic == proto::kAdminMagic && len < (64u << 20)) {
      std::string out(len, '\0');
      if (!len || read_all(&out[0], len)) {
        if (reply && reply_cap) {
          size_t n = out.size() < reply_cap - 1 ? out.size() : reply_cap - 1;
          memcpy(reply, out.data(), n);
          reply[n] = 0;
        }
        result = mccsSuccess;
      }
    }
  }
  close(fd);
  return result;
}

void* mccs_torch_malloc(size_t size, int device, void* stream) {
  (void)stream;
  void* p = nullptr;
  if (size == 0) size = 1;
  mccsResult_t r = mccsMalloc(&p, device, size);
  if (r != mccsSuccess) {
    LOG_ERROR("mccs_torch_malloc(%zu bytes, device %d): %s", size, device, mccsGetErrorString(r));
    return nullptr;
  }
  return p;
}

void mccs_torch_free(void* ptr, size_t size, int device, void* stream) {
  (void)size; (void)device; (void)stream;
  mccsFree(ptr);
}

}  // extern "C"
