// Wire protocol between the client shim (libmccs) and the service daemon.
//
// Two channels per client, as in the reference (src/ipc/mccs/src/command.rs:88-112
// for control, src/ipc/mccs/src/dp.rs:8-28 for the data path):
//   * control: request/reply messages on a Unix SOCK_SEQPACKET connection. Fixed
//     layout structs (no serialisation step); file descriptors travel as
//     SCM_RIGHTS ancillary data.
//   * data path: one pair of single-producer/single-consumer rings in shared memory
//     per (communicator, rank): 128-byte work requests, 64-byte completions, the slot
//     sizes the reference uses. The per-GPU proxy polls the request ring directly,
//     so a collective crosses one thread boundary instead of the reference's two.
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace mccs {
namespace proto {

constexpr uint32_t kMagic = 0x5343434du;  // "MCCS"
constexpr uint32_t kVersion = 10;
constexpr uint32_t kWqDepth = 64;
constexpr uint32_t kCqDepth = 64;
constexpr uint32_t kWrBytes = 128;
constexpr uint32_t kWcBytes = 64;
constexpr uint32_t kIpcHandleBytes = 64;  // cudaIpcMemHandle_t / cudaIpcEventHandle_t

enum MsgType : uint32_t {
  kHello = 1, kWelcome = 2,
  kMalloc = 3, kMallocReply = 4,
  kFree = 5, kFreeReply = 6,
  kCommInit = 7, kCommInitReply = 8,
  kCommDestroy = 9, kCommDestroyReply = 10,
  kRegisterStream = 11, kRegisterStreamReply = 12,
  kCommQuery = 13, kCommQueryReply = 14,
  kGoodbye = 15,
  // client-side launch: a member of a communicator maps what its kernels must address
  kMapScratch = 16, kMapScratchReply = 17,   // a rank's signal pad / status block / FIFOs
  kMapMem = 18, kMapMemReply = 19,           // a peer's allocation named in a plan
  kMapMc = 20, kMapMcReply = 21,             // a multicast region named in a plan
};

enum Status : int32_t {
  kOk = 0,
  kErrInvalidArgument = -1,
  kErrOutOfMemory = -2,
  kErrDevice = -3,          // a CUDA call failed
  kErrProtocol = -4,
  kErrNotFound = -5,
  kErrTimeout = -6,         // a bounded device-side or host-side wait ran out
  kErrAborted = -7,
  kErrMismatch = -8,        // ranks disagreed on a collective's parameters
  kErrUnsupported = -9,
  kErrPeerLost = -10,       // another rank of the communicator went away
  kErrInternal = -11,
  kErrNotConnected = -12,   // client side only: the daemon went away
  kErrBusy = -13,           // memory is still named by a collective that has not been launched
};

enum Backend : uint32_t { kBackendHost = 0, kBackendCuda = 1 };

// How a collective is ordered against the caller's CUDA stream.
//  kSyncEvents: two interprocess events per request, as the reference does
//    (src/libmccs/src/collectives.rs:23-25,68-70): the caller records "submitted",
//    waits for the daemon's completion message, then makes its stream wait for the
//    daemon's "done" event. One blocking round trip per collective.
//  kSyncMemOps: 64-bit semaphores in a pinned host page shared by caller and daemon.
//    The caller enqueues "write submitted" and "wait done" on its stream (stream memory
//    operations) and returns at once; the daemon's proxy polls the "submitted" words
//    from the CPU, launches the kernel once every rank's caller has got there, and
//    enqueues "write done" behind it. No round trip, no blocking wait on the daemon's
//    streams.
enum SyncMode : uint32_t { kSyncEvents = 0, kSyncMemOps = 1 };
constexpr uint32_t kSyncDoneSlot = 0;        // u64 index of the "done" semaphore in the sync page
constexpr uint32_t kSyncFirstStreamSlot = 8; // first "submitted" semaphore
constexpr uint32_t kSyncMaxStreams = 56;
constexpr uint32_t kSyncPageBytes = 4096;

// How the client maps an allocation the daemon made for it.
enum ShareKind : uint32_t {
  kShareHostFd = 0,     // memfd: mmap (host backend)
  kShareVmmFd = 1,      // CUDA VMM allocation exported as POSIX fd
  kShareCudaIpc = 2,    // cudaIpcMemHandle_t (cudaMalloc'ed memory)
  kShareSameProcess = 3 // daemon runs inside the client process: use daemon_va
};

struct Header {
  uint32_t magic;
  uint32_t type;     // MsgType
  uint32_t req_id;   // echoed in the reply
  int32_t status;    // Status (replies)
};

struct Hello {
  Header h;
  uint32_t version;
  int32_t pid;
  int32_t device_affinity;  // -1: none
  uint32_t reserved;
  char app_name[64];
};

struct Welcome {
  Header h;
  uint32_t version;
  int32_t daemon_pid;
  uint32_t backend;       // Backend
  uint32_t num_devices;
  uint64_t session_id;
  uint32_t sync_mode;     // SyncMode
  uint32_t reserved;
};

struct MallocReq {
  Header h;
  int32_t device;
  uint32_t flags;
  uint64_t size;
};

struct MallocReply {
  Header h;
  uint64_t mem_id;
  uint64_t size;          // mapped size (>= requested, rounded to the granularity)
  uint64_t daemon_va;
  uint32_t share_kind;    // ShareKind
  int32_t device;
  uint8_t ipc_handle[kIpcHandleBytes];
};

struct FreeReq { Header h; uint64_t mem_id; };
struct FreeReply { Header h; };

struct CommInitReq {
  Header h;
  uint32_t comm_id;       // user-chosen id: also the tenant key for QoS and overrides
  int32_t rank;
  int32_t nranks;
  int32_t device;
  char root_addr[64];     // accepted for API parity; rendezvous is in-daemon
};

struct CommInitReply {
  Header h;
  uint64_t comm_handle;   // (comm_id << 32) + rank, as the reference composes it
  uint8_t event_handle[kIpcHandleBytes];  // backend event (IPC) ...
  uint64_t event_raw;                     // ... or its in-process handle
  uint32_t dp_bytes;      // size of the data-path segment passed as fd
  uint32_t sync_share_kind;               // ShareKind of the sync page (mem-op mode)
  uint64_t sync_size;                     // 0: no sync page, events are used
  uint64_t sync_daemon_va;
  uint8_t sync_ipc_handle[kIpcHandleBytes];
  uint32_t launch_mode;                   // LaunchMode
  uint32_t fifo_slot_bytes;               // client-side launch: geometry of the ring FIFOs
  uint32_t group_defer;                   // client-side launch: inside a group the library only posts and takes the plans at the end (fused launches are on)
  uint32_t pad_;
};

struct CommDestroyReq { Header h; uint64_t comm_handle; };
struct CommDestroyReply { Header h; };

struct RegisterStreamReq {
  Header h;
  int32_t device;
  uint32_t reserved;
  uint64_t stream;        // client-side stream handle, used only as a key
  uint8_t event_handle[kIpcHandleBytes];
  uint64_t event_raw;
};
struct RegisterStreamReply { Header h; uint64_t stream_id; };

// Who launches the kernels of a communicator. The reference's service always does
// (src/mccs/src/proxy/plan.rs:637-669). With kLaunchClient the daemon still collects the
// ranks' requests, plans, admits and hands out barrier epochs and tickets, but gives the
// finished plan back to each rank's client library, which launches the kernel on the
// caller's own stream: no hand-over between two processes' streams per collective.
enum LaunchMode : uint32_t { kLaunchDaemon = 0, kLaunchClient = 1 };

enum ScratchKind : uint32_t { kScratchPad = 0, kScratchStatus = 1, kScratchFifo = 2 };
struct MapScratchReq { Header h; uint64_t comm_handle; int32_t rank; uint32_t kind; };   // ScratchKind
// share_kind kShareSameProcess (a client inside the daemon's process on a GPU): no descriptor, use daemon_va
struct MapScratchReply { Header h; uint64_t bytes; uint32_t share_kind; uint32_t reserved; uint64_t daemon_va; };   // + 1 fd
struct MapMemReq { Header h; uint64_t comm_handle; uint64_t mem_id; };
struct MapMemReply { Header h; uint64_t bytes; uint32_t share_kind; int32_t device; uint64_t daemon_va; };   // + 1 fd

// A multicast region (the same offsets of every rank's buffer behind one address range).
// On a GPU the reply brings the exported multicast object (+ 1 fd) to map with alignment
// `align`; a client inside the daemon's process uses daemon_va; on the host backend with
// emulated kernels it names the allocation bound per rank and the client builds the
// emulated region from its own mappings of them.
struct MapMcReq { Header h; uint64_t comm_handle; uint64_t mc_id; };
struct MapMcReply {
  Header h;
  uint64_t bytes;
  uint32_t share_kind;
  uint32_t nranks;
  uint64_t align;
  uint64_t daemon_va;
  uint64_t mems[8];
};

struct CommQueryReq { Header h; uint64_t comm_handle; };
struct CommQueryReply {
  Header h;
  int32_t async_error;     // Status, sticky
  uint32_t device_error;   // DevStatus reported by a kernel
  uint64_t launched;       // collectives launched so far
  uint64_t completed;
  uint32_t last_variant;
  uint32_t last_ctas;
  uint64_t config_epoch;   // bumps on every applied reconfiguration
};

union AnyMsg {
  Header h;
  Hello hello; Welcome welcome;
  MallocReq malloc_req; MallocReply malloc_reply;
  FreeReq free_req; FreeReply free_reply;
  CommInitReq comm_init; CommInitReply comm_init_reply;
  CommDestroyReq comm_destroy; CommDestroyReply comm_destroy_reply;
  RegisterStreamReq reg_stream; RegisterStreamReply reg_stream_reply;
  CommQueryReq comm_query; CommQueryReply comm_query_reply;
  MapScratchReq map_scratch; MapScratchReply map_scratch_reply;
  MapMemReq map_mem; MapMemReply map_mem_reply;
  MapMcReq map_mc; MapMcReply map_mc_reply;
  uint8_t raw[256];
};

// ---------------------------------------------------------------------------
// Data path
// ---------------------------------------------------------------------------
enum WrFlags : uint32_t {
  kWrGroupMore = 1u << 0,   // further requests of the same group follow
};

// Client-side launch: what a rank's proxy hands back for one collective, through the
// plan ring of the data-path segment. Addresses are (allocation, offset) pairs; the
// client library turns them into its own mappings.
constexpr uint32_t kPqDepth = 16;
constexpr uint32_t kPlanBytes = 1024;
struct alignas(64) PlanMsg {
  uint64_t user_seq;
  int32_t status;          // Status; anything but kOk: nothing to launch
  int32_t kind;            // CollKind
  int32_t variant, ctas, threads;
  int32_t dtype, op;
  int32_t nranks;
  float scale;
  uint32_t epoch;          // first barrier value of this launch
  uint64_t ticket;         // device-visible sequence number
  uint64_t count;
  uint64_t timeout_ns;
  struct { uint64_t send_mem, send_off, recv_mem, recv_off; } rank[8];
  int8_t ring[32][8];
  uint64_t ring_step_base[32];
  int32_t trace;           // 1: the kernel stamps its start and end time into the status block
  int32_t variant_hint;    // CollArgs::unroll_hint (ar_hybrid: share and CTAs of the in-switch part)
  uint64_t mc_send_id, mc_send_off;   // multicast region of the inputs (0: none) and this rank's offset in it
  uint64_t mc_recv_id, mc_recv_off;
  // Time slices: a large AllReduce of a tenant with competitors is cut into `nslices`
  // independent collectives over sub-ranges, each admitted (and handed out) on its own; this
  // message describes slice `slice` (count and offsets are the slice's). 1 / 0 otherwise.
  int32_t nslices, slice;
  // Fused launches: >= 2 in the answer to the first request of a fused launch (that many
  // consecutive requests of the communicator run in ONE kernel, launched with this plan's
  // shape, epoch and ticket); -1 in the answers to the others, which only describe their
  // buffers; 0 for a request that runs on its own.
  int32_t batch_len;
  int32_t pad1_;
  uint8_t reserved[128];
};
static_assert(sizeof(PlanMsg) == kPlanBytes, "a plan must fill one slot of the plan ring");

struct alignas(64) WorkRequest {
  uint32_t kind;        // CollKind
  uint32_t dtype;       // DataType (AllReduce)
  uint32_t op;          // RedOp (AllReduce)
  uint32_t flags;       // WrFlags
  uint64_t comm_handle;
  uint64_t send_mem, send_off;
  uint64_t recv_mem, recv_off;
  uint64_t count;       // AllReduce: elements; AllGather: bytes per rank
  uint64_t stream_id;   // from RegisterStream
  uint64_t user_seq;    // client-side counter, echoed in the completion
  float scale;          // PreMulSum / SumPostDiv argument
  uint32_t variant;     // Variant requested by the caller (0 = planner decides)
  uint64_t sync_slot;   // mem-op mode: 1 + index of the "submitted" semaphore, 0 = events
  uint64_t sync_value;  // value the caller's stream writes there before this request
  uint64_t reserved[3];
};
static_assert(sizeof(WorkRequest) == kWrBytes, "work request must fill one 128-byte slot");

struct alignas(64) WorkCompletion {
  uint32_t kind;
  int32_t status;       // Status
  uint64_t user_seq;
  uint32_t variant;     // what the planner launched
  uint32_t ctas;
  uint64_t comm_seq;    // sequence number of the collective within the communicator
  uint64_t reserved[4];
};
static_assert(sizeof(WorkCompletion) == kWcBytes, "completion must fill one 64-byte slot");

// Completion state of requests submitted in mem-op mode, at the end of the data-path
// segment. Such requests are not answered one by one (the caller does not wait for
// them, so a completion ring could fill up while the caller sits in a CUDA
// synchronisation that only ends once the daemon has launched more work); the daemon
// counts them here and keeps the first error.
struct alignas(64) DpStatus {
  uint64_t completed;      // mem-op requests the daemon has finished handling (launched or failed)
  int32_t first_error;     // Status of the first failed request, 0 = none
  uint32_t last_variant;
  uint32_t last_ctas;
  uint32_t pad_[11];
};
static_assert(sizeof(DpStatus) == 64, "DpStatus layout is part of the ABI");

inline size_t dp_wq_bytes() { return ((sizeof(uint64_t) * 24 + (size_t)kWqDepth * kWrBytes) + 63) / 64 * 64; }
inline size_t dp_cq_bytes() { return ((sizeof(uint64_t) * 24 + (size_t)kCqDepth * kWcBytes) + 63) / 64 * 64; }
inline size_t dp_pq_bytes() { return ((sizeof(uint64_t) * 24 + (size_t)kPqDepth * kPlanBytes) + 63) / 64 * 64; }
inline size_t dp_pq_offset() { return dp_wq_bytes() + dp_cq_bytes() + sizeof(DpStatus); }
inline size_t dp_segment_bytes() { return dp_pq_offset() + dp_pq_bytes(); }

inline uint64_t make_comm_handle(uint32_t comm_id, int rank) { return ((uint64_t)comm_id << 32) + (uint32_t)rank; }
inline uint32_t handle_comm_id(uint64_t h) { return (uint32_t)(h >> 32); }
inline int handle_rank(uint64_t h) { return (int)(uint32_t)h; }

// ---------------------------------------------------------------------------
// Admin channel (TCP), same framing as the reference's exchange engine
// (src/mccs/src/exchange/engine.rs:33,44-76): u64 magic, u8 type, u32 length, body.
// Type 1 carries a reconfiguration command; the body here is JSON text.
// ---------------------------------------------------------------------------
constexpr uint64_t kAdminMagic = 0x424ab9f2fc4b9d6eull;
enum AdminType : uint8_t { kAdminProxy = 0, kAdminReconfig = 1, kAdminQuery = 2 };

const char* status_string(int32_t s);

}  // namespace proto
}  // namespace mccs
