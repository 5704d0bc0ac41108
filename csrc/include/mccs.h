/* libmccs: client API of the managed collective communication service.
 *
 * An application links against (or dlopens) libmccs.so and talks to the per-host
 * daemon `mccsd`. The daemon owns the GPUs' communication: it allocates the device
 * buffers (the application maps them), keeps the communicators, plans and admits every
 * collective (variant, launch shape, ring order, tenant arbitration) and can change
 * all of that while applications run. A collective call is stream ordered like a
 * kernel launch: the caller's stream will not run anything issued later until the
 * collective has finished. Who launches the kernel is the daemon's choice
 * ([b200] launch in its configuration):
 *   - this library (the default on GPUs for communicators whose ranks are separate
 *     processes on separate GPUs): it maps the peers' buffers, signal pads and
 *     multicast objects and launches its rank's kernel on the caller's stream from the
 *     plan the daemon made; a call blocks until every rank has made the same call and
 *     the plan is back, like a rendezvous;
 *   - the daemon, on its own streams (ranks that share a GPU, clients inside the
 *     daemon's process, the host-staged transport, the host backend), ordered against
 *     the caller's stream in one of two ways ([b200] sync):
 *       stream memory operations (default on GPUs that support them): the library
 *       queues "write submitted" and "wait done" on the caller's stream, on two 64-bit
 *       semaphores in a pinned host page it shares with the daemon, and returns at
 *       once; the daemon polls "submitted" and launches when every rank got there;
 *       errors of a request show up on a later call or in mccsCommFlush. One stream may
 *       carry only one rank of a given communicator;
 *       interprocess events (the reference's scheme): the library records "submitted",
 *       waits for the daemon's completion message, then makes the stream wait for the
 *       daemon's "done" event; the call blocks for one round trip and reports errors.
 * In every arrangement each call involves the daemon, so collectives cannot be recorded
 * into a CUDA graph and replayed; keep them outside stream capture.
 *
 * This is the C form of the reference's Rust API (src/libmccs/src/lib.rs:23-27):
 *   cuda_malloc            -> mccsMalloc          (src/libmccs/src/memory.rs:12)
 *   init_communicator_rank -> mccsCommInitRank    (src/libmccs/src/communicator.rs:15)
 *   register_stream        -> mccsRegisterStream  (src/libmccs/src/communicator.rs:47)
 *   all_gather             -> mccsAllGather       (src/libmccs/src/collectives.rs:15)
 *   all_reduce             -> mccsAllReduce       (src/libmccs/src/collectives.rs:75)
 * plus what the reference leaves out: mccsFree (its cuda_free is unimplemented),
 * communicator destruction, grouped submission, error queries, a C ABI.
 *
 * Environment: MCCS_CONTROL (path of the daemon's control socket, overrides
 * MCCS_PREFIX + "/control.sock"), MCCS_PREFIX (default /tmp/mccs-$USER),
 * MCCS_DEVICE_AFFINITY (advertised to the daemon), MCCS_WC_TIMEOUT_MS.
 *
 * Threading: one communicator (and one CUDA stream used with it) belongs to one
 * host thread at a time, as in the reference (src/ipc/mccs/src/command.rs:96-98).
 */
#ifndef MCCS_H_
#define MCCS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct mccsComm* mccsComm_t;
typedef void* mccsStream_t; /* a cudaStream_t / CUstream (NULL = legacy default stream) */

typedef enum {
  mccsSuccess = 0,
  mccsInvalidArgument = -1,
  mccsOutOfMemory = -2,
  mccsDeviceError = -3,
  mccsProtocolError = -4,
  mccsNotFound = -5,
  mccsTimeout = -6,
  mccsAborted = -7,
  mccsMismatch = -8,
  mccsUnsupported = -9,
  mccsPeerLost = -10,
  mccsInternalError = -11,
  mccsNotConnected = -12,
  mccsBusy = -13            /* mccsFree: a queued collective still names the memory */
} mccsResult_t;

/* Same numbering as the kernels' element types. The reference API exposes only
 * Float16 and Int32 (src/ipc/mccs/src/command.rs:26-31). */
typedef enum {
  mccsInt8 = 0, mccsUint8 = 1, mccsInt32 = 2, mccsUint32 = 3, mccsInt64 = 4, mccsUint64 = 5,
  mccsFloat16 = 6, mccsFloat32 = 7, mccsFloat64 = 8, mccsBfloat16 = 9
} mccsDataType_t;

/* src/ipc/mccs/src/command.rs:33-42. mccsSumPostDiv divides by the communicator
 * size (an average); mccsPreMulSum multiplies every input by `scale` first. */
typedef enum {
  mccsSum = 0, mccsProd = 1, mccsMax = 2, mccsMin = 3, mccsPreMulSum = 4, mccsSumPostDiv = 5
} mccsRedOp_t;

/* Kernel variant request (0 lets the service decide). */
typedef enum {
  mccsAlgoAuto = 0, mccsAlgoArOneShot = 1, mccsAlgoArTwoShot = 2, mccsAlgoArNvlsOneShot = 3,
  mccsAlgoArNvlsTwoShot = 4, mccsAlgoArRing = 5, mccsAlgoAgPull = 6, mccsAlgoAgPush = 7,
  mccsAlgoAgNvls = 8, mccsAlgoAgRing = 9, mccsAlgoLocalCopy = 10,
  mccsAlgoArHybrid = 11,  /* part through the switch, part by peer copies, in one kernel */
  mccsAlgoRsDirect = 12,  /* reduce-scatter by peer loads */
  mccsAlgoRsNvls = 13     /* reduce-scatter in the switch */
} mccsAlgo_t;

/* Connects to the daemon. Optional: every other call connects on first use with
 * the path from the environment. */
mccsResult_t mccsInit(const char* control_socket_path);
mccsResult_t mccsFinalize(void);
/* 0: host backend (no GPU, buffers are host shared memory), 1: CUDA. */
int mccsBackendKind(void);
int mccsDeviceCount(void);

/* Device memory owned by the daemon and mapped here. Only such memory can be
 * passed to collectives. */
mccsResult_t mccsMalloc(void** ptr, int device, size_t size);
mccsResult_t mccsFree(void* ptr);
/* Which allocation a pointer belongs to (any address inside it). */
mccsResult_t mccsMemInfo(const void* ptr, uint64_t* mem_id, uint64_t* offset, uint64_t* alloc_size);

/* Blocks until all `nranks` ranks of `unique_id` have joined. `root_addr` is accepted
 * for source compatibility with the reference and ignored inside one box. */
mccsResult_t mccsCommInitRank(mccsComm_t* comm, uint32_t unique_id, int rank, int nranks, int device,
                              const char* root_addr);
mccsResult_t mccsCommDestroy(mccsComm_t comm);
mccsResult_t mccsCommRank(mccsComm_t comm, int* rank);
mccsResult_t mccsCommSize(mccsComm_t comm, int* nranks);
uint64_t mccsCommHandle(mccsComm_t comm); /* (unique_id << 32) + rank */

/* Optional: streams are registered on first use. */
mccsResult_t mccsRegisterStream(int device, mccsStream_t stream);

/* count: elements. In-place when send == recv. */
mccsResult_t mccsAllReduce(mccsComm_t comm, const void* send, void* recv, size_t count,
                           mccsDataType_t dtype, mccsRedOp_t op, mccsStream_t stream);
mccsResult_t mccsAllReduceEx(mccsComm_t comm, const void* send, void* recv, size_t count,
                             mccsDataType_t dtype, mccsRedOp_t op, float scale, mccsAlgo_t algo,
                             mccsStream_t stream);
/* bytes: per rank. recv holds nranks*bytes; in-place when send == recv + rank*bytes. */
mccsResult_t mccsAllGather(mccsComm_t comm, const void* send, void* recv, size_t bytes,
                           mccsStream_t stream);
mccsResult_t mccsAllGatherEx(mccsComm_t comm, const void* send, void* recv, size_t bytes,
                             mccsAlgo_t algo, mccsStream_t stream);

/* Not in the reference: every rank contributes nranks*count elements and receives the
 * reduction of block `rank` (count elements), at half the traffic of an AllReduce.
 * In-place when recv == send + rank*count elements. */
mccsResult_t mccsReduceScatter(mccsComm_t comm, const void* send, void* recv, size_t count,
                               mccsDataType_t dtype, mccsRedOp_t op, mccsStream_t stream);
mccsResult_t mccsReduceScatterEx(mccsComm_t comm, const void* send, void* recv, size_t count,
                                 mccsDataType_t dtype, mccsRedOp_t op, float scale, mccsAlgo_t algo,
                                 mccsStream_t stream);

/* Deferred waiting. By default every collective call also makes the caller's stream wait
 * for the collective (stream order, like a kernel launch). A caller that issues many
 * collectives from a side stream and only needs the results later (gradient buckets
 * during backward) can switch that off for a communicator and place one wait itself:
 * mccsCommWait makes `stream` wait for every collective submitted on `comm` so far. */
mccsResult_t mccsCommSetDeferredWait(mccsComm_t comm, int on);
mccsResult_t mccsCommWait(mccsComm_t comm, mccsStream_t stream);

/* Calls between GroupStart and GroupEnd are submitted back to back and completed
 * together at GroupEnd (the protocol's GroupCall, src/ipc/mccs/src/command.rs:93-95):
 * the caller's stream is ordered after the whole group, not after each member, so the
 * daemon can queue the members' kernels without a gap. Results of a member are defined
 * for work queued after GroupEnd. */
mccsResult_t mccsGroupStart(void);
mccsResult_t mccsGroupEnd(void);

typedef struct {
  int32_t async_error;     /* mccsResult_t, sticky */
  uint32_t device_error;   /* kernel-reported status, 0 = none */
  uint64_t launched;
  uint64_t completed;
  uint32_t last_variant;   /* mccsAlgo_t the service chose for the last collective */
  uint32_t last_ctas;
  uint64_t config_epoch;   /* number of live reconfigurations applied */
} mccsCommInfo_t;
mccsResult_t mccsCommQuery(mccsComm_t comm, mccsCommInfo_t* info);
mccsResult_t mccsCommGetAsyncError(mccsComm_t comm, mccsResult_t* async_error);
/* Waits (on the host) until the daemon has taken and launched every request posted on
 * this communicator so far, and returns the first error any of them reported. With
 * stream-memory-operation synchronisation collective calls return before the daemon
 * has seen them; this is the point where their errors become visible. It does not
 * wait for the GPU work (synchronise the stream for that). */
mccsResult_t mccsCommFlush(mccsComm_t comm);
/* Variant and CTA count reported with the last completed request of this rank. */
mccsResult_t mccsCommLastPlan(mccsComm_t comm, uint32_t* variant, uint32_t* ctas);
/* Who launches this communicator's kernels: 0 = the daemon, 1 = this library on the
 * caller's stream ([b200] launch = "client" in the daemon's configuration). */
int mccsCommLaunchMode(mccsComm_t comm);

const char* mccsGetErrorString(mccsResult_t r);
const char* mccsAlgoName(int algo);

/* Admin client: sends one framed request (type 1 = reconfiguration, 2 = query) with a
 * JSON body to a daemon's admin port and copies the JSON reply into `reply`. */
mccsResult_t mccsAdminRequest(const char* host, int port, int type, const char* json_body, char* reply,
                              size_t reply_cap);

/* Hooks for torch.cuda.memory.CUDAPluggableAllocator. */
void* mccs_torch_malloc(size_t size, int device, void* stream);
void mccs_torch_free(void* ptr, size_t size, int device, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MCCS_H_ */
