// Structures shared between the host-side planner/launcher and the sm_100a
// collective kernels. Plain C++ (no CUDA headers) so that host-only code and the
// CPU backend can include it.
//
// Role in the system: the reference hands its kernels a device-resident
// communicator (`mccsDevComm`, `mccsDevChannel`, per-peer `mccsDevConnInfo` with
// FIFO head/tail pointers; src/collectives/include/devcomm.h:36-164) plus a chained
// work FIFO. Here one daemon process owns every GPU of the box, so every rank's
// buffers, signal pads and staging FIFOs are addressable from every kernel. The
// whole description of one collective therefore fits in a by-value kernel
// parameter (`CollArgs`); there is no device-resident communicator to keep in sync.
#pragma once
#include <stdint.h>

namespace mccs {

constexpr int kMaxRanks = 8;       // one NVSwitch box
constexpr int kMaxCtas = 148;      // per-rank CTAs ("channels") per collective: one per SM of a B200
constexpr int kMaxRingChannels = 32;  // same limit as the reference (devcomm.h:32)
constexpr int kRingSlots = 8;      // FIFO slots per ring connection (devcomm.h:29)

enum DataType : int32_t {
  kInt8 = 0, kUint8 = 1, kInt32 = 2, kUint32 = 3, kInt64 = 4, kUint64 = 5,
  kFloat16 = 6, kFloat32 = 7, kFloat64 = 8, kBfloat16 = 9,
  kNumDataTypes = 10
};

// Same set as the reference protocol (src/ipc/mccs/src/command.rs:33-42).
enum RedOp : int32_t {
  kSum = 0, kProd = 1, kMax = 2, kMin = 3, kPreMulSum = 4, kSumPostDiv = 5,
  kNumRedOps = 6
};

// kReduceScatter: every rank sends nranks * count elements and receives the reduction of
// block `rank` (count elements).
enum CollKind : int32_t { kAllReduce = 0, kAllGather = 1, kReduceScatter = 2, kNumCollKinds = 3 };
inline bool kind_reduces(int kind) { return kind == kAllReduce || kind == kReduceScatter; }
// Units (elements; bytes for all-gather) one rank sends and receives for CollArgs::count.
inline uint64_t send_units(int kind, uint64_t count, int nranks) { return kind == kReduceScatter ? count * (uint64_t)nranks : count; }
inline uint64_t recv_units(int kind, uint64_t count, int nranks) { return kind == kAllGather ? count * (uint64_t)nranks : count; }

// Kernel variants. `kAuto` lets the planner pick from the tuning table.
enum Variant : int32_t {
  kAuto = 0,
  kArOneShot = 1,    // every rank pulls all peers' data, reduces, stores locally
  kArTwoShot = 2,    // reduce-scatter by peer loads + all-gather by peer stores
  kArNvlsOne = 3,    // multimem.ld_reduce of the whole buffer on every rank
  kArNvlsTwo = 4,    // multimem.ld_reduce own shard + multimem.st broadcast
  kArRing = 5,       // FIFO-staged ring (device FIFOs over NVLink or pinned host)
  kAgPull = 6,       // every rank loads its peers' shards
  kAgPush = 7,       // every rank stores its shard into every peer
  kAgNvls = 8,       // multimem.st of the own shard
  kAgRing = 9,       // FIFO-staged ring
  kLocalCopy = 10,   // single-rank communicator: device copy (or nothing in place)
  kArHybrid = 11,    // head of the buffer through the switch (multimem), rest by peer loads/stores, in one kernel
  kRsDirect = 12,    // reduce-scatter: every rank loads its block from all peers and reduces it
  kRsNvls = 13,      // reduce-scatter: multimem.ld_reduce of the own block
  kNumVariants = 14
};

// Error codes written by kernels into the per-rank status word.
enum DevStatus : uint32_t {
  kDevOk = 0,
  kDevTimeoutStart = 1,   // a peer never arrived at the start barrier
  kDevTimeoutEnd = 2,     // a peer never arrived at the end barrier
  kDevTimeoutRing = 3,    // ring credit / data wait ran out
  kDevAborted = 4,        // host raised the abort word
  kDevBadArgs = 5
};

// Per-rank signal pad, placed in that rank's device memory (or in pinned host
// memory for the host-staged transport) and mapped for all peers. All counters only
// ever grow, so a pad is never reset between collectives.
struct alignas(128) SignalPad {
  // barrier[cta][peer]: written by `peer`, polled by the owner.
  uint32_t barrier[kMaxCtas][kMaxRanks];
  // Ring flow control (per channel). `tail` counts slots filled in the owner's
  // receive FIFO (written by the ring predecessor); `head` counts slots of the
  // owner's *sends* that the ring successor has consumed (written by the successor).
  uint64_t ring_tail[kMaxRingChannels];
  uint64_t ring_head[kMaxRingChannels];
  // Counters of finished CTAs of the owner's kernels (wrap to zero at the grid size, so
  // they need no reset between launches): [kPadBatchCounter] for the fused kernels'
  // caller-visible completion word, [kPadCtaCounter] for StatusBlock::done_seq.
  uint32_t pad_[32];
};
// Launch shape of the single-rank copy kernel: every thread moves kCopyUnroll 16-byte
// packs, one CTA per tile of the message.
constexpr int kCopyThreads = 256;
constexpr int kCopyUnroll = 4;
constexpr uint64_t kCopyTileBytes = (uint64_t)kCopyThreads * kCopyUnroll * 16;
constexpr int kPadBatchCounter = 0;
constexpr int kPadCtaCounter = 1;

// Per-rank status block in pinned, host-mapped memory: the host reads it without
// synchronising the stream.
struct alignas(64) StatusBlock {
  uint32_t error;          // DevStatus, sticky (atomicMax)
  uint32_t error_peer;     // which peer (or ring step) the failed wait was for
  uint64_t done_seq;       // sequence number of the last collective that finished
  uint64_t start_ns;       // globaltimer at kernel start of the last collective (tracing)
  uint64_t end_ns;         // globaltimer at its end
  uint32_t abort;          // host -> device: non-zero makes every wait of this rank give up
  uint32_t pad0_;
  uint64_t pad_[3];
};

struct CollArgs {
  // --- identity -------------------------------------------------------------
  int32_t rank;            // ignored when `emulated` (then rank = blockIdx.y)
  int32_t nranks;
  int32_t emulated;        // 1: all ranks share one GPU and one cooperative launch
  int32_t dtype;           // DataType
  int32_t op;              // RedOp
  int32_t variant;         // Variant
  uint64_t count;          // AllReduce: elements. AllGather: bytes per rank. ReduceScatter: elements per block.
  uint64_t seq;            // collective sequence number (for StatusBlock::done_seq)
  float scale;             // PreMulSum multiplier / SumPostDiv divisor reciprocal
  uint32_t epoch;          // first barrier value this launch may use (uses epoch, epoch+1)
  uint64_t timeout_ns;     // bound for every device-side wait
  int32_t trace;           // 1: record globaltimer start/end into the status block
  int32_t unroll_hint;     // ar_hybrid: low 16 bits = share of the message for the multimem part (1/1000), high 16 bits = its CTAs;
                           // the NVLS all-reduce kernels: in-switch loads in flight per thread (8, or 4 for any other value);
                           // all-gather pull/push: 32 = 256-bit loads and stores where buffers and size allow
  // --- buffers (unicast addresses valid on every GPU of the communicator) -----
  const void* send[kMaxRanks];
  void* recv[kMaxRanks];
  // --- multicast addresses (NVLS variants), null otherwise ---------------------
  const void* mc_send;
  void* mc_recv;
  // --- synchronisation -----------------------------------------------------------
  SignalPad* pad[kMaxRanks];
  StatusBlock* status[kMaxRanks];
  // --- ring ------------------------------------------------------------------------
  int8_t ring[kMaxRingChannels][kMaxRanks];  // ring[c][i] = user rank at position i of channel c's ring
  char* fifo[kMaxRanks];          // base of each rank's receive FIFOs
  uint64_t fifo_slot_bytes;       // bytes per slot
  uint64_t ring_step_base[kMaxRingChannels];  // cumulative steps already used per channel
};

// Several consecutive AllReduces of one communicator with the same element type and
// operator, carried by ONE launch: one barrier before the first and one after the last
// instead of two per collective. The reference fuses the same way, up to 10 work
// elements per work item (src/mccs/src/proxy/plan.rs:122-141,
// src/collectives/include/devcomm.h:66,103-104). `base` gives everything that is per
// launch (identity, op, epoch, pads, status); its own send/recv/count are unused.
constexpr int kMaxBatch = 8;
enum BatchFlags : uint32_t {
  // Every rank's launch was held back by the host until all ranks' inputs existed and all
  // outputs could be overwritten, so the kernel needs no barrier before its first load.
  kBatchSkipStartBarrier = 1u << 0,
};
struct BatchArgs {
  CollArgs base;
  int32_t nops;
  uint32_t flags;                            // BatchFlags
  // Optional completion word for the caller: the last CTA of this rank to finish stores
  // `done_value` to `done_ptr` (null = nobody is told from inside the kernel).
  // `done_counter` is a word in this rank's device memory that counts finished CTAs and
  // wraps to zero at gridDim.x, so it needs no reset between launches.
  uint64_t* done_ptr[kMaxRanks];
  uint64_t done_value[kMaxRanks];
  uint32_t* done_counter[kMaxRanks];
  uint64_t count[kMaxBatch];                 // elements of each member
  const void* send[kMaxBatch][kMaxRanks];
  void* recv[kMaxBatch][kMaxRanks];
  const void* mc_send[kMaxBatch];            // NVLS members only
  void* mc_recv[kMaxBatch];
};

struct LaunchDims {
  int32_t ctas;      // grid.x (per rank)
  int32_t threads;   // block.x
};

inline int dtype_size(int dt) {
  switch (dt) {
    case kInt8: case kUint8: return 1;
    case kFloat16: case kBfloat16: return 2;
    case kInt32: case kUint32: case kFloat32: return 4;
    case kInt64: case kUint64: case kFloat64: return 8;
  }
  return 0;
}

inline const char* variant_name(int v) {
  switch (v) {
    case kAuto: return "auto";
    case kArOneShot: return "ar_oneshot";
    case kArTwoShot: return "ar_twoshot";
    case kArNvlsOne: return "ar_nvls_oneshot";
    case kArNvlsTwo: return "ar_nvls_twoshot";
    case kArRing: return "ar_ring";
    case kAgPull: return "ag_pull";
    case kAgPush: return "ag_push";
    case kAgNvls: return "ag_nvls";
    case kAgRing: return "ag_ring";
    case kLocalCopy: return "local_copy";
    case kArHybrid: return "ar_hybrid";
    case kRsDirect: return "rs_direct";
    case kRsNvls: return "rs_nvls";
  }
  return "?";
}

inline bool variant_is_nvls(int v) { return v == kArNvlsOne || v == kArNvlsTwo || v == kAgNvls || v == kArHybrid || v == kRsNvls; }
inline bool variant_is_ring(int v) { return v == kArRing || v == kAgRing; }

// Number of ring steps one channel consumes for a collective. Every rank and every
// channel advances by the same amount, which keeps the cumulative FIFO counters of
// all connections in step. `elems_or_bytes` is CollArgs::count.
inline uint64_t ring_loops(int kind, uint64_t count, int elem_size, int nranks, int nch,
                           uint64_t slot_bytes) {
  // Elements (bytes for all-gather) one slot can carry.
  uint64_t per_slot = slot_bytes / (kind == kAllGather ? 1 : elem_size);
  uint64_t per_loop = kind == kAllGather ? per_slot * (uint64_t)nch
                                         : per_slot * (uint64_t)nch * (uint64_t)nranks;
  if (count == 0) return 0;
  return (count + per_loop - 1) / per_loop;
}

inline uint64_t ring_steps_per_channel(int kind, uint64_t count, int elem_size, int nranks,
                                       int nch, uint64_t slot_bytes) {
  uint64_t loops = ring_loops(kind, count, elem_size, nranks, nch, slot_bytes);
  uint64_t per_loop = kind == kAllGather ? (uint64_t)(nranks - 1) : 2ull * (nranks - 1);
  return loops * per_loop;
}

}  // namespace mccs
