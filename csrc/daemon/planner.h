// Collective planner: picks the kernel variant and the launch shape for one
// collective from a size-indexed tuning table, then applies feasibility rules.
// It is the counterpart of the reference's schedule step
// (src/mccs/src/proxy/plan.rs:111-166 kernel choice, :602-635 thread/channel sizing),
// which has a single algorithm and sizes 64..512 threads x channels from the byte
// count. Pure host code, no device calls, so it is unit-testable.
#pragma once
#include <stdint.h>

#include <mutex>
#include <shared_mutex>
#include <string>
#include <vector>

#include "../common/value.h"
#include "../kernels/dev_types.h"

namespace mccs {

struct TuneEntry {
  uint64_t max_bytes;   // entry applies to messages of up to this many bytes
  int variant;
  int ctas;
  int threads;
};

// Table for one (collective kind, rank count).
struct TuneTable {
  std::vector<TuneEntry> entries;   // ascending max_bytes; the last one is the catch-all
  const TuneEntry* lookup(uint64_t bytes) const;
};

struct PlanInput {
  int kind = kAllReduce;        // CollKind
  int nranks = 1;
  uint64_t count = 0;           // elements (AllReduce) / bytes per rank (AllGather)
  int dtype = kFloat32;
  int op = kSum;
  bool in_place = false;        // any rank passed aliasing send/recv
  bool aligned16 = true;        // all pointers (and the AllGather byte count) 16-byte aligned
  bool nvls_possible = false;   // backend has NVLS, buffers sit at equal offsets of multicast-able allocations
  bool p2p_possible = true;     // all devices can address each other's memory
  bool host_staged = false;     // transport forces FIFO rings through pinned host memory
  uint32_t carried_variants = ~0u;  // bit v: every connection of the communicator can carry variant v (ConnectionTable)
  bool emulated = false;        // all ranks on one device (single cooperative launch)
  int requested_variant = kAuto;  // from the caller or an override
  int requested_ctas = 0;         // from an override ("channel count"), 0 = table
  int cta_cap = 0;                // QoS quota, 0 = none
  int ring_channels = 1;          // configured channel count for ring variants
  uint64_t fifo_slot_bytes = (4u << 20) / kRingSlots;
};

struct Plan {
  int variant = kAuto;
  LaunchDims dims{1, 512};
  uint64_t bytes = 0;           // message size used for the table lookup and accounting
  bool needs_mc_send = false;   // multicast mapping of the send allocations required
  bool needs_mc_recv = false;
  int status = 0;               // proto::Status; non-zero: cannot run
  std::string note;             // why a requested variant was replaced, for logs
};

class Planner {
 public:
  Planner();
  // Built-in defaults, optionally overlaid by a tuning file (JSON) measured on the box.
  void load_defaults(bool nvls);
  bool load_file(const std::string& path, std::string* err);
  bool load_json(const Value& root, std::string* err);
  Value to_json() const;

  Plan plan(const PlanInput& in) const;
  // Feasibility of one variant for this input ("" = ok, else the reason).
  static std::string infeasible(int variant, const PlanInput& in);
  static int variant_from_name(const std::string& name);  // -1 when unknown
  static uint64_t message_bytes(const PlanInput& in);

 private:
  TuneTable& table(int kind, int nranks);
  const TuneTable* find_table(int kind, int nranks) const;
  TuneTable tables_[kNumCollKinds][kMaxRanks + 1];
  mutable std::shared_mutex mu_;   // tables can be replaced at run time (admin tuning_set) while proxies plan
};

}  // namespace mccs
