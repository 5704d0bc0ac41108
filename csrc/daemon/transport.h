// Transports: the ways one rank's data reaches another rank inside the box, behind one
// interface, chosen per (sender, receiver) connection.
//
// The reference selects a transporter for every connection of a communicator through a
// trait with `can_connect` / `send_setup` / `recv_setup` / `connect` stages
// (src/mccs/src/transport/transporter.rs:84-256); the first registered transporter whose
// `can_connect` accepts the pair wins (src/mccs/src/transport/setup.rs:346-361), and a
// typed catalog holds their configurations (src/mccs/src/transport/catalog.rs:20-80).
// Its transporters are host shared memory and RDMA. Inside one NVSwitch box the peers of
// the interface are:
//
//   nvls         NVLink through the switch with multicast objects: carries the in-switch
//                variants and everything the peer-memory transport carries
//   nvlink_p2p   peer device memory over NVLink (plain loads and stores of a peer's buffer)
//   host_staged  FIFO slots and flags in pinned host memory, for device pairs without peer
//                access, or when configured: carries the FIFO ring variants only
//
// There are no per-connection agents to set up here (one process owns every GPU, the kernels
// get all addresses as launch arguments), so what a connection contributes to its
// communicator is (a) which kernel variants it can carry and (b) where the signal pads and
// FIFOs of its end points must live. Pads and FIFOs are per rank, shared by all of a rank's
// connections; a communicator with one host-staged connection therefore keeps all of them
// in pinned host memory and is limited to what every connection carries.
#pragma once
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "../kernels/dev_types.h"

namespace mccs {

enum TransportKind : int { kTransportNvls = 0, kTransportNvlinkP2P = 1, kTransportHostStaged = 2, kNumTransportKinds = 3 };

// What the probes may ask about the machine (the device backend; a table in tests).
struct TransportEnv {
  std::function<bool(int, int)> peer_access;   // can device a address device b's memory
  std::function<bool(int)> multicast;          // can the device join a multicast object
  bool nvls_enabled = true;                    // [b200] nvls
};

class Transport {
 public:
  virtual ~Transport() = default;
  virtual TransportKind kind() const = 0;
  virtual const char* name() const = 0;
  // Can the rank on `send_dev` deliver to the rank on `recv_dev` this way?
  virtual bool can_connect(const TransportEnv& env, int send_dev, int recv_dev) const = 0;
  // Can a connection of this kind carry kernel variant `variant` (kernels/dev_types.h)?
  virtual bool carries(int variant) const = 0;
  // Signal pads and FIFOs of the end points live in pinned host memory (else device memory).
  virtual bool scratch_in_host_memory() const = 0;
};

// The ordered list of transports a daemon offers. `mode` is `[b200] transport`:
// "auto" = nvls, nvlink_p2p, host_staged in that order; "nvlink" = without host_staged (a pair
// without peer access is then an error); "host_staged" = only that one.
class TransportCatalog {
 public:
  explicit TransportCatalog(const std::string& mode);
  // First transport whose can_connect accepts the pair; null when none does.
  const Transport* select(const TransportEnv& env, int send_dev, int recv_dev) const;
  const std::vector<std::unique_ptr<Transport>>& transports() const { return list_; }

 private:
  std::vector<std::unique_ptr<Transport>> list_;
};

// The chosen transport of every ordered pair of ranks of one communicator.
struct ConnectionTable {
  int nranks = 0;
  const Transport* conn[kMaxRanks][kMaxRanks] = {};   // [sender][receiver], null on the diagonal
  int unconnected_from = -1, unconnected_to = -1;     // first pair no transport accepted

  bool complete() const { return unconnected_from < 0; }
  bool any(TransportKind k) const;
  bool all(TransportKind k) const;
  // Every connection can carry the variant (a single rank has no connections: everything).
  bool carries(int variant) const;
  bool scratch_in_host_memory() const;
  uint32_t carried_variants() const;   // bit v set: carries(v)
  std::string describe() const;        // e.g. "nvls" or "nvlink_p2p x10, host_staged x2"
};

ConnectionTable connect_all(const TransportCatalog& catalog, const TransportEnv& env, const std::vector<int>& devices);

}  // namespace mccs
