// Daemon configuration. The file keeps the reference's TOML schema
// (src/mccs/src/config.rs:14-89 and the shipped mccs.toml) so an existing mccs.toml
// loads unchanged: [control], [comm_default_config], [comm_global_config.*], addrs,
// listen_port, [qos_schedule] and [[comm_patterns_override]]. The RDMA/NIC keys are
// accepted and kept but have no effect inside one NVSwitch box. A new [b200] table
// and [qos.tenants.<id>] tables carry what the NVLink re-target adds: transport
// selection, NVLS on/off, device wait bound, tuning table, tenant weights.
#pragma once
#include <stdint.h>

#include <map>
#include <string>
#include <utility>
#include <vector>

#include "../common/value.h"

namespace mccs {

struct ChannelPattern {
  int channel_id = 0;
  std::vector<int> ring;                      // user ranks in ring order
  std::vector<std::vector<int>> udp_sport;    // kept for schema parity, unused
  std::string net_dev;                        // kept for schema parity, unused
};

struct CommPattern {
  uint32_t communicator_id = 0;
  std::vector<ChannelPattern> channels;
  int ib_traffic_class = -1;
  // Extensions for the NVLink box (all optional).
  std::string allreduce_algo;   // "", "auto", or a variant name
  std::string allgather_algo;
  int ctas = 0;                 // 0: planner decides ("channel count" of the new kernels)
};

struct QosIntervalConfig {
  std::vector<std::pair<uint64_t, uint64_t>> intervals;  // [start,end) in µs within the epoch
  bool allow = true;            // mode = "Allow" | "Deny"
  int enforce_step = 0;         // 0: every collective; N: only when round % N == 0
};

struct QosTenantConfig {
  double weight = 1.0;
  int priority = 0;             // > 0: high-priority stream
  int cta_quota = 0;            // 0: derived from the weight
};

struct Config {
  // [control]
  std::string control_prefix = "/tmp/mccs-${USER}";
  std::string control_path = "control.sock";
  std::string daemon_prefix = "/tmp/mccs-${USER}";
  std::string daemon_basename = "mccs-deamon";
  std::vector<std::string> addrs;
  int listen_port = 5000;       // admin/exchange TCP port; 0 disables, -1 picks a free port
  // [comm_default_config]
  std::vector<uint64_t> buffer_sizes{4u << 20};   // ring FIFO bytes per channel
  int channel_count = 1;
  // [comm_global_config.*] kept verbatim
  Value comm_global_config;
  // [qos_schedule]
  uint64_t qos_epoch_us = 0;
  std::map<uint32_t, QosIntervalConfig> qos_schedule;
  // [qos.tenants.<id>]
  std::map<uint32_t, QosTenantConfig> qos_tenants;
  int qos_cta_budget = 64;       // CTAs shared by contending tenants on one GPU
  uint64_t qos_max_outstanding_bytes = 64ull << 20;  // per tenant, only under contention
  int qos_sm_limit = 148;          // CTAs of kernels that wait on each other allowed in flight per GPU; 0 = unchecked
  uint64_t qos_active_window_us = 5000;  // a tenant counts as a contender this long after its last request
  // [[comm_patterns_override]]
  std::vector<CommPattern> overrides;
  // [b200]
  std::string transport = "auto";   // auto | nvlink | host_staged
  bool nvls = true;
  bool vmm = true;
  std::string sync = "auto";        // auto | events | memops (see proto::SyncMode)
  // Who launches the kernels (proto::LaunchMode). auto: on GPUs the clients themselves, for
  // communicators whose ranks are all other processes, one per GPU, on peer memory (the
  // hand-over between two processes costs more than the kernel of a small collective);
  // the daemon otherwise. daemon / client force one of the two where it is possible.
  std::string launch = "auto";
  bool client_nvls = true;          // client-side launch: also plan the in-switch variants (clients map the multicast objects)
  uint64_t wait_timeout_ms = 10000; // bound of every device-side wait
  std::string tuning_file;
  bool trace = false;
  std::string trace_file;
  int host_devices = 8;
  std::vector<std::pair<int, int>> host_no_peer_access;   // host backend: [[a, b], ...] device pairs without peer access
  bool force_host_backend = false;
  std::string host_kernels = "loops";  // host backend: "loops" (plain CPU collectives) | "emulated" (the kernels on the SIMT emulator)
  int idle_sleep_us = 50;           // sleep between polls once a proxy has been idle for idle_spin_us
  int idle_spin_us = 200000;        // how long an idle proxy keeps busy-polling
  bool pin_threads = true;
  uint64_t init_timeout_ms = 60000; // how long a communicator waits for all its ranks
  // Fused launches: up to this many consecutive AllReduces of a communicator (same type and
  // operator, all queued when the first is planned) share one kernel; 1 = off.
  // What one client (one connection to the control socket) may hold. A tenant is another
  // user's process: without bounds one of them can take the daemon's memory or every byte of
  // a GPU. 0 = no limit.
  int max_clients = 1024;
  int max_allocations_per_client = 65536;
  uint64_t max_bytes_per_client = 0;
  int max_communicators_per_client = 1024;
  int fuse_allreduce = 1;
  // Experiments on the per-call floor; they act on launches that go through the fused
  // kernels only (kernels/batch.cuh) and are all off by default.
  int hybrid_nvls_permille = 750;     // ar_hybrid: share of the message that goes through the switch (1/1000)
  int pack_bytes = 16;             // two-shot AllReduce and AllGather pull/push kernels: bytes per load/store instruction (16, or 32 = sm_100's 256-bit form)
  int nvls_unroll = 4;                // NVLS all-reduce kernels: in-switch loads in flight per thread (4 or 8)
  int hybrid_nvls_ctas = 8;           // ar_hybrid: CTAs that feed the switch; the others exchange the rest by peer copies
  bool single_through_fused = false;  // a lone two-shot AllReduce also uses the fused kernel (one member)
  bool skip_start_barrier = false;    // no barrier before the first load when the host has gated every rank
  bool kernel_writes_done = false;    // the kernel's last CTA releases the caller's stream itself

  std::string control_socket_path() const;   // expanded prefix/path
  const CommPattern* find_override(uint32_t comm_id) const;

  static Config from_value(const Value& root);       // throws std::runtime_error
  static Config from_file(const std::string& path);  // throws
  static Config from_string(const std::string& toml);
  // Parses one override / reconfiguration entry (TOML or JSON tree).
  static CommPattern parse_pattern(const Value& v);
};

}  // namespace mccs
