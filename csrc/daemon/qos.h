// Flow scheduler for tenants that share the GPUs and the NVLink fabric of one box.
//
// The reference arbitrates tenants on an Ethernet fabric: per-communicator route
// pinning plus periodic Allow/Deny send windows checked before each RDMA chunk
// (src/qos-service/src/lib.rs:18-85, enforcement in
// src/mccs/src/transport/net/agent.rs:514-541). Inside an NVSwitch box the contended
// resources are SMs, launch slots and per-GPU link bandwidth, so the same policy
// surface (tenant = communicator id, priority, windows) plus weights is enforced at
// different points:
//   * CTA quota: under contention a tenant's kernels get a share of a per-GPU CTA
//     budget proportional to its weight (bandwidth of co-running kernels follows
//     their CTA counts);
//   * launch admission: weighted fair queueing over bytes with a bound on each
//     tenant's outstanding bytes, decided once per collective (or time slice) for
//     all ranks together;
//   * time slicing: large collectives are cut into slices that are admitted one by
//     one, so a waiting tenant gets the links between slices;
//   * windows: the Allow/Deny interval schedule of the reference, evaluated on the
//     same `now % epoch` clock;
//   * stream priority for tenants marked high priority;
//   * residency: the kernels of one collective wait for each other across GPUs, so all
//     their CTAs must get an SM. A launch is held back while its CTAs plus those of the
//     other tenants' kernels in flight on a shared GPU exceed the SM count: otherwise two
//     tenants whose kernels reached two GPUs in opposite order could each hold the SMs
//     the other one's missing CTAs need, until the device-side bound ends both.
// All decisions are host-side and take the clock as an argument (testable).
#pragma once
#include <stdint.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../common/value.h"
#include "config.h"

namespace mccs {

enum QosDecision { kQosAdmit = 0, kQosDeferWindow = 1, kQosDeferBacklog = 2, kQosDeferFairness = 3, kQosDeferResidency = 4 };

class QosArbiter {
 public:
  QosArbiter();
  void configure(const Config& cfg);
  void set_tenant(uint32_t id, const QosTenantConfig& t);
  void set_schedule(uint64_t epoch_us, const std::map<uint32_t, QosIntervalConfig>& schedule);
  void set_enabled(bool on) { std::lock_guard<std::mutex> g(mu_); enabled_ = on; bump(); }

  void tenant_register(uint32_t id, const std::vector<int>& devices);
  void tenant_unregister(uint32_t id);

  // Tenants other than `id` that share a device with it and were active recently.
  int contenders(uint32_t id, uint64_t now_us);
  // CTA cap for a collective planned now (0 = no cap).
  int cta_cap(uint32_t id, uint64_t now_us);
  // Bytes per time slice for a collective planned now (0 = do not slice).
  uint64_t slice_bytes(uint32_t id, uint64_t now_us);
  int stream_priority(uint32_t id);   // 0 normal, 1 high

  // A planned collective (or slice) asks to launch. `wall_us` is the Unix clock used
  // for the window schedule, `now_us` a monotonic clock.
  // `ctas`: CTAs the launch puts on each of the tenant's GPUs (0 = unknown, not counted).
  QosDecision admit(uint32_t id, uint64_t bytes, uint64_t now_us, uint64_t wall_us, int ctas = 0);
  // Registers that a collective of `id` is planned and waiting for admission.
  void note_waiting(uint32_t id, uint64_t now_us);
  void complete(uint32_t id, uint64_t bytes);
  // Changes whenever something happened that can turn a deferral into an admission (a
  // completion, another tenant's admission, a new policy). A proxy that was told to wait
  // reads this without the arbiter's lock and only asks again when it moved, or after a
  // short time for the reasons that depend on the clock (windows, a competitor going idle).
  uint64_t generation() const { return gen_.load(std::memory_order_acquire); }

  Value stats();
  static bool window_allows(const QosIntervalConfig& w, uint64_t epoch_us, uint64_t wall_us, uint64_t round);

 private:
  struct Tenant {
    QosTenantConfig cfg;
    std::vector<int> devices;
    bool registered = false;
    double vtime = 0;
    uint64_t outstanding_bytes = 0;
    int inflight_ctas = 0;           // most CTAs any launch in flight uses per GPU (a tenant's launches run one after another)
    uint64_t deferred_residency = 0;
    uint64_t last_active_us = 0;
    uint64_t waiting_since_us = 0;   // 0: nothing waiting
    uint64_t round = 0;
    uint64_t admitted = 0, deferred_window = 0, deferred_backlog = 0, deferred_fair = 0;
    uint64_t bytes_admitted = 0;
  };
  Tenant& tenant(uint32_t id);
  bool shares_device(const Tenant& a, const Tenant& b) const;
  bool is_contender(const Tenant& other, uint64_t now_us) const;

  void bump() { gen_.fetch_add(1, std::memory_order_acq_rel); }

  std::mutex mu_;
  std::atomic<uint64_t> gen_{1};
  bool enabled_ = true;
  std::map<uint32_t, Tenant> tenants_;
  uint64_t epoch_us_ = 0;
  std::map<uint32_t, QosIntervalConfig> schedule_;
  int cta_budget_ = 64;
  uint64_t max_outstanding_ = 64ull << 20;
  uint64_t active_window_us_ = 5000;   // a tenant counts as active this long after its last request
  int sm_limit_ = 148;                 // CTAs of waiting-on-each-other kernels that may be in flight per GPU (0 = unchecked)
};

}  // namespace mccs
