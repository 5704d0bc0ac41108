#include "qos.h"

#include <algorithm>
#include <cmath>

namespace mccs {

QosArbiter::QosArbiter() {}

void QosArbiter::configure(const Config& cfg) {
  std::lock_guard<std::mutex> g(mu_);
  epoch_us_ = cfg.qos_epoch_us;
  schedule_ = cfg.qos_schedule;
  cta_budget_ = cfg.qos_cta_budget > 0 ? cfg.qos_cta_budget : 64;
  max_outstanding_ = cfg.qos_max_outstanding_bytes;
  active_window_us_ = cfg.qos_active_window_us;
  sm_limit_ = cfg.qos_sm_limit;
  for (const auto& kv : cfg.qos_tenants) tenants_[kv.first].cfg = kv.second;
  bump();
}

QosArbiter::Tenant& QosArbiter::tenant(uint32_t id) { return tenants_[id]; }

void QosArbiter::set_tenant(uint32_t id, const QosTenantConfig& t) {
  std::lock_guard<std::mutex> g(mu_);
  tenants_[id].cfg = t;
  bump();
}

void QosArbiter::set_schedule(uint64_t epoch_us, const std::map<uint32_t, QosIntervalConfig>& schedule) {
  std::lock_guard<std::mutex> g(mu_);
  epoch_us_ = epoch_us;
  schedule_ = schedule;
  bump();
}

void QosArbiter::tenant_register(uint32_t id, const std::vector<int>& devices) {
  std::lock_guard<std::mutex> g(mu_);
  Tenant& t = tenant(id);
  t.devices = devices;
  t.registered = true;
  // A newcomer starts at the current front of the virtual clock: no credit for the past.
  double vmin = -1;
  for (const auto& kv : tenants_)
    if (kv.second.registered && kv.first != id) vmin = vmin < 0 ? kv.second.vtime : std::min(vmin, kv.second.vtime);
  if (vmin > t.vtime) t.vtime = vmin;
}

void QosArbiter::tenant_unregister(uint32_t id) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = tenants_.find(id);
  if (it == tenants_.end()) return;
  it->second.registered = false;
  it->second.outstanding_bytes = 0;
  it->second.inflight_ctas = 0;
  it->second.waiting_since_us = 0;
  it->second.devices.clear();
  bump();
}

bool QosArbiter::shares_device(const Tenant& a, const Tenant& b) const {
  for (int d : a.devices)
    if (std::find(b.devices.begin(), b.devices.end(), d) != b.devices.end()) return true;
  return false;
}

bool QosArbiter::is_contender(const Tenant& other, uint64_t now_us) const {
  if (!other.registered) return false;
  if (other.waiting_since_us || other.outstanding_bytes) return true;
  return other.last_active_us && now_us - other.last_active_us <= active_window_us_;
}

int QosArbiter::contenders(uint32_t id, uint64_t now_us) {
  std::lock_guard<std::mutex> g(mu_);
  const Tenant& me = tenant(id);
  int n = 0;
  for (const auto& kv : tenants_)
    if (kv.first != id && is_contender(kv.second, now_us) && shares_device(me, kv.second)) n++;
  return n;
}

int QosArbiter::cta_cap(uint32_t id, uint64_t now_us) {
  std::lock_guard<std::mutex> g(mu_);
  if (!enabled_) return 0;
  Tenant& me = tenant(id);
  if (me.cfg.cta_quota > 0) return me.cfg.cta_quota;
  double total = me.cfg.weight;
  int others = 0;
  for (const auto& kv : tenants_) {
    if (kv.first == id || !is_contender(kv.second, now_us) || !shares_device(me, kv.second)) continue;
    total += kv.second.cfg.weight;
    others++;
  }
  if (!others) return 0;
  int cap = (int)std::floor(cta_budget_ * me.cfg.weight / total);
  return std::max(1, cap);
}

uint64_t QosArbiter::slice_bytes(uint32_t id, uint64_t now_us) {
  std::lock_guard<std::mutex> g(mu_);
  if (!enabled_) return 0;
  const Tenant& me = tenant(id);
  for (const auto& kv : tenants_)
    if (kv.first != id && is_contender(kv.second, now_us) && shares_device(me, kv.second))
      return std::max<uint64_t>(max_outstanding_ / 2, 1u << 20);
  return 0;
}

int QosArbiter::stream_priority(uint32_t id) {
  std::lock_guard<std::mutex> g(mu_);
  return tenant(id).cfg.priority > 0 ? 1 : 0;
}

bool QosArbiter::window_allows(const QosIntervalConfig& w, uint64_t epoch_us, uint64_t wall_us, uint64_t round) {
  if (epoch_us == 0) return true;
  // enforce_step gates which rounds are subject to the schedule
  // (src/mccs/src/transport/net/agent.rs:514-535).
  if (w.enforce_step > 0 && round % (uint64_t)w.enforce_step != 0) return true;
  const uint64_t t = wall_us % epoch_us;
  bool inside = false;
  for (const auto& iv : w.intervals)
    if (t >= iv.first && t < iv.second) { inside = true; break; }
  return w.allow ? inside : !inside;
}

void QosArbiter::note_waiting(uint32_t id, uint64_t now_us) {
  std::lock_guard<std::mutex> g(mu_);
  Tenant& t = tenant(id);
  t.last_active_us = now_us;
  if (!t.waiting_since_us) t.waiting_since_us = now_us ? now_us : 1;
}

QosDecision QosArbiter::admit(uint32_t id, uint64_t bytes, uint64_t now_us, uint64_t wall_us, int ctas) {
  std::lock_guard<std::mutex> g(mu_);
  Tenant& me = tenant(id);
  me.last_active_us = now_us;
  if (!me.waiting_since_us) me.waiting_since_us = now_us ? now_us : 1;
  // Residency comes first and holds even with the arbiter switched off: it is what keeps
  // kernels that wait for each other from starving each other of SMs.
  if (sm_limit_ > 0 && ctas > 0) {
    int resident = 0;
    for (const auto& kv : tenants_)
      if (kv.first != id && kv.second.outstanding_bytes > 0 && shares_device(me, kv.second)) resident += kv.second.inflight_ctas;
    // Launches of one tenant run one after another: only a launch that needs more CTAs
    // than the tenant already has in flight adds to what must be resident.
    const bool grows = me.outstanding_bytes == 0 || ctas > me.inflight_ctas;
    if (grows && resident > 0 && resident + ctas > sm_limit_) {
      me.deferred_residency++;
      return kQosDeferResidency;
    }
  }
  auto grant = [&]() {
    me.vtime += (double)bytes / me.cfg.weight;
    me.outstanding_bytes += bytes;
    me.inflight_ctas = std::max(me.inflight_ctas, ctas);
    me.waiting_since_us = 0;
    me.round++;
    me.admitted++;
    me.bytes_admitted += bytes;
    bump();   // a waiter that was admitted no longer holds the others back
    return kQosAdmit;
  };
  if (!enabled_) return grant();

  auto w = schedule_.find(id);
  if (w != schedule_.end() && !window_allows(w->second, epoch_us_, wall_us, me.round)) {
    me.deferred_window++;
    return kQosDeferWindow;
  }

  // Who competes with this tenant right now?
  double vmin_waiting = -1;
  int others = 0;
  for (auto& kv : tenants_) {
    if (kv.first == id || !is_contender(kv.second, now_us) || !shares_device(me, kv.second)) continue;
    others++;
    if (kv.second.waiting_since_us)
      vmin_waiting = vmin_waiting < 0 ? kv.second.vtime : std::min(vmin_waiting, kv.second.vtime);
  }
  if (!others) {
    // Work conserving: alone on its GPUs a tenant is never held back. Keep its
    // virtual clock from running ahead so that it gets no penalty later.
    return grant();
  }
  // Bound the work a tenant may queue on the GPUs ahead of its competitors.
  if (me.outstanding_bytes > 0 && me.outstanding_bytes + bytes > max_outstanding_) {
    me.deferred_backlog++;
    return kQosDeferBacklog;
  }
  // Weighted fair queueing: a tenant that is ahead of a waiting competitor by more
  // than one request's worth of virtual time yields.
  if (vmin_waiting >= 0) {
    const double slack = (double)bytes / me.cfg.weight;
    if (me.vtime > vmin_waiting + slack) {
      me.deferred_fair++;
      return kQosDeferFairness;
    }
  }
  return grant();
}

void QosArbiter::complete(uint32_t id, uint64_t bytes) {
  std::lock_guard<std::mutex> g(mu_);
  Tenant& t = tenant(id);
  t.outstanding_bytes = t.outstanding_bytes > bytes ? t.outstanding_bytes - bytes : 0;
  if (t.outstanding_bytes == 0) t.inflight_ctas = 0;
  bump();
}

Value QosArbiter::stats() {
  std::lock_guard<std::mutex> g(mu_);
  Value out = Value::object();
  out.set("enabled", enabled_);
  out.set("epoch_microsecs", (int64_t)epoch_us_);
  out.set("cta_budget", cta_budget_);
  Value ts = Value::object();
  for (const auto& kv : tenants_) {
    const Tenant& t = kv.second;
    Value v = Value::object();
    v.set("weight", t.cfg.weight);
    v.set("priority", t.cfg.priority);
    v.set("registered", t.registered);
    v.set("admitted", (int64_t)t.admitted);
    v.set("bytes_admitted", (int64_t)t.bytes_admitted);
    v.set("deferred_window", (int64_t)t.deferred_window);
    v.set("deferred_backlog", (int64_t)t.deferred_backlog);
    v.set("deferred_fairness", (int64_t)t.deferred_fair);
    v.set("deferred_residency", (int64_t)t.deferred_residency);
    v.set("inflight_ctas", t.inflight_ctas);
    v.set("outstanding_bytes", (int64_t)t.outstanding_bytes);
    v.set("vtime", t.vtime);
    ts.set(std::to_string(kv.first), v);
  }
  out.set("tenants", ts);
  return out;
}

}  // namespace mccs
