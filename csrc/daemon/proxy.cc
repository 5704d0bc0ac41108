// Data path of the daemon: the per-GPU proxy engine.
//
// For every rank that lives on its device the proxy (1) takes work requests from
// the client's shared-memory ring, (2) posts them into the communicator's
// rendezvous slot for that collective, (3) once every rank has posted, one proxy
// plans the collective for all ranks (variant, CTAs, slices, barrier epochs, NVLS
// mappings), (4) asks the QoS arbiter for admission, slice by slice, (5) launches
// the kernel on the rank's backend stream between the client's "submitted" event
// and the backend's "done" event, and (6) completes the request.
//
// Reference counterparts: check_daemon_command / schedule_all_reduce /
// launch_scheduled_and_record (src/mccs/src/proxy/engine.rs:926-1066,1170-1275) and
// the planner in src/mccs/src/proxy/plan.rs. The reference's per-rank proxies never
// meet on the host: each uploads work to its kernel's FIFO and the kernels find each
// other through connection FIFOs set up at communicator creation. Here the host-side
// meeting is what lets one plan (and one reconfiguration point) hold for all ranks.
#include <string.h>

#include <algorithm>

#include <nvtx3/nvToolsExt.h>   // header-only; ranges cost a pointer check unless a profiler is attached

#include "../common/log.h"
#include "daemon.h"

namespace mccs {

namespace {
// NVTX range for a timeline profiler: planning and every launch show up on the proxy
// thread's row, named after the kernel variant.
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
};
}  // namespace

// NVTX fills its function table on first use, from whichever thread gets there first and
// without synchronisation; doing it once before the proxy threads exist keeps that
// initialisation single-threaded.
void proxy_tracing_init() {
  nvtxRangePushA("mccs init");
  nvtxRangePop();
}

void ProxyEngine::on_start() {
  daemon_->backend()->set_device(device_);
  started_.store(true);
}

void ProxyEngine::add_rank(RankState* rs) {
  std::lock_guard<std::mutex> g(mu_);
  ranks_.push_back(rs);
  version_.fetch_add(1);
}

void ProxyEngine::remove_rank(RankState* rs) {
  uint64_t v;
  {
    std::lock_guard<std::mutex> g(mu_);
    ranks_.erase(std::remove(ranks_.begin(), ranks_.end(), rs), ranks_.end());
    v = version_.fetch_add(1) + 1;
  }
  // Wait until the proxy thread has adopted the new list (it may be mid-iteration).
  if (!started_.load()) return;
  for (int i = 0; i < 20000 && seen_version_.load(std::memory_order_acquire) < v; i++) {
    struct timespec ts = {0, 100000};
    nanosleep(&ts, nullptr);
  }
}

Progress ProxyEngine::progress() {
  passes_.fetch_add(1, std::memory_order_acq_rel);
  if (seen_version_.load(std::memory_order_relaxed) != version_.load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> g(mu_);
    local_ = ranks_;
    seen_version_.store(version_.load(), std::memory_order_release);
  }
  bool any = false;
  spins_++;
  for (RankState* rs : local_) {
    if (rs->gone.load(std::memory_order_relaxed)) continue;
    any |= intake(*rs);
    any |= advance(*rs);
    if ((spins_ & 0x3f) == 0 || any) housekeeping(*rs);
  }
  return any ? Progress::kProgressed : Progress::kIdle;
}

// ---------------------------------------------------------------------------
// (1)+(2): request intake and posting
// ---------------------------------------------------------------------------
bool ProxyEngine::intake(RankState& rs) {
  bool any = false;
  if (rs.have_pending_wc) {
    if (!rs.cq.try_push(&rs.pending_wc)) return false;
    rs.have_pending_wc = false;
    any = true;
  }
  // The reference drains at most 32 requests per visit (daemon/engine.rs:274-435).
  for (int i = 0; i < 32; i++) {
    if (!rs.have_pending_wr) {
      if (!rs.wq.try_pop(&rs.pending_wr)) break;
      rs.have_pending_wr = true;
    }
    if (rs.comm->state.load(std::memory_order_acquire) == kCommError) {
      // A failed communicator takes no new work: answer in order, after whatever
      // was posted before the failure has been completed by advance().
      if (rs.next_launch_seq != rs.next_post_seq || rs.have_pending_wc) break;
      proto::WorkCompletion wc;
      memset(&wc, 0, sizeof wc);
      wc.kind = rs.pending_wr.kind;
      int err = rs.comm->async_error.load();
      wc.status = err ? err : proto::kErrPeerLost;
      wc.user_seq = rs.pending_wr.user_seq;
      LOG_WARN("comm %u rank %d: request %llu arrived after the communicator stopped taking work (status %d)", rs.comm->id,
               rs.rank, (unsigned long long)wc.user_seq, wc.status);
      if (rs.comm->client_launch) {
        if (!publish_plan_error(rs, wc.user_seq, wc.status)) break;
      } else if (rs.pending_wr.sync_slot && rs.dp_status) {
        signal_done(rs, rs.pending_wr.user_seq, wc.status);
        if (rs.dp_status->first_error == 0) rs.dp_status->first_error = wc.status;
        __atomic_store_n(&rs.dp_status->completed, rs.dp_status->completed + 1, __ATOMIC_RELEASE);
      } else if (!rs.cq.try_push(&wc)) { rs.pending_wc = wc; rs.have_pending_wc = true; }
      rs.have_pending_wr = false;
      any = true;
      continue;
    }
    if (!post(rs, rs.pending_wr)) break;
    rs.have_pending_wr = false;
    any = true;
  }
  return any;
}

bool ProxyEngine::post(RankState& rs, const proto::WorkRequest& wr) {
  Communicator& c = *rs.comm;
  const uint64_t seq = rs.next_post_seq;
  CollSlot& s = c.slot(seq);
  if (s.seq.load(std::memory_order_acquire) != seq) return false;   // slot still busy with seq - kCollSlots

  CollOp& op = s.ops[rs.rank];
  op = CollOp();
  op.kind = (int)wr.kind;
  op.dtype = (int)wr.dtype;
  op.op = (int)wr.op;
  op.count = wr.count;
  op.scale = wr.scale;
  op.variant_req = (int)wr.variant;
  op.user_seq = wr.user_seq;
  op.sync_slot = wr.sync_slot;
  op.sync_value = wr.sync_value;
  op.send_mem = wr.send_mem; op.send_off = wr.send_off;
  op.recv_mem = wr.recv_mem; op.recv_off = wr.recv_off;
  op.t_post_us = monotonic_us();
  int status = proto::kOk;
  if (op.kind < 0 || op.kind >= kNumCollKinds) status = proto::kErrInvalidArgument;
  else if (kind_reduces(op.kind) && (op.dtype < 0 || op.dtype >= kNumDataTypes || op.op < 0 || op.op >= kNumRedOps))
    status = proto::kErrInvalidArgument;
  else if (op.variant_req < 0 || op.variant_req >= kNumVariants) status = proto::kErrInvalidArgument;
  // Sizes come from another process: keep count * element size * ranks far from wrapping.
  else if (op.count > (1ull << 44)) status = proto::kErrInvalidArgument;
  if (status == proto::kOk) {
    const uint64_t esz = kind_reduces(op.kind) ? (uint64_t)dtype_size(op.dtype) : 1;
    const uint64_t send_bytes = send_units(op.kind, op.count, c.nranks) * esz;
    const uint64_t recv_bytes = recv_units(op.kind, op.count, c.nranks) * esz;
    int sdev = -1, rdev = -1;
    if (!daemon_->translate(rs.session_id, op.send_mem, op.send_off, send_bytes, &op.send_va, &sdev)) {
      status = proto::kErrNotFound;
    } else if (!daemon_->translate(rs.session_id, op.recv_mem, op.recv_off, recv_bytes, &op.recv_va, &rdev)) {
      daemon_->release_mem_ref(op.send_mem);
      status = proto::kErrNotFound;
    } else {
      op.holds_refs = true;
    }
    if (status == proto::kOk) {
      // Both buffers on the rank's own device, and elements naturally aligned: the kernels
      // load and store whole elements, and a misaligned access is a device fault, not an
      // error code.
      if (sdev != rs.device || rdev != rs.device) status = proto::kErrInvalidArgument;
      else if (((op.send_va | op.recv_va) & (esz - 1)) != 0) status = proto::kErrInvalidArgument;
    }
  }
  if (status != proto::kOk && op.holds_refs) {
    op.holds_refs = false;
    daemon_->release_mem_ref(op.send_mem);
    daemon_->release_mem_ref(op.recv_mem);
  }
  op.user_event = daemon_->lookup_stream_event(rs.session_id, wr.stream_id);
  op.status = status;
  op.valid = status == proto::kOk;
  rs.next_post_seq++;
  if (s.arrived.fetch_add(1, std::memory_order_acq_rel) + 1 == c.nranks) {
    s.t_collected_us.store(op.t_post_us, std::memory_order_relaxed);
    s.state.store(kSlotCollected, std::memory_order_release);
  }
  return true;
}

// Fused launches: a collective whose followers are still arriving (some rank has posted the
// next request, not all have) is worth a short wait, because only requests that every rank has
// posted can join its launch. Ranks post the members of a group microseconds apart; the wait
// ends as soon as the next slots are complete or untouched, and after 50 us in any case.
bool ProxyEngine::followers_still_arriving(Communicator& c, CollSlot& s, uint64_t seq) {
  const Config& cfg = daemon_->config();
  if (cfg.fuse_allreduce <= 1 || s.ops[0].kind != kAllReduce) return false;
  if (monotonic_us() - s.t_collected_us.load(std::memory_order_relaxed) > 50) return false;
  const int limit = std::min(cfg.fuse_allreduce, kMaxBatch);
  for (int k = 1; k < limit; k++) {
    CollSlot& m = c.slot(seq + (uint64_t)k);
    if (m.seq.load(std::memory_order_acquire) != seq + (uint64_t)k) return false;   // still serving an older collective
    const int arrived = m.arrived.load(std::memory_order_acquire);
    if (arrived == 0) return false;              // nobody has posted a follower: nothing to wait for
    if (arrived < c.nranks) return true;         // some have, not all: wait for the rest
  }
  return false;
}

// ---------------------------------------------------------------------------
// (3): planning, done by whichever proxy first sees the slot complete
// ---------------------------------------------------------------------------
int ProxyEngine::ensure_mc(Communicator& c, CollSlot& s, bool for_recv, uint64_t* out_va) {
  std::vector<uint64_t> key;
  for (int r = 0; r < c.nranks; r++) key.push_back(for_recv ? s.ops[r].recv_mem : s.ops[r].send_mem);
  const uint64_t off = for_recv ? s.ops[0].recv_off : s.ops[0].send_off;
  const uint64_t esz = kind_reduces(s.ops[0].kind) ? (uint64_t)dtype_size(s.ops[0].dtype) : 1;
  const uint64_t bytes = (for_recv ? recv_units(s.ops[0].kind, s.ops[0].count, c.nranks)
                                   : send_units(s.ops[0].kind, s.ops[0].count, c.nranks)) * esz;
  std::lock_guard<std::mutex> g(c.mc_mu);
  auto it = c.mc_cache.find(key);
  if (it == c.mc_cache.end()) {
    std::shared_lock<std::shared_mutex> al(daemon_->alloc_mutex());
    std::vector<const Allocation*> allocs;
    for (uint64_t id : key) {
      const Allocation* a = daemon_->find_alloc_locked(id);
      if (!a) return proto::kErrNotFound;
      // only memory of the rank that named it may be bound (checked again here because a
      // region outlives the request that created it)
      const size_t r = allocs.size();
      if (!c.ranks[r] || a->owner_session != c.ranks[r]->session_id) return proto::kErrNotFound;
      allocs.push_back(a);
    }
    McRegion reg;
    int rc = daemon_->backend()->mc_create(allocs, &reg, c.client_launch);
    if (rc != proto::kOk) {
      // Remember the failure so that it is not retried on every collective.
      McRegion none;
      c.mc_cache[key] = none;
      return rc;
    }
    reg.id = ++c.next_mc_id;
    for (int r = 0; r < c.nranks; r++) reg.mems[r] = key[(size_t)r];
    LOG_INFO("comm %u: multicast region of %zu bytes bound for %d ranks", c.id, reg.size, c.nranks);
    it = c.mc_cache.emplace(key, reg).first;
  }
  const McRegion& reg = it->second;
  if (!reg.handle) return proto::kErrUnsupported;
  if (off + bytes > reg.size) return proto::kErrUnsupported;
  for (int r = 0; r < c.nranks; r++) out_va[r] = reg.va[r];
  (for_recv ? s.mc_recv_id : s.mc_send_id) = reg.id;
  return proto::kOk;
}

bool ProxyEngine::plan_slot(Communicator& c, CollSlot& s, uint64_t seq) {
  s.batch_len = 1;
  s.fused_kernel = false;
  s.batch_bytes = 0;
  auto fail = [&](int status) {
    s.status = status;
    s.state.store(kSlotFailed, std::memory_order_release);
    return false;
  };
  const CollOp& o0 = s.ops[0];
  for (int r = 0; r < c.nranks; r++)
    if (!s.ops[r].valid) return fail(s.ops[r].status ? s.ops[r].status : proto::kErrInvalidArgument);
  for (int r = 1; r < c.nranks; r++) {
    const CollOp& o = s.ops[r];
    if (o.kind != o0.kind || o.count != o0.count || (kind_reduces(o0.kind) && (o.dtype != o0.dtype || o.op != o0.op)))
      return fail(proto::kErrMismatch);
    // The multiplier of PreMulSum / SumPostDiv is one per collective (the kernels apply the
    // same factor to every source): ranks that pass different factors disagree.
    if (kind_reduces(o0.kind) && (o0.op == kPreMulSum || o0.op == kSumPostDiv) && o.scale != o0.scale)
      return fail(proto::kErrMismatch);
  }
  Backend* be = daemon_->backend();
  const bool host_backend = be->kind() == proto::kBackendHost;
  PlanInput in;
  in.kind = o0.kind;
  in.nranks = c.nranks;
  in.count = o0.count;
  in.dtype = kind_reduces(o0.kind) ? o0.dtype : kUint8;
  in.op = kind_reduces(o0.kind) ? o0.op : kSum;
  in.emulated = c.emulated;
  in.host_staged = c.host_staged;
  in.fifo_slot_bytes = c.fifo_slot_bytes;
  // Every block boundary the kernels compute from the count must be aligned as well.
  uint64_t bits = o0.kind == kAllGather ? o0.count : o0.kind == kReduceScatter ? o0.count * (uint64_t)dtype_size(o0.dtype) : 0;
  bool same_send_off = true, same_recv_off = true, all_vmm = !host_backend || be->nvls_supported();   // the host backend's emulated multicast binds any of its allocations
  int req = o0.variant_req;
  for (int r = 0; r < c.nranks; r++) {
    const CollOp& o = s.ops[r];
    bits |= o.send_va | o.recv_va;
    if (o0.kind == kAllReduce) in.in_place |= o.send_va == o.recv_va;
    else if (o0.kind == kReduceScatter) in.in_place |= o.recv_va == o.send_va + (uint64_t)r * o.count * (uint64_t)dtype_size(o.dtype);
    else in.in_place |= o.send_va == o.recv_va + (uint64_t)r * o.count;
    same_send_off &= o.send_off == o0.send_off;
    same_recv_off &= o.recv_off == o0.recv_off;
    if (o.variant_req != req) req = kAuto;
  }
  in.aligned16 = (bits & 15u) == 0;
  in.carried_variants = c.conns.carried_variants();
  in.p2p_possible = c.conns.carries(kArTwoShot);
  in.nvls_possible = c.conns.carries(kArNvlsTwo) && !c.emulated &&
                     (!c.client_launch || daemon_->config().client_nvls) &&
                     all_vmm && c.nranks >= 2 &&
                     (o0.kind == kReduceScatter ? same_send_off   // only the inputs are read through the switch
                                                : same_recv_off && (same_send_off || o0.kind == kAllGather));
  {
    std::lock_guard<std::mutex> g(c.cfg_mu);
    const int cfg_variant = o0.kind == kAllReduce ? c.ar_variant : o0.kind == kAllGather ? c.ag_variant : (int)kAuto;
    in.requested_variant = req != kAuto ? req : cfg_variant;
    in.requested_ctas = c.ctas_override;
    in.ring_channels = c.channel_count;
    // The ring order is frozen here, once for all ranks, so that a reconfiguration
    // arriving between two ranks' launches cannot split the collective.
    for (int ch = 0; ch < kMaxRingChannels; ch++) {
      const std::vector<int>& ring = c.rings[(size_t)ch % c.rings.size()];
      for (int i = 0; i < c.nranks; i++) s.ring[ch][i] = (int8_t)ring[(size_t)i];
    }
  }
  const uint64_t now = monotonic_us();
  in.cta_cap = daemon_->qos().cta_cap(c.id, now);

  Plan plan = daemon_->planner().plan(in);
  for (int attempt = 0; attempt < 3 && plan.status == proto::kOk; attempt++) {
    bool redo = false;
    if (plan.needs_mc_send && ensure_mc(c, s, false, s.mc_send) != proto::kOk) redo = true;
    if (!redo && plan.needs_mc_recv && ensure_mc(c, s, true, s.mc_recv) != proto::kOk) redo = true;
    if (redo) {
      in.nvls_possible = false;
      plan = daemon_->planner().plan(in);
      continue;
    }
    if (!be->variant_supported(plan.variant, in.dtype, in.op)) {
      if (in.requested_variant == plan.variant) in.requested_variant = kAuto;
      in.nvls_possible = false;
      Plan alt = daemon_->planner().plan(in);
      if (alt.variant == plan.variant) { plan.status = proto::kErrUnsupported; break; }
      plan = alt;
      continue;
    }
    break;
  }
  if (plan.status != proto::kOk) return fail(plan.status);
  if (!plan.note.empty()) LOG_DEBUG("comm %u seq %llu: %s", c.id, (unsigned long long)seq, plan.note.c_str());

  // Ring variants are limited by the FIFO space that exists per rank.
  if (variant_is_ring(plan.variant)) {
    const int fifo_channels = (int)(c.ranks[0]->fifo_bytes / (c.fifo_slot_bytes * kRingSlots));
    if (fifo_channels < 1) return fail(proto::kErrUnsupported);
    plan.dims.ctas = std::min(plan.dims.ctas, fifo_channels);
  }
  if (c.emulated && !host_backend) {
    int fit = be->max_group_ctas(plan.variant, in.dtype, in.op, plan.dims.threads, c.nranks);
    if (fit < 1) return fail(proto::kErrUnsupported);
    plan.dims.ctas = std::min(plan.dims.ctas, fit);
  }

  // Time slices (all-reduce through non-ring variants only: each slice is an
  // independent collective over a sub-range).
  s.nslices = 1;
  s.slice_count = o0.count;
  const uint64_t slice_bytes = daemon_->qos().slice_bytes(c.id, now);
  if (slice_bytes && o0.kind == kAllReduce && !variant_is_ring(plan.variant) && plan.bytes > slice_bytes &&
      plan.variant != kLocalCopy) {
    const uint64_t esz = (uint64_t)dtype_size(o0.dtype);
    uint64_t n = std::min<uint64_t>((plan.bytes + slice_bytes - 1) / slice_bytes, 64);
    uint64_t per = (o0.count + n - 1) / n;
    const uint64_t quantum = 256 / esz;   // keeps every slice start 256-byte aligned
    per = (per + quantum - 1) / quantum * quantum;
    s.slice_count = per;
    s.nslices = (int)((o0.count + per - 1) / per);
  }
  s.epoch_base = c.barrier_epoch;
  c.barrier_epoch += 2u * (uint32_t)s.nslices;
  s.ticket_base = c.ticket + 1;
  c.ticket += (uint64_t)s.nslices;
  if (variant_is_ring(plan.variant)) {
    const int esz = kind_reduces(o0.kind) ? dtype_size(o0.dtype) : 1;
    const uint64_t steps = ring_steps_per_channel(o0.kind, o0.count, esz, c.nranks, plan.dims.ctas, c.fifo_slot_bytes);
    for (int ch = 0; ch < kMaxRingChannels; ch++) s.ring_step_base[ch] = c.ring_steps[ch];
    for (int ch = 0; ch < plan.dims.ctas; ch++) c.ring_steps[ch] += steps;
  }
  s.plan = plan;
  s.status = proto::kOk;
  s.t_ready_us = now;
  s.admitted_slices.store(0, std::memory_order_relaxed);
  s.group_launch.store(0, std::memory_order_relaxed);
  c.planned.fetch_add(1);
  c.last_variant.store((uint32_t)plan.variant);
  c.last_ctas.store((uint32_t)plan.dims.ctas);
  daemon_->qos().note_waiting(c.id, now);
  s.batch_bytes = plan.bytes;
  extend_batch(c, s, seq, in, now);
  s.state.store(kSlotPlanned, std::memory_order_release);
  return true;
}

// ---------------------------------------------------------------------------
// (3b): fused launches. The reference chains consecutive queued AllReduce tasks with
// equal type and operator into one kernel (src/mccs/src/proxy/plan.rs:122-141). Here the
// proxy that plans a collective looks at the slots right behind it: every one that all
// ranks have already posted, that is an AllReduce of the same type and operator, and
// for which the planner picks the same two-shot variant becomes a follower of this
// slot. The decision is taken once, by one thread, before the head becomes visible as
// planned, so every rank launches the same batch.
// ---------------------------------------------------------------------------
// Do two byte ranges of the same allocation overlap?
static bool ranges_overlap(uint64_t mem_a, uint64_t off_a, uint64_t len_a, uint64_t mem_b, uint64_t off_b, uint64_t len_b) {
  return mem_a == mem_b && off_a < off_b + len_b && off_b < off_a + len_a;
}

// Members of a fused launch run between ONE pair of barriers, so a member must not
// depend on an earlier one: its buffers may share nothing with an earlier member's
// output, and its output nothing with an earlier member's input.
static bool independent_of(const CollSlot& earlier, const CollSlot& m, int nranks) {
  for (int r = 0; r < nranks; r++) {
    const CollOp& e = earlier.ops[r];
    const CollOp& o = m.ops[r];
    const uint64_t eb = e.count * (uint64_t)dtype_size(e.dtype), ob = o.count * (uint64_t)dtype_size(o.dtype);
    if (ranges_overlap(e.recv_mem, e.recv_off, eb, o.send_mem, o.send_off, ob) ||
        ranges_overlap(e.recv_mem, e.recv_off, eb, o.recv_mem, o.recv_off, ob) ||
        ranges_overlap(e.send_mem, e.send_off, eb, o.recv_mem, o.recv_off, ob))
      return false;
  }
  return true;
}

bool ProxyEngine::plan_member(Communicator& c, CollSlot& head, CollSlot& m, const PlanInput& head_in, Plan* out) {
  const CollOp& h0 = head.ops[0];
  const CollOp& o0 = m.ops[0];
  Backend* be = daemon_->backend();
  PlanInput in = head_in;
  in.count = o0.count;
  in.in_place = false;
  uint64_t bits = 0;
  bool same_send_off = true, same_recv_off = true;
  int req = o0.variant_req;
  for (int r = 0; r < c.nranks; r++) {
    const CollOp& o = m.ops[r];
    if (!o.valid || o.kind != kAllReduce || o.count != o0.count || o.dtype != h0.dtype || o.op != h0.op ||
        o.scale != h0.scale)
      return false;   // left to the ordinary path, which also reports mismatches
    bits |= o.send_va | o.recv_va;
    in.in_place |= o.send_va == o.recv_va;
    same_send_off &= o.send_off == o0.send_off;
    same_recv_off &= o.recv_off == o0.recv_off;
    if (o.variant_req != req) req = kAuto;
  }
  in.aligned16 = (bits & 15u) == 0;
  in.carried_variants = head_in.carried_variants;
  in.nvls_possible = c.conns.carries(kArNvlsTwo) && !c.emulated &&
                     be->kind() != proto::kBackendHost && same_recv_off && same_send_off && c.nranks >= 2;
  {
    std::lock_guard<std::mutex> g(c.cfg_mu);
    in.requested_variant = req != kAuto ? req : c.ar_variant;
    in.requested_ctas = c.ctas_override;
  }
  Plan p = daemon_->planner().plan(in);
  if (p.status != proto::kOk || p.variant != head.plan.variant) return false;
  if (p.needs_mc_send && ensure_mc(c, m, false, m.mc_send) != proto::kOk) return false;
  if (p.needs_mc_recv && ensure_mc(c, m, true, m.mc_recv) != proto::kOk) return false;
  *out = p;
  return true;
}

void ProxyEngine::extend_batch(Communicator& c, CollSlot& head, uint64_t seq, const PlanInput& head_in, uint64_t now) {
  const int limit = std::min(daemon_->config().fuse_allreduce, kMaxBatch);
  const bool single = daemon_->config().single_through_fused;
  if (limit <= 1 && !(single && !c.client_launch)) return;   // a lone collective through the fused kernel is a daemon-launch experiment
  Backend* be = daemon_->backend();
  const CollOp& h0 = head.ops[0];
  if (h0.kind != kAllReduce || head.nslices != 1) return;
  if (head.plan.variant != kArTwoShot && head.plan.variant != kArNvlsTwo) return;
  if (!be->batch_supported(head.plan.variant, h0.dtype, h0.op)) return;
  int fit = kMaxCtas;
  if (c.emulated && be->kind() != proto::kBackendHost) {
    fit = be->max_group_batch_ctas(head.plan.variant, h0.dtype, h0.op, head.plan.dims.threads, c.nranks);
    if (fit < 1) return;
  }
  const uint64_t slice_bytes = daemon_->qos().slice_bytes(c.id, now);
  int len = 1;
  int ctas = head.plan.dims.ctas;
  uint64_t bytes = head.plan.bytes;
  while (len < limit) {
    const uint64_t mseq = seq + (uint64_t)len;
    CollSlot& m = c.slot(mseq);
    if (m.seq.load(std::memory_order_acquire) != mseq) break;
    int expect = kSlotCollected;
    if (!m.state.compare_exchange_strong(expect, kSlotPlanning, std::memory_order_acq_rel)) break;
    Plan mp;
    bool independent = true;
    for (int e = 0; e < len && independent; e++)
      independent = independent_of(e == 0 ? head : c.slot(seq + (uint64_t)e), m, c.nranks);
    if (!independent || !plan_member(c, head, m, head_in, &mp) || (slice_bytes && mp.bytes > slice_bytes)) {
      m.state.store(kSlotCollected, std::memory_order_release);   // planned on its own later
      break;
    }
    m.plan = mp;
    m.status = proto::kOk;
    m.nslices = 1;
    m.slice_count = m.ops[0].count;
    m.batch_len = 0;
    m.batch_bytes = 0;
    m.t_ready_us = now;
    m.admitted_slices.store(0, std::memory_order_relaxed);
    m.group_launch.store(0, std::memory_order_relaxed);
    ctas = std::max(ctas, mp.dims.ctas);
    bytes += mp.bytes;
    c.planned.fetch_add(1);
    m.state.store(kSlotPlanned, std::memory_order_release);
    len++;
  }
  if (len == 1 && !single) return;
  head.plan.dims.ctas = std::min(ctas, fit);
  head.batch_len = len;
  head.fused_kernel = true;
  head.batch_bytes = bytes;
  c.fused_launches.fetch_add(1);
  c.fused_members.fetch_add((uint64_t)len);
}

void ProxyEngine::fill_batch_args(Communicator& c, CollSlot& head, uint64_t seq, int rank, BatchArgs* out) {
  BatchArgs& b = *out;
  memset(&b, 0, sizeof b);
  fill_args(c, head, rank, 0, &b.base);
  b.nops = head.batch_len;
  for (int k = 0; k < head.batch_len; k++) {
    CollSlot& m = k == 0 ? head : c.slot(seq + (uint64_t)k);
    b.count[k] = m.ops[0].count;
    for (int r = 0; r < c.nranks; r++) {
      b.send[k][r] = (const void*)m.ops[r].send_va;
      b.recv[k][r] = (void*)m.ops[r].recv_va;
    }
    if (head.plan.needs_mc_send) b.mc_send[k] = (const void*)(m.mc_send[rank] + m.ops[rank].send_off);
    if (head.plan.needs_mc_recv) b.mc_recv[k] = (void*)(m.mc_recv[rank] + m.ops[rank].recv_off);
  }
  const Config& cfg = daemon_->config();
  // Is every rank's launch held back by the host until all clients have arrived? Only
  // then do all inputs exist (and may all outputs be overwritten) when a kernel starts.
  bool all_gated = true;
  for (int k = 0; k < head.batch_len; k++) {
    CollSlot& m = k == 0 ? head : c.slot(seq + (uint64_t)k);
    for (int r = 0; r < c.nranks; r++) all_gated &= c.ranks[(size_t)r]->sync.host != nullptr && m.ops[r].sync_slot != 0;
  }
  if (cfg.skip_start_barrier && all_gated) b.flags |= kBatchSkipStartBarrier;
  if (cfg.kernel_writes_done && !c.host_staged) {
    const bool group = c.emulated || daemon_->backend()->kind() == proto::kBackendHost;
    for (int r = 0; r < c.nranks; r++) {
      if (!group && r != rank) continue;
      RankState& rr = *c.ranks[(size_t)r];
      if (!rr.sync.host || !head.ops[r].sync_slot || !rr.pad) continue;
      b.done_ptr[r] = (uint64_t*)(rr.sync.dev_addr + 8 * proto::kSyncDoneSlot);
      b.done_value[r] = last_member_user_seq(c, head, seq, r);
      b.done_counter[r] = &rr.pad->pad_[kPadBatchCounter];
    }
  }
}

bool ProxyEngine::batch_clients_ready(Communicator& c, CollSlot& head, uint64_t seq, int self_rank) {
  for (int k = 0; k < head.batch_len; k++)
    if (!clients_ready(c, k == 0 ? head : c.slot(seq + (uint64_t)k), self_rank)) return false;
  return true;
}

uint64_t ProxyEngine::last_member_user_seq(Communicator& c, CollSlot& head, uint64_t seq, int rank) {
  return c.slot(seq + (uint64_t)head.batch_len - 1).ops[rank].user_seq;
}

// ---------------------------------------------------------------------------
// (4): admission
// ---------------------------------------------------------------------------
bool ProxyEngine::admit_slice(Communicator& c, CollSlot& s, int slice) {
  if (s.admitted_slices.load(std::memory_order_acquire) > slice) return true;
  std::lock_guard<std::mutex> g(c.admit_mu);
  if (s.admitted_slices.load(std::memory_order_acquire) > slice) return true;
  const uint64_t bytes = s.batch_len > 1 ? s.batch_bytes : s.nslices == 1 ? s.plan.bytes : s.plan.bytes / (uint64_t)s.nslices;
  // CTAs per GPU: one launch per rank and GPU, or every rank's CTAs on the one GPU.
  const int ctas = s.plan.dims.ctas * (c.emulated ? c.nranks : 1);
  // A request that was told to wait is not put to the arbiter again (a lock shared by the
  // proxies of all GPUs) until the arbiter's state moved, or a short time passed for the
  // reasons that follow the clock: 20 us for a closed window, 200 us otherwise (a competitor
  // that stopped issuing work only stops counting after its activity window).
  QosArbiter& qos = daemon_->qos();
  const uint64_t now = monotonic_us();
  const uint64_t gen = qos.generation();
  if (s.defer_slice == slice && s.defer_gen == gen && now < s.defer_retry_us) return false;
  QosDecision d = qos.admit(c.id, bytes, now, wall_us(), ctas);
  if (d != kQosAdmit) {
    s.defer_slice = slice;
    s.defer_gen = gen;
    s.defer_retry_us = now + (d == kQosDeferWindow ? 20 : 200);
    return false;
  }
  s.defer_slice = -1;
  s.admitted_slices.store(slice + 1, std::memory_order_release);
  return true;
}

// ---------------------------------------------------------------------------
// (5): launch
// ---------------------------------------------------------------------------
void ProxyEngine::fill_args(Communicator& c, CollSlot& s, int rank, int slice, CollArgs* out) {
  CollArgs& a = *out;
  memset(&a, 0, sizeof a);
  const CollOp& o0 = s.ops[0];
  const bool group = c.emulated || daemon_->backend()->kind() == proto::kBackendHost;
  a.rank = rank;
  a.nranks = c.nranks;
  a.emulated = group ? 1 : 0;
  a.dtype = kind_reduces(o0.kind) ? o0.dtype : kUint8;
  a.op = kind_reduces(o0.kind) ? o0.op : kSum;
  a.variant = s.plan.variant;
  const uint64_t esz = kind_reduces(o0.kind) ? (uint64_t)dtype_size(o0.dtype) : 1;
  uint64_t first = 0, count = o0.count;
  if (s.nslices > 1) {
    first = (uint64_t)slice * s.slice_count;
    count = std::min<uint64_t>(s.slice_count, o0.count - first);
  }
  const uint64_t off = first * esz;
  a.count = count;
  a.seq = s.ticket_base + (uint64_t)slice;
  a.scale = o0.op == kSumPostDiv ? 1.0f / (float)c.nranks : o0.scale;
  a.epoch = s.epoch_base + 2u * (uint32_t)slice;
  a.timeout_ns = daemon_->timeout_ns();
  a.trace = daemon_->tracer().enabled() ? 1 : 0;
  for (int r = 0; r < c.nranks; r++) {
    a.send[r] = (const void*)(s.ops[r].send_va + off);
    a.recv[r] = (void*)(s.ops[r].recv_va + off);
    a.pad[r] = c.ranks[(size_t)r]->pad;
    a.status[r] = c.ranks[(size_t)r]->status;
    a.fifo[r] = c.ranks[(size_t)r]->fifo;
  }
  if (s.plan.needs_mc_send) a.mc_send = (const void*)(s.mc_send[rank] + s.ops[rank].send_off + off);
  if (s.plan.needs_mc_recv) a.mc_recv = (void*)(s.mc_recv[rank] + s.ops[rank].recv_off + off);
  if (s.plan.variant == kArHybrid) {
    const Config& cfg = daemon_->config();
    const int nvls_ctas = std::min(cfg.hybrid_nvls_ctas, std::max(s.plan.dims.ctas - 1, 0));
    a.unroll_hint = (int32_t)(((uint32_t)nvls_ctas << 16) | (uint32_t)cfg.hybrid_nvls_permille);
  } else if (s.plan.variant == kArNvlsOne || s.plan.variant == kArNvlsTwo) {
    a.unroll_hint = daemon_->config().nvls_unroll;
  } else if (s.plan.variant == kAgPull || s.plan.variant == kAgPush || s.plan.variant == kArTwoShot) {
    a.unroll_hint = daemon_->config().pack_bytes;
  }
  a.fifo_slot_bytes = c.fifo_slot_bytes;
  memcpy(a.ring, s.ring, sizeof a.ring);
  for (int ch = 0; ch < kMaxRingChannels; ch++) a.ring_step_base[ch] = s.ring_step_base[ch];
}

bool ProxyEngine::launch_slices(RankState& rs, CollSlot& s, uint64_t seq) {
  Communicator& c = *rs.comm;
  Backend* be = daemon_->backend();
  const CollOp& op = s.ops[rs.rank];
  if (s.fused_kernel) {
    // One kernel for this slot and its followers.
    if (!admit_slice(c, s, 0)) return false;
    for (int k = 0; k < s.batch_len; k++)
      order_after_client(rs, (k == 0 ? s : c.slot(seq + (uint64_t)k)).ops[rs.rank], rs.stream);
    BatchArgs b;
    fill_batch_args(c, s, seq, rs.rank, &b);
    int rc = be->launch_batch(rs.device, b, s.plan.dims, rs.stream);
    if (rc != proto::kOk) {
      c.async_error.store(rc);
      c.state.store(kCommError);
    } else {
      if (rs.rank == 0) rs.inflight.push_back({b.base.seq, s.batch_bytes});
      rs.last_ticket.store(b.base.seq, std::memory_order_relaxed);
    }
    rs.next_slice = 1;
    // "done" values grow in submission order: the last member's covers the whole batch.
    if (rs.sync.host && op.sync_slot)
      be->stream_write_value64(rs.device, rs.stream, rs.sync.dev_addr + 8 * proto::kSyncDoneSlot,
                               last_member_user_seq(c, s, seq, rs.rank));
    else
      be->event_record(rs.device, rs.backend_event, rs.stream);
    return true;
  }
  while (rs.next_slice < s.nslices) {
    if (!admit_slice(c, s, rs.next_slice)) return false;
    if (rs.next_slice == 0) order_after_client(rs, op, rs.stream);
    CollArgs a;
    fill_args(c, s, rs.rank, rs.next_slice, &a);
    int rc = be->launch(rs.device, op.kind, a, s.plan.dims, rs.stream);
    if (rc != proto::kOk) {
      c.async_error.store(rc);
      c.state.store(kCommError);
      break;   // the request completes with the communicator's error; the client's stream is still released below
    }
    if (rs.rank == 0) {
      const uint64_t bytes = s.nslices == 1 ? s.plan.bytes : s.plan.bytes / (uint64_t)s.nslices;
      rs.inflight.push_back({a.seq, bytes});
    }
    rs.last_ticket.store(a.seq, std::memory_order_relaxed);
    rs.next_slice++;
  }
  if (rs.sync.host && op.sync_slot)
    be->stream_write_value64(rs.device, rs.stream, rs.sync.dev_addr + 8 * proto::kSyncDoneSlot, op.user_seq);
  else
    be->event_record(rs.device, rs.backend_event, rs.stream);
  (void)seq;
  return true;
}

// Mem-op mode: has every rank's stream reached this collective? Each client's stream
// writes a "submitted" value into its semaphore page (host memory) when the work queued
// before the collective is done; the proxies read those words with plain loads. Kernels
// are launched only once all inputs exist, so no kernel sits on SMs waiting for a peer
// whose application is still computing, and no backend stream ever blocks.
bool ProxyEngine::clients_ready(Communicator& c, CollSlot& s, int self_rank) {
  // An event-ordered rank (a client inside the daemon's process) blocks on the host until
  // its kernel is queued, so it is launched at once, as before; its kernel then waits
  // for the others on the device, within the usual bound.
  if (self_rank >= 0 && !(c.ranks[(size_t)self_rank]->sync.host && s.ops[self_rank].sync_slot)) return true;
  for (int r = 0; r < c.nranks; r++) {
    const CollOp& op = s.ops[r];
    const RankState& rr = *c.ranks[(size_t)r];
    if (!rr.sync.host || !op.sync_slot) continue;   // event-ordered client: the stream wait covers it
    const volatile uint64_t* sem = (const volatile uint64_t*)rr.sync.host + proto::kSyncFirstStreamSlot +
                                   (op.sync_slot - 1) % proto::kSyncMaxStreams;
    if ((int64_t)(*sem - op.sync_value) < 0) return false;
  }
  std::atomic_thread_fence(std::memory_order_acquire);
  return true;
}

// Makes `stream` wait for the work the client had queued before this request.
void ProxyEngine::order_after_client(RankState& rs, const CollOp& op, void* stream) {
  Backend* be = daemon_->backend();
  if (rs.sync.host && op.sync_slot) {
    // nothing to queue: clients_ready() has seen the "submitted" value already
  } else if (op.user_event) {
    be->stream_wait_event(rs.device, stream, op.user_event);
  }
}

// A request that ends without a launch must still release the client's stream, which
// (in mem-op mode) already waits for this request's "done" value.
void ProxyEngine::signal_done(RankState& rs, uint64_t user_seq, int status) {
  if (!rs.sync.host) return;
  // The error is published before the stream is released, so that a caller who waited for
  // this request finds it.
  if (status != proto::kOk && rs.dp_status && rs.dp_status->first_error == 0)
    __atomic_store_n(&rs.dp_status->first_error, status, __ATOMIC_RELEASE);
  Communicator& c = *rs.comm;
  void* stream = c.group_stream ? c.group_stream : rs.stream;
  daemon_->backend()->stream_write_value64(rs.device, stream, rs.sync.dev_addr + 8 * proto::kSyncDoneSlot, user_seq);
}

// Emulated communicators (all ranks on one GPU) and the host backend run every rank
// in one launch. Rank 0's proxy issues it; the other ranks wait for it.
bool ProxyEngine::launch_group(Communicator& c, CollSlot& s, uint64_t seq) {
  (void)seq;
  RankState& r0 = *c.ranks[0];
  Backend* be = daemon_->backend();
  if (s.fused_kernel) {
    if (!admit_slice(c, s, 0)) return false;
    for (int k = 0; k < s.batch_len; k++) {
      CollSlot& m = k == 0 ? s : c.slot(seq + (uint64_t)k);
      for (int r = 0; r < c.nranks; r++) order_after_client(*c.ranks[(size_t)r], m.ops[r], c.group_stream);
    }
    BatchArgs b;
    fill_batch_args(c, s, seq, 0, &b);
    int rc = be->launch_batch(r0.device, b, s.plan.dims, c.group_stream);
    if (rc != proto::kOk) {
      c.async_error.store(rc);
      c.state.store(kCommError);
    } else {
      r0.inflight.push_back({b.base.seq, s.batch_bytes});
      r0.last_ticket.store(b.base.seq, std::memory_order_relaxed);
    }
    r0.next_slice = 1;
    for (int r = 0; r < c.nranks; r++) {
      RankState& rr = *c.ranks[(size_t)r];
      if (rr.sync.host && s.ops[r].sync_slot)
        be->stream_write_value64(rr.device, c.group_stream, rr.sync.dev_addr + 8 * proto::kSyncDoneSlot,
                                 last_member_user_seq(c, s, seq, r));
      else
        be->event_record(rr.device, rr.backend_event, c.group_stream);
    }
    s.group_launch.store(2, std::memory_order_release);
    return true;
  }
  while (r0.next_slice < s.nslices) {
    if (!admit_slice(c, s, r0.next_slice)) return false;
    if (r0.next_slice == 0) {
      for (int r = 0; r < c.nranks; r++) order_after_client(*c.ranks[(size_t)r], s.ops[r], c.group_stream);
    }
    CollArgs a;
    fill_args(c, s, 0, r0.next_slice, &a);
    int rc = be->launch(r0.device, s.ops[0].kind, a, s.plan.dims, c.group_stream);
    if (rc != proto::kOk) {
      c.async_error.store(rc);
      c.state.store(kCommError);
      break;
    }
    const uint64_t bytes = s.nslices == 1 ? s.plan.bytes : s.plan.bytes / (uint64_t)s.nslices;
    r0.inflight.push_back({a.seq, bytes});
    r0.last_ticket.store(a.seq, std::memory_order_relaxed);
    r0.next_slice++;
  }
  for (int r = 0; r < c.nranks; r++) {
    RankState& rr = *c.ranks[(size_t)r];
    if (rr.sync.host && s.ops[r].sync_slot)
      be->stream_write_value64(rr.device, c.group_stream, rr.sync.dev_addr + 8 * proto::kSyncDoneSlot, s.ops[r].user_seq);
    else
      be->event_record(rr.device, rr.backend_event, c.group_stream);
  }
  s.group_launch.store(2, std::memory_order_release);
  return true;
}

// ---------------------------------------------------------------------------
// (6): completion
// ---------------------------------------------------------------------------
// Client-side launch: the plan ring carries the answer to every request, the plan itself
// or the reason there is none. A client keeps fewer requests outstanding than the ring has
// places (one outside a group; inside a group it takes the answers before the ring fills),
// so a push only fails while the client is behind; the caller then comes back.
bool ProxyEngine::publish_plan_error(RankState& rs, uint64_t user_seq, int status) {
  proto::PlanMsg m;
  memset(&m, 0, sizeof m);
  m.user_seq = user_seq;
  m.status = status;
  return rs.pq.try_push(&m);
}

bool ProxyEngine::publish_plan(RankState& rs, CollSlot& s, uint64_t seq) {
  Communicator& c = *rs.comm;
  const CollOp& o0 = s.ops[0];
  const uint64_t esz = kind_reduces(o0.kind) ? (uint64_t)dtype_size(o0.dtype) : 1;
  // One plan per time slice, each handed out once that slice is admitted: the client launches
  // them one after another on the caller's stream (a collective that is not sliced is its
  // only slice).
  while (rs.next_slice < s.nslices) {
    const int slice = rs.next_slice;
    if (!admit_slice(c, s, slice)) return false;
    uint64_t first = 0, count = o0.count;
    if (s.nslices > 1) {
      first = (uint64_t)slice * s.slice_count;
      count = std::min<uint64_t>(s.slice_count, o0.count - first);
    }
    const uint64_t off = first * esz;
    proto::PlanMsg m;
    memset(&m, 0, sizeof m);
    m.user_seq = s.ops[rs.rank].user_seq;
    m.status = proto::kOk;
    m.kind = o0.kind;
    m.variant = s.plan.variant;
    m.ctas = s.plan.dims.ctas;
    m.threads = s.plan.dims.threads;
    m.dtype = kind_reduces(o0.kind) ? o0.dtype : kUint8;
    m.op = kind_reduces(o0.kind) ? o0.op : kSum;
    m.nranks = c.nranks;
    m.scale = o0.op == kSumPostDiv ? 1.0f / (float)c.nranks : o0.scale;
    m.epoch = s.epoch_base + 2u * (uint32_t)slice;
    m.ticket = s.ticket_base + (uint64_t)slice;
    m.count = count;
    m.nslices = s.nslices;
    m.slice = slice;
    m.batch_len = s.fused_kernel && s.batch_len >= 2 ? s.batch_len : 0;   // the head of a fused launch
    m.timeout_ns = daemon_->timeout_ns();
    m.trace = daemon_->tracer().enabled() ? 1 : 0;
    if (s.plan.variant == kArHybrid) {
      const Config& cfg = daemon_->config();
      const int nvls_ctas = std::min(cfg.hybrid_nvls_ctas, std::max(s.plan.dims.ctas - 1, 0));
      m.variant_hint = (int32_t)(((uint32_t)nvls_ctas << 16) | (uint32_t)cfg.hybrid_nvls_permille);
    } else if (s.plan.variant == kArNvlsOne || s.plan.variant == kArNvlsTwo) {
      m.variant_hint = daemon_->config().nvls_unroll;
    } else if (s.plan.variant == kAgPull || s.plan.variant == kAgPush || s.plan.variant == kArTwoShot) {
      m.variant_hint = daemon_->config().pack_bytes;
    }
    if (s.plan.needs_mc_send) { m.mc_send_id = s.mc_send_id; m.mc_send_off = s.ops[rs.rank].send_off + off; }
    if (s.plan.needs_mc_recv) { m.mc_recv_id = s.mc_recv_id; m.mc_recv_off = s.ops[rs.rank].recv_off + off; }
    for (int r = 0; r < c.nranks; r++) {
      m.rank[r].send_mem = s.ops[r].send_mem; m.rank[r].send_off = s.ops[r].send_off + off;
      m.rank[r].recv_mem = s.ops[r].recv_mem; m.rank[r].recv_off = s.ops[r].recv_off + off;
    }
    memcpy(m.ring, s.ring, sizeof m.ring);
    for (int ch = 0; ch < kMaxRingChannels; ch++) m.ring_step_base[ch] = s.ring_step_base[ch];
    if (!rs.pq.try_push(&m)) return false;   // the client has not taken the previous slices yet: come back
    if (rs.rank == 0) {
      const uint64_t bytes = s.batch_len > 1 ? s.batch_bytes : s.nslices == 1 ? s.plan.bytes : s.plan.bytes / (uint64_t)s.nslices;
      rs.inflight.push_back({m.ticket, bytes});
    }
    rs.last_ticket.store(m.ticket, std::memory_order_relaxed);
    rs.next_slice++;
  }
  (void)seq;
  return true;
}

// The answer to a request that runs inside the fused launch of an earlier one: only its
// buffers (and multicast regions); the head's plan carries everything else.
bool ProxyEngine::publish_follower_plan(RankState& rs, CollSlot& s) {
  Communicator& c = *rs.comm;
  const CollOp& o0 = s.ops[0];
  proto::PlanMsg m;
  memset(&m, 0, sizeof m);
  m.user_seq = s.ops[rs.rank].user_seq;
  m.status = proto::kOk;
  m.kind = o0.kind;
  m.variant = s.plan.variant;
  m.dtype = o0.dtype;
  m.op = o0.op;
  m.nranks = c.nranks;
  m.count = o0.count;
  m.nslices = 1;
  m.batch_len = -1;
  if (s.plan.needs_mc_send) { m.mc_send_id = s.mc_send_id; m.mc_send_off = s.ops[rs.rank].send_off; }
  if (s.plan.needs_mc_recv) { m.mc_recv_id = s.mc_recv_id; m.mc_recv_off = s.ops[rs.rank].recv_off; }
  for (int r = 0; r < c.nranks; r++) {
    m.rank[r].send_mem = s.ops[r].send_mem; m.rank[r].send_off = s.ops[r].send_off;
    m.rank[r].recv_mem = s.ops[r].recv_mem; m.rank[r].recv_off = s.ops[r].recv_off;
  }
  return rs.pq.try_push(&m);
}

bool ProxyEngine::complete_request(RankState& rs, CollSlot& s, uint64_t seq, int status) {
  const CollOp& op = s.ops[rs.rank];
  if (rs.comm->client_launch) {
    // a published plan is the answer; only failures still need one
    if (status != proto::kOk && !publish_plan_error(rs, op.user_seq, status)) {
      rs.pending_plan_error = status;
      rs.pending_plan_seq = op.user_seq;
    }
    return true;
  }
  if (op.sync_slot && rs.dp_status) {
    // Mem-op request: counted, not answered (see proto::DpStatus).
    proto::DpStatus* d = rs.dp_status;
    if (status != proto::kOk && d->first_error == 0) d->first_error = status;
    d->last_variant = (uint32_t)s.plan.variant;
    d->last_ctas = (uint32_t)s.plan.dims.ctas;
    std::atomic_thread_fence(std::memory_order_release);
    __atomic_store_n(&d->completed, d->completed + 1, __ATOMIC_RELEASE);
    return true;
  }
  proto::WorkCompletion wc;
  memset(&wc, 0, sizeof wc);
  wc.kind = (uint32_t)op.kind;
  wc.status = status;
  wc.user_seq = op.user_seq;
  wc.variant = (uint32_t)s.plan.variant;
  wc.ctas = (uint32_t)s.plan.dims.ctas;
  wc.comm_seq = seq;
  if (!rs.cq.try_push(&wc)) {
    rs.pending_wc = wc;
    rs.have_pending_wc = true;
  }
  return true;
}

void ProxyEngine::finish_slot(Communicator& c, CollSlot& s, uint64_t seq) {
  if (s.finished.fetch_add(1, std::memory_order_acq_rel) + 1 == c.nranks) {
    // Every rank has put its kernel on a stream (or answered with an error): from here a
    // free only has to wait for those streams, so the buffers stop being held busy.
    for (int r = 0; r < c.nranks; r++) {
      CollOp& op = s.ops[r];
      if (!op.holds_refs) continue;
      op.holds_refs = false;
      daemon_->release_mem_ref(op.send_mem);
      daemon_->release_mem_ref(op.recv_mem);
    }
    s.arrived.store(0, std::memory_order_relaxed);
    s.finished.store(0, std::memory_order_relaxed);
    s.admitted_slices.store(0, std::memory_order_relaxed);
    s.defer_slice = -1;
    s.group_launch.store(0, std::memory_order_relaxed);
    s.state.store(kSlotCollecting, std::memory_order_relaxed);
    s.seq.store(seq + kCollSlots, std::memory_order_release);
  }
}

bool ProxyEngine::advance(RankState& rs) {
  Communicator& c = *rs.comm;
  Backend* be = daemon_->backend();
  const bool group = (c.emulated || be->kind() == proto::kBackendHost) && !c.client_launch;
  bool any = false;
  while (rs.next_launch_seq < rs.next_post_seq) {
    if (rs.pending_plan_error) {
      if (!publish_plan_error(rs, rs.pending_plan_seq, rs.pending_plan_error)) break;
      rs.pending_plan_error = 0;
    }
    if (rs.have_pending_wc) {
      if (!rs.cq.try_push(&rs.pending_wc)) break;
      rs.have_pending_wc = false;
    }
    const uint64_t seq = rs.next_launch_seq;
    CollSlot& s = c.slot(seq);
    // The communicator's state is read BEFORE the slot's: a peer only closes its handle
    // after every collective it took part in has been collected, so a slot that still
    // shows "collecting" after the close was observed can never complete. (Read the other
    // way round, a proxy thread that is descheduled between the two loads would fail a
    // collective that completed for everybody else in the meantime.)
    const bool comm_stopped = c.state.load(std::memory_order_acquire) == kCommError;
    int st = s.state.load(std::memory_order_acquire);
    if (comm_stopped) {
      // A failed communicator never launches again; what was posted completes in error.
      // A communicator that is merely being closed (a peer destroyed its handle, no
      // error recorded) still finishes collectives every rank had already joined.
      const int err = c.async_error.load();
      if (err != 0 || st == kSlotCollecting) {
        LOG_WARN("comm %u rank %d: collective %llu ends with status %d (%d of %d ranks had joined it)", c.id, rs.rank,
                 (unsigned long long)seq, err ? err : proto::kErrPeerLost, s.arrived.load(), c.nranks);
        if (s.ops[rs.rank].sync_slot) signal_done(rs, s.ops[rs.rank].user_seq, err ? err : proto::kErrPeerLost);
        complete_request(rs, s, seq, err ? err : proto::kErrPeerLost);
        rs.next_launch_seq++;
        rs.next_slice = 0;
        any = true;
        continue;
      }
    }
    if (st == kSlotCollecting) break;
    if (st == kSlotCollected) {
      if (c.paused.load(std::memory_order_acquire)) break;
      if (followers_still_arriving(c, s, seq)) break;
      int expect = kSlotCollected;
      if (!s.state.compare_exchange_strong(expect, kSlotPlanning, std::memory_order_acq_rel)) break;
      {
        NvtxRange range("mccs plan");
        plan_slot(c, s, seq);
      }
      st = s.state.load(std::memory_order_acquire);
      any = true;
    }
    if (st == kSlotPlanning) break;
    // Bound the work queued on the GPU per rank. Clients can post far ahead of the GPU
    // (calls return before anything runs); without a bound the backend streams fill up,
    // a launch call then blocks this proxy thread, and since a blocked kernel at the head
    // of that stream waits for a peer kernel that another (equally blocked) proxy has to
    // launch, the proxies could wait on each other forever.
    const bool follower = st == kSlotPlanned && s.batch_len == 0;   // went out with its head's launch
    if (st == kSlotPlanned && !follower) {
      RankState& gate = group ? *c.ranks[0] : rs;
      if (gate.status && gate.last_ticket.load(std::memory_order_relaxed) >
                             __atomic_load_n(&gate.status->done_seq, __ATOMIC_ACQUIRE) + kMaxGpuQueue) break;
      if (rs.next_slice == 0 && !(group && s.group_launch.load(std::memory_order_acquire) == 2) &&
          !(s.batch_len > 1 ? batch_clients_ready(c, s, seq, group ? -1 : rs.rank) : clients_ready(c, s, group ? -1 : rs.rank)))
        break;
    }
    int status = proto::kOk;
    const uint64_t t_go_us = daemon_->tracer().enabled() ? monotonic_us() : 0;
    if (st == kSlotFailed) {
      status = s.status;
      if (s.ops[rs.rank].sync_slot) signal_done(rs, s.ops[rs.rank].user_seq, status);
    } else if (follower) {
      // One answer per request: the error, or the member's buffers.
      if (c.state.load() == kCommError) status = c.async_error.load();
      if (status == proto::kOk && c.client_launch && !publish_follower_plan(rs, s)) break;
    } else if (c.client_launch) {
      if (!publish_plan(rs, s, seq)) break;   // the rank's own library launches the kernel
    } else if (group) {
      if (s.group_launch.load(std::memory_order_acquire) != 2) {
        if (rs.rank != 0) break;
        NvtxRange range(variant_name(s.plan.variant));
        if (!launch_group(c, s, seq)) break;
      }
      if (c.state.load() == kCommError) status = c.async_error.load();
    } else {
      {
        NvtxRange range(variant_name(s.plan.variant));
        if (!launch_slices(rs, s, seq)) break;
      }
      if (c.state.load() == kCommError) status = c.async_error.load();
    }
    if (daemon_->tracer().enabled() && st == kSlotPlanned) {
      TraceEvent ev;
      ev.comm_id = c.id; ev.rank = rs.rank; ev.device = rs.device; ev.seq = seq;
      ev.kind = s.ops[rs.rank].kind; ev.variant = s.plan.variant; ev.ctas = s.plan.dims.ctas;
      ev.slices = s.nslices; ev.bytes = s.plan.bytes;
      ev.t_post_us = s.ops[rs.rank].t_post_us; ev.t_ready_us = s.t_ready_us; ev.t_launch_us = monotonic_us();
      ev.t_go_us = t_go_us;
      // Device stamps belong to the most recent finished kernel of this rank.
      if (rs.status) {
        ev.dev_start_ns = __atomic_load_n(&rs.status->start_ns, __ATOMIC_RELAXED);
        ev.dev_end_ns = __atomic_load_n(&rs.status->end_ns, __ATOMIC_RELAXED);
      }
      daemon_->tracer().record(ev);
    }
    complete_request(rs, s, seq, status);
    finish_slot(c, s, seq);
    rs.next_launch_seq++;
    rs.next_slice = 0;
    any = true;
  }
  return any;
}

// Completion accounting for QoS and device error pick-up.
void ProxyEngine::housekeeping(RankState& rs) {
  Communicator& c = *rs.comm;
  if (!rs.status) return;
  if (rs.rank == 0) {
    const uint64_t done = __atomic_load_n(&rs.status->done_seq, __ATOMIC_ACQUIRE);
    while (!rs.inflight.empty() && rs.inflight.front().ticket <= done) {
      daemon_->qos().complete(c.id, rs.inflight.front().bytes);
      c.completed.fetch_add(1);
      rs.inflight.pop_front();
    }
  }
  const uint32_t err = __atomic_load_n(&rs.status->error, __ATOMIC_ACQUIRE);
  if (err != kDevOk && c.device_error.load() == kDevOk) {
    c.device_error.store(err);
    c.async_error.store(err == kDevAborted ? proto::kErrAborted : proto::kErrTimeout);
    c.state.store(kCommError);
    LOG_ERROR("comm %u rank %d: kernel reported %s (detail %u)", c.id, rs.rank,
              err == kDevAborted ? "abort" : "a wait that ran out", rs.status->error_peer);
    // Let the other ranks' kernels give up at once instead of waiting out their bound.
    for (auto& r : c.ranks)
      if (r && r->status) __atomic_store_n(&r->status->abort, 1u, __ATOMIC_RELEASE);
    // Nothing is in flight for QoS purposes any more.
    if (rs.rank == 0) {
      while (!rs.inflight.empty()) { daemon_->qos().complete(c.id, rs.inflight.front().bytes); rs.inflight.pop_front(); }
    }
  }
}

}  // namespace mccs
