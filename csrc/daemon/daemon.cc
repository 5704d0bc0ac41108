// Control plane of the daemon: sessions, allocations, communicator rendezvous,
// teardown, and the process-wide embedded instance. See daemon.h for the map to the
// reference.
#include "daemon.h"

#include <errno.h>
#include <poll.h>
#include <signal.h>
#include <string.h>
#include <unistd.h>

#include <algorithm>

#include "../common/log.h"
#include "../ipc/uds.h"

namespace mccs {

namespace proto {
const char* status_string(int32_t s) {
  switch (s) {
    case kOk: return "ok";
    case kErrInvalidArgument: return "invalid argument";
    case kErrOutOfMemory: return "out of memory";
    case kErrDevice: return "device call failed";
    case kErrProtocol: return "protocol error";
    case kErrNotFound: return "not found";
    case kErrTimeout: return "timed out";
    case kErrAborted: return "aborted";
    case kErrMismatch: return "ranks disagree on the collective";
    case kErrUnsupported: return "unsupported";
    case kErrPeerLost: return "a peer rank went away";
    case kErrInternal: return "internal error";
  }
  return "unknown status";
}
}  // namespace proto

Daemon::Daemon() {}

Daemon::~Daemon() { stop(); }

int Daemon::start(const Config& cfg, std::string* err) {
  cfg_ = cfg;
  BackendOptions bo;
  bo.host_devices = cfg.host_devices;
  bo.host_no_peer_access = cfg.host_no_peer_access;
  bo.allow_vmm = cfg.vmm;
  bo.allow_nvls = cfg.nvls;
  bo.force_host = cfg.force_host_backend;
  bo.allow_memops = cfg.sync != "events";
  bo.emulate_kernels = cfg.host_kernels == "emulated";
  bo.host_memops = cfg.sync == "memops";   // on the host backend only on request ("auto" keeps events there)
  backend_.reset(make_backend(bo));
  if (!backend_) { if (err) *err = "no backend"; return proto::kErrInternal; }
  LOG_INFO("daemon backend: %s", backend_->describe().c_str());
  memops_ = backend_->memops_supported() && cfg.sync != "events";
  if (cfg.sync == "memops" && !memops_) LOG_WARN("b200.sync=memops requested but stream memory operations are unavailable; using events");

  catalog_.reset(new TransportCatalog(cfg.transport));
  auto_launch_ = cfg.launch == "auto";
  client_launch_ = cfg.launch == "client" || (auto_launch_ && backend_->kind() == proto::kBackendCuda);
  if (client_launch_ && !backend_->client_launch_supported()) {
    if (!auto_launch_)
      LOG_WARN("b200.launch=client needs exportable device memory and registered host memory addressable by its host pointer; the daemon launches");
    client_launch_ = false;
  }
  planner_.load_defaults(backend_->nvls_supported() && cfg.nvls);
  if (!cfg.tuning_file.empty()) {
    std::string terr;
    if (!planner_.load_file(cfg.tuning_file, &terr))
      LOG_WARN("tuning file %s not used: %s", cfg.tuning_file.c_str(), terr.c_str());
  }
  qos_.configure(cfg);
  tracer_.set_enabled(cfg.trace);

  control_path_ = cfg.control_socket_path();
  int rc = ipc::make_dirs(ipc::dirname_of(control_path_));
  if (rc < 0) { if (err) *err = "cannot create " + ipc::dirname_of(control_path_); return proto::kErrInternal; }
  listen_fd_ = ipc::uds_listen(control_path_);
  if (listen_fd_ < 0) {
    if (err) *err = "cannot listen on " + control_path_ + ": " + strerror(-listen_fd_);
    return proto::kErrInternal;
  }

  // Admin endpoint (TCP, loopback unless an address list names this host).
  admin_port_ = 0;
  if (cfg.listen_port != 0) {
    extern int admin_listen(int port, int* bound_port);
    admin_fd_ = admin_listen(cfg.listen_port < 0 ? 0 : cfg.listen_port, &admin_port_);
    if (admin_fd_ < 0) {
      LOG_WARN("admin endpoint disabled: cannot bind port %d (%s)", cfg.listen_port, strerror(-admin_fd_));
      admin_fd_ = -1;
      admin_port_ = 0;
    }
  }

  extern void proxy_tracing_init();
  proxy_tracing_init();
  runtimes_.reset(new RuntimeManager(cfg.idle_sleep_us, cfg.idle_spin_us, cfg.pin_threads));
  for (int d = 0; d < backend_->device_count(); d++) {
    auto p = std::make_shared<ProxyEngine>(this, d);
    proxies_.push_back(p);
    runtimes_->submit(p, backend_->cpu_affinity(d));
  }
  stop_.store(false);
  running_.store(true);
  if (admin_fd_ >= 0) admin_thread_ = std::thread([this] { admin_loop(); });
  LOG_INFO("daemon up: control=%s admin_port=%d devices=%d", control_path_.c_str(), admin_port_,
           backend_->device_count());
  return proto::kOk;
}

void Daemon::run() {
  while (!stop_.load(std::memory_order_relaxed)) control_iteration(5);
}

void Daemon::run_in_thread() {
  control_thread_ = std::thread([this] { run(); });
}

void Daemon::stop() {
  if (!running_.exchange(false)) return;
  stop_.store(true);
  if (control_thread_.joinable() && control_thread_.get_id() != std::this_thread::get_id()) control_thread_.join();
  if (admin_thread_.joinable()) admin_thread_.join();
  // Tear down clients and communicators while the proxies still run (they must
  // acknowledge rank removal), then stop the engine threads.
  std::vector<uint64_t> ids;
  {
    std::lock_guard<std::mutex> g(mu_);
    for (auto& kv : sessions_) ids.push_back(kv.first);
  }
  for (uint64_t id : ids) drop_session(id, "daemon shutdown");
  if (runtimes_) runtimes_->stop_all();
  proxies_.clear();
  {
    std::unique_lock<std::shared_mutex> al(alloc_mu_);
    for (auto& kv : allocs_) backend_->release(&kv.second);
    allocs_.clear();
    alloc_use_.clear();
  }
  if (listen_fd_ >= 0) { close(listen_fd_); listen_fd_ = -1; unlink(control_path_.c_str()); }
  if (admin_fd_ >= 0) { close(admin_fd_); admin_fd_ = -1; }
  if (!cfg_.trace_file.empty() && tracer_.enabled()) tracer_.dump(cfg_.trace_file);
  backend_.reset();
}

// ---------------------------------------------------------------------------
// Control loop
// ---------------------------------------------------------------------------
void Daemon::control_iteration(int timeout_ms) {
  std::vector<struct pollfd> fds;
  std::vector<uint64_t> ids;
  {
    std::lock_guard<std::mutex> g(mu_);
    fds.push_back({listen_fd_, POLLIN, 0});
    ids.push_back(0);
    for (auto& kv : sessions_) {
      fds.push_back({kv.second->fd, POLLIN, 0});
      ids.push_back(kv.first);
    }
  }
  int rc = poll(fds.data(), (nfds_t)fds.size(), timeout_ms);
  if (rc > 0) {
    if (fds[0].revents & POLLIN) accept_clients();
    for (size_t i = 1; i < fds.size(); i++) {
      if (!(fds[i].revents & (POLLIN | POLLHUP | POLLERR))) continue;
      Session* s = nullptr;
      {
        std::lock_guard<std::mutex> g(mu_);
        auto it = sessions_.find(ids[i]);
        if (it != sessions_.end()) s = it->second.get();
      }
      if (s) handle_session(*s);
    }
  }
  check_init_timeouts();
}

void Daemon::accept_clients() {
  for (;;) {
    int fd = ipc::uds_accept(listen_fd_);
    if (fd < 0) break;
    // Handshake: the client speaks first.
    proto::AnyMsg m;
    if (ipc::wait_readable(fd, 2000) <= 0) { close(fd); continue; }
    ssize_t n = ipc::uds_recv(fd, &m, sizeof m);
    if (n < (ssize_t)sizeof(proto::Hello) || m.h.magic != proto::kMagic || m.h.type != proto::kHello ||
        m.hello.version != proto::kVersion) {
      LOG_WARN("rejecting client: bad hello (%zd bytes)", n);
      close(fd);
      continue;
    }
    {
      std::lock_guard<std::mutex> g(mu_);
      if (cfg_.max_clients > 0 && (int)sessions_.size() >= cfg_.max_clients) {
        LOG_WARN("rejecting client: %zu clients are connected ([limits] max_clients)", sessions_.size());
        close(fd);
        continue;
      }
    }
    ipc::PeerCred cred{0, 0, 0};
    ipc::uds_peer_cred(fd, &cred);
    auto s = std::make_unique<Session>();
    s->fd = fd;
    s->pid = cred.pid ? (int)cred.pid : m.hello.pid;
    s->same_process = s->pid == (int)getpid();
    s->device_affinity = m.hello.device_affinity;
    m.hello.app_name[sizeof(m.hello.app_name) - 1] = 0;
    s->app = m.hello.app_name;
    proto::AnyMsg r;
    memset(&r, 0, sizeof r);
    {
      std::lock_guard<std::mutex> g(mu_);
      s->id = next_session_id_++;
      r.welcome.session_id = s->id;
    }
    r.h.magic = proto::kMagic;
    r.h.type = proto::kWelcome;
    r.h.req_id = m.h.req_id;
    r.welcome.version = proto::kVersion;
    r.welcome.daemon_pid = (int)getpid();
    r.welcome.backend = backend_->kind();
    r.welcome.num_devices = (uint32_t)backend_->device_count();
    r.welcome.sync_mode = memops_ ? proto::kSyncMemOps : proto::kSyncEvents;
    LOG_INFO("client %llu attached: pid=%d app=%s%s", (unsigned long long)s->id, s->pid, s->app.c_str(),
             s->same_process ? " (same process)" : "");
    ipc::uds_send(fd, &r, sizeof(proto::Welcome));
    std::lock_guard<std::mutex> g(mu_);
    sessions_[s->id] = std::move(s);
  }
}

void Daemon::reply(Session& s, proto::AnyMsg& m, size_t len, const int* fds, int nfds) {
  m.h.magic = proto::kMagic;
  ssize_t n = ipc::uds_send(s.fd, &m, len, fds, nfds);
  if (n < 0) LOG_WARN("reply to client %llu failed: %s", (unsigned long long)s.id, strerror((int)-n));
}

void Daemon::handle_session(Session& s) {
  proto::AnyMsg m;
  memset(&m, 0, sizeof m);
  ssize_t n = ipc::uds_recv(s.fd, &m, sizeof m);
  if (n == -EAGAIN) return;
  if (n <= 0) { drop_session(s.id, n == 0 ? "client closed the connection" : "receive error"); return; }
  if ((size_t)n < sizeof(proto::Header) || m.h.magic != proto::kMagic) {
    drop_session(s.id, "malformed message");
    return;
  }
  // A request shorter than its type's layout is answered as a protocol error (the
  // missing fields were zeroed above, nothing reads past what arrived).
  size_t need = sizeof(proto::Header);
  switch (m.h.type) {
    case proto::kMalloc: need = sizeof(proto::MallocReq); break;
    case proto::kFree: need = sizeof(proto::FreeReq); break;
    case proto::kCommInit: need = sizeof(proto::CommInitReq); break;
    case proto::kCommDestroy: need = sizeof(proto::CommDestroyReq); break;
    case proto::kRegisterStream: need = sizeof(proto::RegisterStreamReq); break;
    case proto::kCommQuery: need = sizeof(proto::CommQueryReq); break;
    case proto::kMapScratch: need = sizeof(proto::MapScratchReq); break;
    case proto::kMapMem: need = sizeof(proto::MapMemReq); break;
    case proto::kMapMc: need = sizeof(proto::MapMcReq); break;
    default: break;
  }
  if ((size_t)n < need) m.h.type = 0;   // falls into the protocol-error reply below
  switch (m.h.type) {
    case proto::kMalloc: on_malloc(s, m.malloc_req); break;
    case proto::kFree: on_free(s, m.free_req); break;
    case proto::kCommInit: on_comm_init(s, m.comm_init); break;
    case proto::kCommDestroy: on_comm_destroy(s, m.comm_destroy); break;
    case proto::kRegisterStream: on_register_stream(s, m.reg_stream); break;
    case proto::kCommQuery: on_comm_query(s, m.comm_query); break;
    case proto::kMapScratch: on_map_scratch(s, m.map_scratch); break;
    case proto::kMapMc: on_map_mc(s, m.map_mc); break;
    case proto::kMapMem: on_map_mem(s, m.map_mem); break;
    case proto::kGoodbye: drop_session(s.id, "client said goodbye"); break;
    default: {
      proto::AnyMsg r;
      memset(&r, 0, sizeof r);
      r.h.type = m.h.type + 1;
      r.h.req_id = m.h.req_id;
      r.h.status = proto::kErrProtocol;
      reply(s, r, sizeof(proto::Header));
    }
  }
}

// ---------------------------------------------------------------------------
// Memory
// ---------------------------------------------------------------------------
static void refresh_stats(Session& s) {
  s.stat_bytes.store(s.alloc_bytes, std::memory_order_relaxed);
  s.stat_allocs.store((int)s.allocs.size(), std::memory_order_relaxed);
  s.stat_comms.store((int)s.comm_ranks.size(), std::memory_order_relaxed);
}

void Daemon::on_malloc(Session& s, const proto::MallocReq& m) {
  proto::AnyMsg r;
  memset(&r, 0, sizeof r);
  r.h.type = proto::kMallocReply;
  r.h.req_id = m.h.req_id;
  Allocation a;
  const bool over = (cfg_.max_allocations_per_client > 0 && (int)s.allocs.size() >= cfg_.max_allocations_per_client) ||
                    (cfg_.max_bytes_per_client > 0 && (m.size > cfg_.max_bytes_per_client || s.alloc_bytes > cfg_.max_bytes_per_client - m.size));
  int rc = over ? proto::kErrOutOfMemory : backend_->alloc(m.device, m.size, &a);
  if (rc != proto::kOk) {
    if (over) LOG_WARN("client %llu (%s): allocation of %llu bytes refused by [limits]", (unsigned long long)s.id, s.app.c_str(),
                       (unsigned long long)m.size);
    r.h.status = rc;
    reply(s, r, sizeof(proto::MallocReply));
    return;
  }
  a.owner_session = s.id;
  s.alloc_bytes += a.size;
  {
    std::unique_lock<std::shared_mutex> al(alloc_mu_);
    a.id = next_mem_id_++;
    allocs_[a.id] = a;
    alloc_use_[a.id];
  }
  s.allocs.insert(a.id);
  refresh_stats(s);
  r.malloc_reply.mem_id = a.id;
  r.malloc_reply.size = a.size;
  r.malloc_reply.daemon_va = a.va;
  r.malloc_reply.device = a.device;
  r.malloc_reply.share_kind = s.same_process ? proto::kShareSameProcess : a.share_kind;
  memcpy(r.malloc_reply.ipc_handle, a.ipc_handle, sizeof a.ipc_handle);
  const bool send_fd = !s.same_process && a.share_fd >= 0;
  LOG_DEBUG("client %llu: malloc dev=%d size=%zu -> mem %llu", (unsigned long long)s.id, m.device, a.size,
            (unsigned long long)a.id);
  reply(s, r, sizeof(proto::MallocReply), send_fd ? &a.share_fd : nullptr, send_fd ? 1 : 0);
}

void Daemon::quiesce_session_streams(Session& s) {
  // Nothing of this client's communicators may still run on a GPU when memory they
  // use goes away. Kernels are bounded, so this returns.
  std::vector<std::pair<int, void*>> streams;
  {
    std::lock_guard<std::mutex> g(mu_);
    for (auto& cr : s.comm_ranks) {
      auto it = comms_.find(cr.first);
      if (it == comms_.end()) continue;
      Communicator& c = *it->second;
      for (auto& r : c.ranks)
        if (r && r->stream) streams.push_back({r->device, r->stream});
      if (c.group_stream && !c.ranks.empty() && c.ranks[0]) streams.push_back({c.ranks[0]->device, c.group_stream});
    }
  }
  for (auto& ds : streams) backend_->stream_sync(ds.first, ds.second);
}

// Waits until every proxy thread has finished what it was doing when this was called. A proxy
// decides on a launch (the communicator is fine, every rank has posted) and then carries it out;
// a communicator that is failed in between is only seen at the proxy's next look. So whoever
// fails a communicator and then takes away memory its collectives name waits here first: after
// it no launch decided on earlier is still being carried out (on the host backend the "kernel"
// runs inside that call; on a GPU it is on a stream by then, which the caller synchronises next).
void Daemon::proxy_grace_period() {
  std::vector<std::pair<ProxyEngine*, uint64_t>> seen;
  for (auto& p : proxies_)
    if (p && p->running()) seen.push_back({p.get(), p->passes()});
  const uint64_t t_end = monotonic_us() + 30ull * 1000 * 1000;
  for (auto& ps : seen) {
    while (ps.first->passes() < ps.second + 2) {
      if (monotonic_us() > t_end) {
        LOG_WARN("a proxy thread has not come round within 30 s; going on");
        return;
      }
      struct timespec ts = {0, 50000};
      nanosleep(&ts, nullptr);
    }
  }
}

void Daemon::drop_mc_regions_using(uint64_t mem_id) {
  std::lock_guard<std::mutex> g(mu_);
  for (auto& kv : comms_) {
    Communicator& c = *kv.second;
    std::lock_guard<std::mutex> mg(c.mc_mu);
    for (auto it = c.mc_cache.begin(); it != c.mc_cache.end();) {
      if (std::find(it->first.begin(), it->first.end(), mem_id) != it->first.end()) {
        backend_->mc_destroy(&it->second);
        it = c.mc_cache.erase(it);
      } else {
        ++it;
      }
    }
  }
}

void Daemon::on_free(Session& s, const proto::FreeReq& m) {
  proto::AnyMsg r;
  memset(&r, 0, sizeof r);
  r.h.type = proto::kFreeReply;
  r.h.req_id = m.h.req_id;
  if (!s.allocs.count(m.mem_id)) {
    r.h.status = proto::kErrNotFound;
    reply(s, r, sizeof(proto::FreeReply));
    return;
  }
  {
    // A collective that was posted but has not been launched on every rank still carries
    // this allocation's address (it may be waiting for peers, for admission, behind a
    // pause or behind the queue bound). Releasing the memory now would turn its launch
    // into a device fault inside the daemon, so the free is refused instead; the client
    // library drains its communicators first and never gets here with work in flight.
    // From here on the id resolves for nobody, so no new request can name it.
    std::unique_lock<std::shared_mutex> al(alloc_mu_);
    auto ut = alloc_use_.find(m.mem_id);
    if (ut != alloc_use_.end()) {
      if (ut->second.busy.load(std::memory_order_acquire) > 0) {
        al.unlock();
        LOG_DEBUG("client %llu: free of mem %llu refused for now, a queued collective still names it", (unsigned long long)s.id,
                 (unsigned long long)m.mem_id);
        r.h.status = proto::kErrBusy;
        reply(s, r, sizeof(proto::FreeReply));
        return;
      }
      ut->second.dying = true;
    }
  }
  // Everything that named the allocation is on a stream by now: wait for it.
  quiesce_session_streams(s);
  drop_mc_regions_using(m.mem_id);
  {
    std::unique_lock<std::shared_mutex> al(alloc_mu_);
    auto it = allocs_.find(m.mem_id);
    if (it != allocs_.end()) {
      s.alloc_bytes -= std::min<uint64_t>(s.alloc_bytes, it->second.size);
      backend_->release(&it->second);
      allocs_.erase(it);
    }
    alloc_use_.erase(m.mem_id);
  }
  s.allocs.erase(m.mem_id);
  refresh_stats(s);
  reply(s, r, sizeof(proto::FreeReply));
}

const Allocation* Daemon::find_alloc_locked(uint64_t mem_id) const {
  auto it = allocs_.find(mem_id);
  return it == allocs_.end() ? nullptr : &it->second;
}

bool Daemon::translate(uint64_t session_id, uint64_t mem_id, uint64_t off, uint64_t bytes, uint64_t* va, int* device) {
  std::shared_lock<std::shared_mutex> al(alloc_mu_);
  auto it = allocs_.find(mem_id);
  if (it == allocs_.end()) return false;
  const Allocation& a = it->second;
  if (a.owner_session != session_id) return false;   // another tenant's memory does not exist for this one
  auto ut = alloc_use_.find(mem_id);
  if (ut == alloc_use_.end() || ut->second.dying) return false;
  // Bounds-checked sub-buffer, like MccsDeviceMemoryHandle::add
  // (src/ipc/mccs/src/command.rs:44-56).
  if (off > a.size || bytes > a.size - off) return false;
  *va = a.va + off;
  *device = a.device;
  ut->second.busy.fetch_add(1, std::memory_order_acq_rel);
  return true;
}

void Daemon::release_mem_ref(uint64_t mem_id) {
  std::shared_lock<std::shared_mutex> al(alloc_mu_);
  auto ut = alloc_use_.find(mem_id);
  if (ut != alloc_use_.end()) ut->second.busy.fetch_sub(1, std::memory_order_acq_rel);
}

void Daemon::release_slot_refs(Communicator& c) {
  for (auto& slot : c.slots)
    for (int r = 0; r < c.nranks; r++) {
      CollOp& op = slot.ops[r];
      if (!op.holds_refs) continue;
      op.holds_refs = false;
      release_mem_ref(op.send_mem);
      release_mem_ref(op.recv_mem);
    }
}

// ---------------------------------------------------------------------------
// Streams
// ---------------------------------------------------------------------------
void Daemon::on_register_stream(Session& s, const proto::RegisterStreamReq& m) {
  proto::AnyMsg r;
  memset(&r, 0, sizeof r);
  r.h.type = proto::kRegisterStreamReply;
  r.h.req_id = m.h.req_id;
  StreamReg reg;
  reg.device = m.device;
  int rc = proto::kOk;
  if (backend_->kind() == proto::kBackendHost) {
    reg.event = nullptr;
  } else if (s.same_process) {
    reg.event = (void*)m.event_raw;
  } else {
    rc = backend_->event_open(m.device, m.event_handle, &reg.event);
    reg.owned = rc == proto::kOk;
  }
  if (rc == proto::kOk) {
    uint64_t id = s.next_stream_id++;
    s.streams[id] = reg;
    {
      std::unique_lock<std::shared_mutex> g(stream_mu_);
      stream_events_[{s.id, id}] = reg.event;
    }
    r.reg_stream_reply.stream_id = id;
  }
  r.h.status = rc;
  reply(s, r, sizeof(proto::RegisterStreamReply));
}

void* Daemon::lookup_stream_event(uint64_t session_id, uint64_t stream_id) {
  if (!stream_id) return nullptr;
  std::shared_lock<std::shared_mutex> g(stream_mu_);
  auto it = stream_events_.find({session_id, stream_id});
  return it == stream_events_.end() ? nullptr : it->second;
}

// ---------------------------------------------------------------------------
// Communicators
// ---------------------------------------------------------------------------
void Daemon::apply_pattern_locked(Communicator& c, const CommPattern& p) {
  // Caller holds c.cfg_mu. Channels come as {channel_id, ring}; the channel count is
  // the number of channels given (src/mccs/src/proxy/engine.rs:269-321).
  if (!p.channels.empty()) {
    std::vector<std::vector<int>> rings;
    std::vector<ChannelPattern> sorted = p.channels;
    std::sort(sorted.begin(), sorted.end(),
              [](const ChannelPattern& a, const ChannelPattern& b) { return a.channel_id < b.channel_id; });
    for (const auto& ch : sorted) rings.push_back(ch.ring);
    c.rings = rings;
    c.channel_count = (int)rings.size();
  }
  if (!p.allreduce_algo.empty()) {
    int v = Planner::variant_from_name(p.allreduce_algo);
    if (v == -2) v = kArRing;
    if (v == -3) v = kArNvlsTwo;
    if (v >= 0) c.ar_variant = v;
  }
  if (!p.allgather_algo.empty()) {
    int v = Planner::variant_from_name(p.allgather_algo);
    if (v == -2) v = kAgRing;
    if (v == -3) v = kAgNvls;
    if (v >= 0) c.ag_variant = v;
  }
  if (p.ctas > 0) c.ctas_override = std::min(p.ctas, kMaxCtas);
  else if (p.ctas < 0) c.ctas_override = 0;
  c.config_epoch++;
}

static bool valid_ring(const std::vector<int>& ring, int nranks) {
  if ((int)ring.size() != nranks) return false;
  std::vector<bool> seen((size_t)nranks, false);
  for (int r : ring) {
    if (r < 0 || r >= nranks || seen[(size_t)r]) return false;
    seen[(size_t)r] = true;
  }
  return true;
}

void Daemon::on_comm_init(Session& s, const proto::CommInitReq& m) {
  auto fail = [&](int status) {
    proto::AnyMsg r;
    memset(&r, 0, sizeof r);
    r.h.type = proto::kCommInitReply;
    r.h.req_id = m.h.req_id;
    r.h.status = status;
    reply(s, r, sizeof(proto::CommInitReply));
  };
  if (m.nranks < 1 || m.nranks > kMaxRanks || m.rank < 0 || m.rank >= m.nranks || m.device < 0 ||
      m.device >= backend_->device_count())
    return fail(proto::kErrInvalidArgument);
  if (cfg_.max_communicators_per_client > 0 && (int)s.comm_ranks.size() >= cfg_.max_communicators_per_client) {
    LOG_WARN("client %llu (%s): communicator %u refused by [limits]", (unsigned long long)s.id, s.app.c_str(), m.comm_id);
    return fail(proto::kErrOutOfMemory);
  }
  Communicator* cptr = nullptr;
  bool complete = false;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = comms_.find(m.comm_id);
    if (it == comms_.end()) {
      auto c = std::make_unique<Communicator>();
      c->id = m.comm_id;
      c->nranks = m.nranks;
      c->devices.assign((size_t)m.nranks, -1);
      c->ranks.resize((size_t)m.nranks);
      c->created_us = monotonic_us();
      for (int i = 0; i < kCollSlots; i++) c->slots[i].seq.store((uint64_t)i);
      it = comms_.emplace(m.comm_id, std::move(c)).first;
    }
    Communicator& c = *it->second;
    if (c.state.load() != kCommInit || c.nranks != m.nranks || c.ranks[(size_t)m.rank]) {
      // The id is in use (or the ranks disagree on the size). If the communicator that holds it
      // is on its way out (a rank has left already: the others are about to, or will be told),
      // the request waits for the id instead of failing; a rank that destroys a communicator and
      // creates its successor under the same id is simply ahead of its peers.
      bool closing = false;
      if (c.state.load() != kCommInit)
        for (auto& r : c.ranks) closing |= r && r->gone.load();
      // (A client waits for the answer before it asks again; one that does not is not given
      // an unbounded list.)
      size_t mine = 0;
      for (const ParkedInit& pi : parked_inits_) mine += pi.session_id == s.id;
      if (closing && mine < 8 && parked_inits_.size() < 1024) {
        parked_inits_.push_back({s.id, m, monotonic_us() + cfg_.init_timeout_ms * 1000});
        return;
      }
      return fail(proto::kErrInvalidArgument);
    }
    auto rs = std::make_unique<RankState>();
    rs->comm = &c;
    rs->rank = m.rank;
    rs->device = m.device;
    rs->session_id = s.id;
    rs->same_process = s.same_process;
    rs->joined.store(true);
    c.devices[(size_t)m.rank] = m.device;
    c.ranks[(size_t)m.rank] = std::move(rs);
    s.comm_ranks.push_back({m.comm_id, m.rank});
    refresh_stats(s);
    pending_inits_.push_back({s.id, m.h.req_id, m.comm_id, m.rank, monotonic_us() + cfg_.init_timeout_ms * 1000});
    int joined = 0;
    for (auto& r : c.ranks) if (r) joined++;
    complete = joined == c.nranks;
    cptr = &c;
  }
  if (!complete) return;   // the reply goes out when the last rank has joined

  int rc = finalize_communicator(*cptr);
  std::vector<PendingInit> mine;
  {
    std::lock_guard<std::mutex> g(mu_);
    for (auto it = pending_inits_.begin(); it != pending_inits_.end();) {
      if (it->comm_id == m.comm_id) { mine.push_back(*it); it = pending_inits_.erase(it); }
      else ++it;
    }
  }
  for (const PendingInit& pi : mine) {
    Session* ps = nullptr;
    {
      std::lock_guard<std::mutex> g(mu_);
      auto it = sessions_.find(pi.session_id);
      if (it != sessions_.end()) ps = it->second.get();
    }
    if (!ps) continue;
    proto::AnyMsg r;
    memset(&r, 0, sizeof r);
    r.h.type = proto::kCommInitReply;
    r.h.req_id = pi.req_id;
    r.h.status = rc;
    if (rc == proto::kOk) {
      RankState& rs = *cptr->ranks[(size_t)pi.rank];
      r.comm_init_reply.comm_handle = proto::make_comm_handle(cptr->id, pi.rank);
      memcpy(r.comm_init_reply.event_handle, rs.event_handle, sizeof rs.event_handle);
      r.comm_init_reply.event_raw = ps->same_process ? (uint64_t)rs.backend_event : 0;
      r.comm_init_reply.dp_bytes = (uint32_t)rs.dp_bytes;
      r.comm_init_reply.launch_mode = cptr->client_launch ? proto::kLaunchClient : proto::kLaunchDaemon;
      r.comm_init_reply.fifo_slot_bytes = (uint32_t)cptr->fifo_slot_bytes;
      r.comm_init_reply.group_defer = cptr->client_launch && cfg_.fuse_allreduce > 1 ? 1u : 0u;
      int fds[2] = {rs.dp_fd, -1};
      int nfds = 1;
      if (rs.sync.host) {
        r.comm_init_reply.sync_size = rs.sync.bytes;
        r.comm_init_reply.sync_share_kind = proto::kShareHostFd;
        fds[nfds++] = rs.sync.fd;
      }
      reply(*ps, r, sizeof(proto::CommInitReply), fds, nfds);
    } else {
      reply(*ps, r, sizeof(proto::CommInitReply));
    }
  }
  if (rc != proto::kOk) destroy_communicator(m.comm_id);
}

int Daemon::finalize_communicator(Communicator& c) {
  const bool host = backend_->kind() == proto::kBackendHost;
  // Device placement: either one device per rank, or (for tests and single-GPU
  // boxes) every rank on the same device, which runs as one cooperative launch.
  bool all_same = true, all_distinct = true;
  for (int a = 0; a < c.nranks; a++)
    for (int b = a + 1; b < c.nranks; b++) {
      if (c.devices[(size_t)a] == c.devices[(size_t)b]) all_distinct = false;
      else all_same = false;
    }
  if (!host && c.nranks > 1 && !all_same && !all_distinct) {
    LOG_ERROR("comm %u: ranks must sit on distinct GPUs, or all on one", c.id);
    return proto::kErrUnsupported;
  }
  c.emulated = !host && c.nranks > 1 && all_same;
  // One transport per (sender, receiver) pair, the first of the catalog that can connect
  // the two devices.
  TransportEnv env;
  env.peer_access = [this](int a, int b) { return backend_->peer_access(a, b); };
  env.multicast = [this](int) { return backend_->nvls_supported(); };
  env.nvls_enabled = cfg_.nvls;
  c.conns = connect_all(*catalog_, env, c.devices);   // the table points into the catalog, which lives as long as the daemon
  if (!c.conns.complete()) {
    LOG_ERROR("comm %u: transport=%s connects no path from rank %d (device %d) to rank %d (device %d)", c.id, cfg_.transport.c_str(),
              c.conns.unconnected_from, c.devices[(size_t)c.conns.unconnected_from], c.conns.unconnected_to,
              c.devices[(size_t)c.conns.unconnected_to]);
    return proto::kErrUnsupported;
  }
  c.host_staged = c.conns.scratch_in_host_memory();
  // Kernels that clients launch themselves: not when several ranks share a GPU (their
  // kernels would be separate launches that wait on one another on one device), and on a
  // GPU not with the pads in pinned host memory (that memory is not exported).
  bool all_remote = true;   // every rank is a process of its own (not a thread of this one)
  for (int r = 0; r < c.nranks; r++) all_remote &= !c.ranks[(size_t)r]->same_process;
  c.client_launch = client_launch_ && (host || (!c.emulated && !c.host_staged)) && (!auto_launch_ || all_remote);
  if (client_launch_ && !auto_launch_ && !c.client_launch)
    LOG_WARN("comm %u: launched by the daemon although b200.launch=client (%s)", c.id,
             c.emulated ? "several ranks on one GPU" : "host-staged transport");

  {
    std::lock_guard<std::mutex> g(c.cfg_mu);
    c.channel_count = cfg_.channel_count;
    std::vector<int> identity;
    for (int r = 0; r < c.nranks; r++) identity.push_back(r);
    c.rings.assign((size_t)c.channel_count, identity);
    if (const CommPattern* p = cfg_.find_override(c.id)) {
      for (const auto& ch : p->channels)
        if (!valid_ring(ch.ring, c.nranks)) {
          LOG_ERROR("comm %u: override ring of channel %d is not a permutation of the ranks", c.id, ch.channel_id);
          return proto::kErrInvalidArgument;
        }
      apply_pattern_locked(c, *p);
      c.config_epoch = 0;
    }
  }
  const uint64_t buffer = cfg_.buffer_sizes[0];
  c.fifo_slot_bytes = buffer / kRingSlots / 16 * 16;
  if (c.fifo_slot_bytes < 16) return proto::kErrInvalidArgument;
  const int fifo_channels = std::max(c.channel_count, 4);
  const size_t fifo_bytes = (size_t)fifo_channels * c.fifo_slot_bytes * kRingSlots;

  const int prio = qos_.stream_priority(c.id) > 0 ? -1 : 0;   // lower number = higher priority
  for (int r = 0; r < c.nranks; r++) {
    RankState& rs = *c.ranks[(size_t)r];
    int rc;
    void* p = nullptr;
    if ((rc = backend_->scratch_alloc(rs.device, sizeof(SignalPad), c.host_staged, c.client_launch, &p)) != proto::kOk) return rc;
    rs.pad = (SignalPad*)p;
    if (c.nranks > 1) {
      if ((rc = backend_->scratch_alloc(rs.device, fifo_bytes, c.host_staged, c.client_launch, &p)) != proto::kOk) return rc;
      rs.fifo = (char*)p;
      rs.fifo_bytes = fifo_bytes;
    }
    if ((rc = backend_->hostmem_alloc(sizeof(StatusBlock), c.client_launch, &p)) != proto::kOk) return rc;
    rs.status = (StatusBlock*)p;
    // Stream-memory-operation ordering only for clients in other processes. A client
    // that lives in the daemon's own process has its stream in the same CUDA context
    // as the backend streams; streams of one context can share a hardware queue, and a
    // "wait for done" blocking the client's stream could then hold up the very backend
    // stream that has to produce "done". Such clients use ordinary events, which are
    // cheap inside one process.
    // (The host backend has no hardware queues: there every client may use the page.)
    if (memops_ && (!rs.same_process || host) && !c.client_launch) {
      if ((rc = backend_->sync_page_create(rs.device, &rs.sync)) != proto::kOk) return rc;
    }
    if ((rc = backend_->stream_create(rs.device, prio, &rs.stream)) != proto::kOk) return rc;
    if ((rc = backend_->event_create(rs.device, &rs.backend_event, rs.event_handle)) != proto::kOk) return rc;
    // Data-path segment: request ring followed by completion ring.
    const size_t wq_bytes = proto::dp_wq_bytes();
    rs.dp_bytes = proto::dp_segment_bytes();
    rs.dp_fd = ipc::memfd_make("mccs-dp", rs.dp_bytes);
    if (rs.dp_fd < 0) return proto::kErrOutOfMemory;
    rs.dp_mem = ipc::map_shared(rs.dp_fd, rs.dp_bytes);
    if (!rs.dp_mem) return proto::kErrOutOfMemory;
    rs.dp_status = (proto::DpStatus*)((char*)rs.dp_mem + wq_bytes + proto::dp_cq_bytes());
    memset(rs.dp_status, 0, sizeof(proto::DpStatus));
    rs.wq.init(rs.dp_mem, proto::kWqDepth, proto::kWrBytes);
    rs.cq.init((char*)rs.dp_mem + wq_bytes, proto::kCqDepth, proto::kWcBytes);
    rs.pq.init((char*)rs.dp_mem + proto::dp_pq_offset(), proto::kPqDepth, proto::kPlanBytes);
  }
  if (c.emulated || host) {
    int rc = backend_->stream_create(c.ranks[0]->device, prio, &c.group_stream);
    if (rc != proto::kOk) return rc;
  }
  std::vector<int> devs(c.devices.begin(), c.devices.end());
  qos_.tenant_register(c.id, devs);
  c.state.store(kCommActive);
  for (int r = 0; r < c.nranks; r++) proxies_[(size_t)c.ranks[(size_t)r]->device]->add_rank(c.ranks[(size_t)r].get());
  int sem_ranks = 0;
  for (auto& r : c.ranks) sem_ranks += r->sync.host != nullptr;
  LOG_INFO("comm %u ready: %d ranks, %s%s, %d ring channel(s), %d rank(s) ordered by semaphores, %d by events", c.id, c.nranks,
           c.conns.describe().c_str(), c.emulated ? " (single-device emulation)" : "",
           c.channel_count, sem_ranks, c.nranks - sem_ranks);
  return proto::kOk;
}

// Second (third, ...) pass for requests that wait for their id: through on_comm_init again
// once the old communicator is gone, answered with an error when their time is up.
void Daemon::retry_parked_inits() {
  if (parked_inits_.empty()) return;
  std::vector<ParkedInit> parked;
  parked.swap(parked_inits_);
  const uint64_t now = monotonic_us();
  for (ParkedInit& pi : parked) {
    Session* ps = nullptr;
    bool id_taken = false;
    {
      std::lock_guard<std::mutex> g(mu_);
      auto it = sessions_.find(pi.session_id);
      if (it != sessions_.end()) ps = it->second.get();
      auto cit = comms_.find(pi.req.comm_id);
      id_taken = cit != comms_.end() && cit->second->state.load() != kCommInit;
    }
    if (!ps) continue;   // the client went away while it waited
    if (!id_taken) {
      on_comm_init(*ps, pi.req);
    } else if (now > pi.deadline_us) {
      proto::AnyMsg r;
      memset(&r, 0, sizeof r);
      r.h.type = proto::kCommInitReply;
      r.h.req_id = pi.req.h.req_id;
      r.h.status = proto::kErrInvalidArgument;
      reply(*ps, r, sizeof(proto::CommInitReply));
    } else {
      parked_inits_.push_back(pi);
    }
  }
}

void Daemon::check_init_timeouts() {
  retry_parked_inits();
  const uint64_t now = monotonic_us();
  std::vector<PendingInit> expired;
  {
    std::lock_guard<std::mutex> g(mu_);
    for (auto it = pending_inits_.begin(); it != pending_inits_.end();) {
      if (now > it->deadline_us) { expired.push_back(*it); it = pending_inits_.erase(it); }
      else ++it;
    }
  }
  for (const PendingInit& pi : expired) {
    Session* ps = nullptr;
    {
      std::lock_guard<std::mutex> g(mu_);
      auto it = sessions_.find(pi.session_id);
      if (it != sessions_.end()) ps = it->second.get();
    }
    if (ps) {
      proto::AnyMsg r;
      memset(&r, 0, sizeof r);
      r.h.type = proto::kCommInitReply;
      r.h.req_id = pi.req_id;
      r.h.status = proto::kErrTimeout;
      reply(*ps, r, sizeof(proto::CommInitReply));
      auto& v = ps->comm_ranks;
      v.erase(std::remove(v.begin(), v.end(), std::make_pair(pi.comm_id, pi.rank)), v.end());
      refresh_stats(*ps);
    }
    bool empty = false;
    {
      std::lock_guard<std::mutex> g(mu_);
      auto it = comms_.find(pi.comm_id);
      if (it != comms_.end() && it->second->state.load() == kCommInit) {
        it->second->ranks[(size_t)pi.rank].reset();
        it->second->devices[(size_t)pi.rank] = -1;
        empty = true;
        for (auto& r : it->second->ranks) if (r) empty = false;
      }
    }
    if (empty) destroy_communicator(pi.comm_id);
  }
}

// Takes one rank out of a communicator (client destroyed it or went away). The
// communicator cannot run collectives any more; the remaining ranks see errors.
void Daemon::detach_rank(Communicator& c, int rank, int status) {
  RankState* rs = c.ranks[(size_t)rank].get();
  if (!rs || rs->gone.load()) return;
  if (status != proto::kOk && c.state.load() == kCommActive) {
    c.async_error.store(status);
    c.state.store(kCommError);
  }
  // Make any kernel of this communicator that still waits give up now.
  if (status != proto::kOk)
    for (auto& r : c.ranks)
      if (r && r->status) __atomic_store_n(&r->status->abort, 1u, __ATOMIC_RELEASE);
  if (c.state.load() != kCommInit) proxies_[(size_t)rs->device]->remove_rank(rs);
  rs->gone.store(true);
  if (rs->stream) backend_->stream_sync(rs->device, rs->stream);
  if (c.group_stream) backend_->stream_sync(rs->device, c.group_stream);
}

void Daemon::destroy_communicator(uint32_t comm_id) {
  std::unique_ptr<Communicator> c;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = comms_.find(comm_id);
    if (it == comms_.end()) return;
    c = std::move(it->second);
    comms_.erase(it);
    for (auto pit = pending_inits_.begin(); pit != pending_inits_.end();)
      pit = pit->comm_id == comm_id ? pending_inits_.erase(pit) : pit + 1;
  }
  qos_.tenant_unregister(comm_id);
  for (auto& r : c->ranks) {
    if (!r) continue;
    if (!r->gone.load() && c->state.load() != kCommInit) proxies_[(size_t)r->device]->remove_rank(r.get());
    if (r->stream) { backend_->stream_sync(r->device, r->stream); }
  }
  if (c->group_stream && c->ranks[0]) {
    backend_->stream_sync(c->ranks[0]->device, c->group_stream);
    backend_->stream_destroy(c->ranks[0]->device, c->group_stream);
  }
  release_slot_refs(*c);   // collectives that never completed on every rank
  {
    std::lock_guard<std::mutex> mg(c->mc_mu);
    for (auto& kv : c->mc_cache) backend_->mc_destroy(&kv.second);
    c->mc_cache.clear();
  }
  for (auto& r : c->ranks) {
    if (!r) continue;
    if (r->stream) backend_->stream_destroy(r->device, r->stream);
    if (r->backend_event) backend_->event_destroy(r->device, r->backend_event);
    if (r->pad) backend_->scratch_free(r->device, r->pad, sizeof(SignalPad), c->host_staged);
    if (r->fifo) backend_->scratch_free(r->device, r->fifo, r->fifo_bytes, c->host_staged);
    if (r->status) backend_->hostmem_free(r->status);
    if (r->sync.host) backend_->sync_page_destroy(r->device, &r->sync);
    if (r->dp_mem) ipc::unmap_shared(r->dp_mem, r->dp_bytes);
    if (r->dp_fd >= 0) close(r->dp_fd);
  }
  LOG_INFO("comm %u destroyed", comm_id);
}

void Daemon::on_comm_destroy(Session& s, const proto::CommDestroyReq& m) {
  proto::AnyMsg r;
  memset(&r, 0, sizeof r);
  r.h.type = proto::kCommDestroyReply;
  r.h.req_id = m.h.req_id;
  const uint32_t id = proto::handle_comm_id(m.comm_handle);
  const int rank = proto::handle_rank(m.comm_handle);
  auto cr = std::make_pair(id, rank);
  auto it = std::find(s.comm_ranks.begin(), s.comm_ranks.end(), cr);
  if (it == s.comm_ranks.end()) {
    r.h.status = proto::kErrNotFound;
    reply(s, r, sizeof(proto::CommDestroyReply));
    return;
  }
  s.comm_ranks.erase(it);
  refresh_stats(s);
  Communicator* c = nullptr;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto cit = comms_.find(id);
    if (cit != comms_.end()) c = cit->second.get();
  }
  bool last = false;
  if (c) {
    // An orderly destroy leaves the communicator usable by nobody, but is no error
    // for the ranks that have not called destroy yet unless they keep using it.
    detach_rank(*c, rank, proto::kOk);
    last = true;
    for (auto& rr : c->ranks) if (rr && !rr->gone.load()) last = false;
    // No error is recorded: the communicator just stops taking work. A rank that
    // still submits afterwards gets "peer lost" for that request.
    if (!last && c->state.load() == kCommActive) c->state.store(kCommError);
  }
  if (last) destroy_communicator(id);
  reply(s, r, sizeof(proto::CommDestroyReply));
}

// Client-side launch: a member of a communicator maps another member's signal pad, status
// block or FIFOs (its kernels address all of them).
void Daemon::on_map_scratch(Session& s, const proto::MapScratchReq& m) {
  proto::AnyMsg r;
  memset(&r, 0, sizeof r);
  r.h.type = proto::kMapScratchReply;
  r.h.req_id = m.h.req_id;
  const uint32_t id = proto::handle_comm_id(m.comm_handle);
  const auto me = std::make_pair(id, proto::handle_rank(m.comm_handle));
  int fd = -1;
  size_t bytes = 0;
  uint32_t share_kind = proto::kShareHostFd;
  int status = proto::kErrNotFound;
  if (std::find(s.comm_ranks.begin(), s.comm_ranks.end(), me) != s.comm_ranks.end()) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = comms_.find(id);
    if (it != comms_.end() && it->second->client_launch && m.rank >= 0 && m.rank < it->second->nranks &&
        it->second->ranks[(size_t)m.rank]) {
      RankState& rs = *it->second->ranks[(size_t)m.rank];
      void* p = m.kind == proto::kScratchPad ? (void*)rs.pad : m.kind == proto::kScratchStatus ? (void*)rs.status
                : m.kind == proto::kScratchFifo ? (void*)rs.fifo : nullptr;
      status = p ? backend_->scratch_export(p, &fd, &bytes, &share_kind) : proto::kErrNotFound;
      r.map_scratch_reply.daemon_va = (uint64_t)p;
    }
  }
  // A client inside this process on a GPU uses the daemon's own mappings.
  const bool direct = s.same_process && backend_->kind() == proto::kBackendCuda;
  r.h.status = status;
  r.map_scratch_reply.bytes = bytes;
  r.map_scratch_reply.share_kind = direct ? (uint32_t)proto::kShareSameProcess : share_kind;
  if (!direct) r.map_scratch_reply.daemon_va = 0;
  if (status == proto::kOk && direct) reply(s, r, sizeof(proto::MapScratchReply));
  else if (status == proto::kOk) reply(s, r, sizeof(proto::MapScratchReply), &fd, 1);
  else reply(s, r, sizeof(proto::MapScratchReply));
}

// Client-side launch: an allocation named in a plan. Only allocations of sessions that
// hold a rank of the same communicator as the requester can be mapped.
void Daemon::on_map_mem(Session& s, const proto::MapMemReq& m) {
  proto::AnyMsg r;
  memset(&r, 0, sizeof r);
  r.h.type = proto::kMapMemReply;
  r.h.req_id = m.h.req_id;
  const uint32_t id = proto::handle_comm_id(m.comm_handle);
  const auto me = std::make_pair(id, proto::handle_rank(m.comm_handle));
  int status = proto::kErrNotFound;
  int fd = -1;
  if (std::find(s.comm_ranks.begin(), s.comm_ranks.end(), me) != s.comm_ranks.end()) {
    std::set<uint64_t> members;
    {
      std::lock_guard<std::mutex> g(mu_);
      auto it = comms_.find(id);
      if (it != comms_.end() && it->second->client_launch)
        for (auto& rr : it->second->ranks)
          if (rr) members.insert(rr->session_id);
    }
    std::shared_lock<std::shared_mutex> al(alloc_mu_);
    auto it = allocs_.find(m.mem_id);
    const bool direct = s.same_process && backend_->kind() == proto::kBackendCuda;
    if (it != allocs_.end() && members.count(it->second.owner_session) && (direct || it->second.share_fd >= 0)) {
      status = proto::kOk;
      fd = direct ? -1 : it->second.share_fd;
      r.map_mem_reply.bytes = it->second.size;
      r.map_mem_reply.share_kind = direct ? (uint32_t)proto::kShareSameProcess : it->second.share_kind;
      r.map_mem_reply.device = it->second.device;
      r.map_mem_reply.daemon_va = direct ? it->second.va : 0;
    }
  }
  r.h.status = status;
  if (status == proto::kOk && fd < 0) reply(s, r, sizeof(proto::MapMemReply));
  else if (status == proto::kOk) reply(s, r, sizeof(proto::MapMemReply), &fd, 1);
  else reply(s, r, sizeof(proto::MapMemReply));
}

// Client-side launch: a multicast region named in a plan.
void Daemon::on_map_mc(Session& s, const proto::MapMcReq& m) {
  proto::AnyMsg r;
  memset(&r, 0, sizeof r);
  r.h.type = proto::kMapMcReply;
  r.h.req_id = m.h.req_id;
  const uint32_t id = proto::handle_comm_id(m.comm_handle);
  const int rank = proto::handle_rank(m.comm_handle);
  int status = proto::kErrNotFound;
  int fd = -1;
  if (std::find(s.comm_ranks.begin(), s.comm_ranks.end(), std::make_pair(id, rank)) != s.comm_ranks.end()) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = comms_.find(id);
    if (it != comms_.end() && it->second->client_launch && rank >= 0 && rank < it->second->nranks) {
      Communicator& c = *it->second;
      std::lock_guard<std::mutex> mg(c.mc_mu);
      for (const auto& kv : c.mc_cache) {
        const McRegion& reg = kv.second;
        if (!reg.handle || reg.id != m.mc_id) continue;
        const bool host = backend_->kind() == proto::kBackendHost;
        const bool direct = s.same_process && !host;
        if (!host && !direct && reg.share_fd < 0) { status = proto::kErrUnsupported; break; }
        status = proto::kOk;
        r.map_mc_reply.bytes = reg.size;
        r.map_mc_reply.align = reg.gran;
        r.map_mc_reply.nranks = (uint32_t)reg.nranks;
        r.map_mc_reply.share_kind = host ? (uint32_t)proto::kShareHostFd : direct ? (uint32_t)proto::kShareSameProcess : (uint32_t)proto::kShareVmmFd;
        if (direct) r.map_mc_reply.daemon_va = reg.va[rank];
        if (host) for (int q = 0; q < reg.nranks; q++) r.map_mc_reply.mems[q] = reg.mems[q];
        if (!host && !direct) fd = reg.share_fd;
        break;
      }
    }
  }
  r.h.status = status;
  if (status == proto::kOk && fd >= 0) reply(s, r, sizeof(proto::MapMcReply), &fd, 1);
  else reply(s, r, sizeof(proto::MapMcReply));
}

void Daemon::on_comm_query(Session& s, const proto::CommQueryReq& m) {
  proto::AnyMsg r;
  memset(&r, 0, sizeof r);
  r.h.type = proto::kCommQueryReply;
  r.h.req_id = m.h.req_id;
  std::lock_guard<std::mutex> g(mu_);
  auto it = comms_.find(proto::handle_comm_id(m.comm_handle));
  if (it == comms_.end()) {
    r.h.status = proto::kErrNotFound;
  } else {
    Communicator& c = *it->second;
    r.comm_query_reply.async_error = c.async_error.load();
    r.comm_query_reply.device_error = c.device_error.load();
    r.comm_query_reply.launched = c.planned.load();
    r.comm_query_reply.completed = c.completed.load();
    r.comm_query_reply.last_variant = c.last_variant.load();
    r.comm_query_reply.last_ctas = c.last_ctas.load();
    std::lock_guard<std::mutex> cg(c.cfg_mu);
    r.comm_query_reply.config_epoch = c.config_epoch;
  }
  reply(s, r, sizeof(proto::CommQueryReply));
}

// A client that disappears (crash, kill, exit without cleanup) shows up as EOF on its
// control connection. Its communicators fail, its memory is released
// (src/mccs/src/daemon/engine.rs:448-465, src/mccs/src/proxy/engine.rs:1091-1114).
void Daemon::drop_session(uint64_t session_id, const char* why) {
  std::unique_ptr<Session> s;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = sessions_.find(session_id);
    if (it == sessions_.end()) return;
    s = std::move(it->second);
    sessions_.erase(it);
  }
  LOG_INFO("client %llu detached (%s)", (unsigned long long)s->id, why);
  std::vector<uint32_t> to_destroy;
  for (auto& cr : s->comm_ranks) {
    Communicator* c = nullptr;
    {
      std::lock_guard<std::mutex> g(mu_);
      auto cit = comms_.find(cr.first);
      if (cit != comms_.end()) c = cit->second.get();
    }
    if (!c) continue;
    if (c->state.load() == kCommInit) {
      // Rendezvous never completed: the other ranks get an error reply.
      std::vector<PendingInit> others;
      {
        std::lock_guard<std::mutex> g(mu_);
        for (auto it = pending_inits_.begin(); it != pending_inits_.end();) {
          if (it->comm_id == cr.first) { others.push_back(*it); it = pending_inits_.erase(it); }
          else ++it;
        }
      }
      for (const PendingInit& pi : others) {
        if (pi.session_id == session_id) continue;
        std::lock_guard<std::mutex> g(mu_);
        auto sit = sessions_.find(pi.session_id);
        if (sit == sessions_.end()) continue;
        proto::AnyMsg r;
        memset(&r, 0, sizeof r);
        r.h.type = proto::kCommInitReply;
        r.h.req_id = pi.req_id;
        r.h.status = proto::kErrPeerLost;
        reply(*sit->second, r, sizeof(proto::CommInitReply));
        auto& v = sit->second->comm_ranks;
        v.erase(std::remove(v.begin(), v.end(), std::make_pair(pi.comm_id, pi.rank)), v.end());
        refresh_stats(*sit->second);
      }
      to_destroy.push_back(cr.first);
      continue;
    }
    detach_rank(*c, cr.second, proto::kErrPeerLost);
    bool last = true;
    for (auto& rr : c->ranks) if (rr && !rr->gone.load()) last = false;
    if (last) to_destroy.push_back(cr.first);
  }
  // The communicators this client was part of are failed now, but a proxy of a surviving rank
  // may be in the middle of a launch it decided on just before, and its kernels may be reading
  // this client's buffers: let those launches end, then wait for the streams of every rank of
  // those communicators. Only then can the memory go.
  if (!s->allocs.empty() && !s->comm_ranks.empty()) {
    proxy_grace_period();
    quiesce_session_streams(*s);
    // Kernels that surviving clients launched themselves run on their streams, out of the
    // daemon's reach. They have been told to give up (abort word); give them a moment to do
    // so before multicast bindings of the dead client's memory are taken apart under them:
    // every surviving rank is through its last ticket or has reported an error. Bounded: a
    // client that got a plan and never launched must not hold the daemon up.
    const uint64_t t_end = monotonic_us() + 2ull * 1000 * 1000;
    for (auto& cr : s->comm_ranks) {
      Communicator* c = nullptr;
      {
        std::lock_guard<std::mutex> g(mu_);
        auto cit = comms_.find(cr.first);
        if (cit != comms_.end()) c = cit->second.get();
      }
      if (!c || c->state.load() == kCommInit || !c->client_launch) continue;
      for (auto& r : c->ranks) {
        if (!r || r->gone.load() || !r->status) continue;
        while (__atomic_load_n(&r->status->done_seq, __ATOMIC_ACQUIRE) < r->last_ticket.load(std::memory_order_relaxed) &&
               __atomic_load_n(&r->status->error, __ATOMIC_ACQUIRE) == kDevOk && monotonic_us() < t_end) {
          struct timespec ts = {0, 50000};
          nanosleep(&ts, nullptr);
        }
      }
    }
  }
  for (uint32_t id : to_destroy) destroy_communicator(id);
  for (uint64_t mem : s->allocs) {
    drop_mc_regions_using(mem);
    std::unique_lock<std::shared_mutex> al(alloc_mu_);
    auto it = allocs_.find(mem);
    if (it != allocs_.end()) { backend_->release(&it->second); allocs_.erase(it); }
    alloc_use_.erase(mem);
  }
  {
    std::unique_lock<std::shared_mutex> g(stream_mu_);
    for (auto& kv : s->streams) {
      stream_events_.erase({s->id, kv.first});
      if (kv.second.owned && kv.second.event) backend_->event_destroy(kv.second.device, kv.second.event);
    }
  }
  if (s->fd >= 0) close(s->fd);
}

// ---------------------------------------------------------------------------
// Embedded instance
// ---------------------------------------------------------------------------
static std::mutex g_embedded_mu;
static std::unique_ptr<Daemon> g_embedded;
static std::string g_control_path, g_describe;

static int start_embedded(const Config& cfg) {
  std::lock_guard<std::mutex> g(g_embedded_mu);
  if (g_embedded && g_embedded->running()) return proto::kOk;
  g_embedded.reset(new Daemon());
  std::string err;
  int rc = g_embedded->start(cfg, &err);
  if (rc != proto::kOk) {
    LOG_ERROR("embedded daemon failed to start: %s", err.c_str());
    g_embedded.reset();
    return rc;
  }
  g_control_path = g_embedded->control_path();
  g_describe = g_embedded->backend()->describe();
  g_embedded->run_in_thread();
  return proto::kOk;
}

extern "C" int mccsd_start(const char* config_toml) {
  try {
    Config cfg = Config::from_string(config_toml ? config_toml : "");
    return start_embedded(cfg);
  } catch (const std::exception& e) {
    LOG_ERROR("bad daemon configuration: %s", e.what());
    return proto::kErrInvalidArgument;
  }
}

extern "C" int mccsd_start_file(const char* config_path) {
  try {
    Config cfg = Config::from_file(config_path);
    return start_embedded(cfg);
  } catch (const std::exception& e) {
    LOG_ERROR("bad daemon configuration %s: %s", config_path, e.what());
    return proto::kErrInvalidArgument;
  }
}

extern "C" void mccsd_stop() {
  std::lock_guard<std::mutex> g(g_embedded_mu);
  if (g_embedded) { g_embedded->stop(); g_embedded.reset(); }
}

extern "C" const char* mccsd_control_path() { return g_control_path.c_str(); }
extern "C" int mccsd_admin_port() {
  std::lock_guard<std::mutex> g(g_embedded_mu);
  return g_embedded ? g_embedded->admin_port() : 0;
}
extern "C" int mccsd_backend_kind() {
  std::lock_guard<std::mutex> g(g_embedded_mu);
  return g_embedded && g_embedded->backend() ? (int)g_embedded->backend()->kind() : -1;
}
extern "C" const char* mccsd_describe() { return g_describe.c_str(); }
extern "C" const char* mccsd_admin(int type, const char* json_body) {
  static thread_local std::string out;
  std::lock_guard<std::mutex> g(g_embedded_mu);
  if (!g_embedded) { out = "{\"status\":\"error\",\"error\":\"daemon not running\"}"; return out.c_str(); }
  try {
    out = g_embedded->admin_request(type, parse_json(json_body ? json_body : "{}")).to_json();
  } catch (const std::exception& e) {
    Value v = Value::object();
    v.set("status", "error");
    v.set("error", e.what());
    out = v.to_json();
  }
  return out.c_str();
}

}  // namespace mccs
