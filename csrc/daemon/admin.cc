// Admin endpoint of the daemon: live reconfiguration of communicators, QoS updates,
// pause/resume, statistics and trace dumps, over TCP with the framing the
// reference's exchange engine uses (src/mccs/src/exchange/engine.rs:33,44-76:
// u64 magic, u8 type, u32 length, body). The reference fans a
// `CommPatternReconfig` out to every proxy, which then suspends the communicator,
// shuts its transport agents down and reconnects the rings
// (src/mccs/src/proxy/engine.rs:787-840, proxy/init.rs:213-400). Here the new
// pattern is swapped in under the communicator's configuration lock and becomes
// part of the plan of the next collective; since one plan serves all ranks, every
// rank switches at the same collective and nothing has to drain.
#include <arpa/inet.h>
#include <errno.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <unistd.h>

#include "../common/log.h"
#include "daemon.h"

namespace mccs {

int admin_listen(int port, int* bound_port) {
  int fd = socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) return -errno;
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in addr;
  memset(&addr, 0, sizeof addr);
  addr.sin_family = AF_INET;
  addr.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  addr.sin_port = htons((uint16_t)port);
  if (bind(fd, (sockaddr*)&addr, sizeof addr) < 0) { int e = -errno; close(fd); return e; }
  if (listen(fd, 16) < 0) { int e = -errno; close(fd); return e; }
  socklen_t len = sizeof addr;
  getsockname(fd, (sockaddr*)&addr, &len);
  *bound_port = ntohs(addr.sin_port);
  return fd;
}

static bool read_full(int fd, void* buf, size_t n, int timeout_ms) {
  char* p = (char*)buf;
  while (n) {
    struct pollfd pf = {fd, POLLIN, 0};
    int rc = poll(&pf, 1, timeout_ms);
    if (rc <= 0) return false;
    ssize_t k = read(fd, p, n);
    if (k <= 0) return false;
    p += k;
    n -= (size_t)k;
  }
  return true;
}

static bool write_full(int fd, const void* buf, size_t n) {
  const char* p = (const char*)buf;
  while (n) {
    ssize_t k = send(fd, p, n, MSG_NOSIGNAL);
    if (k <= 0) return false;
    p += k;
    n -= (size_t)k;
  }
  return true;
}

void Daemon::admin_loop() {
  while (!stop_.load(std::memory_order_relaxed)) {
    struct pollfd pf = {admin_fd_, POLLIN, 0};
    int rc = poll(&pf, 1, 50);
    if (rc <= 0) continue;
    int fd = accept4(admin_fd_, nullptr, nullptr, SOCK_CLOEXEC);
    if (fd < 0) continue;
    handle_admin_connection(fd);
    close(fd);
  }
}

void Daemon::handle_admin_connection(int fd) {
  // One or more framed requests per connection; each gets a framed JSON reply.
  for (;;) {
    uint8_t hdr[13];
    if (!read_full(fd, hdr, sizeof hdr, 2000)) return;
    uint64_t magic;
    uint32_t len;
    memcpy(&magic, hdr, 8);
    uint8_t type = hdr[8];
    memcpy(&len, hdr + 9, 4);
    if (magic != proto::kAdminMagic || len > (16u << 20)) {
      LOG_WARN("admin: bad frame (magic %llx, len %u)", (unsigned long long)magic, len);
      return;
    }
    std::string body(len, '\0');
    if (len && !read_full(fd, &body[0], len, 5000)) return;
    Value reply;
    try {
      reply = admin_request(type, body.empty() ? Value::object() : parse_json(body));
    } catch (const std::exception& e) {
      reply = Value::object();
      reply.set("status", "error");
      reply.set("error", e.what());
    }
    std::string out = reply.to_json();
    uint8_t rh[13];
    memcpy(rh, &proto::kAdminMagic, 8);
    rh[8] = type;
    uint32_t olen = (uint32_t)out.size();
    memcpy(rh + 9, &olen, 4);
    if (!write_full(fd, rh, sizeof rh) || !write_full(fd, out.data(), out.size())) return;
  }
}

static bool ring_is_permutation(const std::vector<int>& ring, int nranks) {
  if ((int)ring.size() != nranks) return false;
  std::vector<bool> seen((size_t)nranks, false);
  for (int r : ring) {
    if (r < 0 || r >= nranks || seen[(size_t)r]) return false;
    seen[(size_t)r] = true;
  }
  return true;
}

int Daemon::apply_reconfig(const CommPattern& p, std::string* err) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = comms_.find(p.communicator_id);
  if (it == comms_.end()) {
    if (err) *err = "no communicator " + std::to_string(p.communicator_id);
    return proto::kErrNotFound;
  }
  Communicator& c = *it->second;
  if (c.state.load(std::memory_order_acquire) == kCommInit) {
    if (err) *err = "communicator " + std::to_string(p.communicator_id) + " is still waiting for ranks";
    return proto::kErrNotFound;
  }
  if (p.channels.size() > (size_t)kMaxRingChannels) {
    if (err) *err = "too many channels";
    return proto::kErrInvalidArgument;
  }
  for (const auto& ch : p.channels)
    if (!ring_is_permutation(ch.ring, c.nranks)) {
      if (err) *err = "ring of channel " + std::to_string(ch.channel_id) + " is not a permutation of the ranks";
      return proto::kErrInvalidArgument;
    }
  for (const std::string* algo : {&p.allreduce_algo, &p.allgather_algo})
    if (!algo->empty() && Planner::variant_from_name(*algo) == -1) {
      if (err) *err = "unknown algorithm '" + *algo + "'";
      return proto::kErrInvalidArgument;
    }
  std::lock_guard<std::mutex> cg(c.cfg_mu);
  apply_pattern_locked(c, p);
  LOG_INFO("comm %u reconfigured: %d channel(s), ar=%s ag=%s ctas=%d (config epoch %llu)", c.id, c.channel_count,
           variant_name(c.ar_variant), variant_name(c.ag_variant), c.ctas_override,
           (unsigned long long)c.config_epoch);
  return proto::kOk;
}

Value Daemon::stats() {
  Value out = Value::object();
  out.set("backend", backend_ ? backend_->describe() : "");
  out.set("control", control_path_);
  out.set("admin_port", admin_port_);
  Value comms = Value::object();
  {
    std::lock_guard<std::mutex> g(mu_);
    out.set("clients", (int64_t)sessions_.size());
    // what every client holds (the quantities the [limits] table bounds)
    Value holders = Value::array();
    for (auto& kv : sessions_) {
      const Session& s = *kv.second;
      Value h = Value::object();
      h.set("id", (int64_t)s.id);
      h.set("pid", s.pid);
      h.set("app", s.app);
      h.set("allocations", s.stat_allocs.load(std::memory_order_relaxed));
      h.set("allocated_bytes", (int64_t)s.stat_bytes.load(std::memory_order_relaxed));
      h.set("communicators", s.stat_comms.load(std::memory_order_relaxed));
      holders.push(h);
    }
    out.set("client_list", holders);
    for (auto& kv : comms_) {
      Communicator& c = *kv.second;
      Value v = Value::object();
      v.set("nranks", c.nranks);
      v.set("state", c.state.load());
      v.set("async_error", c.async_error.load());
      v.set("device_error", (int64_t)c.device_error.load());
      v.set("planned", (int64_t)c.planned.load());
      v.set("completed", (int64_t)c.completed.load());
      v.set("fused_launches", (int64_t)c.fused_launches.load());
      v.set("fused_members", (int64_t)c.fused_members.load());
      v.set("last_variant", variant_name((int)c.last_variant.load()));
      v.set("last_ctas", (int64_t)c.last_ctas.load());
      // Placement fields are written while the communicator is being set up, outside
      // the registry lock; they are final once its state has left "init".
      const bool ready = c.state.load(std::memory_order_acquire) != kCommInit;
      v.set("client_launch", ready && c.client_launch);
      v.set("emulated", ready && c.emulated);
      v.set("host_staged", ready && c.host_staged);
      v.set("transport", ready ? c.conns.describe() : std::string("-"));
      v.set("paused", c.paused.load());
      Value devs = Value::array();
      for (int d : c.devices) devs.push(d);
      v.set("devices", devs);
      {
        std::lock_guard<std::mutex> cg(c.cfg_mu);
        v.set("config_epoch", (int64_t)c.config_epoch);
        v.set("channel_count", c.channel_count);
        v.set("allreduce_algo", variant_name(c.ar_variant));
        v.set("allgather_algo", variant_name(c.ag_variant));
        v.set("ctas", c.ctas_override);
        Value rings = Value::array();
        for (auto& ring : c.rings) {
          Value rv = Value::array();
          for (int r : ring) rv.push(r);
          rings.push(rv);
        }
        v.set("rings", rings);
      }
      comms.set(std::to_string(c.id), v);
    }
  }
  out.set("communicators", comms);
  out.set("qos", qos_.stats());
  {
    std::shared_lock<std::shared_mutex> al(alloc_mu_);
    int64_t bytes = 0;
    for (auto& kv : allocs_) bytes += (int64_t)kv.second.size;
    out.set("allocations", (int64_t)allocs_.size());
    out.set("allocated_bytes", bytes);
  }
  return out;
}

Value Daemon::admin_request(int type, const Value& body) {
  Value reply = Value::object();
  auto ok = [&]() { reply.set("status", "ok"); return reply; };
  auto bad = [&](const std::string& why) {
    reply.set("status", "error");
    reply.set("error", why);
    return reply;
  };
  std::string cmd = body["cmd"].as_string();
  if (type == proto::kAdminReconfig && cmd.empty()) cmd = "reconfig";

  if (cmd == "reconfig") {
    // {"comm_patterns_reconfig": [ {communicator_id, channels:[{channel_id, ring}], ...} ]}
    const Value& list = body.has("comm_patterns_reconfig") ? body["comm_patterns_reconfig"] : body["patterns"];
    int applied = 0;
    for (const Value& pv : list.items()) {
      CommPattern p = Config::parse_pattern(pv);
      std::string err;
      int rc = apply_reconfig(p, &err);
      if (rc != proto::kOk) return bad(err);
      applied++;
    }
    reply.set("applied", applied);
    return ok();
  }
  if (cmd == "stats") {
    reply.set("stats", stats());
    return ok();
  }
  if (cmd == "qos_set") {
    for (const auto& kv : body["tenants"].fields()) {
      QosTenantConfig t;
      t.weight = kv.second["weight"].as_double(1.0);
      t.priority = (int)kv.second["priority"].as_int(0);
      t.cta_quota = (int)kv.second["cta_quota"].as_int(0);
      if (t.weight <= 0) return bad("tenant weight must be positive");
      qos_.set_tenant((uint32_t)std::stoul(kv.first), t);
    }
    if (body.has("schedule") || body.has("epoch_microsecs")) {
      std::map<uint32_t, QosIntervalConfig> sched;
      for (const auto& kv : body["schedule"].fields()) {
        QosIntervalConfig qi;
        for (const Value& iv : kv.second["intervals"].items())
          qi.intervals.push_back({(uint64_t)iv.at(0).as_int(), (uint64_t)iv.at(1).as_int()});
        qi.allow = kv.second["mode"].as_string("Allow") != "Deny";
        qi.enforce_step = (int)kv.second["enforce_step"].as_int(0);
        sched[(uint32_t)std::stoul(kv.first)] = qi;
      }
      qos_.set_schedule((uint64_t)body["epoch_microsecs"].as_int(0), sched);
    }
    if (body.has("enabled")) qos_.set_enabled(body["enabled"].as_bool(true));
    return ok();
  }
  if (cmd == "pause" || cmd == "resume") {
    std::lock_guard<std::mutex> g(mu_);
    auto it = comms_.find((uint32_t)body["communicator_id"].as_int());
    if (it == comms_.end()) return bad("no such communicator");
    it->second->paused.store(cmd == "pause");
    return ok();
  }
  if (cmd == "trace") {
    if (body.has("enabled")) tracer_.set_enabled(body["enabled"].as_bool());
    if (body["clear"].as_bool(false)) tracer_.clear();
    if (body.has("dump")) {
      if (!tracer_.dump(body["dump"].as_string())) return bad("cannot write trace file");
    }
    if (body["inline"].as_bool(false)) reply.set("trace", tracer_.to_chrome_json());
    return ok();
  }
  if (cmd == "tuning_get") {
    reply.set("tuning", planner_.to_json());
    return ok();
  }
  if (cmd == "tuning_set") {
    std::string err;
    if (!planner_.load_json(body["tuning"], &err)) return bad(err);
    return ok();
  }
  if (cmd == "hwinfo") {
    // What the daemon sees of the box: devices, the CPUs local to each (where its proxy
    // thread is pinned), the peer-access matrix and in-switch multicast support. The
    // reference's get_hwinfo example prints the NVML affinity part of this
    // (src/experimental/examples/get_hwinfo.rs).
    Value hw = Value::object();
    hw.set("backend", backend_->kind() == proto::kBackendCuda ? "cuda" : "host");
    hw.set("describe", backend_->describe());
    hw.set("nvls", backend_->nvls_supported());
    hw.set("memops", backend_->memops_supported());
    Value devs = Value::array();
    const int n = backend_->device_count();
    for (int d = 0; d < n; d++) {
      Value dv = Value::object();
      dv.set("index", d);
      dv.set("cpu_affinity", backend_->cpu_affinity(d));
      Value peers = Value::array();
      for (int e = 0; e < n; e++) peers.push(d == e || backend_->peer_access(d, e));
      dv.set("peer_access", peers);
      devs.push(dv);
    }
    hw.set("devices", devs);
    reply.set("hwinfo", hw);
    return ok();
  }
  if (cmd == "shutdown") {
    stop_.store(true);
    return ok();
  }
  return bad("unknown admin command '" + cmd + "'");
}

}  // namespace mccs
