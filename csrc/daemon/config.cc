#include "config.h"

#include <set>
#include <string>
#include <stdexcept>

#include "../kernels/dev_types.h"

namespace mccs {

std::string Config::control_socket_path() const {
  std::string prefix = expand_env(control_prefix);
  if (!prefix.empty() && prefix.back() == '/') prefix.pop_back();
  return prefix + "/" + expand_env(control_path);
}

const CommPattern* Config::find_override(uint32_t comm_id) const {
  for (const auto& p : overrides)
    if (p.communicator_id == comm_id) return &p;
  return nullptr;
}

CommPattern Config::parse_pattern(const Value& v) {
  CommPattern p;
  if (!v.has("communicator_id")) throw std::runtime_error("comm pattern without communicator_id");
  p.communicator_id = (uint32_t)v["communicator_id"].as_int();
  for (const Value& c : v["channels"].items()) {
    ChannelPattern ch;
    ch.channel_id = (int)c["channel_id"].as_int();
    for (const Value& r : c["ring"].items()) ch.ring.push_back((int)r.as_int());
    for (const Value& t : c["udp_sport"].items()) {
      std::vector<int> triple;
      for (const Value& x : t.items()) triple.push_back((int)x.as_int());
      ch.udp_sport.push_back(triple);
    }
    ch.net_dev = c["net_dev"].as_string();
    p.channels.push_back(ch);
  }
  if (v.has("ib_traffic_class")) p.ib_traffic_class = (int)v["ib_traffic_class"].as_int();
  p.allreduce_algo = v["allreduce_algo"].as_string();
  p.allgather_algo = v["allgather_algo"].as_string();
  p.ctas = (int)v["ctas"].as_int(0);
  return p;
}

static void check_keys(const Value& table, const std::set<std::string>& allowed, const char* where) {
  for (const auto& kv : table.fields())
    if (!allowed.count(kv.first))
      throw std::runtime_error(std::string("unknown key '") + kv.first + "' in " + where);
}

Config Config::from_value(const Value& root) {
  Config c;
  // The reference rejects unknown top-level fields (serde deny_unknown_fields,
  // src/mccs/src/config.rs:74-76); so does this loader.
  check_keys(root,
             {"control", "comm_default_config", "comm_global_config", "addrs", "listen_port",
              "mccs_daemon_basename", "mccs_daemon_prefix", "qos_schedule", "qos",
              "comm_patterns_override", "b200", "limits"},
             "the top level");
  if (root.has("control")) {
    const Value& t = root["control"];
    c.control_prefix = t["prefix"].as_string(c.control_prefix);
    c.control_path = t["path"].as_string(c.control_path);
  }
  c.daemon_prefix = root["mccs_daemon_prefix"].as_string(c.daemon_prefix);
  c.daemon_basename = root["mccs_daemon_basename"].as_string(c.daemon_basename);
  for (const Value& a : root["addrs"].items()) c.addrs.push_back(a.as_string());
  c.listen_port = (int)root["listen_port"].as_int(c.listen_port);
  if (root.has("comm_default_config")) {
    const Value& t = root["comm_default_config"];
    if (t.has("buffer_sizes")) {
      c.buffer_sizes.clear();
      for (const Value& b : t["buffer_sizes"].items()) c.buffer_sizes.push_back((uint64_t)b.as_int());
      if (c.buffer_sizes.empty()) throw std::runtime_error("buffer_sizes must not be empty");
    }
    c.channel_count = (int)t["channel_count"].as_int(c.channel_count);
    if (c.channel_count < 1 || c.channel_count > 32) throw std::runtime_error("channel_count out of range 1..32");
  }
  c.comm_global_config = root["comm_global_config"];
  if (root.has("qos_schedule")) {
    const Value& q = root["qos_schedule"];
    c.qos_epoch_us = (uint64_t)q["epoch_microsecs"].as_int();
    for (const auto& kv : q["schedule"].fields()) {
      QosIntervalConfig qi;
      for (const Value& iv : kv.second["intervals"].items()) {
        if (iv.size() != 2) throw std::runtime_error("qos interval must be [start, end]");
        qi.intervals.push_back({(uint64_t)iv.at(0).as_int(), (uint64_t)iv.at(1).as_int()});
      }
      std::string mode = kv.second["mode"].as_string("Allow");
      if (mode != "Allow" && mode != "Deny") throw std::runtime_error("qos mode must be Allow or Deny");
      qi.allow = mode == "Allow";
      qi.enforce_step = (int)kv.second["enforce_step"].as_int(0);
      c.qos_schedule[(uint32_t)std::stoul(kv.first)] = qi;
    }
  }
  if (root.has("qos")) {
    const Value& q = root["qos"];
    c.qos_cta_budget = (int)q["cta_budget"].as_int(c.qos_cta_budget);
    c.qos_max_outstanding_bytes = (uint64_t)q["max_outstanding_bytes"].as_int((int64_t)c.qos_max_outstanding_bytes);
    c.qos_active_window_us = (uint64_t)q["active_window_us"].as_int((int64_t)c.qos_active_window_us);
    c.qos_sm_limit = (int)q["sm_limit"].as_int(c.qos_sm_limit);
    for (const auto& kv : q["tenants"].fields()) {
      QosTenantConfig t;
      t.weight = kv.second["weight"].as_double(1.0);
      t.priority = (int)kv.second["priority"].as_int(0);
      t.cta_quota = (int)kv.second["cta_quota"].as_int(0);
      if (t.weight <= 0) throw std::runtime_error("tenant weight must be positive");
      c.qos_tenants[(uint32_t)std::stoul(kv.first)] = t;
    }
  }
  for (const Value& p : root["comm_patterns_override"].items()) c.overrides.push_back(parse_pattern(p));
  if (root.has("limits")) {
    const Value& l = root["limits"];
    check_keys(l, {"max_clients", "max_allocations_per_client", "max_bytes_per_client", "max_communicators_per_client"}, "[limits]");
    c.max_clients = (int)l["max_clients"].as_int(c.max_clients);
    c.max_allocations_per_client = (int)l["max_allocations_per_client"].as_int(c.max_allocations_per_client);
    c.max_bytes_per_client = (uint64_t)l["max_bytes_per_client"].as_int((int64_t)c.max_bytes_per_client);
    c.max_communicators_per_client = (int)l["max_communicators_per_client"].as_int(c.max_communicators_per_client);
    if (c.max_clients < 0 || c.max_allocations_per_client < 0 || c.max_communicators_per_client < 0)
      throw std::runtime_error("[limits] values must not be negative");
  }
  if (root.has("b200")) {
    const Value& b = root["b200"];
    check_keys(b,
               {"transport", "nvls", "vmm", "sync", "wait_timeout_ms", "tuning_file", "trace", "trace_file",
                "host_devices", "force_host_backend", "idle_sleep_us", "idle_spin_us", "pin_threads", "init_timeout_ms", "fuse_allreduce", "client_nvls",
                "single_through_fused", "skip_start_barrier", "kernel_writes_done", "host_kernels",
                "hybrid_nvls_permille", "hybrid_nvls_ctas", "launch", "nvls_unroll", "pack_bytes", "host_no_peer_access"},
               "[b200]");
    c.transport = b["transport"].as_string(c.transport);
    if (c.transport != "auto" && c.transport != "nvlink" && c.transport != "host_staged")
      throw std::runtime_error("b200.transport must be auto, nvlink or host_staged");
    c.nvls = b["nvls"].as_bool(c.nvls);
    c.vmm = b["vmm"].as_bool(c.vmm);
    c.sync = b["sync"].as_string(c.sync);
    if (c.sync != "auto" && c.sync != "events" && c.sync != "memops")
      throw std::runtime_error("b200.sync must be auto, events or memops");
    c.launch = b["launch"].as_string(c.launch);
    if (c.launch != "auto" && c.launch != "daemon" && c.launch != "client") throw std::runtime_error("b200.launch must be auto, daemon or client");
    c.wait_timeout_ms = (uint64_t)b["wait_timeout_ms"].as_int((int64_t)c.wait_timeout_ms);
    c.tuning_file = b["tuning_file"].as_string();
    c.trace = b["trace"].as_bool(c.trace);
    c.trace_file = b["trace_file"].as_string();
    c.host_devices = (int)b["host_devices"].as_int(c.host_devices);
    if (b.has("host_no_peer_access"))
      for (const Value& pr : b["host_no_peer_access"].items()) {
        if (pr.size() != 2) throw std::runtime_error("b200.host_no_peer_access must be a list of [a, b] device pairs");
        c.host_no_peer_access.push_back({(int)pr.at(0).as_int(), (int)pr.at(1).as_int()});
      }
    c.force_host_backend = b["force_host_backend"].as_bool(c.force_host_backend);
    c.host_kernels = b["host_kernels"].as_string(c.host_kernels);
    if (c.host_kernels != "loops" && c.host_kernels != "emulated")
      throw std::runtime_error("b200.host_kernels must be loops or emulated");
    c.idle_sleep_us = (int)b["idle_sleep_us"].as_int(c.idle_sleep_us);
    c.idle_spin_us = (int)b["idle_spin_us"].as_int(c.idle_spin_us);
    c.pin_threads = b["pin_threads"].as_bool(c.pin_threads);
    c.init_timeout_ms = (uint64_t)b["init_timeout_ms"].as_int((int64_t)c.init_timeout_ms);
    c.hybrid_nvls_permille = (int)b["hybrid_nvls_permille"].as_int(c.hybrid_nvls_permille);
    c.hybrid_nvls_ctas = (int)b["hybrid_nvls_ctas"].as_int(c.hybrid_nvls_ctas);
    c.nvls_unroll = (int)b["nvls_unroll"].as_int(c.nvls_unroll);
    if (c.nvls_unroll != 4 && c.nvls_unroll != 8) throw std::runtime_error("b200.nvls_unroll must be 4 or 8");
    c.pack_bytes = (int)b["pack_bytes"].as_int(c.pack_bytes);
    if (c.pack_bytes != 16 && c.pack_bytes != 32) throw std::runtime_error("b200.pack_bytes must be 16 or 32");
    if (c.hybrid_nvls_permille < 0 || c.hybrid_nvls_permille > 1000 || c.hybrid_nvls_ctas < 0 || c.hybrid_nvls_ctas > kMaxCtas)
      throw std::runtime_error("b200.hybrid_nvls_permille must be 0..1000 and hybrid_nvls_ctas 0..148");
    c.single_through_fused = b["single_through_fused"].as_bool(c.single_through_fused);
    c.skip_start_barrier = b["skip_start_barrier"].as_bool(c.skip_start_barrier);
    c.kernel_writes_done = b["kernel_writes_done"].as_bool(c.kernel_writes_done);
    c.client_nvls = b["client_nvls"].as_bool(c.client_nvls);
    c.fuse_allreduce = (int)b["fuse_allreduce"].as_int(c.fuse_allreduce);
    if (c.fuse_allreduce < 1 || c.fuse_allreduce > kMaxBatch)
      throw std::runtime_error("b200.fuse_allreduce must be between 1 and " + std::to_string(kMaxBatch));
  }
  return c;
}

Config Config::from_string(const std::string& toml) { return from_value(parse_toml(toml)); }
Config Config::from_file(const std::string& path) { return from_string(read_text_file(path)); }

}  // namespace mccs
