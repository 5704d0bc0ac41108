// Admin tool for live reconfiguration, the reference's ring_config
// (src/mccs_examples/ring_config/src/main.rs:36-58): reads a TOML file with
// `mccs_addrs`, `mccs_port` and `[[comm_patterns_reconfig]]` entries (the format of
// eval/dynamic-config/reconfig-patch.toml) and sends the command to every daemon
// listed. Entries may also carry `allreduce_algo`, `allgather_algo` and `ctas`.
//   ring_config --config patch.toml [--port P] [--addr A]
//   ring_config --stats [--port P]            (prints the daemon's statistics)
//   ring_config --hwinfo [--port P]           (devices, CPU affinity, peer access, NVLS)
#include <stdio.h>
#include <stdlib.h>

#include <string>
#include <vector>

#include "../common/value.h"
#include "app_common.h"

int main(int argc, char** argv) {
  app::Options o(argc, argv, {"stats", "hwinfo"});
  o.require({}, "usage: ring_config --config patch.toml [--port P] [--addr A] | --stats | --hwinfo");
  std::vector<std::string> addrs;
  int port = (int)o.num("port", 5000);
  mccs::Value body = mccs::Value::object();
  int type = 1;
  if (o.flag("stats") || o.flag("hwinfo")) {
    body.set("cmd", o.flag("stats") ? "stats" : "hwinfo");
    type = 2;
  } else {
    if (!o.has("config")) { fprintf(stderr, "usage: ring_config --config patch.toml [--port P] [--addr A] | --stats | --hwinfo\n"); return 2; }
    mccs::Value cfg;
    try {
      cfg = mccs::parse_toml(mccs::read_text_file(o.str("config")));
    } catch (const std::exception& e) {
      fprintf(stderr, "ring_config: %s\n", e.what());
      return 2;
    }
    for (const mccs::Value& a : cfg["mccs_addrs"].items()) addrs.push_back(a.as_string());
    if (cfg.has("mccs_port") && !o.has("port")) port = (int)cfg["mccs_port"].as_int();
    body.set("comm_patterns_reconfig", cfg["comm_patterns_reconfig"]);
  }
  if (o.has("addr")) addrs = {o.str("addr")};
  if (addrs.empty()) addrs.push_back("127.0.0.1");
  int failures = 0;
  std::vector<char> reply(1 << 22);
  for (const std::string& a : addrs) {
    mccsResult_t r = mccsAdminRequest(a.c_str(), port, type, body.to_json().c_str(), reply.data(), reply.size());
    if (r != mccsSuccess) {
      fprintf(stderr, "%s:%d: %s\n", a.c_str(), port, mccsGetErrorString(r));
      failures++;
      continue;
    }
    printf("%s:%d: %s\n", a.c_str(), port, reply.data());
  }
  return failures ? 1 : 0;
}
