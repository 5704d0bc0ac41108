// mccsd: the per-host service daemon.
//   mccsd [--config mccs.toml] [--host <index>] [--check]
// Same command line as the reference binary (src/mccs/src/main.rs:16-24): the
// configuration defaults to ./mccs.toml when that file exists; --host selects this
// machine's entry of `addrs` and is only informational inside a single box. SIGINT
// and SIGTERM end the control loop (main.rs:26-31,67-73); clients then see their
// control connection close. --check reads the configuration, prints what it understood
// and exits without starting anything (0 = the file is acceptable).
#include <signal.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include "../common/log.h"
#include "daemon.h"

static mccs::Daemon* g_daemon = nullptr;
static void on_signal(int) {
  if (g_daemon) g_daemon->stop_requested();
}

int main(int argc, char** argv) {
  std::string config_path;
  int host = 0;
  bool check_only = false;
  for (int i = 1; i < argc; i++) {
    if ((!strcmp(argv[i], "--config") || !strcmp(argv[i], "-c")) && i + 1 < argc) config_path = argv[++i];
    else if ((!strcmp(argv[i], "--host") || !strcmp(argv[i], "-h")) && i + 1 < argc) host = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--check")) check_only = true;
    else if (!strcmp(argv[i], "--help")) {
      printf("usage: mccsd [--config mccs.toml] [--host <index>] [--check]\n");
      return 0;
    } else {
      fprintf(stderr, "mccsd: unknown argument '%s'\n", argv[i]);
      return 2;
    }
  }
  if (mccs::log_level() < mccs::kLogInfo && !getenv("MCCS_LOG")) mccs::set_log_level(mccs::kLogInfo);
  mccs::Config cfg;
  try {
    if (!config_path.empty()) cfg = mccs::Config::from_file(config_path);
    else if (access("mccs.toml", R_OK) == 0) cfg = mccs::Config::from_file("mccs.toml");
  } catch (const std::exception& e) {
    fprintf(stderr, "mccsd: %s\n", e.what());
    return 2;
  }
  if (check_only) {
    printf("configuration ok: control %s/%s, admin port %d, %d ring channel(s), buffers of %llu bytes, transport %s, launch %s, "
           "%zu tenant policies, %zu communicator overrides, %zu window schedules\n",
           cfg.control_prefix.c_str(), cfg.control_path.c_str(), cfg.listen_port, cfg.channel_count,
           (unsigned long long)cfg.buffer_sizes[0], cfg.transport.c_str(), cfg.launch.c_str(), cfg.qos_tenants.size(),
           cfg.overrides.size(), cfg.qos_schedule.size());
    return 0;
  }
  LOG_INFO("mccsd starting (host index %d)", host);
  mccs::Daemon daemon;
  std::string err;
  if (daemon.start(cfg, &err) != 0) {
    fprintf(stderr, "mccsd: %s\n", err.c_str());
    return 1;
  }
  g_daemon = &daemon;
  struct sigaction sa;
  memset(&sa, 0, sizeof sa);
  sa.sa_handler = on_signal;
  sigaction(SIGINT, &sa, nullptr);
  sigaction(SIGTERM, &sa, nullptr);
  // Tells a parent that spawned us (tests, launch scripts) that clients may connect.
  printf("MCCSD_READY control=%s admin_port=%d backend=%s\n", daemon.control_path().c_str(), daemon.admin_port(),
         daemon.backend()->kind() == mccs::proto::kBackendCuda ? "cuda" : "host");
  fflush(stdout);
  daemon.run();
  g_daemon = nullptr;
  daemon.stop();
  LOG_INFO("mccsd stopped");
  return 0;
}
