// Host-side unit tests of the native code (no GPU needed): IPC rings, fd passing,
// TOML/JSON, configuration schema, planner rules, ring step accounting, the QoS
// arbiter on a simulated clock, CPU list parsing. The reference has unit tests only
// for its in-process channel (src/ipc/core/src/channel/flavors/sequential.rs:85-108).
// Run by tests/test_native_host.py; exit code = number of failed checks.
#include <stdio.h>
#include <string.h>
#include <sys/wait.h>
#include <unistd.h>

#include <atomic>
#include <thread>

#include "../common/protocol.h"
#include "../common/value.h"
#include "../daemon/config.h"
#include "../daemon/planner.h"
#include "../daemon/qos.h"
#include "../daemon/runtime.h"
#include "../daemon/trace.h"
#include "../daemon/transport.h"
#include "../ipc/shm_ring.h"
#include "../ipc/uds.h"
#include "../kernels/dev_types.h"

using namespace mccs;

static int g_failed = 0, g_checks = 0;
#define CHECK(cond)                                                      \
  do {                                                                   \
    g_checks++;                                                          \
    if (!(cond)) { g_failed++; printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond); } \
  } while (0)

static void test_ring() {
  const size_t bytes = ipc::Ring::bytes_needed(8, 64);
  std::vector<uint8_t> mem(bytes + 64);
  void* base = (void*)(((uintptr_t)mem.data() + 63) & ~(uintptr_t)63);
  ipc::Ring prod, cons;
  prod.init(base, 8, 64);
  cons.attach(base);
  uint8_t item[64], out[64];
  CHECK(cons.empty());
  CHECK(!cons.try_pop(out));
  for (int i = 0; i < 8; i++) { memset(item, i, 64); CHECK(prod.try_push(item)); }
  CHECK(!prod.try_push(item));   // full
  CHECK(cons.size() == 8);
  for (int i = 0; i < 8; i++) { CHECK(cons.try_pop(out)); CHECK(out[0] == i && out[63] == i); }
  // wrap-around under concurrency
  const int total = 200000;
  std::thread t([&] {
    uint8_t it[64];
    for (int i = 0; i < total;) { memcpy(it, &i, 4); if (prod.try_push(it)) i++; }
  });
  int expect = 0, bad = 0;
  while (expect < total) {
    if (cons.try_pop(out)) { int v; memcpy(&v, out, 4); bad += v != expect; expect++; }
  }
  t.join();
  CHECK(bad == 0);
}

static void test_uds_fd_passing() {
  char path[64];
  snprintf(path, sizeof path, "/tmp/mccs-ut-%d.sock", (int)getpid());
  int lfd = ipc::uds_listen(path);
  CHECK(lfd >= 0);
  pid_t pid = fork();
  if (pid == 0) {
    int fd = ipc::uds_connect(path);
    int mfd = ipc::memfd_make("ut", 4096);
    char* p = (char*)ipc::map_shared(mfd, 4096);
    strcpy(p, "through the fd");
    const char msg[] = "hello";
    ipc::uds_send(fd, msg, sizeof msg, &mfd, 1);
    char ack[8];
    ipc::wait_readable(fd, 2000);
    ipc::uds_recv(fd, ack, sizeof ack);
    _exit(0);
  }
  int cfd = -1;
  for (int i = 0; i < 200 && cfd < 0; i++) { cfd = ipc::uds_accept(lfd); if (cfd < 0) usleep(5000); }
  CHECK(cfd >= 0);
  ipc::PeerCred cred{};
  CHECK(ipc::uds_peer_cred(cfd, &cred) == 0);
  CHECK(cred.pid == pid);
  char buf[32];
  std::vector<int> fds;
  CHECK(ipc::wait_readable(cfd, 2000) == 1);
  ssize_t n = ipc::uds_recv(cfd, buf, sizeof buf, &fds);
  CHECK(n == 6 && !strcmp(buf, "hello"));
  CHECK(fds.size() == 1);
  if (!fds.empty()) {
    char* p = (char*)ipc::map_shared(fds[0], 4096);
    CHECK(p && !strcmp(p, "through the fd"));
    close(fds[0]);
  }
  ipc::uds_send(cfd, "ok", 3);
  int st = 0;
  waitpid(pid, &st, 0);
  // Peer death shows as end of stream.
  CHECK(ipc::wait_readable(cfd, 1000) == 1);
  CHECK(ipc::uds_recv(cfd, buf, sizeof buf) == 0);
  close(cfd);
  close(lfd);
  unlink(path);
}

static void test_toml_json() {
  const char* text =
      "a = 1\nname = \"x y\" # comment\nf = 2.5\nflag = true\narr = [1, 2,\n 3]\n"
      "[t.sub]\nk = 'lit'\n[[items]]\nid = 1\nring = [0,1]\n[[items]]\nid = 2\n"
      "inline = { p = 1, q = [ [1,2,3], [4,5,6] ], s = \"z\" }\n[qos_schedule.schedule.99]\nmode = \"Allow\"\n";
  Value v = parse_toml(text);
  CHECK(v["a"].as_int() == 1);
  CHECK(v["name"].as_string() == "x y");
  CHECK(v["f"].as_double() == 2.5);
  CHECK(v["flag"].as_bool());
  CHECK(v["arr"].size() == 3 && v["arr"].at(2).as_int() == 3);
  CHECK(v["t"]["sub"]["k"].as_string() == "lit");
  CHECK(v["items"].size() == 2 && v["items"].at(1)["id"].as_int() == 2);
  CHECK(v["items"].at(1)["inline"]["q"].at(1).at(2).as_int() == 6);
  CHECK(v["qos_schedule"]["schedule"]["99"]["mode"].as_string() == "Allow");
  Value back = parse_json(v.to_json());
  CHECK(back.to_json() == v.to_json());
  bool threw = false;
  try { parse_toml("a = \n"); } catch (const ParseError&) { threw = true; }
  CHECK(threw);
  threw = false;
  try { parse_toml("a = 1\na = 2\n"); } catch (const ParseError&) { threw = true; }
  CHECK(threw);
  CHECK(parse_json("{\"k\": [1, 2.5, \"s\\n\", null, true]}")["k"].at(2).as_string() == "s\n");
}

static void test_config() {
  // The reference's shipped file must load unchanged.
  Config c = Config::from_string(
      "mccs_daemon_basename = \"mccs-deamon\"\nmccs_daemon_prefix = \"/tmp/mccs-${USER}\"\n"
      "addrs = [\"0.0.0.0\", \"192.168.211.2\"]\nlisten_port = 5000\n"
      "[control]\nprefix = \"/tmp/mccs-${USER}\"\npath = \"control.sock\"\n"
      "[comm_default_config]\nbuffer_sizes = [4194304]\nchannel_count = 2\n"
      "[comm_global_config]\n[comm_global_config.net_rdma]\ngid_index = 3\n[comm_global_config.shm]\nlocality = \"Sender\"\n"
      "[qos_schedule]\nepoch_microsecs = 85000\n[qos_schedule.schedule.99]\nintervals = [[0, 35000]]\nmode = \"Allow\"\n"
      "[qos_schedule.schedule.100]\nintervals = [[35000, 69000]]\nmode = \"Deny\"\nenforce_step = 2\n"
      "[[comm_patterns_override]]\ncommunicator_id = 138\n"
      "channels = [ { channel_id = 0, ring = [0,1,2,3], udp_sport = [[3,4,49200]], net_dev = \"mlx5_0\" },\n"
      "             { channel_id = 1, ring = [3,2,1,0] } ]\nib_traffic_class = 106\n");
  CHECK(c.channel_count == 2);
  CHECK(c.buffer_sizes[0] == 4194304);
  CHECK(c.qos_epoch_us == 85000);
  CHECK(c.qos_schedule.size() == 2);
  CHECK(c.qos_schedule[99].allow && c.qos_schedule[99].intervals[0].second == 35000);
  CHECK(!c.qos_schedule[100].allow && c.qos_schedule[100].enforce_step == 2);
  CHECK(c.overrides.size() == 1);
  CHECK(c.find_override(138) && c.find_override(138)->channels[1].ring[0] == 3);
  CHECK(c.find_override(138)->ib_traffic_class == 106);
  CHECK(!c.find_override(7));
  CHECK(c.control_socket_path().find("${") == std::string::npos);
  CHECK(c.control_socket_path().rfind("/control.sock") != std::string::npos);
  bool threw = false;
  try { Config::from_string("bogus_key = 1\n"); } catch (const std::exception&) { threw = true; }
  CHECK(threw);   // unknown top-level keys are rejected
  Config lim = Config::from_string("[limits]\nmax_clients = 3\nmax_bytes_per_client = 1073741824\n");
  CHECK(lim.max_clients == 3 && lim.max_bytes_per_client == (1ull << 30) && lim.max_allocations_per_client == 65536 &&
        lim.max_communicators_per_client == 1024);
  bool refused = false;
  try { Config::from_string("[limits]\nmax_clients = -1\n"); } catch (const std::exception&) { refused = true; }
  CHECK(refused);
  Config d = Config::from_string("[b200]\ntransport = \"host_staged\"\nwait_timeout_ms = 500\n[qos.tenants.7]\nweight = 2.0\npriority = 1\n");
  CHECK(d.transport == "host_staged" && d.wait_timeout_ms == 500);
  CHECK(d.qos_tenants[7].weight == 2.0 && d.qos_tenants[7].priority == 1);
}

static void test_planner() {
  Planner p;
  p.load_defaults(true);
  PlanInput in;
  in.kind = kAllReduce; in.nranks = 8; in.dtype = kBfloat16; in.op = kSum;
  in.count = 256u << 20; in.nvls_possible = true;
  Plan pl = p.plan(in);
  CHECK(pl.status == 0 && pl.variant == kArNvlsTwo && pl.needs_mc_send && pl.needs_mc_recv);
  in.nvls_possible = false;
  pl = p.plan(in);
  CHECK(pl.variant == kArTwoShot);
  // small + out of place: one-shot family; in place forbids it
  in.count = 4096; in.nvls_possible = true;
  CHECK(p.plan(in).variant == kArNvlsOne);
  in.in_place = true;
  CHECK(p.plan(in).variant != kArNvlsOne && p.plan(in).variant != kArOneShot);
  in.in_place = false;
  // integer types and max never go to NVLS
  in.dtype = kInt32; in.count = 1 << 24;
  CHECK(!variant_is_nvls(p.plan(in).variant));
  in.dtype = kFloat32; in.op = kMax;
  CHECK(!variant_is_nvls(p.plan(in).variant));
  in.op = kSum;
  // host-staged transport: ring only, channel count from the configuration
  in.host_staged = true; in.ring_channels = 2;
  pl = p.plan(in);
  CHECK(pl.variant == kArRing && pl.dims.ctas == 2);
  in.count = 1024;   // tiny: one channel, small CTA (plan.rs:602-635)
  pl = p.plan(in);
  CHECK(pl.variant == kArRing && pl.dims.ctas == 1 && pl.dims.threads >= 64);
  in.host_staged = false;
  // requested variant honoured when feasible, replaced (with a note) when not
  in.count = 1 << 20; in.requested_variant = kArRing;
  CHECK(p.plan(in).variant == kArRing);
  in.requested_variant = kAgPull;
  pl = p.plan(in);
  CHECK(pl.variant != kAgPull && !pl.note.empty());
  in.requested_variant = kAuto;
  // the hybrid variant is only ever taken on request, needs both multicast mappings, and
  // falls back (with a note) where the switch path is not available
  in.count = 64u << 20; in.nvls_possible = true; in.requested_variant = kArHybrid;
  pl = p.plan(in);
  CHECK(pl.status == 0 && pl.variant == kArHybrid && pl.needs_mc_send && pl.needs_mc_recv && pl.dims.ctas == 72);
  in.nvls_possible = false;
  pl = p.plan(in);
  CHECK(pl.variant == kArTwoShot && !pl.note.empty());
  in.nvls_possible = true; in.requested_variant = kAuto;
  CHECK(Planner::variant_from_name("ar_hybrid") == kArHybrid);
  // reduce-scatter: its own table; in the switch only for float sums on aligned blocks;
  // variants of other collectives are refused for it and its variants for them
  {
    PlanInput rs = in;
    rs.kind = kReduceScatter; rs.count = 8u << 20; rs.requested_variant = kAuto; rs.in_place = true;
    Plan q = p.plan(rs);
    CHECK(q.status == 0 && q.variant == kRsNvls && q.needs_mc_send && !q.needs_mc_recv);
    CHECK(q.bytes == (uint64_t)(8u << 20) * (uint64_t)rs.nranks * (uint64_t)dtype_size(rs.dtype));
    rs.nvls_possible = false;
    q = p.plan(rs);
    CHECK(q.status == 0 && q.variant == kRsDirect);
    rs.nvls_possible = true; rs.dtype = kInt32;
    CHECK(p.plan(rs).variant == kRsDirect);
    rs.dtype = in.dtype; rs.requested_variant = kArTwoShot;
    q = p.plan(rs);
    CHECK(q.status == 0 && (q.variant == kRsNvls || q.variant == kRsDirect) && !q.note.empty());
    PlanInput ar = in;
    ar.requested_variant = kRsDirect;
    q = p.plan(ar);
    CHECK(q.status == 0 && q.variant != kRsDirect && !q.note.empty());
    rs.requested_variant = kAuto; rs.nranks = 1;
    CHECK(p.plan(rs).variant == kLocalCopy);
  }
  // QoS cap and override
  in.count = 256u << 20; in.cta_cap = 5;
  CHECK(p.plan(in).dims.ctas == 5);
  in.cta_cap = 0; in.requested_ctas = 24;
  CHECK(p.plan(in).dims.ctas == 24);
  in.requested_ctas = 0;
  // single rank
  in.nranks = 1;
  CHECK(p.plan(in).variant == kLocalCopy);
  // all-gather
  PlanInput g;
  g.kind = kAllGather; g.nranks = 4; g.count = 16 << 10; g.nvls_possible = true;
  CHECK(p.plan(g).variant == kAgNvls);
  g.aligned16 = false;
  CHECK(p.plan(g).variant != kAgNvls);
  // tuning table round trip and override
  std::string err;
  Value t = parse_json("{\"allreduce\": {\"8\": [[65536, \"ar_oneshot\", 4, 256], [-1, \"ar_twoshot\", 48, 512]]}}");
  CHECK(p.load_json(t, &err));
  PlanInput q;
  q.kind = kAllReduce; q.nranks = 8; q.dtype = kFloat32; q.count = 1 << 24;
  pl = p.plan(q);
  CHECK(pl.variant == kArTwoShot && pl.dims.ctas == 48);
  q.count = 1024;
  pl = p.plan(q);
  CHECK(pl.variant == kArOneShot && pl.dims.threads == 256);
  CHECK(!p.load_json(parse_json("{\"allreduce\": {\"8\": [[1, \"nope\", 4]]}}"), &err));
  {
    // parsers refuse absurd nesting instead of recursing until the stack runs out
    std::string deep(100000, '[');
    bool threw = false;
    try { parse_json(deep); } catch (const std::exception&) { threw = true; }
    CHECK(threw);
    threw = false;
    try { parse_toml("a = " + deep); } catch (const std::exception&) { threw = true; }
    CHECK(threw);
  }
  Planner p2;
  CHECK(p2.load_json(p.to_json(), &err));
  CHECK(p2.to_json().to_json() == p.to_json().to_json());
}

// Transport selection per connection (the reference's "first can_connect wins",
// src/mccs/src/transport/setup.rs:346-361), against a table standing in for the machine.
static void test_transports() {
  bool access[4][4];
  for (auto& row : access) for (bool& x : row) x = true;
  bool multicast = true;
  TransportEnv env;
  env.peer_access = [&](int a, int b) { return access[a][b]; };
  env.multicast = [&](int) { return multicast; };
  const std::vector<int> four = {0, 1, 2, 3};

  // a healthy NVSwitch box: every pair through the switch, everything can run, scratch on the devices
  TransportCatalog automatic("auto");
  CHECK(automatic.transports().size() == 3);
  ConnectionTable t = connect_all(automatic, env, four);
  CHECK(t.complete() && t.all(kTransportNvls) && !t.scratch_in_host_memory());
  CHECK(t.carries(kArNvlsTwo) && t.carries(kArTwoShot) && t.carries(kArRing) && t.carries(kAgNvls));
  CHECK(t.describe() == "nvls");

  // multicast switched off (configuration) or not supported: plain peer memory
  env.nvls_enabled = false;
  t = connect_all(automatic, env, four);
  CHECK(t.all(kTransportNvlinkP2P) && t.carries(kArTwoShot) && t.carries(kAgPush) && !t.carries(kArNvlsTwo) && !t.carries(kArHybrid));
  env.nvls_enabled = true;
  multicast = false;
  t = connect_all(automatic, env, four);
  CHECK(t.all(kTransportNvlinkP2P) && !t.carries(kRsNvls) && t.carries(kRsDirect));
  multicast = true;

  // one pair of GPUs without peer access: that connection (both directions) is host-staged,
  // the others are not; the communicator keeps its scratch in host memory and is limited to
  // what every connection carries, the FIFO rings
  access[1][2] = false;
  t = connect_all(automatic, env, four);
  CHECK(t.complete());
  CHECK(t.conn[1][2]->kind() == kTransportHostStaged && t.conn[2][1]->kind() == kTransportHostStaged);
  CHECK(t.conn[0][1]->kind() == kTransportNvls && t.conn[3][2]->kind() == kTransportNvls);
  CHECK(t.any(kTransportHostStaged) && !t.all(kTransportHostStaged) && t.scratch_in_host_memory());
  CHECK(t.carries(kArRing) && t.carries(kAgRing) && !t.carries(kArTwoShot) && !t.carries(kAgPull) && !t.carries(kArNvlsTwo));
  CHECK(t.carried_variants() == ((1u << kArRing) | (1u << kAgRing)));
  CHECK(t.describe() == "host_staged x2, nvls x10");
  // ... and the planner follows: whatever is asked for, a ring runs
  {
    Planner p;
    p.load_defaults(true);
    PlanInput in;
    in.kind = kAllReduce; in.nranks = 4; in.count = 1 << 22; in.dtype = kFloat32;
    in.carried_variants = t.carried_variants();
    in.host_staged = t.scratch_in_host_memory();
    in.p2p_possible = t.carries(kArTwoShot);
    in.ring_channels = 2;
    CHECK(p.plan(in).variant == kArRing);
    in.requested_variant = kArTwoShot;
    Plan pl = p.plan(in);
    CHECK(pl.status == 0 && pl.variant == kArRing && !pl.note.empty());
    in.kind = kAllGather; in.requested_variant = kAuto;
    CHECK(p.plan(in).variant == kAgRing);
  }
  // a communicator that does not include the pair is not affected
  t = connect_all(automatic, env, {0, 1, 3});
  CHECK(t.all(kTransportNvls) && !t.scratch_in_host_memory());

  // transport = "nvlink": no host-staged fall-back, the pair stays unconnected and is named
  TransportCatalog nvlink_only("nvlink");
  t = connect_all(nvlink_only, env, four);
  CHECK(!t.complete() && t.unconnected_from == 1 && t.unconnected_to == 2);
  access[1][2] = true;
  CHECK(connect_all(nvlink_only, env, four).complete());

  // transport = "host_staged": every connection, whatever the machine could do
  TransportCatalog staged("host_staged");
  t = connect_all(staged, env, four);
  CHECK(t.all(kTransportHostStaged) && t.scratch_in_host_memory() && t.carries(kArRing) && !t.carries(kArOneShot));

  // ranks that share a device (the single-GPU form) are peers by construction, never multicast
  t = connect_all(automatic, env, {0, 0, 0});
  CHECK(t.all(kTransportNvlinkP2P) && t.carries(kArTwoShot) && !t.carries(kArNvlsOne));
  // a single rank has no connections and no limits
  t = connect_all(automatic, env, {2});
  CHECK(t.complete() && t.carries(kLocalCopy) && !t.scratch_in_host_memory() && t.describe() == "no connections");
}

static void test_ring_steps() {
  // 8 ranks, 1 channel, 512 KiB slots: a 16 MiB fp32 all-reduce needs
  // ceil(4Mi elems / (131072*8)) = 4 loops of 2*(8-1) steps.
  CHECK(ring_loops(kAllReduce, 4u << 20, 4, 8, 1, 512 << 10) == 4);
  CHECK(ring_steps_per_channel(kAllReduce, 4u << 20, 4, 8, 1, 512 << 10) == 4 * 14);
  CHECK(ring_steps_per_channel(kAllReduce, 4u << 20, 4, 8, 2, 512 << 10) == 2 * 14);
  CHECK(ring_steps_per_channel(kAllGather, 1 << 20, 1, 4, 2, 512 << 10) == 1 * 3);
  CHECK(ring_steps_per_channel(kAllReduce, 0, 4, 8, 1, 512 << 10) == 0);
  CHECK(ring_steps_per_channel(kAllReduce, 1, 2, 2, 1, 512 << 10) == 2);
}

static void test_qos() {
  // Windows: the reference's Allow/Deny semantics on now % epoch.
  QosIntervalConfig allow;
  allow.intervals = {{0, 35000}};
  CHECK(QosArbiter::window_allows(allow, 85000, 10, 0));
  CHECK(!QosArbiter::window_allows(allow, 85000, 40000, 0));
  CHECK(QosArbiter::window_allows(allow, 85000, 85000 + 34999, 0));
  QosIntervalConfig deny = allow;
  deny.allow = false;
  CHECK(!QosArbiter::window_allows(deny, 85000, 10, 0));
  CHECK(QosArbiter::window_allows(deny, 85000, 40000, 0));
  allow.enforce_step = 2;
  CHECK(QosArbiter::window_allows(allow, 85000, 40000, 1));    // odd rounds are not gated
  CHECK(!QosArbiter::window_allows(allow, 85000, 40000, 2));

  Config cfg;
  cfg.qos_tenants[1].weight = 2.0;
  cfg.qos_tenants[2].weight = 1.0;
  cfg.qos_cta_budget = 60;
  cfg.qos_max_outstanding_bytes = 32u << 20;
  QosArbiter q;
  q.configure(cfg);
  q.tenant_register(1, {0, 1});
  q.tenant_register(2, {1, 2});
  q.tenant_register(3, {5});
  uint64_t now = 1000;
  // Alone: no cap, always admitted.
  CHECK(q.cta_cap(1, now) == 0);
  CHECK(q.admit(1, 8 << 20, now, 0) == kQosAdmit);
  q.complete(1, 8 << 20);
  // Contention: tenants 1 and 2 share device 1; tenant 3 does not take part.
  q.note_waiting(2, now);
  CHECK(q.contenders(1, now) == 1);
  CHECK(q.contenders(3, now) == 0);
  CHECK(q.cta_cap(1, now) == 40);   // 60 * 2/3
  CHECK(q.cta_cap(2, now) == 20);
  CHECK(q.cta_cap(3, now) == 0);
  CHECK(q.slice_bytes(1, now) > 0 && q.slice_bytes(3, now) == 0);
  // Weighted fair queueing: with both always backlogged, admitted bytes approach 2:1.
  uint64_t b1 = 0, b2 = 0;
  const uint64_t sz = 8 << 20;
  for (int round = 0; round < 300; round++) {
    now += 100;
    q.note_waiting(1, now);
    q.note_waiting(2, now);
    if (q.admit(1, sz, now, 0) == kQosAdmit) { b1 += sz; q.complete(1, sz); }
    q.note_waiting(1, now);
    if (q.admit(2, sz, now, 0) == kQosAdmit) { b2 += sz; q.complete(2, sz); }
  }
  const double ratio = (double)b1 / (double)b2;
  CHECK(ratio > 1.7 && ratio < 2.3);
  // Backlog bound: outstanding bytes of a contended tenant are limited.
  QosArbiter r;
  r.configure(cfg);
  r.tenant_register(1, {0});
  r.tenant_register(2, {0});
  r.note_waiting(2, 10);
  int admitted = 0;
  for (int i = 0; i < 10; i++) admitted += r.admit(1, 16u << 20, 10, 0) == kQosAdmit;
  CHECK(admitted == 2);   // 32 MiB outstanding allowed
  r.complete(1, 16u << 20);
  CHECK(r.admit(1, 16u << 20, 11, 0) != kQosDeferBacklog);
  // Window schedule applied at admission.
  std::map<uint32_t, QosIntervalConfig> sched;
  sched[1].intervals = {{0, 1000}};
  r.set_schedule(10000, sched);
  r.complete(1, 64u << 20);
  // Tenant 2 was waiting all along and is behind in virtual time: it goes first.
  CHECK(r.admit(1, 1024, 12, 500) == kQosDeferFairness);
  CHECK(r.admit(2, 48u << 20, 12, 500) == kQosAdmit);
  r.complete(2, 48u << 20);
  CHECK(r.admit(1, 1024, 12, 5000) == kQosDeferWindow);
  CHECK(r.admit(1, 1024, 12, 10500) == kQosAdmit);
  r.set_enabled(false);
  CHECK(r.admit(1, 1024, 12, 5000) == kQosAdmit);
  CHECK(r.stats()["tenants"]["1"]["deferred_window"].as_int() == 1);
  // Residency: kernels that wait on each other must all get an SM. Tenants 1 and 2 share
  // GPU 0, tenant 3 sits on other GPUs; the limit is 148 CTAs per GPU.
  QosArbiter s;
  s.configure(cfg);
  s.set_enabled(false);                       // the rule holds with the arbiter switched off, too
  s.tenant_register(1, {0, 1});
  s.tenant_register(2, {0, 2});
  s.tenant_register(3, {4, 5});
  CHECK(s.admit(1, 1 << 20, 1, 0, 128) == kQosAdmit);
  CHECK(s.admit(2, 1 << 20, 1, 0, 64) == kQosDeferResidency);    // 128 + 64 > 148
  CHECK(s.admit(2, 1 << 20, 1, 0, 20) == kQosAdmit);             // 128 + 20 fits
  CHECK(s.admit(3, 1 << 20, 1, 0, 128) == kQosAdmit);            // no GPU in common with anybody
  CHECK(s.admit(1, 1 << 20, 2, 0, 128) == kQosAdmit);            // same size as what tenant 1 already has in flight
  CHECK(s.admit(2, 1 << 20, 2, 0, 21) == kQosDeferResidency);    // growing to 21 would make 149
  s.complete(1, 2 << 20);
  CHECK(s.admit(2, 1 << 20, 3, 0, 128) == kQosAdmit);            // tenant 1 has nothing in flight any more
  CHECK(s.admit(1, 1 << 20, 3, 0, 64) == kQosDeferResidency);
  s.complete(2, 2 << 20);
  CHECK(s.admit(1, 1 << 20, 4, 0, 200) == kQosAdmit);            // alone, even more CTAs than SMs are its own business
  CHECK(s.stats()["tenants"]["2"]["deferred_residency"].as_int() == 2);
  // Generation: moves on what can turn a deferral into an admission (a completion, another
  // tenant's admission, a policy change), so that a deferred request need not poll the lock.
  {
    QosArbiter q2;
    Config c2 = Config::from_string("[qos]\nmax_outstanding_bytes = 1048576\n");
    q2.configure(c2);
    q2.tenant_register(1, {0});
    q2.tenant_register(2, {0});
    const uint64_t g0 = q2.generation();
    CHECK(q2.admit(1, 1 << 20, 1000, 0, 8) == kQosAdmit);
    const uint64_t g1 = q2.generation();
    CHECK(g1 != g0);                                         // an admission
    q2.note_waiting(2, 1001);
    CHECK(q2.admit(1, 1 << 20, 1002, 0, 8) == kQosDeferBacklog);
    CHECK(q2.generation() == g1);                            // a deferral changes nothing
    q2.complete(1, 1 << 20);
    CHECK(q2.generation() != g1);                            // a completion
    const uint64_t g2 = q2.generation();
    QosTenantConfig tc;
    tc.weight = 3.0;
    q2.set_tenant(2, tc);
    CHECK(q2.generation() != g2);                            // a policy change
  }
}

// Forty tenants on one GPU, asked for the way the proxies do it: a request that was told to
// wait asks again only when the arbiter's generation moved or a short time went by. First on a
// simulated clock, in one thread (the figures are then exact: everybody is served, shares
// follow the weights, the number of questions stays within a small multiple of the
// admissions), then by eight threads on the real clock for the locking (shares then depend on
// how the machine schedules the threads and are not asked for).
static void test_qos_many_tenants() {
  constexpr int kTenants = 40, kThreads = 8, kPerThread = kTenants / kThreads;
  Config cfg;
  for (int t = 0; t < kTenants; t++) cfg.qos_tenants[(uint32_t)(100 + t)].weight = (double)(1 << (t % 3));   // 1, 2, 4
  cfg.qos_max_outstanding_bytes = 8u << 20;
  const uint64_t sz = 1 << 20;
  struct Asker { uint32_t id; bool deferred = false; uint64_t gen = 0, retry_us = 0; int inflight = 0; uint64_t bytes = 0; };
  auto ask = [&](QosArbiter& q, Asker& m, uint64_t now, uint64_t* asks, uint64_t* admissions) {
    if (m.inflight) {               // the "kernel" of the previous admission is through
      q.complete(m.id, sz);
      m.inflight = 0;
    }
    if (m.deferred && q.generation() == m.gen && now < m.retry_us) return;
    m.gen = q.generation();
    q.note_waiting(m.id, now);
    (*asks)++;
    if (q.admit(m.id, sz, now, 0, 4) == kQosAdmit) {
      m.deferred = false;
      m.inflight = 1;
      m.bytes += sz;
      (*admissions)++;
    } else {
      m.deferred = true;
      m.retry_us = now + 200;
    }
  };
  {
    QosArbiter q;
    q.configure(cfg);
    std::vector<Asker> all((size_t)kTenants);
    for (int t = 0; t < kTenants; t++) { all[(size_t)t].id = (uint32_t)(100 + t); q.tenant_register(all[(size_t)t].id, {0}); }
    // One round = what concurrent proxies do in one stretch of time: the transfers admitted
    // in the round before complete, every tenant has its next request waiting, and the
    // requests are put to the arbiter one after the other (starting with another tenant each
    // round).
    uint64_t asks = 0, admissions = 0, now = 1000;
    for (int round = 0; round < 20000; round++) {
      now += 10;
      for (Asker& m : all)
        if (m.inflight) { q.complete(m.id, sz); m.inflight = 0; }
      for (Asker& m : all) q.note_waiting(m.id, now);
      for (int k = 0; k < kTenants; k++) ask(q, all[(size_t)((round + k) % kTenants)], now, &asks, &admissions);
    }
    double by_weight[3] = {0, 0, 0};
    bool all_served = true;
    for (int t = 0; t < kTenants; t++) {
      all_served &= all[(size_t)t].bytes > 0;
      by_weight[t % 3] += (double)all[(size_t)t].bytes;
    }
    // classes 0, 1, 2 hold 14, 13 and 13 tenants of weight 1, 2 and 4
    const double per1 = by_weight[0] / 14, per2 = by_weight[1] / 13, per4 = by_weight[2] / 13;
    CHECK(all_served && admissions > 2000);
    CHECK(per2 / per1 > 1.8 && per2 / per1 < 2.2);
    CHECK(per4 / per1 > 3.6 && per4 / per1 < 4.4);
    CHECK(asks < 40 * admissions);
    if (getenv("MCCS_TEST_VERBOSE"))
      printf("qos, 40 tenants, simulated clock: %llu admissions, %llu questions, shares 1 : %.2f : %.2f\n",
             (unsigned long long)admissions, (unsigned long long)asks, per2 / per1, per4 / per1);
  }
  QosArbiter q;
  q.configure(cfg);
  for (int t = 0; t < kTenants; t++) q.tenant_register((uint32_t)(100 + t), {0});
  std::atomic<uint64_t> asks{0}, admissions{0};
  std::vector<uint64_t> bytes((size_t)kTenants, 0);
  const uint64_t t_end = monotonic_us() + 500000;
  std::vector<std::thread> threads;
  for (int w = 0; w < kThreads; w++)
    threads.emplace_back([&, w]() {
      Asker mine[kPerThread];
      for (int k = 0; k < kPerThread; k++) mine[k].id = (uint32_t)(100 + w * kPerThread + k);
      uint64_t my_asks = 0, my_admissions = 0;
      while (monotonic_us() < t_end)
        for (Asker& m : mine) ask(q, m, monotonic_us(), &my_asks, &my_admissions);
      for (Asker& m : mine) {
        if (m.inflight) q.complete(m.id, sz);
        bytes[(size_t)(m.id - 100)] = m.bytes;
      }
      asks.fetch_add(my_asks);
      admissions.fetch_add(my_admissions);
    });
  for (auto& t : threads) t.join();
  bool all_served = true;
  for (int t = 0; t < kTenants; t++) all_served &= bytes[(size_t)t] > 0;
  CHECK(all_served);
  CHECK(admissions.load() >= (uint64_t)kTenants && asks.load() >= admissions.load());
  Value st = q.stats();
  CHECK(st["tenants"]["100"]["outstanding_bytes"].as_int() == 0 && st["tenants"]["139"]["outstanding_bytes"].as_int() == 0);
  if (getenv("MCCS_TEST_VERBOSE"))
    printf("qos, 40 tenants, 8 threads: %llu admissions, %llu questions\n", (unsigned long long)admissions.load(),
           (unsigned long long)asks.load());
}

static void test_misc() {
  std::vector<int> c = parse_cpu_list("0-3,8,10-11");
  CHECK(c.size() == 7 && c[4] == 8 && c[6] == 11);
  CHECK(parse_cpu_list("").empty());
  CHECK(sizeof(proto::WorkRequest) == 128 && sizeof(proto::WorkCompletion) == 64);
  CHECK(proto::handle_comm_id(proto::make_comm_handle(138, 5)) == 138);
  CHECK(proto::handle_rank(proto::make_comm_handle(138, 5)) == 5);
  CHECK(sizeof(StatusBlock) == 64);
  CHECK(sizeof(CollArgs) < 4000);   // must fit the kernel parameter space
  CHECK(Planner::variant_from_name("ar_nvls_twoshot") == kArNvlsTwo);
  CHECK(Planner::variant_from_name("whatever") == -1);
}

int main() {
  test_ring();
  test_uds_fd_passing();
  test_toml_json();
  test_config();
  test_planner();
  test_transports();
  test_ring_steps();
  test_qos();
  test_qos_many_tenants();
  test_misc();
  printf("%d checks, %d failed\n", g_checks, g_failed);
  return g_failed;
}
