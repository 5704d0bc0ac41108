// A hostile tenant: speaks the control protocol and the shared-memory request ring with
// random, truncated and out-of-range contents against an in-process daemon (host
// backend), under AddressSanitizer (`make asan`). A tenant is another user's process, so
// nothing it sends may crash the daemon, make it touch memory outside the tenant's own
// allocations, or disturb a well-behaved tenant, which is checked at the end.
//
// The reference trusts its clients: most of its error paths are unwrap()/panic!
// (src/mccs/src/daemon/engine.rs:86-99,263).
#include <signal.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <unistd.h>

#include <random>
#include <string>
#include <vector>

#include "../common/protocol.h"
#include "../daemon/daemon.h"
#include "../include/mccs.h"
#include "../ipc/shm_ring.h"
#include "../ipc/uds.h"
#include "../kernels/dev_types.h"

using namespace mccs;

namespace {

std::mt19937_64 rng(987654321);

// Where the run is, for the watchdog: a daemon that stops answering must end the run with
// its place, not hang it.
volatile int g_stage = 0;
volatile long g_step = 0, g_posted = 0, g_answered = 0;
void on_alarm(int) {
  char buf[160];
  int n = snprintf(buf, sizeof buf, "fuzz_protocol: stuck in stage %d at step %ld (posted %ld, answered %ld)\n", g_stage, g_step,
                   g_posted, g_answered);
  if (write(2, buf, (size_t)n) < 0) {}
  _exit(3);
}

int connect_and_hello(const std::string& path) {
  int fd = ipc::uds_connect(path);
  if (fd < 0) return fd;
  proto::AnyMsg m;
  memset(&m, 0, sizeof m);
  m.h.magic = proto::kMagic;
  m.h.type = proto::kHello;
  m.hello.version = proto::kVersion;
  m.hello.pid = 1;   // claims to be someone else: the daemon goes by the socket's credentials
  m.hello.device_affinity = -1;
  snprintf(m.hello.app_name, sizeof m.hello.app_name, "fuzzer");
  ipc::uds_send(fd, &m, sizeof(proto::Hello));
  if (ipc::wait_readable(fd, 2000) <= 0) { close(fd); return -1; }
  ipc::uds_recv(fd, &m, sizeof m);
  return fd;
}

// Drains whatever the daemon answered; closes passed descriptors.
void drain(int fd, std::vector<int>* keep_fds = nullptr, proto::AnyMsg* last = nullptr) {
  while (ipc::wait_readable(fd, 3) > 0) {
    proto::AnyMsg r;
    std::vector<int> fds;
    ssize_t n = ipc::uds_recv(fd, &r, sizeof r, &fds);
    if (n <= 0) break;
    if (last) *last = r;
    for (int f : fds) {
      if (keep_fds) keep_fds->push_back(f);
      else close(f);
    }
  }
}

uint64_t wild_u64() {
  switch (rng() % 6) {
    case 0: return 0;
    case 1: return ~0ull;
    case 2: return 1ull << 63;
    case 3: return rng() % 64;
    case 4: return (1ull << (rng() % 64)) - (rng() % 3);
    default: return rng();
  }
}


// A tenant that speaks the raw protocol: one connection, its own allocations (mapped here
// through the descriptor the host backend hands out) and communicators.
struct RawTenant {
  int fd = -1;
  bool open(const std::string& path) { fd = connect_and_hello(path); return fd >= 0; }
  bool request(proto::AnyMsg& m, size_t len, proto::AnyMsg* rep, std::vector<int>* fds) {
    m.h.magic = proto::kMagic;
    if (ipc::uds_send(fd, &m, len) < 0) return false;
    if (ipc::wait_readable(fd, 5000) <= 0) return false;
    memset(rep, 0, sizeof *rep);
    return ipc::uds_recv(fd, rep, sizeof *rep, fds) > 0;
  }
  // Allocation of `bytes` on `device`; returns the id and a host mapping of the memory.
  bool alloc(int device, size_t bytes, uint64_t* mem_id, void** host) {
    proto::AnyMsg m, rep;
    memset(&m, 0, sizeof m);
    m.h.type = proto::kMalloc;
    m.malloc_req.device = device;
    m.malloc_req.size = bytes;
    std::vector<int> fds;
    if (!request(m, sizeof(proto::MallocReq), &rep, &fds) || rep.h.status != 0) return false;
    *mem_id = rep.malloc_reply.mem_id;
    // This test shares the daemon's process, where host-backend memory is addressable as
    // it is; out of process the reply carries a descriptor to map.
    if (fds.empty()) *host = (void*)rep.malloc_reply.daemon_va;
    else *host = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fds[0], 0);
    for (int f : fds) close(f);
    return *host != nullptr && *host != MAP_FAILED;
  }
  int free_mem(uint64_t mem_id) {
    proto::AnyMsg m, rep;
    memset(&m, 0, sizeof m);
    m.h.type = proto::kFree;
    m.free_req.mem_id = mem_id;
    std::vector<int> fds;
    if (!request(m, sizeof(proto::FreeReq), &rep, &fds)) return -1000;
    for (int f : fds) close(f);
    return rep.h.status;
  }
  void send_comm_init(uint32_t id, int nranks, int rank, int device) {
    proto::AnyMsg m;
    memset(&m, 0, sizeof m);
    m.h.magic = proto::kMagic;
    m.h.type = proto::kCommInit;
    m.comm_init.comm_id = id;
    m.comm_init.nranks = nranks;
    m.comm_init.rank = rank;
    m.comm_init.device = device;
    ipc::uds_send(fd, &m, sizeof(proto::CommInitReq));
  }
  struct Rings { uint64_t handle = 0; void* dp = nullptr; size_t bytes = 0; ipc::Ring wq, cq; };
  bool recv_comm_init(Rings* out) {
    proto::AnyMsg rep;
    std::vector<int> fds;
    if (ipc::wait_readable(fd, 5000) <= 0) return false;
    memset(&rep, 0, sizeof rep);
    if (ipc::uds_recv(fd, &rep, sizeof rep, &fds) <= 0 || rep.h.status != 0 || fds.empty()) return false;
    out->handle = rep.comm_init_reply.comm_handle;
    out->bytes = rep.comm_init_reply.dp_bytes;
    out->dp = mmap(nullptr, out->bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fds[0], 0);
    for (int f : fds) close(f);
    if (out->dp == MAP_FAILED) return false;
    out->wq.attach(out->dp);
    out->cq.attach((char*)out->dp + proto::dp_wq_bytes());
    return true;
  }
};

proto::WorkRequest make_wr(uint64_t handle, int kind, uint64_t send_mem, uint64_t recv_mem, uint64_t count, uint64_t user_seq) {
  proto::WorkRequest wr;
  memset(&wr, 0, sizeof wr);
  wr.kind = (uint32_t)kind;
  wr.dtype = kFloat32;
  wr.op = kSum;
  wr.variant = kAuto;
  wr.comm_handle = handle;
  wr.send_mem = send_mem;
  wr.recv_mem = recv_mem;
  wr.count = count;
  wr.user_seq = user_seq;
  return wr;
}

bool wait_completion(ipc::Ring& cq, proto::WorkCompletion* wc, int ms) {
  for (int i = 0; i < ms * 10; i++) {
    if (cq.try_pop(wc)) return true;
    usleep(100);
  }
  return false;
}

// Tenant isolation on the data path, and memory that is freed under a queued collective.
// Returns the number of failed expectations.
int isolation_and_busy_checks(const std::string& path) {
  int bad = 0;
  auto expect = [&](bool ok, const char* what) { if (!ok) { fprintf(stderr, "isolation check failed: %s\n", what); bad++; } };
  RawTenant victim, thief;
  if (!victim.open(path) || !thief.open(path)) { fprintf(stderr, "isolation check: cannot connect\n"); return 1; }
  uint64_t vmem = 0, tmem = 0;
  float *vhost = nullptr, *thost = nullptr;
  expect(victim.alloc(0, 4096, &vmem, (void**)&vhost), "victim allocation");
  expect(thief.alloc(0, 4096 * 2, &tmem, (void**)&thost), "thief allocation");
  if (bad) return bad;
  for (int i = 0; i < 1024; i++) { vhost[i] = 1000.0f + (float)i; thost[i] = -1.0f; thost[1024 + i] = -1.0f; }
  RawTenant::Rings tr;
  thief.send_comm_init(9400, 1, 0, 0);
  expect(thief.recv_comm_init(&tr), "thief communicator");
  if (bad) return bad;
  // 1. read: AllReduce of the victim's buffer into the thief's own (a single-rank
  //    communicator turns that into a copy); 2. write: the thief's data over the victim's;
  // 3. the same two through AllGather. Memory ids are small consecutive numbers, so a
  //    tenant can guess them: none of the four may be carried out.
  struct Case { int kind; uint64_t send, recv; const char* what; } cases[] = {
      {kAllReduce, vmem, tmem, "AllReduce reading a foreign buffer"},
      {kAllReduce, tmem, vmem, "AllReduce writing a foreign buffer"},
      {kAllGather, vmem, tmem, "AllGather reading a foreign buffer"},
      {kAllGather, tmem, vmem, "AllGather writing a foreign buffer"},
  };
  uint64_t useq = 0;
  for (const Case& c : cases) {
    proto::WorkRequest wr = make_wr(tr.handle, c.kind, c.send, c.recv, c.kind == kAllGather ? 4096 : 1024, useq++);
    expect(tr.wq.try_push(&wr), "posting");
    proto::WorkCompletion wc;
    memset(&wc, 0, sizeof wc);
    expect(wait_completion(tr.cq, &wc, 5000), "a completion for the foreign request");
    expect(wc.status != 0, c.what);
  }
  bool untouched = true, nothing_leaked = true;
  for (int i = 0; i < 1024; i++) {
    if (vhost[i] != 1000.0f + (float)i) untouched = false;
    if (thost[i] != -1.0f) nothing_leaked = false;
  }
  expect(untouched, "the victim's bytes are unchanged");
  expect(nothing_leaked, "the thief's buffer holds none of the victim's bytes");
  // A request on its own memory still works for the same tenant.
  {
    proto::WorkRequest wr = make_wr(tr.handle, kAllReduce, tmem, tmem, 1024, useq++);
    wr.recv_off = 4096;
    tr.wq.try_push(&wr);
    proto::WorkCompletion wc;
    memset(&wc, 0, sizeof wc);
    expect(wait_completion(tr.cq, &wc, 5000) && wc.status == 0, "the tenant's own request is served");
  }

  // Free under a queued collective: rank 0 of a two-rank communicator posts, rank 1 does not
  // yet, so the request sits in its rendezvous slot with the buffer's address resolved. A
  // raw free of that buffer must be refused; once rank 1 has joined and the collective has
  // gone out on both ranks, the same free succeeds.
  RawTenant peer;
  expect(peer.open(path), "second rank connects");
  uint64_t pmem = 0;
  float* phost = nullptr;
  expect(peer.alloc(1, 4096, &pmem, (void**)&phost), "second rank allocation");
  RawTenant::Rings r0, r1;
  victim.send_comm_init(9401, 2, 0, 0);
  peer.send_comm_init(9401, 2, 1, 1);
  expect(victim.recv_comm_init(&r0) && peer.recv_comm_init(&r1), "two-rank communicator");
  if (bad) return bad;
  for (int i = 0; i < 1024; i++) phost[i] = 1.0f;
  proto::WorkRequest w0 = make_wr(r0.handle, kAllReduce, vmem, vmem, 1024, 0);
  expect(r0.wq.try_push(&w0), "rank 0 posts");
  usleep(20000);   // the proxy has taken it by now; rank 1 has not posted
  expect(victim.free_mem(vmem) == proto::kErrBusy, "free of a buffer named by a queued collective is refused");
  proto::WorkRequest w1 = make_wr(r1.handle, kAllReduce, pmem, pmem, 1024, 0);
  expect(r1.wq.try_push(&w1), "rank 1 posts");
  proto::WorkCompletion wc;
  memset(&wc, 0, sizeof wc);
  expect(wait_completion(r0.cq, &wc, 5000) && wc.status == 0, "the collective completes on rank 0");
  expect(wait_completion(r1.cq, &wc, 5000) && wc.status == 0, "the collective completes on rank 1");
  expect(vhost[5] == 1005.0f + 1.0f && phost[5] == 1005.0f + 1.0f, "its result is the sum");
  int st = proto::kErrBusy;
  for (int i = 0; i < 2000 && st == proto::kErrBusy; i++) { st = victim.free_mem(vmem); if (st == proto::kErrBusy) usleep(1000); }
  expect(st == 0, "the free succeeds once the collective has been launched everywhere");
  // a request that names the freed id is refused, not run on a stale address
  proto::WorkRequest w2 = make_wr(r0.handle, kAllReduce, vmem, vmem, 1024, 1);
  r0.wq.try_push(&w2);
  proto::WorkRequest w3 = make_wr(r1.handle, kAllReduce, pmem, pmem, 1024, 1);
  r1.wq.try_push(&w3);
  memset(&wc, 0, sizeof wc);
  expect(wait_completion(r0.cq, &wc, 5000) && wc.status != 0, "a request naming freed memory fails");
  wait_completion(r1.cq, &wc, 5000);
  close(victim.fd); close(thief.fd); close(peer.fd);
  return bad;
}

}  // namespace

int main(int argc, char** argv) {
  const int rounds = argc > 1 ? atoi(argv[1]) : 3000;
  // "client": the daemon hands plans back instead of launching ([b200] launch = "client");
  // the hostile tenant then also asks for mappings of scratch memory, foreign allocations
  // and multicast regions, and reads plans instead of completions.
  const bool client_mode = argc > 2 && std::string(argv[2]) == "client";
  const std::string prefix = "/tmp/mccs-fuzz-" + std::to_string((long)getpid());
  const std::string cfg = "listen_port = 0\nmccs_daemon_prefix = \"" + prefix + "\"\n[control]\nprefix = \"" + prefix +
                          "\"\npath = \"control.sock\"\n[comm_default_config]\nbuffer_sizes = [65536]\nchannel_count = 2\n"
                          "[b200]\nforce_host_backend = true\nhost_devices = 2\nwait_timeout_ms = 2000\ninit_timeout_ms = 300\n" +
                          std::string(client_mode ? "launch = \"client\"\nclient_nvls = true\n" : "");
  setenv("MCCS_LOG", "error", 0);
  if (getenv("FUZZ_SEED")) rng.seed(strtoull(getenv("FUZZ_SEED"), nullptr, 0));   // another run of the same length, other contents
  signal(SIGALRM, on_alarm);
  alarm(getenv("FUZZ_ALARM") ? (unsigned)atoi(getenv("FUZZ_ALARM")) : 600u);
  if (mccsd_start(cfg.c_str()) != 0) { fprintf(stderr, "daemon did not start\n"); return 2; }
  const std::string path = mccsd_control_path();

  // 1. control messages: every type, random length, random fields
  int fd = connect_and_hello(path);
  if (fd < 0) { fprintf(stderr, "cannot connect\n"); return 2; }
  g_stage = 1;
  for (int i = 0; i < rounds; i++) {
    g_step = i;
    proto::AnyMsg m;
    for (size_t k = 0; k < sizeof m.raw; k++) m.raw[k] = (uint8_t)rng();
    m.h.magic = (rng() % 50 == 0) ? (uint32_t)rng() : proto::kMagic;
    m.h.type = (rng() % 10 == 0) ? (uint32_t)rng() : (uint32_t)(rng() % 24);
    switch (m.h.type) {
      case proto::kMalloc: m.malloc_req.device = (int32_t)(rng() % 5) - 1; m.malloc_req.size = (rng() % 3) ? 4096 * (1 + rng() % 4) : wild_u64(); break;
      case proto::kFree: m.free_req.mem_id = rng() % 40; break;
      case proto::kCommInit:
        m.comm_init.comm_id = 9000 + (uint32_t)(rng() % 4);
        m.comm_init.nranks = (int32_t)(rng() % 12) - 1;
        m.comm_init.rank = (int32_t)(rng() % 12) - 1;
        m.comm_init.device = (int32_t)(rng() % 5) - 1;
        break;
      case proto::kCommDestroy: m.comm_destroy.comm_handle = ((uint64_t)(9000 + rng() % 4) << 32) + rng() % 3; break;
      case proto::kMapScratch:
        m.map_scratch.comm_handle = (rng() % 2) ? wild_u64() : ((uint64_t)(9000 + rng() % 4) << 32) + rng() % 3;
        m.map_scratch.rank = (int32_t)(rng() % 12) - 2;
        m.map_scratch.kind = (uint32_t)(rng() % 5);
        break;
      case proto::kMapMem:
        m.map_mem.comm_handle = (rng() % 2) ? wild_u64() : ((uint64_t)(9000 + rng() % 4) << 32) + rng() % 3;
        m.map_mem.mem_id = rng() % 40;
        break;
      case proto::kMapMc:
        m.map_mc.comm_handle = (rng() % 2) ? wild_u64() : ((uint64_t)(9000 + rng() % 4) << 32) + rng() % 3;
        m.map_mc.mc_id = rng() % 6;
        break;
      case proto::kCommQuery: m.comm_query.comm_handle = (rng() % 2) ? wild_u64() : ((uint64_t)(9000 + rng() % 4) << 32) + rng() % 3; break;
      default: break;
    }
    const size_t len = (rng() % 4 == 0) ? rng() % (sizeof m + 1) : sizeof m;
    if (ipc::uds_send(fd, &m, len) < 0) {
      // the daemon hung up on us (malformed frame): that is its right; come back
      close(fd);
      fd = connect_and_hello(path);
      if (fd < 0) { fprintf(stderr, "daemon no longer accepts connections\n"); return 1; }
      continue;
    }
    drain(fd);
  }
  close(fd);

  // 2. data path: a real single-rank communicator, then garbage in its request ring
  fd = connect_and_hello(path);
  proto::AnyMsg m;
  memset(&m, 0, sizeof m);
  m.h.magic = proto::kMagic;
  m.h.type = proto::kMalloc;
  m.malloc_req.device = 0;
  m.malloc_req.size = 65536;
  ipc::uds_send(fd, &m, sizeof(proto::MallocReq));
  proto::AnyMsg rep;
  memset(&rep, 0, sizeof rep);
  std::vector<int> fds;
  ipc::wait_readable(fd, 2000);
  ipc::uds_recv(fd, &rep, sizeof rep, &fds);
  const uint64_t mem_id = rep.malloc_reply.mem_id;
  for (int f : fds) close(f);
  fds.clear();
  memset(&m, 0, sizeof m);
  m.h.magic = proto::kMagic;
  m.h.type = proto::kCommInit;
  m.comm_init.comm_id = 9100;
  m.comm_init.nranks = 1;
  m.comm_init.rank = 0;
  m.comm_init.device = 0;
  ipc::uds_send(fd, &m, sizeof(proto::CommInitReq));
  ipc::wait_readable(fd, 2000);
  ipc::uds_recv(fd, &rep, sizeof rep, &fds);
  if (rep.h.status != 0 || fds.empty()) { fprintf(stderr, "single-rank communicator refused (%d)\n", rep.h.status); return 1; }
  const size_t dp_bytes = rep.comm_init_reply.dp_bytes;
  void* dp = mmap(nullptr, dp_bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fds[0], 0);
  for (int f : fds) close(f);
  if (dp == MAP_FAILED) { fprintf(stderr, "cannot map the data-path segment\n"); return 1; }
  ipc::Ring wq, cq, pq;
  wq.attach(dp);
  cq.attach((char*)dp + proto::dp_wq_bytes());
  pq.attach((char*)dp + proto::dp_pq_offset());
  if (client_mode && rep.comm_init_reply.launch_mode != proto::kLaunchClient) { fprintf(stderr, "the communicator is not in client-launch mode\n"); return 1; }
  // A client that launches its own kernels also owns their completion: the kernel's last
  // store is its ticket into the rank's status block, which is what lets the daemon hand out
  // further plans. The fuzzer runs no kernel, so it writes the ticket itself.
  StatusBlock* my_status = nullptr;
  if (client_mode) {
    memset(&m, 0, sizeof m);
    m.h.magic = proto::kMagic;
    m.h.type = proto::kMapScratch;
    m.map_scratch.comm_handle = rep.comm_init_reply.comm_handle;
    m.map_scratch.rank = 0;
    m.map_scratch.kind = proto::kScratchStatus;
    ipc::uds_send(fd, &m, sizeof(proto::MapScratchReq));
    proto::AnyMsg sr;
    memset(&sr, 0, sizeof sr);
    std::vector<int> sfds;
    ipc::wait_readable(fd, 2000);
    ipc::uds_recv(fd, &sr, sizeof sr, &sfds);
    if (sr.h.status == 0 && !sfds.empty())
      my_status = (StatusBlock*)mmap(nullptr, sr.map_scratch_reply.bytes, PROT_READ | PROT_WRITE, MAP_SHARED, sfds[0], 0);
    for (int f : sfds) close(f);
    if (!my_status || my_status == MAP_FAILED) { fprintf(stderr, "cannot map the status block\n"); return 1; }
  }
  long posted = 0, answered = 0;
  // every request is answered exactly once: by a completion, or (client-side launch) by a
  // plan or the reason there is none
  auto reap = [&]() {
    proto::WorkCompletion wc;
    while (cq.try_pop(&wc)) answered++;
    proto::PlanMsg plan;
    while (client_mode && pq.try_pop(&plan)) {
      answered++;
      if (plan.status == 0) __atomic_store_n(&my_status->done_seq, plan.ticket, __ATOMIC_RELEASE);
    }
  };
  g_stage = 2;
  for (int i = 0; i < rounds; i++) {
    g_step = i; g_posted = posted; g_answered = answered;
    proto::WorkRequest wr;
    uint8_t* raw = (uint8_t*)&wr;
    for (size_t k = 0; k < sizeof wr; k++) raw[k] = (uint8_t)rng();
    wr.kind = (uint32_t)(rng() % 4);
    wr.dtype = (uint32_t)(rng() % 12);
    wr.op = (uint32_t)(rng() % 8);
    wr.variant = (uint32_t)(rng() % 14);
    wr.comm_handle = rep.comm_init_reply.comm_handle;
    wr.send_mem = (rng() % 4) ? mem_id : wild_u64();
    wr.recv_mem = (rng() % 4) ? mem_id : wild_u64();
    wr.send_off = (rng() % 2) ? rng() % 70000 : wild_u64();
    wr.recv_off = (rng() % 2) ? rng() % 70000 : wild_u64();
    wr.count = (rng() % 2) ? rng() % 20000 : wild_u64();
    wr.sync_slot = 0;   // the host backend has no semaphore page; events are not used either
    wr.stream_id = rng() % 3;
    wr.user_seq = (uint64_t)i;
    while (!wq.try_push(&wr)) {
      reap();
      usleep(50);
    }
    posted++;
    reap();
    // the library keeps one request in flight in this mode (the plan ring is that deep)
    for (int spin = 0; client_mode && spin < 20000 && answered < posted; spin++) { usleep(50); reap(); }
  }
  for (int spin = 0; spin < 20000 && answered < posted; spin++) {
    reap();
    usleep(100);
  }
  if (client_mode) {
    // A tenant that posts far ahead of the answers it takes (a group that never ends): the
    // request ring and the plan ring fill up and the daemon has to sit on answers it cannot
    // deliver. Nothing may be lost or answered twice once the tenant reads again.
    g_stage = 25;
    long burst = 0;
    for (int i = 0; i < 400; i++) {
      proto::WorkRequest wr = make_wr(rep.comm_init_reply.comm_handle, kAllReduce, mem_id, mem_id, 16, (uint64_t)(rounds + i));
      wr.flags = proto::kWrGroupMore;
      if (!wq.try_push(&wr)) break;
      burst++;
    }
    posted += burst;
    usleep(100000);
    for (int spin = 0; spin < 40000 && answered < posted; spin++) { reap(); usleep(50); }
    usleep(20000);
    reap();   // a second answer to any of them would show up here
  }
  const bool all_answered = answered == posted;
  // The segment is writable by the tenant: scribble over the ring headers (geometry and
  // both indices) while the proxy keeps polling them. Whatever it makes of the contents,
  // it must stay inside the segment.
  for (int i = 0; i < 200; i++) {
    const int which = (int)(rng() % (client_mode ? 3 : 2));
    ipc::RingHeader* h = (ipc::RingHeader*)(which == 0 ? dp : which == 1 ? (void*)((char*)dp + proto::dp_wq_bytes())
                                                                        : (void*)((char*)dp + proto::dp_pq_offset()));
    h->depth = (uint32_t)wild_u64();
    h->slot_bytes = (uint32_t)wild_u64();
    h->tail.store(wild_u64());
    if (rng() % 3 == 0) h->head.store(wild_u64());
    usleep(200);
  }
  munmap(dp, dp_bytes);
  close(fd);   // no goodbye: the daemon cleans up after us
  if (!all_answered) { fprintf(stderr, "only %ld of %ld requests were answered\n", answered, posted); return 1; }

  g_stage = 3;
  // 3. a well-behaved tenant still gets service
  setenv("MCCS_CONTROL", path.c_str(), 1);
  int bad = 0;
  float* buf = nullptr;
  mccsComm_t comm = nullptr;
  bad += mccsInit(nullptr) != mccsSuccess;
  bad += mccsMalloc((void**)&buf, 0, 4096) != mccsSuccess;
  bad += mccsCommInitRank(&comm, 9200, 0, 1, 0, nullptr) != mccsSuccess;
  if (buf && comm) {
    for (int i = 0; i < 1024; i++) buf[i] = (float)i;
    // Sanitizer builds carry no emulated kernels, so in client-launch mode the library
    // gets its plan and then has nothing to run it with: "unsupported", and nothing worse.
    const mccsResult_t ar = mccsAllReduce(comm, buf, buf, 1024, mccsFloat32, mccsSum, nullptr);
    bad += client_mode ? (ar != mccsUnsupported) : (ar != mccsSuccess);
    bad += buf[1023] != 1023.0f;
    if (client_mode) {
      // Isolation: another tenant (own connection, own communicator) asks to map the good
      // tenant's buffer and status block. Both belong to a communicator it is no part of.
      uint64_t good_mem = 0;
      mccsMemInfo(buf, &good_mem, nullptr, nullptr);
      int fd2 = connect_and_hello(path);
      proto::AnyMsg q, a;
      memset(&q, 0, sizeof q);
      q.h.magic = proto::kMagic;
      q.h.type = proto::kCommInit;
      q.comm_init.comm_id = 9300;
      q.comm_init.nranks = 1;
      ipc::uds_send(fd2, &q, sizeof(proto::CommInitReq));
      std::vector<int> got;
      ipc::wait_readable(fd2, 2000);
      ipc::uds_recv(fd2, &a, sizeof a, &got);
      const uint64_t own_handle = a.comm_init_reply.comm_handle;
      for (int f : got) close(f);
      got.clear();
      for (uint64_t handle : {own_handle, (uint64_t)mccsCommHandle(comm)}) {
        memset(&q, 0, sizeof q);
        q.h.magic = proto::kMagic;
        q.h.type = proto::kMapMem;
        q.map_mem.comm_handle = handle;
        q.map_mem.mem_id = good_mem;
        ipc::uds_send(fd2, &q, sizeof(proto::MapMemReq));
        ipc::wait_readable(fd2, 2000);
        memset(&a, 0, sizeof a);
        ipc::uds_recv(fd2, &a, sizeof a, &got);
        if (a.h.status == 0 || !got.empty()) { fprintf(stderr, "a foreign tenant was handed another tenant's buffer\n"); bad++; }
        for (int f : got) close(f);
        got.clear();
      }
      memset(&q, 0, sizeof q);
      q.h.magic = proto::kMagic;
      q.h.type = proto::kMapScratch;
      q.map_scratch.comm_handle = mccsCommHandle(comm);
      q.map_scratch.rank = 0;
      q.map_scratch.kind = proto::kScratchStatus;
      ipc::uds_send(fd2, &q, sizeof(proto::MapScratchReq));
      ipc::wait_readable(fd2, 2000);
      memset(&a, 0, sizeof a);
      ipc::uds_recv(fd2, &a, sizeof a, &got);
      if (a.h.status == 0 || !got.empty()) { fprintf(stderr, "a foreign tenant was handed another tenant's status block\n"); bad++; }
      for (int f : got) close(f);
      close(fd2);
    }
    bad += mccsCommDestroy(comm) != mccsSuccess;
    bad += mccsFree(buf) != mccsSuccess;
  }
  mccsFinalize();
  if (!client_mode) {
    g_stage = 4;
    bad += isolation_and_busy_checks(path);
  }
  mccsd_stop();
  printf("fuzz_protocol: %d control frames, %ld ring requests answered, good tenant %s\n", rounds, answered,
         bad ? "FAILED" : "served");
  return bad ? 1 : 0;
}
