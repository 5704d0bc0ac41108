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
  mccsd_stop();
  printf("fuzz_protocol: %d control frames, %ld ring requests answered, good tenant %s\n", rounds, answered,
         bad ? "FAILED" : "served");
  return bad ? 1 : 0;
}
