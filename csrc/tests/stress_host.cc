// End-to-end stress of the host-side machinery in ONE process, meant to run under
// ThreadSanitizer and AddressSanitizer (`make tsan`, `make asan`): the daemon with the
// host backend, and client threads that go through the public C API — control socket,
// fd passing, shared-memory rings, per-GPU proxy threads, rendezvous slots, planner,
// QoS admission, completions — while an operator thread fires admin requests
// (statistics, live reconfiguration, pause/resume, tuning table, tracing).
//
// The reference has no sanitizer or race-detection run of any kind; its cross-thread
// state rests on `unsafe impl Send/Sync` (src/mccs/src/proxy/engine.rs:77,
// src/mccs/src/comm/mod.rs:115).
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <atomic>
#include <string>
#include <thread>
#include <vector>

#include "../daemon/daemon.h"
#include "../include/mccs.h"

namespace {

std::atomic<int> g_failures{0};

#define EXPECT(cond)                                                          \
  do {                                                                        \
    if (!(cond)) {                                                            \
      fprintf(stderr, "%s:%d: EXPECT(%s) failed\n", __FILE__, __LINE__, #cond); \
      g_failures.fetch_add(1);                                                \
    }                                                                         \
  } while (0)

struct App {
  uint32_t comm_id;
  std::vector<int> devices;   // device of each rank
  int iters;
};

void run_rank(const App& app, int rank) {
  const int n = (int)app.devices.size();
  const int dev = app.devices[(size_t)rank];
  const size_t count = 4096 + 17;   // odd on purpose: tail path
  float* send = nullptr;
  float* recv = nullptr;
  uint8_t* gath = nullptr;
  EXPECT(mccsMalloc((void**)&send, dev, count * sizeof(float)) == mccsSuccess);
  EXPECT(mccsMalloc((void**)&recv, dev, count * sizeof(float)) == mccsSuccess);
  EXPECT(mccsMalloc((void**)&gath, dev, 1024 * (size_t)n) == mccsSuccess);
  if (!send || !recv || !gath) return;
  float* multi[4] = {nullptr, nullptr, nullptr, nullptr};   // independent buffers: these may share one fused launch
  for (int k = 0; k < 4; k++) EXPECT(mccsMalloc((void**)&multi[k], dev, (64 + 16 * (size_t)k) * sizeof(float)) == mccsSuccess);
  // Several lives of the communicator: creation and teardown race with the operator's
  // statistics and reconfiguration requests and with the other tenants' traffic.
  // The last life takes the id of the one before it: ranks that are ahead of their peers ask
  // for the id while the old communicator is still being let go of, and wait for it.
  for (int life = 0; life < 4; life++) {
  mccsComm_t comm = nullptr;
  EXPECT(mccsCommInitRank(&comm, app.comm_id + 100u * (uint32_t)(life < 3 ? life : 2), rank, n, dev, nullptr) == mccsSuccess);
  if (!comm) return;
  for (int it = 0; it < app.iters; it++) {
    for (size_t i = 0; i < count; i++) send[i] = (float)(rank + 1) + (float)(i % 7) + (float)it;
    if (it % 5 == 4) {
      // a group of back-to-back in-place reductions
      EXPECT(mccsGroupStart() == mccsSuccess);
      memcpy(recv, send, count * sizeof(float));
      for (int k = 0; k < 8; k++)
        EXPECT(mccsAllReduce(comm, recv, recv, 256, mccsFloat32, mccsMax, nullptr) == mccsSuccess);
      EXPECT(mccsGroupEnd() == mccsSuccess);
      float want = (float)n + (float)it;   // max over ranks of (rank+1) + 0 + it at i == 0
      EXPECT(recv[0] == want);
      for (int k = 0; k < 4; k++)
        for (int i = 0; i < 64 + 16 * k; i++) multi[k][i] = (float)(rank + k + i % 3);
      EXPECT(mccsGroupStart() == mccsSuccess);
      for (int k = 0; k < 4; k++)
        EXPECT(mccsAllReduce(comm, multi[k], multi[k], 64 + 16 * (size_t)k, mccsFloat32, mccsSum, nullptr) == mccsSuccess);
      {
        const mccsResult_t ge = mccsGroupEnd();
        if (ge != mccsSuccess) fprintf(stderr, "comm %u rank %d iteration %d: group of independent buffers ended with %d (%s)\n",
                                       app.comm_id, rank, it, (int)ge, mccsGetErrorString(ge));
        EXPECT(ge == mccsSuccess);
      }
      for (int k = 0; k < 4; k++) {
        const int last = 64 + 16 * k - 1;
        EXPECT(multi[k][last] == (float)(n * (n - 1) / 2) + (float)n * (float)(k + last % 3));
      }
      continue;
    }
    EXPECT(mccsAllReduce(comm, send, recv, count, mccsFloat32, mccsSum, nullptr) == mccsSuccess);
    const float want0 = (float)(n * (n + 1) / 2) + (float)n * (float)it;
    EXPECT(recv[0] == want0);
    EXPECT(recv[count - 1] == want0 + (float)n * (float)((count - 1) % 7));
    memset(gath + 1024 * (size_t)rank, rank + 1, 1024);
    EXPECT(mccsAllGather(comm, gath + 1024 * (size_t)rank, gath, 1024, nullptr) == mccsSuccess);
    for (int r = 0; r < n; r++) EXPECT(gath[1024 * (size_t)r + 1023] == (uint8_t)(r + 1));
    // reduce-scatter of the first n * 512 elements: block `rank` of the sum lands in recv
    if (it % 3 == 0 && (size_t)n * 512 <= count) {
      EXPECT(mccsReduceScatter(comm, send, recv, 512, mccsFloat32, mccsSum, nullptr) == mccsSuccess);
      const size_t at = (size_t)rank * 512 + 511;
      EXPECT(recv[511] == (float)(n * (n + 1) / 2) + (float)n * ((float)(at % 7) + (float)it));
    }
  }
  mccsCommInfo_t info;
  EXPECT(mccsCommQuery(comm, &info) == mccsSuccess);
  EXPECT(info.async_error == 0);
  EXPECT(mccsCommDestroy(comm) == mccsSuccess);
  }
  EXPECT(mccsFree(send) == mccsSuccess);
  EXPECT(mccsFree(recv) == mccsSuccess);
  EXPECT(mccsFree(gath) == mccsSuccess);
  for (int k = 0; k < 4; k++) EXPECT(mccsFree(multi[k]) == mccsSuccess);
}

void operator_thread(const std::vector<App>& apps, std::atomic<bool>* stop) {
  int round = 0;
  while (!stop->load()) {
    App a = apps[(size_t)round % apps.size()];
    a.comm_id += 100u * (uint32_t)((round / 7) % 3);
    const int n = (int)a.devices.size();
    std::string ring = "[";
    for (int i = 0; i < n; i++) ring += std::to_string((round % 2) ? n - 1 - i : i) + (i + 1 < n ? "," : "]");
    const std::string reconfig = "{\"cmd\":\"reconfig\",\"patterns\":[{\"communicator_id\":" + std::to_string(a.comm_id) +
                                 ",\"channels\":[{\"channel_id\":0,\"ring\":" + ring + "}],\"allreduce_algo\":\"" +
                                 ((round % 3) ? "auto" : "ring") + "\"}]}";
    // A communicator may not exist yet or any more: both answers are fine, a crash is not.
    (void)mccs::mccsd_admin(1, reconfig.c_str());
    EXPECT(strstr(mccs::mccsd_admin(2, "{\"cmd\":\"stats\"}"), "\"ok\"") != nullptr);
    EXPECT(strstr(mccs::mccsd_admin(2, "{\"cmd\":\"tuning_get\"}"), "allreduce") != nullptr);
    const std::string id = std::to_string(a.comm_id);
    (void)mccs::mccsd_admin(2, ("{\"cmd\":\"pause\",\"communicator_id\":" + id + "}").c_str());
    usleep(300);
    (void)mccs::mccsd_admin(2, ("{\"cmd\":\"resume\",\"communicator_id\":" + id + "}").c_str());
    (void)mccs::mccsd_admin(2, (round % 2) ? "{\"cmd\":\"trace\",\"enabled\":true}" : "{\"cmd\":\"trace\",\"enabled\":false,\"clear\":true}");
    (void)mccs::mccsd_admin(2, "{\"cmd\":\"qos_set\",\"tenants\":{\"7001\":{\"weight\":2.0},\"7002\":{\"weight\":1.0}}}");
    usleep(500);
    round++;
  }
}

}  // namespace

int main(int argc, char** argv) {
  const int iters = argc > 1 ? atoi(argv[1]) : 60;
  // "memops": the stream-memory-operation protocol (semaphore page, counted completions,
  // launches gated on every rank's semaphore) instead of events and completion messages
  const bool memops = argc > 2 && std::string(argv[2]) == "memops";
  const std::string prefix = "/tmp/mccs-stress-" + std::to_string((long)getpid());
  const std::string cfg =
      "listen_port = -1\nmccs_daemon_prefix = \"" + prefix + "\"\n[control]\nprefix = \"" + prefix +
      "\"\npath = \"control.sock\"\n[comm_default_config]\nbuffer_sizes = [65536]\nchannel_count = 2\n"
      "[b200]\nforce_host_backend = true\nhost_devices = 4\nwait_timeout_ms = 20000\nfuse_allreduce = 4\n" +
      std::string(memops ? "sync = \"memops\"\n" : "") +
      "[qos.tenants.7001]\nweight = 2.0\n[qos.tenants.7002]\nweight = 1.0\n";
  if (mccs::mccsd_start(cfg.c_str()) != 0) {
    fprintf(stderr, "daemon did not start\n");
    return 2;
  }
  setenv("MCCS_CONTROL", mccs::mccsd_control_path(), 1);
  if (mccsInit(nullptr) != mccsSuccess) {
    fprintf(stderr, "mccsInit failed\n");
    return 2;
  }
  // Three tenants whose device sets overlap, so every proxy serves several ranks.
  const std::vector<App> apps = {{7001, {0, 1, 2, 3}, iters}, {7002, {0, 1}, iters}, {7003, {2, 3, 1}, iters}};
  std::atomic<bool> stop{false};
  std::thread op(operator_thread, std::cref(apps), &stop);
  std::vector<std::thread> ranks;
  for (const App& a : apps)
    for (int r = 0; r < (int)a.devices.size(); r++) ranks.emplace_back(run_rank, std::cref(a), r);
  for (auto& t : ranks) t.join();
  stop.store(true);
  op.join();
  mccsFinalize();
  mccs::mccsd_stop();
  const int f = g_failures.load();
  printf("stress_host%s: %d failure(s)\n", memops ? " (memops)" : "", f);
  return f ? 1 : 0;
}
