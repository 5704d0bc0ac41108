// The service daemon: control plane (client sessions, allocations, communicator
// rendezvous), one proxy engine per GPU (data path: takes work requests from the
// clients' rings, plans, admits and launches collectives) and the admin endpoint
// (live reconfiguration, QoS updates, statistics, traces).
//
// Reference map: Control (src/mccs/src/control.rs:86-355), DaemonEngine
// (src/mccs/src/daemon/engine.rs:77-456), ProxyEngine
// (src/mccs/src/proxy/engine.rs:50-75,736-751 and proxy/plan.rs), communicator
// registry (src/mccs/src/comm/mod.rs:80-109), ExchangeEngine
// (src/mccs/src/exchange/engine.rs:44-166). Structural differences, on purpose:
//   * the per-client daemon engine and the per-GPU proxy are merged on the data
//     path: the proxy polls each (communicator, rank) ring itself, so a collective
//     crosses one thread boundary, not two;
//   * all ranks of a communicator live in this process, so "bootstrap" is an
//     in-memory rendezvous per collective: the proxies of the ranks meet in a slot,
//     one of them plans for all, and every kernel receives all ranks' buffer
//     addresses as launch parameters;
//   * reconfiguration needs no drain: a new ring order / algorithm / CTA count
//     becomes part of the plan of the next collective, which all ranks share.
#pragma once
#include <atomic>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <shared_mutex>
#include <string>
#include <thread>
#include <vector>

#include "../common/protocol.h"
#include "../device/backend.h"
#include "../ipc/shm_ring.h"
#include "config.h"
#include "planner.h"
#include "transport.h"
#include "qos.h"
#include "runtime.h"
#include "trace.h"

namespace mccs {

constexpr int kCollSlots = 128;   // in-flight rendezvous slots per communicator
constexpr uint64_t kMaxGpuQueue = 48;   // collectives (slices) a rank may have launched but not finished

class Daemon;
class Communicator;

struct StreamReg {
  int device = 0;
  void* event = nullptr;   // the client's "work submitted" event, opened here
  bool owned = false;      // opened through IPC (must be destroyed)
};

struct Session {
  uint64_t id = 0;
  int fd = -1;
  int pid = 0;
  bool same_process = false;
  std::string app;
  int device_affinity = -1;
  std::set<uint64_t> allocs;
  uint64_t alloc_bytes = 0;                // sum of their sizes (for the per-client limit)
  // Copies of the three counts for the statistics, which another thread reads.
  std::atomic<uint64_t> stat_bytes{0};
  std::atomic<int> stat_allocs{0}, stat_comms{0};
  std::map<uint64_t, StreamReg> streams;   // stream_id -> registration
  uint64_t next_stream_id = 1;
  std::vector<std::pair<uint32_t, int>> comm_ranks;
};

// One rank's view of one collective, filled in by that rank's proxy.
struct CollOp {
  bool valid = false;
  int status = 0;          // proto::Status of the translation step
  int kind = 0, dtype = 0, op = 0;
  uint64_t count = 0;
  float scale = 1.0f;
  int variant_req = 0;
  uint64_t send_va = 0, recv_va = 0;
  uint64_t send_mem = 0, recv_mem = 0, send_off = 0, recv_off = 0;
  void* user_event = nullptr;
  uint64_t sync_slot = 0, sync_value = 0;   // mem-op mode (see proto::SyncMode)
  uint64_t user_seq = 0;
  uint64_t t_post_us = 0;
  bool holds_refs = false;   // send_mem and recv_mem are held busy (Daemon::translate)
};

enum SlotState : int { kSlotCollecting = 0, kSlotCollected = 1, kSlotPlanning = 2, kSlotPlanned = 3, kSlotFailed = 4 };

struct CollSlot {
  std::atomic<uint64_t> seq{0};        // the collective this slot serves right now
  std::atomic<int> arrived{0};
  std::atomic<int> state{kSlotCollecting};
  std::atomic<int> finished{0};        // ranks that launched everything and completed the request
  std::atomic<int> admitted_slices{0};
  // the last deferral of a slice by the QoS arbiter (under Communicator::admit_mu)
  int defer_slice = -1;
  uint64_t defer_gen = 0, defer_retry_us = 0;
  std::atomic<int> group_launch{0};    // emulated/host: 0 idle, 1 launching, 2 launched
  CollOp ops[kMaxRanks];
  Plan plan;
  int status = 0;
  int nslices = 1;
  uint64_t slice_count = 0;            // elements (bytes for all-gather) per slice
  uint32_t epoch_base = 0;
  uint64_t ticket_base = 0;            // device-visible sequence numbers, one per slice
  uint64_t ring_step_base[kMaxRingChannels];
  uint64_t mc_send[kMaxRanks];
  uint64_t mc_recv[kMaxRanks];
  uint64_t mc_send_id = 0, mc_recv_id = 0;    // McRegion::id of the two (client-side launch names them in the plan)
  int8_t ring[kMaxRingChannels][kMaxRanks];   // ring order per channel, fixed at plan time
  uint64_t t_ready_us = 0;
  std::atomic<uint64_t> t_collected_us{0};   // when the last rank's request arrived
  // Fused launches. A head slot carries `batch_len` collectives (itself and the next
  // batch_len - 1 slots) in one kernel; a follower slot has batch_len == 0 and launches
  // nothing of its own. Written by the planning proxy before the slot becomes "planned".
  int batch_len = 1;
  bool fused_kernel = false;           // head: launched through the fused kernel (always when batch_len > 1)
  uint64_t batch_bytes = 0;            // head: bytes of all members together (admission)
};

struct RankState {
  Communicator* comm = nullptr;
  int rank = 0;
  int device = 0;
  uint64_t session_id = 0;
  bool same_process = false;
  // data path segment shared with the client
  int dp_fd = -1;
  void* dp_mem = nullptr;
  size_t dp_bytes = 0;
  ipc::Ring wq, cq;
  ipc::Ring pq;                        // plans handed back to the client (client-side launch)
  proto::DpStatus* dp_status = nullptr;
  // device resources
  void* stream = nullptr;
  void* backend_event = nullptr;
  uint8_t event_handle[proto::kIpcHandleBytes] = {0};
  SignalPad* pad = nullptr;
  StatusBlock* status = nullptr;
  char* fifo = nullptr;
  size_t fifo_bytes = 0;
  SyncPage sync;                       // semaphore page shared with the client (mem-op mode)
  // proxy-owned progress state
  int pending_plan_error = 0;          // client-side launch: an error answer that did not fit the plan ring yet
  uint64_t pending_plan_seq = 0;
  uint64_t next_post_seq = 0;
  uint64_t next_launch_seq = 0;
  int next_slice = 0;
  bool have_pending_wr = false;
  proto::WorkRequest pending_wr;
  bool have_pending_wc = false;
  proto::WorkCompletion pending_wc;
  struct Inflight { uint64_t ticket; uint64_t bytes; };
  std::deque<Inflight> inflight;       // rank 0 only: admitted, not yet seen finished
  uint64_t traced_ticket = 0;
  std::atomic<uint64_t> last_ticket{0};  // ticket of the newest kernel launched for this rank (rank 0's is read by every proxy of a one-launch group)
  std::atomic<bool> joined{false};
  std::atomic<bool> gone{false};       // its client went away
};

enum CommState : int { kCommInit = 0, kCommActive = 1, kCommError = 2, kCommClosed = 3 };

class Communicator {
 public:
  uint32_t id = 0;
  int nranks = 0;
  bool emulated = false;       // all ranks on one device: one launch covers every rank
  ConnectionTable conns;       // the transport chosen for every (sender, receiver) pair
  bool host_staged = false;    // = conns.scratch_in_host_memory(): pads and FIFOs in pinned host memory
  bool client_launch = false;  // the ranks' client libraries launch the kernels; the daemon plans and admits
  std::vector<int> devices;    // device of each rank
  std::vector<std::unique_ptr<RankState>> ranks;
  std::atomic<int> state{kCommInit};
  std::atomic<int> async_error{0};
  std::atomic<uint32_t> device_error{0};
  std::atomic<uint64_t> planned{0}, completed{0};
  std::atomic<uint64_t> fused_launches{0}, fused_members{0};
  std::atomic<uint32_t> last_variant{0}, last_ctas{0};
  std::atomic<bool> paused{false};
  uint64_t created_us = 0;
  void* group_stream = nullptr;   // emulated mode: the one stream that runs all ranks

  CollSlot slots[kCollSlots];

  // --- mutable configuration, applied at plan time -----------------------------
  std::mutex cfg_mu;
  std::vector<std::vector<int>> rings;   // per channel: user ranks in ring order
  int channel_count = 1;
  int ar_variant = kAuto, ag_variant = kAuto;
  int ctas_override = 0;
  uint64_t config_epoch = 0;
  // --- plan-time counters (only touched by the thread that plans) -----------------
  uint32_t barrier_epoch = 1;
  uint64_t ticket = 0;
  uint64_t ring_steps[kMaxRingChannels] = {0};
  uint64_t fifo_slot_bytes = 0;
  // --- multicast registrations, keyed by the allocation ids of all ranks ------------
  std::mutex mc_mu;
  std::map<std::vector<uint64_t>, McRegion> mc_cache;
  uint64_t next_mc_id = 0;   // under mc_mu
  std::mutex admit_mu;

  CollSlot& slot(uint64_t seq) { return slots[seq % kCollSlots]; }
};

// One per device. Owns the progress of every rank that lives on that device.
class ProxyEngine : public Engine {
 public:
  ProxyEngine(Daemon* d, int device) : daemon_(d), device_(device) {
    name_ = "proxy" + std::to_string(device);
  }
  Progress progress() override;
  const char* name() const override { return name_.c_str(); }
  void on_start() override;

  void add_rank(RankState* rs);
  // Removes the rank and returns once the proxy thread no longer touches it.
  void remove_rank(RankState* rs);
  bool running() const { return started_.load(); }
  // Passes through progress() so far. Two more than a value read earlier means: whatever the
  // proxy thread was doing at that moment (a launch it had already decided on) is over.
  uint64_t passes() const { return passes_.load(std::memory_order_acquire); }

 private:
  bool intake(RankState& rs);
  bool post(RankState& rs, const proto::WorkRequest& wr);
  bool advance(RankState& rs);
  bool plan_slot(Communicator& c, CollSlot& s, uint64_t seq);
  void extend_batch(Communicator& c, CollSlot& head, uint64_t seq, const PlanInput& head_in, uint64_t now);
  bool plan_member(Communicator& c, CollSlot& head, CollSlot& m, const PlanInput& head_in, Plan* out);
  void fill_batch_args(Communicator& c, CollSlot& head, uint64_t seq, int rank, BatchArgs* b);
  bool batch_clients_ready(Communicator& c, CollSlot& head, uint64_t seq, int self_rank);
  uint64_t last_member_user_seq(Communicator& c, CollSlot& head, uint64_t seq, int rank);
  bool launch_group(Communicator& c, CollSlot& s, uint64_t seq);
  bool launch_slices(RankState& rs, CollSlot& s, uint64_t seq);
  bool admit_slice(Communicator& c, CollSlot& s, int slice);
  void fill_args(Communicator& c, CollSlot& s, int rank, int slice, CollArgs* a);
  bool complete_request(RankState& rs, CollSlot& s, uint64_t seq, int status);
  void signal_done(RankState& rs, uint64_t user_seq, int status);
  bool publish_plan(RankState& rs, CollSlot& s, uint64_t seq);
  bool publish_follower_plan(RankState& rs, CollSlot& s);
  bool followers_still_arriving(Communicator& c, CollSlot& s, uint64_t seq);
  bool publish_plan_error(RankState& rs, uint64_t user_seq, int status);
  void order_after_client(RankState& rs, const CollOp& op, void* stream);
  bool clients_ready(Communicator& c, CollSlot& s, int self_rank);
  void finish_slot(Communicator& c, CollSlot& s, uint64_t seq);
  void housekeeping(RankState& rs);
  int ensure_mc(Communicator& c, CollSlot& s, bool for_recv, uint64_t* out_va);

  Daemon* daemon_;
  int device_;
  std::string name_;
  std::mutex mu_;
  std::vector<RankState*> ranks_;        // guarded by mu_
  std::atomic<uint64_t> version_{0};
  std::atomic<uint64_t> seen_version_{0};
  std::atomic<uint64_t> passes_{0};
  std::vector<RankState*> local_;        // proxy thread's copy
  std::atomic<bool> started_{false};
  uint64_t spins_ = 0;
};

struct DaemonStartOptions {
  std::string config_text;   // TOML text; empty = defaults
  std::string config_path;   // or a file
};

class Daemon {
 public:
  Daemon();
  ~Daemon();
  // Builds backend, sockets and engines. Returns a proto::Status.
  int start(const Config& cfg, std::string* err);
  // Runs the control loop on the calling thread until stop() (standalone binary) ...
  void run();
  // ... or on a thread of its own (daemon embedded in a client process).
  void run_in_thread();
  void stop();
  // Async-signal-safe: only asks the control loop to end.
  void stop_requested() { stop_.store(true); }
  bool running() const { return running_.load(); }

  const Config& config() const { return cfg_; }
  Backend* backend() { return backend_.get(); }
  Planner& planner() { return planner_; }
  QosArbiter& qos() { return qos_; }
  Tracer& tracer() { return tracer_; }
  std::string control_path() const { return control_path_; }
  int admin_port() const { return admin_port_; }
  uint64_t timeout_ns() const { return cfg_.wait_timeout_ms * 1000000ull; }
  bool memops() const { return memops_; }

  // Allocation lookup for the data path (shared lock).
  // Resolves (mem id, offset, length) of a request posted by `session_id` to a device
  // address. Fails unless the allocation belongs to that session (ids are guessable, so a
  // tenant could otherwise name another tenant's memory; the reference resolves ids in a
  // per-client map, src/mccs/src/daemon/engine.rs:188-209) and is not being freed. On
  // success the allocation is held busy until release_mem_ref(): a free that arrives
  // while a posted collective has not been launched on every rank is refused.
  bool translate(uint64_t session_id, uint64_t mem_id, uint64_t off, uint64_t bytes, uint64_t* va, int* device);
  void release_mem_ref(uint64_t mem_id);
  // Drops what the not yet finished collectives of a communicator still hold.
  void release_slot_refs(Communicator& c);
  const Allocation* find_alloc_locked(uint64_t mem_id) const;   // caller holds alloc_mu_ (shared)
  std::shared_mutex& alloc_mutex() { return alloc_mu_; }
  void* lookup_stream_event(uint64_t session_id, uint64_t stream_id);

  // Admin operations (also used by tests directly).
  Value admin_request(int type, const Value& body);
  int apply_reconfig(const CommPattern& p, std::string* err);
  Value stats();

 private:
  friend class ProxyEngine;
  void control_iteration(int timeout_ms);
  void accept_clients();
  void handle_session(Session& s);
  void drop_session(uint64_t session_id, const char* why);
  void reply(Session& s, proto::AnyMsg& m, size_t len, const int* fds = nullptr, int nfds = 0);
  void on_malloc(Session& s, const proto::MallocReq& m);
  void on_free(Session& s, const proto::FreeReq& m);
  void on_comm_init(Session& s, const proto::CommInitReq& m);
  void on_comm_destroy(Session& s, const proto::CommDestroyReq& m);
  void on_register_stream(Session& s, const proto::RegisterStreamReq& m);
  void on_comm_query(Session& s, const proto::CommQueryReq& m);
  void on_map_scratch(Session& s, const proto::MapScratchReq& m);
  void on_map_mem(Session& s, const proto::MapMemReq& m);
  void on_map_mc(Session& s, const proto::MapMcReq& m);
  int finalize_communicator(Communicator& c);
  void fail_pending_inits(Communicator& c, int status);
  void check_init_timeouts();
  void detach_rank(Communicator& c, int rank, int status);
  void destroy_communicator(uint32_t comm_id);
  void quiesce_session_streams(Session& s);
  void proxy_grace_period();
  void drop_mc_regions_using(uint64_t mem_id);
  void admin_loop();
  void handle_admin_connection(int fd);
  void apply_pattern_locked(Communicator& c, const CommPattern& p);

  Config cfg_;
  std::unique_ptr<Backend> backend_;
  Planner planner_;
  QosArbiter qos_;
  Tracer tracer_;
  std::unique_ptr<RuntimeManager> runtimes_;
  std::vector<std::shared_ptr<ProxyEngine>> proxies_;

  std::string control_path_;
  int listen_fd_ = -1;
  int admin_fd_ = -1;
  int admin_port_ = 0;
  std::thread control_thread_;
  std::thread admin_thread_;
  std::atomic<bool> running_{false};
  bool memops_ = false;
  bool client_launch_ = false;
  std::unique_ptr<TransportCatalog> catalog_;   // the transports this daemon offers ([b200] transport), in selection order
  bool auto_launch_ = false;      // b200.launch = auto: per communicator, see finalize_communicator
  std::atomic<bool> stop_{false};

  std::mutex mu_;   // sessions_, comms_, pending_inits_
  std::map<uint64_t, std::unique_ptr<Session>> sessions_;
  std::map<uint32_t, std::unique_ptr<Communicator>> comms_;
  struct PendingInit { uint64_t session_id; uint32_t req_id; uint32_t comm_id; int rank; uint64_t deadline_us; };
  std::vector<PendingInit> pending_inits_;
  // Requests for an id whose previous communicator is still being let go of by its other
  // ranks: answered (by a second pass through on_comm_init) once the id is free.
  struct ParkedInit { uint64_t session_id; proto::CommInitReq req; uint64_t deadline_us; };
  std::vector<ParkedInit> parked_inits_;   // control thread only
  void retry_parked_inits();
  uint64_t next_session_id_ = 1;

  mutable std::shared_mutex alloc_mu_;
  std::map<uint64_t, Allocation> allocs_;
  struct AllocUse { std::atomic<int> busy{0}; bool dying = false; };
  std::map<uint64_t, AllocUse> alloc_use_;   // same keys as allocs_, same lock
  uint64_t next_mem_id_ = 1;

  // registrations for the data path's stream lookup
  std::shared_mutex stream_mu_;
  std::map<std::pair<uint64_t, uint64_t>, void*> stream_events_;
};

// Process-wide embedded daemon (used by the Python package, tests and bench).
extern "C" {
int mccsd_start(const char* config_toml);     // proto::Status; idempotent
int mccsd_start_file(const char* config_path);
void mccsd_stop();
const char* mccsd_control_path();
int mccsd_admin_port();
int mccsd_backend_kind();                     // proto::Backend, -1 when not running
const char* mccsd_describe();
const char* mccsd_admin(int type, const char* json_body);   // returns JSON text (thread-local storage)
}

}  // namespace mccs
