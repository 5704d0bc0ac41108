// Per-collective trace ring of the daemon: host timestamps for request arrival,
// rendezvous completion, admission and launch, plus device globaltimer stamps taken
// by the kernels when tracing is on. Dumped as chrome://tracing JSON. The reference
// only has log lines tagged with a debug id (src/mccs/src/transport/op.rs:114-142).
#pragma once
#include <stdint.h>

#include <atomic>
#include <mutex>
#include <string>
#include <vector>

#include "../common/value.h"

namespace mccs {

struct TraceEvent {
  uint32_t comm_id = 0;
  int32_t rank = 0;
  int32_t device = 0;
  uint64_t seq = 0;
  int32_t kind = 0;
  int32_t variant = 0;
  int32_t ctas = 0;
  int32_t slices = 1;
  uint64_t bytes = 0;
  uint64_t t_post_us = 0;     // work request taken from the client's ring
  uint64_t t_ready_us = 0;    // all ranks arrived and the plan exists
  uint64_t t_go_us = 0;       // every gate passed (queue bound, all clients' streams arrived, admission may still defer)
  uint64_t t_launch_us = 0;   // last slice enqueued on the backend stream
  uint64_t dev_start_ns = 0;  // previous collective's device stamps (read back lazily)
  uint64_t dev_end_ns = 0;
};

class Tracer {
 public:
  explicit Tracer(size_t capacity = 1 << 16) : cap_(capacity) {}
  void set_enabled(bool on) { enabled_.store(on, std::memory_order_relaxed); }
  bool enabled() const { return enabled_.load(std::memory_order_relaxed); }
  void record(const TraceEvent& e);
  std::vector<TraceEvent> snapshot();
  Value to_chrome_json();
  bool dump(const std::string& path);
  void clear();

 private:
  std::mutex mu_;
  std::atomic<bool> enabled_{false};
  size_t cap_;
  size_t next_ = 0;
  std::vector<TraceEvent> buf_;
};

uint64_t monotonic_us();
uint64_t wall_us();

}  // namespace mccs
