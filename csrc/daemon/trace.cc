#include "trace.h"

#include <stdio.h>
#include <sys/time.h>
#include <time.h>

#include "../kernels/dev_types.h"

namespace mccs {

uint64_t monotonic_us() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000ull + (uint64_t)ts.tv_nsec / 1000ull;
}

uint64_t wall_us() {
  struct timeval tv;
  gettimeofday(&tv, nullptr);
  return (uint64_t)tv.tv_sec * 1000000ull + (uint64_t)tv.tv_usec;
}

void Tracer::record(const TraceEvent& e) {
  if (!enabled()) return;
  std::lock_guard<std::mutex> g(mu_);
  if (buf_.size() < cap_) buf_.push_back(e);
  else buf_[next_ % cap_] = e;
  next_++;
}

std::vector<TraceEvent> Tracer::snapshot() {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<TraceEvent> out;
  if (buf_.size() < cap_) return buf_;
  for (size_t i = 0; i < cap_; i++) out.push_back(buf_[(next_ + i) % cap_]);
  return out;
}

void Tracer::clear() {
  std::lock_guard<std::mutex> g(mu_);
  buf_.clear();
  next_ = 0;
}

Value Tracer::to_chrome_json() {
  Value events = Value::array();
  for (const TraceEvent& e : snapshot()) {
    auto span = [&](const char* phase, uint64_t t0, uint64_t t1) {
      if (!t0 || t1 < t0) return;
      Value ev = Value::object();
      char name[96];
      snprintf(name, sizeof name, "%s %s #%llu", phase, variant_name(e.variant), (unsigned long long)e.seq);
      ev.set("name", name);
      ev.set("ph", "X");
      ev.set("ts", (int64_t)t0);
      ev.set("dur", (int64_t)(t1 - t0));
      ev.set("pid", (int64_t)e.comm_id);
      ev.set("tid", (int64_t)e.rank);
      Value args = Value::object();
      args.set("bytes", (int64_t)e.bytes);
      args.set("ctas", e.ctas);
      args.set("slices", e.slices);
      args.set("device", e.device);
      ev.set("args", args);
      events.push(ev);
    };
    span("rendezvous", e.t_post_us, e.t_ready_us);
    if (e.t_go_us >= e.t_ready_us && e.t_go_us <= e.t_launch_us) {
      span("wait for clients", e.t_ready_us, e.t_go_us);
      span("admit+launch", e.t_go_us, e.t_launch_us);
    } else {
      span("admit+launch", e.t_ready_us, e.t_launch_us);
    }
    if (e.dev_start_ns && e.dev_end_ns >= e.dev_start_ns) {
      Value ev = Value::object();
      ev.set("name", std::string("device ") + variant_name(e.variant));
      ev.set("ph", "X");
      ev.set("ts", (double)e.dev_start_ns / 1000.0);
      ev.set("dur", (double)(e.dev_end_ns - e.dev_start_ns) / 1000.0);
      ev.set("pid", (int64_t)e.comm_id);
      ev.set("tid", (int64_t)(1000 + e.rank));
      events.push(ev);
    }
  }
  Value root = Value::object();
  root.set("traceEvents", events);
  root.set("displayTimeUnit", "us");
  return root;
}

bool Tracer::dump(const std::string& path) {
  FILE* f = fopen(path.c_str(), "w");
  if (!f) return false;
  std::string s = to_chrome_json().to_json();
  fwrite(s.data(), 1, s.size(), f);
  fclose(f);
  return true;
}

}  // namespace mccs
