#include "runtime.h"

#include <pthread.h>
#include <sched.h>
#include <stdlib.h>
#include <time.h>
#include <unistd.h>

#include "../common/log.h"

namespace mccs {

std::vector<int> parse_cpu_list(const std::string& s) {
  std::vector<int> out;
  size_t i = 0;
  while (i < s.size()) {
    size_t j = s.find(',', i);
    if (j == std::string::npos) j = s.size();
    std::string tok = s.substr(i, j - i);
    i = j + 1;
    if (tok.empty()) continue;
    size_t dash = tok.find('-');
    int a = atoi(tok.c_str());
    int b = dash == std::string::npos ? a : atoi(tok.c_str() + dash + 1);
    for (int c = a; c <= b && c < 4096; c++) out.push_back(c);
  }
  return out;
}

Runtime::Runtime(std::string name, std::string cpu_list, int idle_sleep_us, int idle_spin_us)
    : name_(std::move(name)), cpu_list_(std::move(cpu_list)), idle_sleep_us_(idle_sleep_us), idle_spin_us_(idle_spin_us) {}

Runtime::~Runtime() { stop(); }

void Runtime::add(std::shared_ptr<Engine> e) {
  std::lock_guard<std::mutex> g(mu_);
  pending_.push_back(std::move(e));
  count_++;
  has_pending_.store(true, std::memory_order_release);
}

size_t Runtime::engine_count() { return count_.load(); }

void Runtime::start() { thread_ = std::thread([this] { mainloop(); }); }

void Runtime::stop() {
  stop_.store(true);
  if (thread_.joinable()) thread_.join();
}

void Runtime::mainloop() {
  pthread_setname_np(pthread_self(), name_.substr(0, 15).c_str());
  std::vector<int> cpus = parse_cpu_list(cpu_list_);
  if (!cpus.empty()) {
    cpu_set_t set;
    CPU_ZERO(&set);
    for (int c : cpus) if (c < CPU_SETSIZE) CPU_SET(c, &set);
    if (sched_setaffinity(0, sizeof set, &set) != 0)
      LOG_DEBUG("%s: sched_setaffinity(%s) failed", name_.c_str(), cpu_list_.c_str());
  }
  std::vector<std::shared_ptr<Engine>> engines;
  unsigned idle_rounds = 0;
  uint64_t idle_since_ns = 0;
  auto now_ns = [] {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
  };
  while (!stop_.load(std::memory_order_relaxed)) {
    if (has_pending_.load(std::memory_order_acquire)) {
      std::vector<std::shared_ptr<Engine>> fresh;
      {
        std::lock_guard<std::mutex> g(mu_);
        fresh.swap(pending_);
        has_pending_.store(false, std::memory_order_release);
      }
      for (auto& e : fresh) { e->on_start(); engines.push_back(std::move(e)); }
    }
    bool any = false;
    for (size_t i = 0; i < engines.size();) {
      Progress p = engines[i]->progress();
      if (p == Progress::kCompleted) {
        LOG_DEBUG("%s: engine %s completed", name_.c_str(), engines[i]->name());
        engines.erase(engines.begin() + (long)i);
        count_--;
        continue;
      }
      if (p == Progress::kProgressed) any = true;
      i++;
    }
    if (any) {
      idle_rounds = 0;
      idle_since_ns = 0;
    } else if (engines.empty()) {
      usleep(1000);
    } else {
      // Busy-poll through short gaps (the time a kernel runs, the time between two
      // requests of a training step); only a runtime that has seen nothing for
      // `idle_spin_us` starts to sleep between polls. A sleeping poller costs every
      // request a timer wake-up, which is more than a small collective takes.
      __builtin_ia32_pause();
      if ((++idle_rounds & 0xff) == 0 && idle_sleep_us_ > 0) {
        const uint64_t t = now_ns();
        if (!idle_since_ns) idle_since_ns = t;
        else if (t - idle_since_ns > (uint64_t)idle_spin_us_ * 1000ull) usleep((useconds_t)idle_sleep_us_);
      }
    }
  }
}

void RuntimeManager::submit(std::shared_ptr<Engine> e, const std::string& cpu_list) {
  std::lock_guard<std::mutex> g(mu_);
  if (e->scheduling_hint() == SchedulingHint::kCompact) {
    if (!compact_) {
      runtimes_.emplace_back(new Runtime("mccs-compact", "", idle_sleep_us_ > 0 ? idle_sleep_us_ : 100, 1000));
      compact_ = runtimes_.back().get();
      compact_->start();
    }
    compact_->add(std::move(e));
    return;
  }
  std::string name = std::string("mccs-") + e->name();
  runtimes_.emplace_back(new Runtime(name, pin_ ? cpu_list : "", idle_sleep_us_, idle_spin_us_));
  runtimes_.back()->add(std::move(e));
  runtimes_.back()->start();
}

void RuntimeManager::stop_all() {
  std::vector<std::unique_ptr<Runtime>> rts;
  {
    std::lock_guard<std::mutex> g(mu_);
    rts.swap(runtimes_);
    compact_ = nullptr;
  }
  for (auto& r : rts) r->stop();
}

size_t RuntimeManager::runtime_count() {
  std::lock_guard<std::mutex> g(mu_);
  return runtimes_.size();
}

}  // namespace mccs
