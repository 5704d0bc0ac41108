// Engine runtime: the daemon's work is split into engines that are polled by
// runtime threads, like the reference (`trait Engine` src/mccs/src/engine.rs:1-18;
// `Runtime::mainloop` src/mccs/src/runtime/executor.rs:62-115; `RuntimeManager`
// src/mccs/src/runtime/manager.rs:30-98). A Dedicated engine gets a thread of its
// own, pinned to the CPUs next to its GPU; Compact engines share one thread.
// Unlike the reference's pure busy-poll, a runtime backs off with short sleeps
// after a stretch of idle polls so that an idle daemon does not burn cores.
#pragma once
#include <atomic>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace mccs {

enum class Progress { kIdle, kProgressed, kCompleted };
enum class SchedulingHint { kDedicated, kCompact };

class Engine {
 public:
  virtual ~Engine() {}
  virtual Progress progress() = 0;
  virtual SchedulingHint scheduling_hint() const { return SchedulingHint::kDedicated; }
  virtual const char* name() const = 0;
  // Called once on the runtime thread before the first progress().
  virtual void on_start() {}
};

class Runtime {
 public:
  Runtime(std::string name, std::string cpu_list, int idle_sleep_us, int idle_spin_us);
  ~Runtime();
  void add(std::shared_ptr<Engine> e);
  void start();
  void stop();     // asks the loop to end and joins
  size_t engine_count();

 private:
  void mainloop();
  std::string name_;
  std::string cpu_list_;
  int idle_sleep_us_;
  int idle_spin_us_;
  std::mutex mu_;
  std::vector<std::shared_ptr<Engine>> pending_;
  std::atomic<bool> has_pending_{false};
  std::atomic<bool> stop_{false};
  std::atomic<size_t> count_{0};
  std::thread thread_;
};

class RuntimeManager {
 public:
  RuntimeManager(int idle_sleep_us, int idle_spin_us, bool pin)
      : idle_sleep_us_(idle_sleep_us), idle_spin_us_(idle_spin_us), pin_(pin) {}
  ~RuntimeManager() { stop_all(); }
  // cpu_list: "0-3,8" style list for thread affinity ("" = no pinning).
  void submit(std::shared_ptr<Engine> e, const std::string& cpu_list);
  void stop_all();
  size_t runtime_count();

 private:
  int idle_sleep_us_;
  int idle_spin_us_;
  bool pin_;
  std::mutex mu_;
  std::vector<std::unique_ptr<Runtime>> runtimes_;
  Runtime* compact_ = nullptr;
};

// Parses "0-3,8,10-11" into CPU numbers.
std::vector<int> parse_cpu_list(const std::string& s);

}  // namespace mccs
