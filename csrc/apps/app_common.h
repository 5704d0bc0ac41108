// Shared pieces of the example/benchmark applications: command line parsing in the
// style of the reference apps (structopt long options,
// src/mccs_examples/allreduce_bench/src/main.rs:17-60) and a small device helper
// that works on the CUDA backend (driver API, loaded at run time) and on the
// daemon's host backend (plain memory).
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <map>
#include <string>
#include <vector>

#include "../include/mccs.h"

namespace app {

class Options {
 public:
  // `flags` lists options that take no value.
  Options(int argc, char** argv, const std::vector<std::string>& flags = {});
  bool has(const std::string& key) const { return kv_.count(key) != 0; }
  std::string str(const std::string& key, const std::string& dflt = "") const;
  long long num(const std::string& key, long long dflt) const;
  double real(const std::string& key, double dflt) const;
  bool flag(const std::string& key) const { return has(key); }
  void require(const std::vector<std::string>& keys, const char* usage) const;

 private:
  std::map<std::string, std::string> kv_;
};

// Device access for buffers returned by mccsMalloc.
class Device {
 public:
  explicit Device(int index);
  bool cuda() const { return cuda_; }
  void upload(void* dst, const void* src, size_t bytes);
  void download(void* dst, const void* src, size_t bytes);
  void sync_stream(mccsStream_t stream);
  // Event pair timing on a stream (returns milliseconds); host clock on the host backend.
  void timer_start(mccsStream_t stream);
  double timer_stop(mccsStream_t stream);

 private:
  bool cuda_ = false;
  int index_ = 0;
  void* ev0_ = nullptr;
  void* ev1_ = nullptr;
  double host_t0_ = 0;
};

double now_seconds();
void check(mccsResult_t r, const char* what);   // prints and exits on failure
size_t dtype_bytes(mccsDataType_t t);
bool parse_dtype(const std::string& s, mccsDataType_t* out);
int parse_algo(const std::string& s);            // -1 when unknown
void spin_sleep_us(uint64_t us);
std::string name_prefix(const std::string& name);  // "[name] " or ""

}  // namespace app
