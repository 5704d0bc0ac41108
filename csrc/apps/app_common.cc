#include "app_common.h"

#include <cuda.h>
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include <algorithm>

namespace app {

Options::Options(int argc, char** argv, const std::vector<std::string>& flags) {
  for (int i = 1; i < argc; i++) {
    std::string a = argv[i];
    if (a.rfind("--", 0) != 0) { fprintf(stderr, "unexpected argument '%s'\n", a.c_str()); exit(2); }
    std::string key = a.substr(2);
    size_t eq = key.find('=');
    if (eq != std::string::npos) { kv_[key.substr(0, eq)] = key.substr(eq + 1); continue; }
    if (key == "help" || std::find(flags.begin(), flags.end(), key) != flags.end()) { kv_[key] = "1"; continue; }
    if (i + 1 >= argc) { fprintf(stderr, "option --%s needs a value\n", key.c_str()); exit(2); }
    kv_[key] = argv[++i];
  }
}
std::string Options::str(const std::string& key, const std::string& dflt) const {
  auto it = kv_.find(key);
  return it == kv_.end() ? dflt : it->second;
}
long long Options::num(const std::string& key, long long dflt) const {
  auto it = kv_.find(key);
  return it == kv_.end() ? dflt : strtoll(it->second.c_str(), nullptr, 0);
}
double Options::real(const std::string& key, double dflt) const {
  auto it = kv_.find(key);
  return it == kv_.end() ? dflt : strtod(it->second.c_str(), nullptr);
}
void Options::require(const std::vector<std::string>& keys, const char* usage) const {
  if (has("help")) { printf("%s\n", usage); exit(0); }
  for (const auto& k : keys)
    if (!has(k)) { fprintf(stderr, "missing --%s\n%s\n", k.c_str(), usage); exit(2); }
}

namespace {
struct Drv {
  bool ok = false;
  decltype(&cuInit) init = nullptr;
  decltype(&cuDeviceGet) device_get = nullptr;
  decltype(&cuDevicePrimaryCtxRetain) retain = nullptr;
  decltype(&cuCtxSetCurrent) set_current = nullptr;
  decltype(&cuMemcpyHtoD) htod = nullptr;
  decltype(&cuMemcpyDtoH) dtoh = nullptr;
  decltype(&cuStreamSynchronize) stream_sync = nullptr;
  decltype(&cuEventCreate) ev_create = nullptr;
  decltype(&cuEventRecord) ev_record = nullptr;
  decltype(&cuEventSynchronize) ev_sync = nullptr;
  decltype(&cuEventElapsedTime) ev_elapsed = nullptr;
} g;

template <typename F> bool sym(void* lib, const char* n, F* out) {
  void* p = dlsym(lib, n);
  if (!p) return false;
  *out = reinterpret_cast<F>(p);
  return true;
}
bool load() {
  static bool tried = false;
  if (tried) return g.ok;
  tried = true;
  void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_LOCAL);
  if (!lib) return false;
  g.ok = sym(lib, "cuInit", &g.init) && sym(lib, "cuDeviceGet", &g.device_get) &&
         sym(lib, "cuDevicePrimaryCtxRetain", &g.retain) && sym(lib, "cuCtxSetCurrent", &g.set_current) &&
         sym(lib, "cuMemcpyHtoD_v2", &g.htod) && sym(lib, "cuMemcpyDtoH_v2", &g.dtoh) &&
         sym(lib, "cuStreamSynchronize", &g.stream_sync) && sym(lib, "cuEventCreate", &g.ev_create) &&
         sym(lib, "cuEventRecord", &g.ev_record) && sym(lib, "cuEventSynchronize", &g.ev_sync) &&
         sym(lib, "cuEventElapsedTime", &g.ev_elapsed);
  if (g.ok && g.init(0) != CUDA_SUCCESS) g.ok = false;
  return g.ok;
}
void cu(CUresult r, const char* what) {
  if (r != CUDA_SUCCESS) { fprintf(stderr, "%s failed (CUDA error %d)\n", what, (int)r); exit(1); }
}
}  // namespace

Device::Device(int index) : index_(index) {
  cuda_ = mccsBackendKind() == 1;
  if (!cuda_) return;
  if (!load()) { fprintf(stderr, "the daemon runs on CUDA but libcuda.so.1 is not loadable\n"); exit(1); }
  CUdevice dev;
  cu(g.device_get(&dev, index), "cuDeviceGet");
  CUcontext ctx;
  cu(g.retain(&ctx, dev), "cuDevicePrimaryCtxRetain");
  cu(g.set_current(ctx), "cuCtxSetCurrent");
  CUevent e0, e1;
  cu(g.ev_create(&e0, CU_EVENT_DEFAULT), "cuEventCreate");
  cu(g.ev_create(&e1, CU_EVENT_DEFAULT), "cuEventCreate");
  ev0_ = e0; ev1_ = e1;
}
void Device::upload(void* dst, const void* src, size_t bytes) {
  if (cuda_) cu(g.htod((CUdeviceptr)dst, src, bytes), "cuMemcpyHtoD");
  else memcpy(dst, src, bytes);
}
void Device::download(void* dst, const void* src, size_t bytes) {
  if (cuda_) cu(g.dtoh(dst, (CUdeviceptr)src, bytes), "cuMemcpyDtoH");
  else memcpy(dst, src, bytes);
}
void Device::sync_stream(mccsStream_t stream) {
  if (cuda_) cu(g.stream_sync((CUstream)stream), "cuStreamSynchronize");
}
void Device::timer_start(mccsStream_t stream) {
  if (cuda_) cu(g.ev_record((CUevent)ev0_, (CUstream)stream), "cuEventRecord");
  else host_t0_ = now_seconds();
}
double Device::timer_stop(mccsStream_t stream) {
  if (!cuda_) return (now_seconds() - host_t0_) * 1e3;
  cu(g.ev_record((CUevent)ev1_, (CUstream)stream), "cuEventRecord");
  cu(g.ev_sync((CUevent)ev1_), "cuEventSynchronize");
  float ms = 0;
  cu(g.ev_elapsed(&ms, (CUevent)ev0_, (CUevent)ev1_), "cuEventElapsedTime");
  return ms;
}

double now_seconds() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (double)ts.tv_sec + (double)ts.tv_nsec * 1e-9;
}
void check(mccsResult_t r, const char* what) {
  if (r != mccsSuccess) { fprintf(stderr, "%s: %s\n", what, mccsGetErrorString(r)); exit(1); }
}
size_t dtype_bytes(mccsDataType_t t) {
  switch (t) {
    case mccsInt8: case mccsUint8: return 1;
    case mccsFloat16: case mccsBfloat16: return 2;
    case mccsInt32: case mccsUint32: case mccsFloat32: return 4;
    default: return 8;
  }
}
bool parse_dtype(const std::string& s, mccsDataType_t* out) {
  static const std::map<std::string, mccsDataType_t> m = {
      {"int8", mccsInt8}, {"uint8", mccsUint8}, {"int32", mccsInt32}, {"uint32", mccsUint32},
      {"int64", mccsInt64}, {"uint64", mccsUint64}, {"half", mccsFloat16}, {"fp16", mccsFloat16},
      {"float16", mccsFloat16}, {"float", mccsFloat32}, {"fp32", mccsFloat32}, {"float32", mccsFloat32},
      {"double", mccsFloat64}, {"bf16", mccsBfloat16}, {"bfloat16", mccsBfloat16}};
  auto it = m.find(s);
  if (it == m.end()) return false;
  *out = it->second;
  return true;
}
int parse_algo(const std::string& s) {
  for (int a = 0; a <= 10; a++)
    if (s == mccsAlgoName(a)) return a;
  return -1;
}
void spin_sleep_us(uint64_t us) {
  // The reference's traffic generator spins for its compute phases
  // (src/mccs_examples/traffic_gen/src/main.rs:171-204); long phases sleep first.
  const double end = now_seconds() + (double)us * 1e-6;
  if (us > 2000) {
    struct timespec ts = {(time_t)((us - 1000) / 1000000), (long)(((us - 1000) % 1000000) * 1000)};
    nanosleep(&ts, nullptr);
  }
  while (now_seconds() < end) {}
}
std::string name_prefix(const std::string& name) { return name.empty() ? "" : "[" + name + "] "; }

}  // namespace app
