// Trace-driven traffic generator: replays (collective, size, compute interval)
// traces the way the reference's traffic_gen does
// (src/mccs_examples/traffic_gen/src/main.rs:24-44,129-237) and reads the same TOML
// files (workloads/*.toml: communicator_id, cuda_devices[], [[traces]] size / type /
// compute_interval in microseconds).
//   traffic_gen --rank R --config trace.toml [--iters 20] [--save-path times.csv]
//               [--verbose] [--name tag] [--root-addr A]
// Each iteration spins for the compute interval, issues the fp16 AllReduce (or, beyond the
// reference's trace types, the fp16 ReduceScatter, type "reduce_scatter") or the
// AllGather of `size` bytes and synchronises the stream; rank 0 prints the total run
// time (the job completion time of the reference's figure 9) and can save the
// per-iteration times; the first 20 iterations are dropped from the statistics.
#include <stdio.h>
#include <stdlib.h>

#include <algorithm>
#include <string>
#include <vector>

#include "../common/value.h"
#include "app_common.h"

struct Trace { size_t size; bool all_reduce; bool reduce_scatter = false; uint64_t compute_us; };

int main(int argc, char** argv) {
  const char* usage = "usage: traffic_gen --rank R --config trace.toml [--iters 20] [--save-path f.csv] [--verbose] [--name X]";
  app::Options o(argc, argv, {"verbose"});
  o.require({"rank", "config"}, usage);
  const int rank = (int)o.num("rank", 0);
  const int iters = (int)o.num("iters", 20);
  const std::string prefix = app::name_prefix(o.str("name"));
  mccs::Value cfg;
  try {
    cfg = mccs::parse_toml(mccs::read_text_file(o.str("config")));
  } catch (const std::exception& e) {
    fprintf(stderr, "traffic_gen: %s\n", e.what());
    return 2;
  }
  const mccs::Value& devs = cfg.has("cuda_devices") ? cfg["cuda_devices"] : cfg["communicator_devices"];
  const int n = (int)devs.size();
  if (rank < 0 || rank >= n) { fprintf(stderr, "rank %d outside cuda_devices[%d]\n", rank, n); return 2; }
  const int dev = (int)devs.at((size_t)rank).as_int();
  const uint32_t comm_id = (uint32_t)(cfg.has("communicator_id") ? cfg["communicator_id"] : cfg["comm_id"]).as_int();
  std::vector<Trace> traces;
  for (const mccs::Value& t : cfg["traces"].items()) {
    Trace tr;
    tr.size = (size_t)(t.has("size") ? t["size"] : t["message_size"]).as_int();
    const std::string type = (t.has("type") ? t["type"] : t["op_type"]).as_string();
    tr.all_reduce = type == "all_reduce" || type == "AllReduce";
    tr.reduce_scatter = type == "reduce_scatter" || type == "ReduceScatter";   // `size` = the whole input of a rank
    tr.compute_us = (uint64_t)t["compute_interval"].as_int();
    traces.push_back(tr);
  }
  if (traces.empty()) { fprintf(stderr, "no traces in the configuration\n"); return 2; }
  size_t buffer = 0;
  for (const Trace& t : traces) buffer = std::max(buffer, t.all_reduce || t.reduce_scatter ? t.size : t.size * (size_t)n);
  buffer = (buffer + (size_t)n - 1) / (size_t)n * (size_t)n;
  buffer = (buffer + 255) / 256 * 256;

  app::check(mccsInit(nullptr), "mccsInit");
  app::Device device(dev);
  char* buf = nullptr;
  app::check(mccsMalloc((void**)&buf, dev, buffer), "mccsMalloc");
  {
    std::vector<uint8_t> host(buffer, 0);   // zeros: repeated sums stay finite
    device.upload(buf, host.data(), buffer);
  }
  mccsComm_t comm;
  app::check(mccsCommInitRank(&comm, comm_id, rank, n, dev, o.str("root-addr", "127.0.0.1").c_str()), "mccsCommInitRank");
  app::check(mccsRegisterStream(dev, nullptr), "mccsRegisterStream");
  printf("%sRank %d: start warmup\n", prefix.c_str(), rank);
  const size_t per_rank = buffer / (size_t)n / 16 * 16;
  for (int i = 0; i < 5; i++)
    app::check(mccsAllGather(comm, buf + (size_t)rank * per_rank, buf, per_rank, nullptr), "mccsAllGather");
  device.sync_stream(nullptr);
  printf("%sRank %d: warmup done\n", prefix.c_str(), rank);

  std::vector<double> round_ms;
  const double global_start = app::now_seconds();
  double start = global_start;
  for (int iter = 0; iter < iters; iter++) {
    for (const Trace& t : traces) {
      app::spin_sleep_us(t.compute_us);
      if (t.all_reduce) {
        app::check(mccsAllReduce(comm, buf, buf, t.size / 2, mccsFloat16, mccsSum, nullptr), "mccsAllReduce");
      } else if (t.reduce_scatter) {
        const size_t block = t.size / 2 / (size_t)n / 8 * 8;   // fp16 elements per block, 16-byte multiples
        if (block)
          app::check(mccsReduceScatter(comm, buf, buf + (size_t)rank * block * 2, block, mccsFloat16, mccsSum, nullptr), "mccsReduceScatter");
      } else {
        const size_t sz = t.size / 16 * 16;
        app::check(mccsAllGather(comm, buf + (size_t)rank * sz, buf, sz, nullptr), "mccsAllGather");
      }
      device.sync_stream(nullptr);
    }
    const double end = app::now_seconds();
    const double ms = (end - start) * 1e3;
    start = end;
    if (o.flag("verbose") && rank == 0) printf("%s[Rank 0] Iter %d time: %.3f ms\n", prefix.c_str(), iter, ms);
    round_ms.push_back(ms);
    if (iter == 20) round_ms.clear();
  }
  const double run_ms = (app::now_seconds() - global_start) * 1e3;
  if (rank == 0) {
    printf("%sRank %d: run time: %llu ms\n", prefix.c_str(), rank, (unsigned long long)run_ms);
    if (!round_ms.empty()) {
      std::vector<double> s = round_ms;
      std::sort(s.begin(), s.end());
      double sum = 0;
      for (double x : s) sum += x;
      printf("%s(mean, median, min, max) = (%.3f, %.3f, %.3f, %.3f) ms over %zu iterations\n", prefix.c_str(),
             sum / (double)s.size(), s[s.size() / 2], s.front(), s.back(), s.size());
    }
    if (o.has("save-path")) {
      FILE* f = fopen(o.str("save-path").c_str(), "w");
      if (f) {
        fprintf(f, "iteration,time_ms\n");
        for (size_t i = 0; i < round_ms.size(); i++) fprintf(f, "%zu,%.6f\n", i, round_ms[i]);
        fclose(f);
      }
    }
  }
  mccsCommDestroy(comm);
  mccsFree(buf);
  mccsFinalize();
  return 0;
}
