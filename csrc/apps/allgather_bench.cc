// AllGather bandwidth benchmark of one rank; options of the reference's
// allgather_bench (src/mccs_examples/allgather_bench/src/main.rs:96-176): --size is
// the per-rank contribution (elements of 4 bytes unless --size-in-byte), the gather
// runs in place (send = recv + rank*size), the first result is verified, algorithm
// bandwidth counts the total gathered bytes and bus bandwidth is alg*(n-1)/n.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "app_common.h"

int main(int argc, char** argv) {
  const char* usage =
      "usage: allgather_bench --rank R --num-ranks N --cuda-device-idx D --size S [--size-in-byte]\n"
      "       --communicator ID [--root-addr A] [--round 20] [--epoch 1] [--algo auto] [--name X]";
  app::Options o(argc, argv, {"size-in-byte"});
  o.require({"rank", "num-ranks", "cuda-device-idx", "size", "communicator"}, usage);
  const int rank = (int)o.num("rank", 0), n = (int)o.num("num-ranks", 1), dev = (int)o.num("cuda-device-idx", 0);
  size_t bytes = (size_t)o.num("size", 0);
  if (!o.flag("size-in-byte")) bytes *= 4;
  const int rounds = (int)o.num("round", 20), epochs = (int)o.num("epoch", 1);
  const int algo = app::parse_algo(o.str("algo", "auto"));
  if (algo < 0) { fprintf(stderr, "unknown --algo\n"); return 2; }
  const std::string prefix = app::name_prefix(o.str("name"));

  app::check(mccsInit(nullptr), "mccsInit");
  app::Device device(dev);
  char* buf = nullptr;
  app::check(mccsMalloc((void**)&buf, dev, bytes * n), "mccsMalloc");
  std::vector<uint8_t> host(bytes * n, 0);
  for (size_t i = 0; i < bytes; i++) host[(size_t)rank * bytes + i] = (uint8_t)(rank * 31 + i % 251);
  device.upload(buf, host.data(), bytes * n);
  mccsComm_t comm;
  app::check(mccsCommInitRank(&comm, (uint32_t)o.num("communicator", 0), rank, n, dev, o.str("root-addr", "127.0.0.1").c_str()),
             "mccsCommInitRank");
  app::check(mccsRegisterStream(dev, nullptr), "mccsRegisterStream");
  auto run = [&]() {
    app::check(mccsAllGatherEx(comm, buf + (size_t)rank * bytes, buf, bytes, (mccsAlgo_t)algo, nullptr), "mccsAllGather");
  };
  run();
  device.sync_stream(nullptr);
  device.download(host.data(), buf, bytes * n);
  for (int r = 0; r < n; r++)
    for (size_t i = 0; i < bytes; i += 997)
      if (host[(size_t)r * bytes + i] != (uint8_t)(r * 31 + i % 251)) {
        fprintf(stderr, "%sRank %d: wrong byte from rank %d at %zu\n", prefix.c_str(), rank, r, i);
        return 1;
      }
  for (int i = 0; i < 5; i++) run();
  device.sync_stream(nullptr);
  for (int e = 0; e < epochs; e++) {
    const double t0 = app::now_seconds();
    device.timer_start(nullptr);
    for (int i = 0; i < rounds; i++) run();
    const double dev_ms = device.timer_stop(nullptr);
    device.sync_stream(nullptr);
    const double host_s = app::now_seconds() - t0;
    const double total = (double)bytes * n * rounds;
    const double factor = n > 1 ? (double)(n - 1) / n : 1.0;
    uint32_t variant = 0, ctas = 0;
    mccsCommLastPlan(comm, &variant, &ctas);
    printf("%sRank %d: Algorithm bandwidth: %.3f GB/s, Bus bandwidth: %.3f GB/s (host clock) | device events: "
           "alg %.3f GB/s, bus %.3f GB/s, %.3f us/op | %s x%u CTAs\n",
           prefix.c_str(), rank, total / host_s / 1e9, total / host_s / 1e9 * factor, total / (dev_ms * 1e-3) / 1e9,
           total / (dev_ms * 1e-3) / 1e9 * factor, dev_ms * 1e3 / rounds, mccsAlgoName((int)variant), ctas);
  }
  app::check(mccsCommDestroy(comm), "mccsCommDestroy");
  mccsFree(buf);
  mccsFinalize();
  return 0;
}
