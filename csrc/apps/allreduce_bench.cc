// AllReduce bandwidth benchmark of one rank, command line compatible with the
// reference's allreduce_bench (src/mccs_examples/allreduce_bench/src/main.rs:17-60):
//   --root-addr A --rank R --num-ranks N --cuda-device-idx D --size S [--size-in-byte]
//   --communicator ID [--round 20] [--epoch 1] [--name tag]
// plus --dtype (half|bf16|float|int32, default half), --algo and --out-of-place.
// Like the reference it runs the buffer in place, does 1 + 5 warm-up rounds and then
// `round` x `epoch` timed operations, and prints "Algorithm bandwidth" and "Bus
// bandwidth" (factor 2(n-1)/n, main.rs:166-181). It reports both the reference's
// host-clock figure and a device-event figure.
#include <stdio.h>
#include <stdlib.h>

#include <vector>

#include "app_common.h"

int main(int argc, char** argv) {
  const char* usage =
      "usage: allreduce_bench --rank R --num-ranks N --cuda-device-idx D --size S [--size-in-byte]\n"
      "       --communicator ID [--root-addr A] [--round 20] [--epoch 1] [--dtype half] [--algo auto] [--name X]";
  app::Options o(argc, argv, {"size-in-byte", "out-of-place", "check"});
  o.require({"rank", "num-ranks", "cuda-device-idx", "size", "communicator"}, usage);
  const int rank = (int)o.num("rank", 0), n = (int)o.num("num-ranks", 1), dev = (int)o.num("cuda-device-idx", 0);
  mccsDataType_t dt = mccsFloat16;
  if (!app::parse_dtype(o.str("dtype", "half"), &dt)) { fprintf(stderr, "unknown dtype\n%s\n", usage); return 2; }
  const size_t esz = app::dtype_bytes(dt);
  size_t bytes = (size_t)o.num("size", 0);
  if (!o.flag("size-in-byte")) bytes *= esz;    // the reference's default unit is elements of the type
  const size_t count = bytes / esz;
  const int rounds = (int)o.num("round", 20), epochs = (int)o.num("epoch", 1);
  const int algo = app::parse_algo(o.str("algo", "auto"));
  if (algo < 0) { fprintf(stderr, "unknown --algo\n"); return 2; }
  const std::string prefix = app::name_prefix(o.str("name"));

  app::check(mccsInit(nullptr), "mccsInit");
  app::Device device(dev);
  void* buf = nullptr;
  void* out = nullptr;
  app::check(mccsMalloc(&buf, dev, bytes), "mccsMalloc");
  if (o.flag("out-of-place")) app::check(mccsMalloc(&out, dev, bytes), "mccsMalloc");
  else out = buf;
  std::vector<uint8_t> host(bytes, 0);
  device.upload(buf, host.data(), bytes);
  mccsComm_t comm;
  app::check(mccsCommInitRank(&comm, (uint32_t)o.num("communicator", 0), rank, n, dev, o.str("root-addr", "127.0.0.1").c_str()),
             "mccsCommInitRank");
  app::check(mccsRegisterStream(dev, nullptr), "mccsRegisterStream");
  auto run = [&]() {
    app::check(mccsAllReduceEx(comm, buf, out, count, dt, mccsSum, 1.0f, (mccsAlgo_t)algo, nullptr), "mccsAllReduce");
  };
  printf("%sRank %d: warmup\n", prefix.c_str(), rank);
  for (int i = 0; i < 6; i++) run();
  device.sync_stream(nullptr);
  for (int e = 0; e < epochs; e++) {
    const double t0 = app::now_seconds();
    device.timer_start(nullptr);
    for (int i = 0; i < rounds; i++) run();
    const double dev_ms = device.timer_stop(nullptr);
    device.sync_stream(nullptr);
    const double host_s = app::now_seconds() - t0;
    const double alg_host = (double)bytes * rounds / host_s / 1e9;
    const double alg_dev = (double)bytes * rounds / (dev_ms * 1e-3) / 1e9;
    const double factor = n > 1 ? 2.0 * (n - 1) / n : 1.0;
    uint32_t variant = 0, ctas = 0;
    mccsCommLastPlan(comm, &variant, &ctas);
    printf("%sRank %d: Algorithm bandwidth: %.3f GB/s, Bus bandwidth: %.3f GB/s (host clock) | device events: "
           "alg %.3f GB/s, bus %.3f GB/s, %.3f us/op | %s x%u CTAs\n",
           prefix.c_str(), rank, alg_host, alg_host * factor, alg_dev, alg_dev * factor, dev_ms * 1e3 / rounds,
           mccsAlgoName((int)variant), ctas);
  }
  app::check(mccsCommDestroy(comm), "mccsCommDestroy");
  if (out != buf) mccsFree(out);
  mccsFree(buf);
  mccsFinalize();
  return 0;
}
