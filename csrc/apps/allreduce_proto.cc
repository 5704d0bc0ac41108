// Correctness probe: int32 sum AllReduce with a closed-form expected value, the exit
// code tells pass/fail. Same check as the reference's allreduce_proto
// (src/mccs_examples/allreduce_proto/src/main.rs:75-116): every rank contributes
// 2042 + rank, so each element must become 2042*n + n(n-1)/2.
#include <stdio.h>
#include <stdlib.h>

#include <vector>

#include "app_common.h"

int main(int argc, char** argv) {
  const char* usage = "usage: allreduce_proto --rank R --num-ranks N --cuda-device-idx D [--communicator 42] [--size 33554432] [--algo auto]";
  app::Options o(argc, argv);
  o.require({"rank", "num-ranks", "cuda-device-idx"}, usage);
  const int rank = (int)o.num("rank", 0), n = (int)o.num("num-ranks", 1), dev = (int)o.num("cuda-device-idx", 0);
  const size_t count = (size_t)o.num("size", 32 << 20) / 4;
  const int algo = app::parse_algo(o.str("algo", "auto"));
  if (algo < 0) { fprintf(stderr, "unknown --algo\n"); return 2; }
  app::check(mccsInit(nullptr), "mccsInit");
  app::Device device(dev);
  int32_t* buf = nullptr;
  app::check(mccsMalloc((void**)&buf, dev, count * 4), "mccsMalloc");
  std::vector<int32_t> host(count, 2042 + rank);
  device.upload(buf, host.data(), count * 4);
  mccsComm_t comm;
  app::check(mccsCommInitRank(&comm, (uint32_t)o.num("communicator", 42), rank, n, dev, o.str("root-addr", "127.0.0.1").c_str()),
             "mccsCommInitRank");
  app::check(mccsAllReduceEx(comm, buf, buf, count, mccsInt32, mccsSum, 1.0f, (mccsAlgo_t)algo, nullptr), "mccsAllReduce");
  device.sync_stream(nullptr);
  device.download(host.data(), buf, count * 4);
  const int32_t want = 2042 * n + n * (n - 1) / 2;
  size_t bad = 0;
  for (size_t i = 0; i < count; i++) bad += host[i] != want;
  printf("Rank %d: all-reduce of %zu int32: %s (expected %d, %zu mismatches)\n", rank, count, bad ? "FAILED" : "passed", want, bad);
  mccsCommDestroy(comm);
  mccsFree(buf);
  mccsFinalize();
  return bad ? 1 : 0;
}
