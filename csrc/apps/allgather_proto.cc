// Correctness probe for AllGather: rank r contributes the int32 value 1883 + r, the
// gathered buffer must hold every rank's value in rank order; exit code = pass/fail
// (counterpart of src/mccs_examples/allgather_proto).
#include <stdio.h>
#include <stdlib.h>

#include <vector>

#include "app_common.h"

int main(int argc, char** argv) {
  const char* usage = "usage: allgather_proto --rank R --num-ranks N --cuda-device-idx D [--communicator 43] [--size 33554432] [--algo auto]";
  app::Options o(argc, argv);
  o.require({"rank", "num-ranks", "cuda-device-idx"}, usage);
  const int rank = (int)o.num("rank", 0), n = (int)o.num("num-ranks", 1), dev = (int)o.num("cuda-device-idx", 0);
  const size_t count = (size_t)o.num("size", 32 << 20) / 4;   // per rank
  const int algo = app::parse_algo(o.str("algo", "auto"));
  if (algo < 0) { fprintf(stderr, "unknown --algo\n"); return 2; }
  app::check(mccsInit(nullptr), "mccsInit");
  app::Device device(dev);
  int32_t* buf = nullptr;
  app::check(mccsMalloc((void**)&buf, dev, count * 4 * n), "mccsMalloc");
  std::vector<int32_t> host(count * n, 0);
  for (size_t i = 0; i < count; i++) host[(size_t)rank * count + i] = 1883 + rank;
  device.upload(buf, host.data(), count * 4 * n);
  mccsComm_t comm;
  app::check(mccsCommInitRank(&comm, (uint32_t)o.num("communicator", 43), rank, n, dev, o.str("root-addr", "127.0.0.1").c_str()),
             "mccsCommInitRank");
  app::check(mccsAllGatherEx(comm, buf + (size_t)rank * count, buf, count * 4, (mccsAlgo_t)algo, nullptr), "mccsAllGather");
  device.sync_stream(nullptr);
  device.download(host.data(), buf, count * 4 * n);
  size_t bad = 0;
  for (int r = 0; r < n; r++)
    for (size_t i = 0; i < count; i++) bad += host[(size_t)r * count + i] != 1883 + r;
  printf("Rank %d: all-gather of %zu int32 per rank: %s (%zu mismatches)\n", rank, count, bad ? "FAILED" : "passed", bad);
  mccsCommDestroy(comm);
  mccsFree(buf);
  mccsFinalize();
  return bad ? 1 : 0;
}
