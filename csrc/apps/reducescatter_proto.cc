// Correctness probe for ReduceScatter (a collective this service adds to the reference's
// AllReduce and AllGather): rank r contributes the int32 value 1883 + r + block index in
// every element of every block; rank q must receive n * 1883 + n(n-1)/2 + n * q in its
// block. In place: the result lands in block `rank` of the input. Exit code = pass/fail,
// like the other probes (src/mccs_examples/allreduce_proto).
#include <stdio.h>
#include <stdlib.h>

#include <vector>

#include "app_common.h"

int main(int argc, char** argv) {
  const char* usage = "usage: reducescatter_proto --rank R --num-ranks N --cuda-device-idx D [--communicator 44] [--size 33554432] [--algo auto]";
  app::Options o(argc, argv);
  o.require({"rank", "num-ranks", "cuda-device-idx"}, usage);
  const int rank = (int)o.num("rank", 0), n = (int)o.num("num-ranks", 1), dev = (int)o.num("cuda-device-idx", 0);
  const size_t count = (size_t)o.num("size", 32 << 20) / 4 / (size_t)n;   // elements per block
  const int algo = app::parse_algo(o.str("algo", "auto"));
  if (algo < 0 || count == 0) { fprintf(stderr, "unknown --algo or --size too small\n"); return 2; }
  app::check(mccsInit(nullptr), "mccsInit");
  app::Device device(dev);
  int32_t* buf = nullptr;
  app::check(mccsMalloc((void**)&buf, dev, count * 4 * n), "mccsMalloc");
  std::vector<int32_t> host(count * n);
  for (int q = 0; q < n; q++)
    for (size_t i = 0; i < count; i++) host[(size_t)q * count + i] = 1883 + rank + q;
  device.upload(buf, host.data(), count * 4 * n);
  mccsComm_t comm;
  app::check(mccsCommInitRank(&comm, (uint32_t)o.num("communicator", 44), rank, n, dev, o.str("root-addr", "127.0.0.1").c_str()),
             "mccsCommInitRank");
  app::check(mccsReduceScatterEx(comm, buf, buf + (size_t)rank * count, count, mccsInt32, mccsSum, 1.0f, (mccsAlgo_t)algo, nullptr),
             "mccsReduceScatter");
  device.sync_stream(nullptr);
  device.download(host.data(), buf, count * 4 * n);
  const int32_t want = n * 1883 + n * (n - 1) / 2 + n * rank;
  size_t bad = 0;
  for (size_t i = 0; i < count; i++) bad += host[(size_t)rank * count + i] != want;
  // the other blocks of the input are untouched
  for (int q = 0; q < n; q++)
    for (size_t i = 0; q != rank && i < count; i++) bad += host[(size_t)q * count + i] != 1883 + rank + q;
  printf("Rank %d: reduce-scatter of %zu int32 per block: %s (%zu mismatches)\n", rank, count, bad ? "FAILED" : "passed", bad);
  mccsCommDestroy(comm);
  mccsFree(buf);
  mccsFinalize();
  return bad ? 1 : 0;
}
