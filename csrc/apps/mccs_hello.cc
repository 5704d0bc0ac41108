// Smallest client: allocate through the daemon, write, read back (the reference's
// cuda_hello, src/mccs_examples/cuda_hello).
#include <stdio.h>

#include <vector>

#include "app_common.h"

int main(int argc, char** argv) {
  app::Options o(argc, argv);
  o.require({}, "usage: mccs_hello [--cuda-device-idx 0]");
  const int dev = (int)o.num("cuda-device-idx", 0);
  app::check(mccsInit(nullptr), "mccsInit");
  printf("backend: %s, %d device(s)\n", mccsBackendKind() == 1 ? "cuda" : "host", mccsDeviceCount());
  app::Device device(dev);
  void* p = nullptr;
  app::check(mccsMalloc(&p, dev, 1 << 20), "mccsMalloc");
  std::vector<int> in(1024), out(1024, 0);
  for (int i = 0; i < 1024; i++) in[i] = i * 7;
  device.upload(p, in.data(), 4096);
  device.download(out.data(), p, 4096);
  uint64_t id = 0, off = 0, size = 0;
  mccsMemInfo(p, &id, &off, &size);
  const bool ok = in == out;
  printf("allocation %llu of %llu bytes at %p: %s\n", (unsigned long long)id, (unsigned long long)size, p,
         ok ? "round trip ok" : "MISMATCH");
  mccsFree(p);
  mccsFinalize();
  return ok ? 0 : 1;
}
