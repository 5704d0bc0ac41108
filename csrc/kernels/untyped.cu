// Kernels that do not depend on the element type: AllGather (bytes), the ring
// AllGather and the single-rank copy, plus their lookup function.
#define MCCS_UNTYPED_KERNELS 1
#include "collectives.cuh"

namespace mccs {
namespace dev {

extern "C" const void* mccs_kfn_untyped(int variant) {
  switch (variant) {
    case kAgPull: return (const void*)&ag_direct_kernel<kAgModePull>;
    case kAgPush: return (const void*)&ag_direct_kernel<kAgModePush>;
    case kAgNvls: return (const void*)&ag_direct_kernel<kAgModeNvls>;
    case kAgRing: return (const void*)&ag_ring_kernel;
    case kLocalCopy: return (const void*)&local_copy_kernel;
  }
  return nullptr;
}

}  // namespace dev
}  // namespace mccs
