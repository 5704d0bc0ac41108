// One translation unit per element type (compiled with -DMCCS_T=<type>
// -DMCCS_TNAME=<suffix> [-DMCCS_NVLS=1]): instantiates the typed AllReduce kernels
// and exports a lookup function used by the launcher. The reference builds one
// object per (collective, op, type) the same way (src/collectives/gen_rules.sh:5-40).
#include "collectives.cuh"

namespace mccs {
namespace dev {

#define MCCS_CAT2(a, b) a##b
#define MCCS_CAT(a, b) MCCS_CAT2(a, b)

template <typename Op>
static const void* typed_kernel(int variant) {
  switch (variant) {
    case kArOneShot: return (const void*)&ar_oneshot_kernel<MCCS_T, Op>;
    case kArTwoShot: return (const void*)&ar_twoshot_kernel<MCCS_T, Op>;
    case kArRing: return (const void*)&ar_ring_kernel<MCCS_T, Op>;
  }
  return nullptr;
}

extern "C" const void* MCCS_CAT(mccs_kfn_, MCCS_TNAME)(int variant, int op) {
#ifdef MCCS_NVLS
  if (variant == kArNvlsOne || variant == kArNvlsTwo) {
    if (op != kSum && op != kSumPostDiv) return nullptr;
    return variant == kArNvlsTwo ? (const void*)&ar_nvls_kernel<MCCS_T, true>
                                 : (const void*)&ar_nvls_kernel<MCCS_T, false>;
  }
#endif
  switch (op) {
    case kSum: case kPreMulSum: case kSumPostDiv: return typed_kernel<OpSum>(variant);
    case kProd: return typed_kernel<OpProd>(variant);
    case kMax: return typed_kernel<OpMax>(variant);
    case kMin: return typed_kernel<OpMin>(variant);
  }
  return nullptr;
}

}  // namespace dev
}  // namespace mccs
