// One translation unit per element type (same -DMCCS_T / -DMCCS_TNAME / -DMCCS_NVLS
// scheme as inst_dtype.cu): instantiates the fused AllReduce, hybrid and reduce-scatter
// kernels and exports their lookup function.
#include "batch.cuh"
#include "hybrid.cuh"
#include "scatter.cuh"

namespace mccs {
namespace dev {

#define MCCS_CAT2(a, b) a##b
#define MCCS_CAT(a, b) MCCS_CAT2(a, b)

extern "C" const void* MCCS_CAT(mccs_kfn_batch_, MCCS_TNAME)(int variant, int op) {
#ifdef MCCS_NVLS
  if (variant == kArHybrid) {
    if (op != kSum && op != kSumPostDiv) return nullptr;
    return (const void*)&ar_hybrid_kernel<MCCS_T>;
  }
  if (variant == kArNvlsTwo) {
    if (op != kSum && op != kSumPostDiv) return nullptr;
    return (const void*)&ar_nvls_batch_kernel<MCCS_T>;
  }
  if (variant == kRsNvls) {
    if (op != kSum && op != kSumPostDiv) return nullptr;
    return (const void*)&rs_nvls_kernel<MCCS_T>;
  }
#endif
  if (variant == kRsDirect) {
    switch (op) {
      case kSum: case kPreMulSum: case kSumPostDiv: return (const void*)&rs_direct_kernel<MCCS_T, OpSum>;
      case kProd: return (const void*)&rs_direct_kernel<MCCS_T, OpProd>;
      case kMax: return (const void*)&rs_direct_kernel<MCCS_T, OpMax>;
      case kMin: return (const void*)&rs_direct_kernel<MCCS_T, OpMin>;
    }
    return nullptr;
  }
  if (variant != kArTwoShot) return nullptr;
  switch (op) {
    case kSum: case kPreMulSum: case kSumPostDiv: return (const void*)&ar_twoshot_batch_kernel<MCCS_T, OpSum>;
    case kProd: return (const void*)&ar_twoshot_batch_kernel<MCCS_T, OpProd>;
    case kMax: return (const void*)&ar_twoshot_batch_kernel<MCCS_T, OpMax>;
    case kMin: return (const void*)&ar_twoshot_batch_kernel<MCCS_T, OpMin>;
  }
  return nullptr;
}

}  // namespace dev
}  // namespace mccs
