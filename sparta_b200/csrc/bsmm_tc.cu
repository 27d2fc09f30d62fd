// placeholder until the tcgen05 kernels land
#include "bsmm.cuh"
namespace sparta {
bool bsmm_tc_available() { return false; }
bool bsmm_tc_supported(const BsmmParams&) { return false; }
int bsmm_tc(const BsmmParams&, cudaStream_t) { return SPARTA_ERR_UNSUPPORTED; }
}  // namespace sparta
