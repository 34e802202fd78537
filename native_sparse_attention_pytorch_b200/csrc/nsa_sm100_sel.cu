// Tensor-core (tcgen05 / TMA) family for the selected-block branch.
#include "nsa_common.cuh"
#include "nsa_kernels.h"

namespace nsa {

int64_t sm100_sel_workspace_bytes(const nsa_sel_fwd_args&, bool) { return NSA_ERR_UNSUPPORTED; }
int sm100_sel_fwd(const nsa_sel_fwd_args&, cudaStream_t) { return NSA_ERR_UNSUPPORTED; }
int sm100_sel_bwd(const nsa_sel_bwd_args&, cudaStream_t) { return NSA_ERR_UNSUPPORTED; }

}  // namespace nsa
