// Tensor-core (tcgen05 / TMEM) stages of the KDA op for BF16 operands.
#include "kda_common.cuh"

namespace kda {

bool tc_supported(const KdaParams& p) { (void)p; return false; }
cudaError_t tc_fwd(const KdaParams& p, cudaStream_t s) { (void)p; (void)s; return cudaErrorNotSupported; }
cudaError_t tc_bwd(const KdaParams& p, cudaStream_t s) { (void)p; (void)s; return cudaErrorNotSupported; }

}  // namespace kda
