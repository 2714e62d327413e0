// Tensor-core GEMM regime (placeholder until the tcgen05 kernel lands): reports "not covered" so the
// dispatcher keeps the multi-token GEMV kernels.
#include "common.cuh"
#include "kernels.h"

namespace mcu {

bool gemm_tc_supported(int, int, int, int) { return false; }

cudaError_t launch_gemm_tc(int, const void *, const void *, const __half *, int, int, int, int, const float *, float *,
                           float *, int, cudaStream_t, int *launches) {
    if (launches != nullptr) *launches = 0;
    return cudaErrorNotSupported;
}

}  // namespace mcu
