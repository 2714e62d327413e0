// The streaming matmul kernels whose activation prologue is GEMV_PRO_SWIGLU (see gemv_stream_kernel.cuh).
#undef MCU_TRACE  // the diagnostic stamps live in gemv_stream.cu alone
#include "gemv_stream_kernel.cuh"

namespace mcu {

cudaError_t launch_gemv_stream_swiglu(int kind, int T, bool short_cfg, const GemvStreamParams &p, int gx, int smem, cudaStream_t s) {
    return launch_all_kinds<GEMV_PRO_SWIGLU>(kind, T, short_cfg, p, gx, smem, s);
}

}  // namespace mcu
