// mcu_linear_static_scratch: the decode-regime quantized linear for callers that must not allocate.
//
// The quantized activations (the only scratch this path needs) live in a fixed array in device
// memory that is part of the library image, so the call performs no cudaMalloc / cudaFree and uses no
// context workspace.  Every GPU that loads the library carries the array until the process exits.
#include "../../include/marmot_cuda.h"

#include "common.cuh"
#include "kernels.h"

#include <cstdio>
#include <mutex>

namespace mcu {

// Limits of the fixed scratch: up to 8 tokens, K up to 16384.
constexpr size_t SS_MAX_T = MCU_STATIC_SCRATCH_MAX_T;
constexpr size_t SS_MAX_K = MCU_STATIC_SCRATCH_MAX_K;
constexpr size_t SS_QS_BYTES = SS_MAX_T * SS_MAX_K;                                // int8 quants, padded rows
constexpr size_t SS_D_BYTES = SS_MAX_T * (SS_MAX_K / Q8_0_VALUES) * sizeof(float);  // one scale per 32 (Q8_0) or 256
constexpr size_t SS_BSUMS_BYTES = SS_MAX_T * (SS_MAX_K / QK_K) * 16 * sizeof(int16_t);
constexpr size_t SS_TOTAL = SS_QS_BYTES + SS_D_BYTES + SS_BSUMS_BYTES;  // 160 KiB

// In host code this name is only a handle for the symbol, not a device address: the address the
// kernels need comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_static_scratch[SS_TOTAL];

constexpr int SS_MAX_DEVICES = 64;
static std::mutex g_ss_mutex;
static unsigned char *g_ss_addr[SS_MAX_DEVICES] = {};

// Device address of the scratch array on the current device (looked up on the first call there).
static int static_scratch_address(unsigned char **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return set_error(MCU_ERROR_DEVICE_NOT_AVAILABLE, cudaGetErrorString(e));
    if (dev < 0 || dev >= SS_MAX_DEVICES) return set_error(MCU_ERROR_DEVICE_NOT_AVAILABLE, "device index out of range");
    std::lock_guard<std::mutex> lock(g_ss_mutex);
    if (g_ss_addr[dev] == nullptr) {
        unsigned char *ptr = nullptr;
        e = cudaGetSymbolAddress((void **)&ptr, g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            char msg[160];
            snprintf(msg, sizeof(msg), "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
            return set_error(e == cudaSuccess ? MCU_ERROR_BACKEND_INIT_FAILED : MCU_ERROR_DEVICE_NOT_AVAILABLE, msg);
        }
        g_ss_addr[dev] = ptr;
    }
    *out = g_ss_addr[dev];
    return MCU_SUCCESS;
}

}  // namespace mcu

using namespace mcu;

extern "C" int mcu_linear_static_scratch(void *cuda_stream, int kind, const float *x_dev, size_t ldx,
                                         const void *w_dev, size_t T, size_t K, size_t F, const float *bias_dev,
                                         float *out_dev, size_t ldo) {
    if (!kind_supported(kind)) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "quant kind has no CUDA kernel");
    if (T == 0 || F == 0) return MCU_SUCCESS;
    if (x_dev == nullptr || w_dev == nullptr || out_dev == nullptr)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "Tensor argument must not be null");
    if (T > SS_MAX_T || K > SS_MAX_K) {
        char msg[200];
        snprintf(msg, sizeof(msg),
                 "mcu_linear_static_scratch handles at most T=%zu tokens and K=%zu (got T=%zu, K=%zu): its scratch is a "
                 "fixed array; use mcu_linear for larger problems",
                 SS_MAX_T, SS_MAX_K, T, K);
        return set_error(MCU_ERROR_INVALID_ARGUMENT, msg);
    }
    if (K == 0 || ldx < K || ldo < F) return set_error(MCU_ERROR_DIMENSION_MISMATCH, "bad K or row stride");
    if (F > ((size_t)1 << 30) || ldx > ((size_t)1 << 30) || ldo > ((size_t)1 << 30))
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "dimension or row stride too large");
    if ((uintptr_t)w_dev & (kind == MCU_KIND_Q4_K ? 15 : 1))
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "weight blocks are not aligned");
    unsigned char *scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    cudaStream_t s = (cudaStream_t)cuda_stream;
    // Every byte the GEMV reads is rewritten by the packer of this call (quants incl. the zero padding of a
    // ragged last block, scales and block sums for all T rows), so nothing in the array has to start at zero.
    ActBuffers ab;
    ab.qs = (int8_t *)scratch;
    ab.d = (float *)(scratch + SS_QS_BYTES);
    ab.bsums = (int16_t *)(scratch + SS_QS_BYTES + SS_D_BYTES);
    cudaError_t e = launch_quantize_act(kind, x_dev, (int)ldx, (int)T, (int)K, ab, nullptr, s);
    if (e == cudaSuccess)
        e = launch_gemv(kind, w_dev, nullptr, ab, (int)T, (int)K, (int)F, bias_dev, out_dev, nullptr, (int)ldo, s);
    if (e != cudaSuccess) return set_error(MCU_ERROR_INVALID_OPERATION, cudaGetErrorString(e));
    count_launches(2);
    return MCU_SUCCESS;
}
