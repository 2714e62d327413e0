// Block dequantizers, bit-exact with the reference CPU code:
//   Q4_K  out = (d*sc)*q - (dmin*m)      src/backends/cpu/quantization/formats/q4k_gguf.c:133-166
//   Q6_K  out = (d*sc)*q, q in [-32,31]  src/backends/cpu/quantization/formats/q6k_gguf.c:63-99
//   Q8_0  out = (float)q * d             src/backends/cpu/quantization/formats/q8_gguf.c:110-114,189-200
// Every product is rounded separately (no FMA), as the reference's scalar build does.
#include "common.cuh"
#include "kernels.h"

namespace mcu {

// Each thread produces four consecutive values (one float4 when the tail allows).
__global__ void __launch_bounds__(256)
dequantize_q4_k_kernel(const uint8_t *__restrict__ blocks, size_t n_values, float *__restrict__ out) {
    const size_t q4 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // index of the group of 4 values
    const size_t e0 = q4 * 4;
    if (e0 >= n_values) return;
    const size_t blk = e0 / QK_K;
    const int e = (int)(e0 - blk * QK_K);
    const uint8_t *b = blocks + blk * Q4_K_BYTES;
    const float d = half_bits_to_float(*(const uint16_t *)b);
    const float dmin = half_bits_to_float(*(const uint16_t *)(b + 2));
    const int g = e >> 6, hi = (e >> 5) & 1, l = e & 31;
    int sc, mn;
    k4_scale_min(2 * g + hi, b + 4, sc, mn);
    const float dl = __fmul_rn(d, (float)sc), ml = __fmul_rn(dmin, (float)mn);
    const uint32_t w = *(const uint32_t *)(b + 16 + g * 32 + l);
    float r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t byte = (w >> (8 * i)) & 0xFFu;
        const float q = (float)(hi ? (byte >> 4) : (byte & 0xFu));
        r[i] = __fsub_rn(__fmul_rn(dl, q), ml);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
        if (e0 + i < n_values) out[e0 + i] = r[i];
}

__global__ void __launch_bounds__(256)
dequantize_q6_k_kernel(const uint8_t *__restrict__ blocks, size_t n_values, float *__restrict__ out) {
    const size_t q4 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t e0 = q4 * 4;
    if (e0 >= n_values) return;
    const size_t blk = e0 / QK_K;
    const int e = (int)(e0 - blk * QK_K);
    const uint8_t *b = blocks + blk * Q6_K_BYTES;
    const float d = half_bits_to_float((uint16_t)(b[208] | (b[209] << 8)));
    const int n = e >> 7, c = (e >> 5) & 3, l = e & 31;  // value = 128n + 32c + l
    const uint8_t *ql = b + n * 64 + (c & 1) * 32 + l;
    const uint8_t *qh = b + 128 + n * 32 + l;
    const int8_t sc = (int8_t)b[192 + n * 8 + 2 * c + (l >> 4)];
    const float ds = __fmul_rn(d, (float)sc);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int lo = (c & 2) ? (ql[i] >> 4) : (ql[i] & 0xF);
        const int h2 = (qh[i] >> (2 * c)) & 3;
        const int q = (lo | (h2 << 4)) - 32;
        if (e0 + i < n_values) out[e0 + i] = __fmul_rn(ds, (float)q);
    }
}

__global__ void __launch_bounds__(256)
dequantize_q8_0_kernel(const uint8_t *__restrict__ blocks, size_t n_values, float *__restrict__ out) {
    const size_t q4 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t e0 = q4 * 4;
    if (e0 >= n_values) return;
    const size_t blk = e0 / Q8_0_VALUES;
    const int e = (int)(e0 - blk * Q8_0_VALUES);
    const uint8_t *b = blocks + blk * Q8_0_BYTES;
    const float d = half_bits_to_float((uint16_t)(b[0] | (b[1] << 8)));
#pragma unroll
    for (int i = 0; i < 4; ++i)
        if (e0 + i < n_values) out[e0 + i] = __fmul_rn((float)(int8_t)b[2 + e + i], d);
}

cudaError_t launch_dequantize(int kind, const void *blocks, size_t n_values, float *out, cudaStream_t s) {
    if (n_values == 0) return cudaSuccess;
    const size_t groups = (n_values + 3) / 4;
    const unsigned grid = (unsigned)((groups + 255) / 256);
    const uint8_t *b = (const uint8_t *)blocks;
    if (kind == KIND_Q4_K) dequantize_q4_k_kernel<<<grid, 256, 0, s>>>(b, n_values, out);
    else if (kind == KIND_Q6_K) dequantize_q6_k_kernel<<<grid, 256, 0, s>>>(b, n_values, out);
    else if (kind == KIND_Q8_0) dequantize_q8_0_kernel<<<grid, 256, 0, s>>>(b, n_values, out);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

}  // namespace mcu
