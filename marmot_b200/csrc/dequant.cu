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
dequantize_q4_k_kernel(const uint8_t *__restrict__ blocks, size_t n_values, float *__restrict__ out,
                       const int32_t *__restrict__ row_ids, size_t row_values, size_t row_bytes) {
    const size_t q4 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // index of the group of 4 values
    const size_t e0 = q4 * 4;
    if (e0 >= n_values) return;
    size_t er = e0;  // value index inside the source row (gather) or inside the whole buffer
    if (row_ids != nullptr) {
        const size_t t = e0 / row_values;
        er = e0 - t * row_values;
        blocks += (size_t)row_ids[t] * row_bytes;
    }
    const size_t blk = er / QK_K;
    const int e = (int)(er - blk * QK_K);
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
dequantize_q6_k_kernel(const uint8_t *__restrict__ blocks, size_t n_values, float *__restrict__ out,
                       const int32_t *__restrict__ row_ids, size_t row_values, size_t row_bytes) {
    const size_t q4 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t e0 = q4 * 4;
    if (e0 >= n_values) return;
    size_t er = e0;
    if (row_ids != nullptr) {
        const size_t t = e0 / row_values;
        er = e0 - t * row_values;
        blocks += (size_t)row_ids[t] * row_bytes;
    }
    const size_t blk = er / QK_K;
    const int e = (int)(er - blk * QK_K);
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
dequantize_q8_0_kernel(const uint8_t *__restrict__ blocks, size_t n_values, float *__restrict__ out,
                       const int32_t *__restrict__ row_ids, size_t row_values, size_t row_bytes) {
    const size_t q4 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t e0 = q4 * 4;
    if (e0 >= n_values) return;
    size_t er = e0;
    if (row_ids != nullptr) {
        const size_t t = e0 / row_values;
        er = e0 - t * row_values;
        blocks += (size_t)row_ids[t] * row_bytes;
    }
    const size_t blk = er / Q8_0_VALUES;
    const int e = (int)(er - blk * Q8_0_VALUES);
    const uint8_t *b = blocks + blk * Q8_0_BYTES;
    const float d = half_bits_to_float((uint16_t)(b[0] | (b[1] << 8)));
#pragma unroll
    for (int i = 0; i < 4; ++i)
        if (e0 + i < n_values) out[e0 + i] = __fmul_rn((float)(int8_t)b[2 + e + i], d);
}

static cudaError_t launch_dequant_any(int kind, const void *blocks, size_t n_values, float *out, const int32_t *row_ids,
                                      size_t row_values, size_t row_bytes, cudaStream_t s) {
    if (n_values == 0) return cudaSuccess;
    const size_t groups = (n_values + 3) / 4;
    const unsigned grid = (unsigned)((groups + 255) / 256);
    const uint8_t *b = (const uint8_t *)blocks;
    if (kind == KIND_Q4_K) dequantize_q4_k_kernel<<<grid, 256, 0, s>>>(b, n_values, out, row_ids, row_values, row_bytes);
    else if (kind == KIND_Q6_K) dequantize_q6_k_kernel<<<grid, 256, 0, s>>>(b, n_values, out, row_ids, row_values, row_bytes);
    else if (kind == KIND_Q8_0) dequantize_q8_0_kernel<<<grid, 256, 0, s>>>(b, n_values, out, row_ids, row_values, row_bytes);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

cudaError_t launch_dequantize(int kind, const void *blocks, size_t n_values, float *out, cudaStream_t s) {
    return launch_dequant_any(kind, blocks, n_values, out, nullptr, 0, 0, s);
}

// out[t][:] = dequantised row row_ids[t] of a [rows][dim] table; dim a multiple of 4.
cudaError_t launch_dequantize_rows(int kind, const void *table, size_t dim, size_t row_bytes, const int32_t *row_ids,
                                   size_t n_rows, float *out, cudaStream_t s) {
    if (dim % 4) return cudaErrorInvalidValue;
    return launch_dequant_any(kind, table, n_rows * dim, out, row_ids, dim, row_bytes, s);
}

}  // namespace mcu
