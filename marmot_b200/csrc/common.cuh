// Shared device helpers for the quantized-matmul kernels (sm_100a).
//
// Block formats are the GGUF layouts of the reference (include/marmot/quant_block.h:48-52,
// 91-97, 111-117 in the reference tree).  Arithmetic that must match the reference's scalar
// CPU code bit for bit uses the explicit round-to-nearest intrinsics (__fmul_rn, __fsub_rn, ...)
// so the compiler cannot contract a multiply and an add into one FMA.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mcu {

constexpr int QK_K = 256;
constexpr int Q8_0_VALUES = 32;
constexpr int Q4_K_BYTES = 144;
constexpr int Q6_K_BYTES = 210;
constexpr int Q8_0_BYTES = 34;

enum Kind : int { KIND_Q8_0 = 5, KIND_Q4_K = 9, KIND_Q6_K = 11 };

__host__ __device__ inline int block_values(int kind) { return kind == KIND_Q8_0 ? Q8_0_VALUES : QK_K; }
__host__ __device__ inline int block_bytes(int kind) {
    return kind == KIND_Q4_K ? Q4_K_BYTES : kind == KIND_Q6_K ? Q6_K_BYTES : Q8_0_BYTES;
}
__host__ __device__ inline bool kind_supported(int kind) {
    return kind == KIND_Q8_0 || kind == KIND_Q4_K || kind == KIND_Q6_K;
}

// Quantized activations, structure-of-arrays (values identical to the reference's Q8_K / Q8_0
// activation blocks, matmul_quant_pack.c:23-62,106-169; only the memory layout differs).
//   K-quant weights  -> Q8_K: per 256 values one f32 scale, int8 quants, int16 sums per 16.
//   Q8_0 weights     -> Q8_0: per 32 values one scale (the f32 value of the fp16-rounded scale).
// Inside every 256-value block of a Q8_K row the 32-value groups are stored "split":
// position = b*128 + g*32 + i for value 64*g + 32*b + i, i.e. the four groups paired with low
// nibbles first, then the four groups paired with high nibbles.  For Q4_K the eight lanes that
// share a block then read eight distinct 16-byte chunks (no shared-memory bank conflicts).
struct ActView {
    const int8_t *qs;     // [T][kp]
    const float *d;       // [T][nb]
    const int16_t *bsums; // [T][nb*16] (Q8_K only; natural order)
    int kp;               // padded K = nb * block_values
    int nb;               // blocks per row
};

__device__ __forceinline__ int q8k_split_pos(int v /*0..255*/) {
    const int g = v >> 6, b = (v >> 5) & 1, i = v & 31;
    return b * 128 + g * 32 + i;
}

__device__ __forceinline__ float half_bits_to_float(uint16_t bits) {
    return __half2float(__ushort_as_half(bits));
}

// 6-bit (scale, min) pair j of a Q4_K block; same bit selection as get_scale_min_k4
// (src/backends/cpu/quantization/common/kquant_common.h:29-37).
__device__ __forceinline__ void k4_scale_min(int j, const uint8_t *q, int &sc, int &mn) {
    if (j < 4) {
        sc = q[j] & 63;
        mn = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

// Same selection from the three 32-bit words of the packed scales (little endian bytes 0..11).
__device__ __forceinline__ void k4_scale_min_w(int j, uint32_t w0, uint32_t w1, uint32_t w2, int &sc, int &mn) {
    // byte k of the 12-byte field
    auto byte_at = [&](int k) -> uint32_t {
        const uint32_t w = k < 4 ? w0 : (k < 8 ? w1 : w2);
        return (w >> (8 * (k & 3))) & 0xFFu;
    };
    if (j < 4) {
        sc = (int)(byte_at(j) & 63u);
        mn = (int)(byte_at(j + 4) & 63u);
    } else {
        sc = (int)((byte_at(j + 4) & 0xFu) | ((byte_at(j - 4) >> 6) << 4));
        mn = (int)((byte_at(j + 4) >> 4) | ((byte_at(j) >> 6) << 4));
    }
}

__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace mcu
