// Quantized matmul with f16 activations: the reference's path for FLOAT16 inputs (matmul_quant_dispatch.c:449-470,
// cpu_quant_matmul_dispatch_fp16_tile -> cpu_vec_dot_{q4_k,q6_k,q8_0}_f16, vec_dot_impl.h:419-447,973-1023,1082-1127).
// Nothing is packed: every weight value is formed in f32 exactly as those functions form it, multiplied by the
// widened activation and added in f32 (products and sums rounded separately).  The reference keeps one running sum per
// output; here a warp owns an output row, its lanes take every 32nd group of four values and the partial sums meet
// in a shuffle tree, so only the order of the f32 additions differs.
//
// Q6_K follows cpu_vec_dot_q6_k_f16 as it stands: value idx of a block takes scale sc[idx / 128], the nibble idx of
// ql counted linearly (even idx low, odd idx high) and bits (idx % 4) of qh[idx / 4] -- not the layout the
// dequantizer reads.  The reference's golden output for this path (g_matmul_q6_k_output_from_f16) pins that reading.
#include "common.cuh"
#include "kernels.h"

namespace mcu {

constexpr int F16_MAX_T = 8;  // tokens per pass over a weight row

// the values e .. e+3 (e a multiple of 4) of a weight row
template <int KIND>
__device__ __forceinline__ void row_values4(const uint8_t *row, int e, float (&r)[4]) {
    if (KIND == KIND_Q4_K) {
        const uint8_t *b = row + (size_t)(e >> 8) * Q4_K_BYTES;
        const int v = e & 255, g = v >> 6, hi = (v >> 5) & 1, l = v & 31;
        const float d = half_bits_to_float(*(const uint16_t *)b), dmin = half_bits_to_float(*(const uint16_t *)(b + 2));
        int sc, mn;
        k4_scale_min(2 * g + hi, b + 4, sc, mn);
        const float dl = __fmul_rn(d, (float)sc), ml = __fmul_rn(dmin, (float)mn);
        const uint32_t w = *(const uint32_t *)(b + 16 + g * 32 + l);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t byte = (w >> (8 * i)) & 0xFFu;
            r[i] = __fsub_rn(__fmul_rn(dl, (float)(hi ? (byte >> 4) : (byte & 0xFu))), ml);
        }
    } else if (KIND == KIND_Q6_K) {
        const uint8_t *b = row + (size_t)(e >> 8) * Q6_K_BYTES;
        const int idx = e & 255;
        const float d = half_bits_to_float((uint16_t)(b[208] | (b[209] << 8)));
        const float scale = __fmul_rn(d, (float)(int8_t)b[192 + idx / 128]);
        const uint32_t ql2 = (uint32_t)b[idx / 2] | ((uint32_t)b[idx / 2 + 1] << 8);  // nibbles idx .. idx+3
        const uint32_t qh = b[128 + idx / 4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int lo = (int)((ql2 >> (4 * i)) & 0xFu), hi = (int)((qh >> (2 * i)) & 3u);
            r[i] = __fmul_rn(scale, (float)((lo | (hi << 4)) - 32));
        }
    } else {
        const uint8_t *b = row + (size_t)(e >> 5) * Q8_0_BYTES;
        const float d = half_bits_to_float((uint16_t)(b[0] | (b[1] << 8)));
        const int l = e & 31;
#pragma unroll
        for (int i = 0; i < 4; ++i) r[i] = __fmul_rn((float)(int8_t)b[2 + l + i], d);
    }
}

// grid (ceil(F / 8), ceil(T / F16_MAX_T)); one warp per weight row, eight tokens per pass.
template <int KIND>
__global__ void __launch_bounds__(256)
linear_f16_kernel(const uint8_t *__restrict__ W, size_t row_bytes, const __half *__restrict__ x, size_t ldx, int T, int K,
                  int F, const float *__restrict__ bias, float *__restrict__ out32, __half *__restrict__ out16, size_t ldo) {
    const int lane = threadIdx.x & 31;
    const int f = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (f >= F) return;
    const int t0 = blockIdx.y * F16_MAX_T, tt = min(F16_MAX_T, T - t0);
    const uint8_t *row = W + (size_t)f * row_bytes;
    const bool vec = ((uintptr_t)x & 7) == 0 && (ldx & 3) == 0;
    float acc[F16_MAX_T];
#pragma unroll
    for (int t = 0; t < F16_MAX_T; ++t) acc[t] = 0.0f;
    for (int e = lane * 4; e < K; e += 128) {
        float w[4];
        row_values4<KIND>(row, e, w);
#pragma unroll
        for (int t = 0; t < F16_MAX_T; ++t) {
            if (t >= tt) break;
            const __half *xr = x + (size_t)(t0 + t) * ldx + e;
            float a[4];
            if (vec && e + 3 < K) {
                const uint2 raw = __ldg((const uint2 *)xr);
                const float2 lo = __half22float2(*(const __half2 *)&raw.x), hi = __half22float2(*(const __half2 *)&raw.y);
                a[0] = lo.x, a[1] = lo.y, a[2] = hi.x, a[3] = hi.y;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) a[i] = e + i < K ? __half2float(xr[i]) : 0.0f;  // past K the product is dropped
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (e + i < K) acc[t] = __fadd_rn(acc[t], __fmul_rn(w[i], a[i]));
        }
    }
#pragma unroll
    for (int t = 0; t < F16_MAX_T; ++t) {
        if (t >= tt) break;
        float v = warp_sum(acc[t]);
        if (lane == 0) {
            if (bias != nullptr) v = __fadd_rn(v, bias[f]);
            if (out16 != nullptr) out16[(size_t)(t0 + t) * ldo + f] = __float2half_rn(v);
            else out32[(size_t)(t0 + t) * ldo + f] = v;
        }
    }
}

cudaError_t launch_linear_f16(int kind, const void *W, const __half *x, size_t ldx, int T, int K, int F, const float *bias,
                              float *out32, __half *out16, size_t ldo, cudaStream_t s) {
    if (T <= 0 || F <= 0) return cudaSuccess;
    const int bv = block_values(kind);
    const size_t row_bytes = (size_t)((K + bv - 1) / bv) * block_bytes(kind);
    const dim3 grid((unsigned)((F + 7) / 8), (unsigned)((T + F16_MAX_T - 1) / F16_MAX_T));
    const uint8_t *w = (const uint8_t *)W;
    if (kind == KIND_Q4_K) linear_f16_kernel<KIND_Q4_K><<<grid, 256, 0, s>>>(w, row_bytes, x, ldx, T, K, F, bias, out32, out16, ldo);
    else if (kind == KIND_Q6_K) linear_f16_kernel<KIND_Q6_K><<<grid, 256, 0, s>>>(w, row_bytes, x, ldx, T, K, F, bias, out32, out16, ldo);
    else if (kind == KIND_Q8_0) linear_f16_kernel<KIND_Q8_0><<<grid, 256, 0, s>>>(w, row_bytes, x, ldx, T, K, F, bias, out32, out16, ldo);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

}  // namespace mcu
