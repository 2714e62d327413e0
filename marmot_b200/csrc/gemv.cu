// Decode-regime quantized matmul (T <= 8 tokens): one warp per weight row, packed super-blocks
// streamed straight from HBM, nibbles / 6-bit values unpacked in registers, int8 dot products
// with dp4a, per-block f32 scaling in the reference's operation order, warp-shuffle reduction.
//
// Per super-block the integer sums are exact, and the f32 term
//   Q4_K: (a.d*d)*isum - (a.d*dmin)*msum   (vec_dot_impl.h:688-732 of the reference)
//   Q6_K: (a.d*d)*isum                     (vec_dot_impl.h:783-828)
//   Q8_0: (float)isum * (d_w*d_a)          (vec_dot_impl.h:452-479)
// is rounded exactly like the reference; only the order in which the block terms of one row are
// added differs (lanes add in parallel), which is a ~1e-7 relative effect.
#include "common.cuh"
#include "kernels.h"

namespace mcu {

__device__ __forceinline__ uint32_t ld_u32_align2(const uint8_t *p) {
    const uint16_t *h = (const uint16_t *)p;
    return (uint32_t)__ldg(h) | ((uint32_t)__ldg(h + 1) << 16);
}

// ---------------------------------------------------------------------------------------------
// Q4_K: eight lanes per super-block (lane8 = 2g + h owns qs bytes [16*lane8, 16*lane8+16)),
// four super-blocks per warp iteration.
// ---------------------------------------------------------------------------------------------
template <int T>
__global__ void __launch_bounds__(256)
gemv_q4_k_kernel(const uint8_t *__restrict__ W, const uint8_t *__restrict__ W2, ActView a, int F,
                 const float *__restrict__ bias, float *__restrict__ out, float *__restrict__ out2, int ldo) {
    const int lane = threadIdx.x & 31, lane8 = lane & 7, sub = lane >> 3;
    const int g = lane8 >> 1, h = lane8 & 1;
    const int nb = a.nb;
    const int rows = W2 != nullptr ? 2 * F : F;
    const int warps = gridDim.x * (blockDim.x >> 5);
    for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
        const bool second = r >= F;
        const int f = second ? r - F : r;
        const uint8_t *wrow = (second ? W2 : W) + (size_t)f * nb * Q4_K_BYTES;
        float acc[T];
#pragma unroll
        for (int t = 0; t < T; ++t) acc[t] = 0.0f;
        for (int b0 = 0; b0 < nb; b0 += 4) {
            const int blk = b0 + sub;
            const bool ok = blk < nb;
            uint4 hdr = make_uint4(0, 0, 0, 0), qv = make_uint4(0, 0, 0, 0);
            if (ok) {
                const uint4 *bp = (const uint4 *)(wrow + (size_t)blk * Q4_K_BYTES);
                hdr = __ldg(bp);
                qv = __ldg(bp + 1 + lane8);
            }
            const float d = half_bits_to_float((uint16_t)(hdr.x & 0xFFFFu));
            const float dmin = half_bits_to_float((uint16_t)(hdr.x >> 16));
            int sc_lo, m_lo, sc_hi, m_hi;
            k4_scale_min_w(2 * g, hdr.y, hdr.z, hdr.w, sc_lo, m_lo);
            k4_scale_min_w(2 * g + 1, hdr.y, hdr.z, hdr.w, sc_hi, m_hi);
            const uint32_t lo[4] = {qv.x & 0x0F0F0F0Fu, qv.y & 0x0F0F0F0Fu, qv.z & 0x0F0F0F0Fu, qv.w & 0x0F0F0F0Fu};
            const uint32_t hi[4] = {(qv.x >> 4) & 0x0F0F0F0Fu, (qv.y >> 4) & 0x0F0F0F0Fu, (qv.z >> 4) & 0x0F0F0F0Fu,
                                    (qv.w >> 4) & 0x0F0F0F0Fu};
#pragma unroll
            for (int t = 0; t < T; ++t) {
                int p = 0, s = 0;
                float ad = 0.0f;
                if (ok) {
                    const int8_t *qa = a.qs + (size_t)t * a.kp + (size_t)blk * QK_K + lane8 * 16;
                    const int4 alo = __ldg((const int4 *)qa);
                    const int4 ahi = __ldg((const int4 *)(qa + 128));
                    int dlo = __dp4a((int)lo[0], alo.x, 0);
                    dlo = __dp4a((int)lo[1], alo.y, dlo);
                    dlo = __dp4a((int)lo[2], alo.z, dlo);
                    dlo = __dp4a((int)lo[3], alo.w, dlo);
                    int dhi = __dp4a((int)hi[0], ahi.x, 0);
                    dhi = __dp4a((int)hi[1], ahi.y, dhi);
                    dhi = __dp4a((int)hi[2], ahi.z, dhi);
                    dhi = __dp4a((int)hi[3], ahi.w, dhi);
                    p = sc_lo * dlo + sc_hi * dhi;
                    const int16_t *bs = a.bsums + ((size_t)t * nb + blk) * 16;
                    s = m_lo * (int)__ldg(bs + 4 * g + h) + m_hi * (int)__ldg(bs + 4 * g + 2 + h);
                    ad = __ldg(a.d + (size_t)t * nb + blk);
                }
#pragma unroll
                for (int o = 1; o < 8; o <<= 1) {
                    p += __shfl_xor_sync(0xffffffffu, p, o);
                    s += __shfl_xor_sync(0xffffffffu, s, o);
                }
                if (lane8 == 0 && ok) {
                    const float dd = __fmul_rn(ad, d), dm = __fmul_rn(ad, dmin);
                    acc[t] = __fadd_rn(acc[t], __fsub_rn(__fmul_rn(dd, (float)p), __fmul_rn(dm, (float)s)));
                }
            }
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
            const float v = warp_sum(acc[t]);
            if (lane == 0) {
                const float y = bias != nullptr ? __fadd_rn(v, bias[f]) : v;
                (second ? out2 : out)[(size_t)t * ldo + f] = y;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Q6_K: sixteen lanes per super-block; lane16 -> half n = lane16/8 and four consecutive l.
// Block bytes are only 2-byte aligned (210-byte stride), so words are assembled from u16 loads.
// ---------------------------------------------------------------------------------------------
template <int T>
__global__ void __launch_bounds__(256)
gemv_q6_k_kernel(const uint8_t *__restrict__ W, const uint8_t *__restrict__ W2, ActView a, int F,
                 const float *__restrict__ bias, float *__restrict__ out, float *__restrict__ out2, int ldo) {
    const int lane = threadIdx.x & 31, lane16 = lane & 15, sub = lane >> 4;
    const int n = lane16 >> 3, l4 = (lane16 & 7) * 4;
    const int nb = a.nb;
    const int rows = W2 != nullptr ? 2 * F : F;
    const int warps = gridDim.x * (blockDim.x >> 5);
    for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
        const bool second = r >= F;
        const int f = second ? r - F : r;
        const uint8_t *wrow = (second ? W2 : W) + (size_t)f * nb * Q6_K_BYTES;
        float acc[T];
#pragma unroll
        for (int t = 0; t < T; ++t) acc[t] = 0.0f;
        for (int b0 = 0; b0 < nb; b0 += 2) {
            const int blk = b0 + sub;
            const bool ok = blk < nb;
            uint32_t qw[4] = {0, 0, 0, 0};
            int sc[4] = {0, 0, 0, 0};
            float d = 0.0f;
            if (ok) {
                const uint8_t *bp = wrow + (size_t)blk * Q6_K_BYTES;
                const uint32_t qla = ld_u32_align2(bp + n * 64 + l4);
                const uint32_t qlb = ld_u32_align2(bp + n * 64 + 32 + l4);
                const uint32_t qh = ld_u32_align2(bp + 128 + n * 32 + l4);
                d = half_bits_to_float(__ldg((const uint16_t *)(bp + 208)));
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t src = (c & 1) ? qlb : qla;
                    const uint32_t lo4 = (c & 2) ? ((src >> 4) & 0x0F0F0F0Fu) : (src & 0x0F0F0F0Fu);
                    const uint32_t h2 = (qh >> (2 * c)) & 0x03030303u;
                    qw[c] = __vsub4(lo4 | (h2 << 4), 0x20202020u);
                    sc[c] = (int)(int8_t)__ldg(bp + 192 + n * 8 + 2 * c + (l4 >> 4));
                }
            }
#pragma unroll
            for (int t = 0; t < T; ++t) {
                int p = 0;
                float ad = 0.0f;
                if (ok) {
                    const int8_t *qa = a.qs + (size_t)t * a.kp + (size_t)blk * QK_K;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        // value 128n + 32c + l sits at split position (c&1)*128 + (2n + c/2)*32 + l
                        const int av = __ldg((const int *)(qa + (c & 1) * 128 + (2 * n + (c >> 1)) * 32 + l4));
                        p += sc[c] * __dp4a((int)qw[c], av, 0);
                    }
                    ad = __ldg(a.d + (size_t)t * nb + blk);
                }
#pragma unroll
                for (int o = 1; o < 16; o <<= 1) p += __shfl_xor_sync(0xffffffffu, p, o);
                if (lane16 == 0 && ok) acc[t] = __fadd_rn(acc[t], __fmul_rn(__fmul_rn(ad, d), (float)p));
            }
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
            const float v = warp_sum(acc[t]);
            if (lane == 0) {
                const float y = bias != nullptr ? __fadd_rn(v, bias[f]) : v;
                (second ? out2 : out)[(size_t)t * ldo + f] = y;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Q8_0: one lane per 32-value block (34 bytes, 2-byte aligned).
// ---------------------------------------------------------------------------------------------
template <int T>
__global__ void __launch_bounds__(256)
gemv_q8_0_kernel(const uint8_t *__restrict__ W, const uint8_t *__restrict__ W2, ActView a, int F,
                 const float *__restrict__ bias, float *__restrict__ out, float *__restrict__ out2, int ldo) {
    const int lane = threadIdx.x & 31;
    const int nb = a.nb;
    const int rows = W2 != nullptr ? 2 * F : F;
    const int warps = gridDim.x * (blockDim.x >> 5);
    for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
        const bool second = r >= F;
        const int f = second ? r - F : r;
        const uint8_t *wrow = (second ? W2 : W) + (size_t)f * nb * Q8_0_BYTES;
        float acc[T];
#pragma unroll
        for (int t = 0; t < T; ++t) acc[t] = 0.0f;
        for (int blk = lane; blk < nb; blk += 32) {
            const uint16_t *bp = (const uint16_t *)(wrow + (size_t)blk * Q8_0_BYTES);
            const float d = half_bits_to_float(__ldg(bp));
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = (uint32_t)__ldg(bp + 1 + 2 * i) | ((uint32_t)__ldg(bp + 2 + 2 * i) << 16);
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const int4 *qa = (const int4 *)(a.qs + (size_t)t * a.kp + (size_t)blk * Q8_0_VALUES);
                const int4 a0 = __ldg(qa), a1 = __ldg(qa + 1);
                int s = __dp4a((int)w[0], a0.x, 0);
                s = __dp4a((int)w[1], a0.y, s);
                s = __dp4a((int)w[2], a0.z, s);
                s = __dp4a((int)w[3], a0.w, s);
                s = __dp4a((int)w[4], a1.x, s);
                s = __dp4a((int)w[5], a1.y, s);
                s = __dp4a((int)w[6], a1.z, s);
                s = __dp4a((int)w[7], a1.w, s);
                const float ad = __ldg(a.d + (size_t)t * nb + blk);
                acc[t] = __fadd_rn(acc[t], __fmul_rn((float)s, __fmul_rn(d, ad)));
            }
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
            const float v = warp_sum(acc[t]);
            if (lane == 0) {
                const float y = bias != nullptr ? __fadd_rn(v, bias[f]) : v;
                (second ? out2 : out)[(size_t)t * ldo + f] = y;
            }
        }
    }
}

template <int T>
static cudaError_t launch_t(int kind, const uint8_t *W, const uint8_t *W2, const ActView &av, int F, const float *bias,
                            float *out, float *out2, int ldo, cudaStream_t s) {
    const int rows = W2 != nullptr ? 2 * F : F;
    const int sms = device_sm_count();
    // eight warps per CTA; enough CTAs for eight resident CTAs per SM, but no more than the rows need
    const int grid = max(1, min((rows + 7) / 8, sms * 8));
    if (kind == KIND_Q4_K) gemv_q4_k_kernel<T><<<grid, 256, 0, s>>>(W, W2, av, F, bias, out, out2, ldo);
    else if (kind == KIND_Q6_K) gemv_q6_k_kernel<T><<<grid, 256, 0, s>>>(W, W2, av, F, bias, out, out2, ldo);
    else gemv_q8_0_kernel<T><<<grid, 256, 0, s>>>(W, W2, av, F, bias, out, out2, ldo);
    return cudaGetLastError();
}

cudaError_t launch_gemv(int kind, const void *W, const void *W2, const ActBuffers &a, int T, int K, int F,
                        const float *bias, float *out, float *out2, int ldo, cudaStream_t s) {
    if (T <= 0 || F <= 0) return cudaSuccess;
    if (T > GEMV_MAX_T) return cudaErrorInvalidValue;
    const int bv = block_values(kind);
    ActView av;
    av.qs = a.qs;
    av.d = a.d;
    av.bsums = a.bsums;
    av.nb = (K + bv - 1) / bv;
    av.kp = av.nb * bv;
    const uint8_t *w = (const uint8_t *)W, *w2 = (const uint8_t *)W2;
    switch (T) {
    case 1: return launch_t<1>(kind, w, w2, av, F, bias, out, out2, ldo, s);
    case 2: return launch_t<2>(kind, w, w2, av, F, bias, out, out2, ldo, s);
    case 3: return launch_t<3>(kind, w, w2, av, F, bias, out, out2, ldo, s);
    case 4: return launch_t<4>(kind, w, w2, av, F, bias, out, out2, ldo, s);
    case 5: return launch_t<5>(kind, w, w2, av, F, bias, out, out2, ldo, s);
    case 6: return launch_t<6>(kind, w, w2, av, F, bias, out, out2, ldo, s);
    case 7: return launch_t<7>(kind, w, w2, av, F, bias, out, out2, ldo, s);
    default: return launch_t<8>(kind, w, w2, av, F, bias, out, out2, ldo, s);
    }
}

}  // namespace mcu
