// Activation quantizers: f32 rows -> Q8_K / Q8_0 values, bit-identical to the reference's
// matmul packers (src/backends/cpu/ops/matmul/quantized/matmul_quant_pack.c:23-62,106-169,
// scalar helpers src/backends/cpu/quantization/common/block.c:175-183,221-232).
#include "common.cuh"
#include "kernels.h"

#include <float.h>

namespace mcu {

// round-to-nearest-even through the 1.5*2^23 bit trick, as cpu_quant_matmul_nearest_int
// (matmul_quant_pack.c:11-21)
__device__ __forceinline__ int nearest_int(float v) {
    v = fminf(fmaxf(v, -4194303.0f), 4194303.0f);
    const float shifted = __fadd_rn(v, 12582912.0f);
    return (__float_as_int(shifted) & 0x007fffff) - 0x00400000;
}

// One warp per (token, 256-value block).  Lane l owns values l, l+32, ..., l+224.
__global__ void __launch_bounds__(256)
quantize_q8_k_kernel(const float *__restrict__ x, int ldx, int T, int K, int nb, int8_t *__restrict__ qs,
                     float *__restrict__ dq, int16_t *__restrict__ bsums, __half *__restrict__ xh) {
    const int lane = threadIdx.x & 31;
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= T * nb) return;
    const int t = w / nb, blk = w - t * nb;
    const float *row = x + (size_t)t * ldx + (size_t)blk * QK_K;
    const int len = min(QK_K, K - blk * QK_K);

    float v[8];
    float best_abs = 0.0f, best_val = 0.0f;
    int best_idx = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int idx = lane + 32 * i;
        v[i] = idx < len ? row[idx] : 0.0f;
        const float a = fabsf(v[i]);
        if (a > best_abs) {  // strict: the first occurrence wins
            best_abs = a;
            best_val = v[i];
            best_idx = idx;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, best_abs, o);
        const float ov = __shfl_xor_sync(0xffffffffu, best_val, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_idx, o);
        if (oa > best_abs || (oa == best_abs && oi < best_idx)) {
            best_abs = oa;
            best_val = ov;
            best_idx = oi;
        }
    }
    int8_t *qrow = qs + (size_t)t * nb * QK_K + (size_t)blk * QK_K;
    int16_t *brow = bsums + ((size_t)t * nb + blk) * 16;
    __half *hrow = xh != nullptr ? xh + (size_t)t * nb * QK_K + (size_t)blk * QK_K : nullptr;
    if (!(best_abs > 0.0f)) {
        // all-zero block: d = 0, zero quants (matmul_quant_pack.c:121-126)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            qrow[(i & 1) * 128 + (i >> 1) * 32 + lane] = 0;
            if (hrow != nullptr) hrow[lane + 32 * i] = __float2half_rn(0.0f);
        }
        if (lane < 16) brow[lane] = 0;
        if (lane == 0) dq[(size_t)t * nb + blk] = 0.0f;
        return;
    }
    const float iscale = __fdiv_rn(-127.0f, best_val);
    const float d = __fdiv_rn(1.0f, iscale);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int q = nearest_int(__fmul_rn(iscale, v[i]));
        q = min(q, 127);
        qrow[(i & 1) * 128 + (i >> 1) * 32 + lane] = (int8_t)q;
        if (hrow != nullptr) hrow[lane + 32 * i] = __float2half_rn(__fmul_rn(d, (float)q));
        // sums over 16 consecutive values: the 16 lanes of a half warp
        int s = q;
        s += __shfl_xor_sync(0xffffffffu, s, 8);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        if ((lane & 15) == 0) brow[2 * i + (lane >> 4)] = (int16_t)s;
    }
    if (lane == 0) dq[(size_t)t * nb + blk] = d;
}

// One warp per (token, 32-value block); lane = value.
__global__ void __launch_bounds__(256)
quantize_q8_0_kernel(const float *__restrict__ x, int ldx, int T, int K, int nb, int8_t *__restrict__ qs,
                     float *__restrict__ dq, __half *__restrict__ xh) {
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    const long total = (long)T * nb;
    for (long w = (long)blockIdx.x * wpb + (threadIdx.x >> 5); w < total; w += (long)gridDim.x * wpb) {
        const int t = (int)(w / nb), blk = (int)(w - (long)t * nb);
        const int k = blk * Q8_0_VALUES + lane;
        const float v = k < K ? x[(size_t)t * ldx + k] : 0.0f;
        float amax = fabsf(v);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        float scale = __fdiv_rn(amax, 127.0f);
        if (scale < FLT_MIN) scale = 1.0f;
        const float inv = __fdiv_rn(1.0f, scale);
        int q = (int)roundf(__fmul_rn(v, inv));
        q = max(-127, min(127, q));
        const float d_stored = __half2float(__float2half_rn(scale));
        qs[(size_t)t * nb * Q8_0_VALUES + k] = (int8_t)q;
        if (xh != nullptr) xh[(size_t)t * nb * Q8_0_VALUES + k] = __float2half_rn(__fmul_rn(d_stored, (float)q));
        if (lane == 0) dq[(size_t)t * nb + blk] = d_stored;
    }
}

// Which value of a row goes to position k (see ACT_ORDER_* in kernels.h).
__device__ __forceinline__ int act_order_source(int k, int order) {
    if (order == ACT_ORDER_QUAD) return (k & ~3) | ((k & 1) << 1) | ((k >> 1) & 1);
    if (order == ACT_ORDER_FRAG16) {
        const int p = k & 15;
        return (k & ~15) | (((p & 7) >> 1) << 2) | (p >> 3) | ((p & 1) << 1);
    }
    return k;
}

// fp16 operands for the tensor-core path: xh[t][k] = (d*q) * 2^-e_t, with one exponent per token chosen so
// that the largest magnitude of the row is about 2^14.  The power-of-two scale is exact, keeps large
// activations inside the fp16 range (and tiny ones out of the subnormals); the matmul epilogue multiplies
// the row back by rowscale[t] = 2^e_t.  One CTA per token.
__global__ void __launch_bounds__(256)
half_acts_kernel(int kq, int perm, const int8_t *__restrict__ qs, const float *__restrict__ dq, int nb, int kp,
                 __half *__restrict__ xh, float *__restrict__ rowscale) {
    __shared__ float red[8];
    __shared__ float inv_s;
    const int t = blockIdx.x;
    const float *drow = dq + (size_t)t * nb;
    float m = 0.0f;
    for (int b = threadIdx.x; b < nb; b += blockDim.x) m = fmaxf(m, fabsf(drow[b]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float mm = 0.0f;
        for (int i = 0; i < 8; ++i) mm = fmaxf(mm, red[i]);
        mm *= 127.0f;  // bound of |d*q| over the row
        int e = 0;
        if (mm > 0.0f && mm < 3.0e38f) {
            (void)frexpf(mm, &e);  // mm = f * 2^e, f in [0.5, 1)
            e -= 14;
            e = max(-100, min(100, e));
        }
        inv_s = ldexpf(1.0f, -e);
        rowscale[t] = ldexpf(1.0f, e);
    }
    __syncthreads();
    const float inv = inv_s;
    const int8_t *qrow = qs + (size_t)t * kp;
    __half *hrow = xh + (size_t)t * kp;
    const int bv = kq ? QK_K : Q8_0_VALUES;
    for (int k = threadIdx.x; k < kp; k += blockDim.x) {
        const int src = act_order_source(k, perm);
        const int blk = src / bv;
        const int pos = kq ? blk * QK_K + q8k_split_pos(src - blk * QK_K) : src;
        hrow[k] = __float2half_rn(__fmul_rn(__fmul_rn(drow[blk], inv), (float)qrow[pos]));
    }
}

// Quantise-and-stage in one kernel for the tensor-core matmul, which needs neither the int8 values nor the block
// sums in global memory: one CTA per token quantises the row block by block exactly as the kernels above (values
// and scales kept in shared memory), then writes xh and rowscale exactly as half_acts_kernel.  Launched with
// programmatic stream serialization: everything before griddepcontrol.wait is independent of earlier kernels.
// Sixteen staged values from sixteen quantised ones: position p of the group takes source act_order_source(p, ORDER)
// (every order permutes inside aligned groups of sixteen), so the indices resolve at compile time.
template <int ORDER>
__device__ __forceinline__ void stage_group16(const int8_t *q16, float sc, __half *dst) {
    const uint4 raw = *(const uint4 *)q16;
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float f[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) f[j] = __fmul_rn(sc, (float)(int8_t)(w[j >> 2] >> (8 * (j & 3))));
    uint32_t o[8];
#pragma unroll
    for (int p2 = 0; p2 < 8; ++p2) {
        const __half2 h = __floats2half2_rn(f[act_order_source(2 * p2, ORDER)], f[act_order_source(2 * p2 + 1, ORDER)]);
        o[p2] = *(const uint32_t *)&h;
    }
    uint4 *d = (uint4 *)dst;
    d[0] = make_uint4(o[0], o[1], o[2], o[3]);
    d[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// GLU: 0 = the row as it is; 1 = silu(x) * x2; 2 = gelu(x) * x2.  The SiLU uses the fast exponential and division
// (relative error about 1e-6): its result is quantised to eight bits right here, three orders of magnitude coarser.
template <bool KQ, int GLU>
__global__ void __launch_bounds__(256)
act_half_fused_kernel(const float *__restrict__ x, int ldx, ActSource src, int K, int nb, int perm,
                      __half *__restrict__ xh, float *__restrict__ rowscale) {
    extern __shared__ __align__(16) uint8_t act_sm[];
    constexpr int BV = KQ ? QK_K : Q8_0_VALUES;
    const int kp = nb * BV;
    int8_t *q_s = (int8_t *)act_sm;
    float *d_s = (float *)(act_sm + ((kp + 15) & ~15));
    __shared__ float red[8];
    __shared__ float inv_s;
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (src.row_lo != nullptr && (t < *src.row_lo || t >= *src.row_hi)) return;  // not this rank's row
    const size_t row_off = (size_t)(src.row_index != nullptr ? src.row_index[t] : t) * ldx;
    const float *xrow = x + row_off;
    const float *urow = GLU != 0 ? src.x2 + row_off : nullptr;
    const float *arow = nullptr, *nrow = xrow;  // norm: what is added, and where the sum is read back from
    float norm_inv = 1.0f;
    if (GLU == 0 && src.norm) {
        arow = src.add != nullptr ? src.add + row_off : nullptr;
        float *orow = src.x_out != nullptr ? src.x_out + row_off : nullptr;
        float sum = 0.0f;
        for (int i = threadIdx.x; i < K; i += blockDim.x) {
            const float v = arow != nullptr ? __fadd_rn(xrow[i], arow[i]) : xrow[i];
            if (orow != nullptr) orow[i] = v;
            sum += v * v;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) red[warp] = sum;
        __syncthreads();
        if (threadIdx.x == 0) {
            float s = 0.0f;
            for (int i = 0; i < 8; ++i) s += red[i];
            inv_s = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(s, (float)K), src.eps)));
        }
        __syncthreads();
        norm_inv = inv_s;
        __syncthreads();  // red and inv_s are used again below
        if (orow != nullptr) {  // the packer reads the sums back (other threads' elements too: all written before
            nrow = orow;        // the barriers above) instead of adding again
            arow = nullptr;
        }
    }
    auto value = [&](int k) -> float {
        if (GLU == 0 && src.norm) {
            const float v = arow != nullptr ? __fadd_rn(nrow[k], arow[k]) : nrow[k];
            float y = __fmul_rn(v, norm_inv);
            if (src.norm_w != nullptr) y = __fmul_rn(y, __fadd_rn(src.norm_w[k], src.w_off));
            return y;
        }
        const float g = xrow[k];
        if constexpr (GLU == 0) return g;
        float a;
        if constexpr (GLU == 2) a = __fmul_rn(__fmul_rn(0.5f, g), __fadd_rn(1.0f, erff(__fmul_rn(g, 0.7071067811865475f))));
        else a = __fdividef(g, __fadd_rn(1.0f, __expf(-g)));
        return __fmul_rn(a, urow[k]);
    };
    if (KQ) {
        for (int blk = warp; blk < nb; blk += 8) {
            const int len = min(QK_K, K - blk * QK_K);
            float v[8];
            float best_abs = 0.0f, best_val = 0.0f;
            int best_idx = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int idx = lane + 32 * i;
                v[i] = idx < len ? value(blk * QK_K + idx) : 0.0f;
                const float a = fabsf(v[i]);
                if (a > best_abs) {
                    best_abs = a;
                    best_val = v[i];
                    best_idx = idx;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float oa = __shfl_xor_sync(0xffffffffu, best_abs, o);
                const float ov = __shfl_xor_sync(0xffffffffu, best_val, o);
                const int oi = __shfl_xor_sync(0xffffffffu, best_idx, o);
                if (oa > best_abs || (oa == best_abs && oi < best_idx)) {
                    best_abs = oa;
                    best_val = ov;
                    best_idx = oi;
                }
            }
            float d = 0.0f, iscale = 0.0f;
            if (best_abs > 0.0f) {
                iscale = __fdiv_rn(-127.0f, best_val);
                d = __fdiv_rn(1.0f, iscale);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                int q = best_abs > 0.0f ? min(nearest_int(__fmul_rn(iscale, v[i])), 127) : 0;
                q_s[blk * QK_K + lane + 32 * i] = (int8_t)q;
            }
            if (lane == 0) d_s[blk] = d;
        }
    } else {
        for (int blk = warp; blk < nb; blk += 8) {
            const int k = blk * Q8_0_VALUES + lane;
            const float v = k < K ? value(k) : 0.0f;
            float amax = fabsf(v);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            float scale = __fdiv_rn(amax, 127.0f);
            if (scale < FLT_MIN) scale = 1.0f;
            const float inv = __fdiv_rn(1.0f, scale);
            int q = (int)roundf(__fmul_rn(v, inv));
            q = max(-127, min(127, q));
            q_s[k] = (int8_t)q;
            if (lane == 0) d_s[blk] = __half2float(__float2half_rn(scale));
        }
    }
    __syncthreads();
    float m = 0.0f;
    for (int b = threadIdx.x; b < nb; b += blockDim.x) m = fmaxf(m, fabsf(d_s[b]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float mm = 0.0f;
        for (int i = 0; i < 8; ++i) mm = fmaxf(mm, red[i]);
        mm *= 127.0f;
        int e = 0;
        if (mm > 0.0f && mm < 3.0e38f) {
            (void)frexpf(mm, &e);
            e -= 14;
            e = max(-100, min(100, e));
        }
        inv_s = ldexpf(1.0f, -e);
        rowscale[t] = ldexpf(1.0f, e);
    }
    __syncthreads();
    const float inv = inv_s;
    __half *hrow = xh + (size_t)t * kp;
    for (int g = threadIdx.x; g < kp / 16; g += blockDim.x) {
        const float sc = __fmul_rn(d_s[(16 * g) / BV], inv);
        if (perm == ACT_ORDER_QUAD) stage_group16<ACT_ORDER_QUAD>(q_s + 16 * g, sc, hrow + 16 * g);
        else if (perm == ACT_ORDER_FRAG16) stage_group16<ACT_ORDER_FRAG16>(q_s + 16 * g, sc, hrow + 16 * g);
        else stage_group16<ACT_ORDER_NATURAL>(q_s + 16 * g, sc, hrow + 16 * g);
    }
}

size_t act_half_fused_smem(int kind, int K) {
    const int bv = block_values(kind), nb = (K + bv - 1) / bv;
    return (size_t)((nb * bv + 15) & ~15) + (size_t)nb * sizeof(float);
}

cudaError_t launch_act_half_fused_from(int kind, const float *x, int ldx, const ActSource &src, int T, int K, int k_order,
                                       __half *xh, float *rowscale, cudaStream_t s) {
    if (T <= 0) return cudaSuccess;
    const int bv = block_values(kind), nb = (K + bv - 1) / bv;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)T, 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.dynamicSmemBytes = act_half_fused_smem(kind, K);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const bool kq = kind != KIND_Q8_0;
    const int glu = src.x2 != nullptr ? (src.glu == 2 ? 2 : 1) : 0;
#define MCU_STAGE(KQ, GLU) cudaLaunchKernelEx(&cfg, act_half_fused_kernel<KQ, GLU>, x, ldx, src, K, nb, k_order, xh, rowscale)
    if (glu == 0) return kq ? MCU_STAGE(true, 0) : MCU_STAGE(false, 0);
    if (glu == 1) return kq ? MCU_STAGE(true, 1) : MCU_STAGE(false, 1);
    return kq ? MCU_STAGE(true, 2) : MCU_STAGE(false, 2);
#undef MCU_STAGE
}

cudaError_t launch_act_half_fused(int kind, const float *x, int ldx, int T, int K, int k_order, __half *xh,
                                  float *rowscale, cudaStream_t s) {
    return launch_act_half_fused_from(kind, x, ldx, ActSource{}, T, K, k_order, xh, rowscale, s);
}

cudaError_t launch_half_acts(int kind, const ActBuffers &a, int T, int K, int k_order, __half *xh, float *rowscale,
                             cudaStream_t s) {
    if (T <= 0) return cudaSuccess;
    const int bv = block_values(kind), nb = (K + bv - 1) / bv;
    half_acts_kernel<<<T, 256, 0, s>>>(kind != KIND_Q8_0, k_order, a.qs, a.d, nb, nb * bv, xh, rowscale);
    return cudaGetLastError();
}

cudaError_t launch_quantize_act(int kind, const float *x, int ldx, int T, int K, const ActBuffers &a, __half *xh,
                                cudaStream_t s) {
    if (T <= 0) return cudaSuccess;
    if (kind == KIND_Q8_0) {
        const int nb = (K + Q8_0_VALUES - 1) / Q8_0_VALUES;
        const long warps = (long)T * nb;
        const int blocks = (int)min((warps + 7) / 8, (long)148 * 16);
        quantize_q8_0_kernel<<<blocks, 256, 0, s>>>(x, ldx, T, K, nb, a.qs, a.d, xh);
    } else {
        const int nb = (K + QK_K - 1) / QK_K;
        const long warps = (long)T * nb;
        quantize_q8_k_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, s>>>(x, ldx, T, K, nb, a.qs, a.d, a.bsums, xh);
    }
    return cudaGetLastError();
}

}  // namespace mcu
