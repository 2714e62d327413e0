// Activation packers shared by the kernels that quantize f32 activations themselves: f32 -> Q8_K (K-quant weights)
// or Q8_0 (Q8_0 weights), value for value what the reference's packers produce (matmul_quant_pack.c:23-62,106-169).
#pragma once

#include "common.cuh"

// How the packers read activations (and the prologues' operands).  Read-only cache loads by default; a kernel that
// reads what OTHER CTAs of the same launch wrote earlier (the persistent decode step) defines this as __ldcg before
// including the header, because the non-coherent path may serve a line cached before the write.
#ifndef MCU_ACT_LOAD
#define MCU_ACT_LOAD(ptr) __ldg(ptr)
#endif

namespace mcu {

// Q8_K packer, matmul_quant_pack.c:106-142 of the reference.  LPB lanes share one 256-value block, lane `sl` of the
// group owns the NV = 256 / LPB consecutive values NV*sl ..; groups are aligned runs of LPB lanes of one warp.  Few
// lanes per block when there are many blocks, all 32 when there are few: either way a warp issues all the loads of a
// block before it uses any, so the packing costs one trip to L2.  cvt.rni (round to nearest even) equals the
// reference's 1.5*2^23 rounding trick for |v| < 2^22, and |iscale*x| <= 127 here.
template <int LPB>
__device__ __forceinline__ void load_values_q8_k(const float *row, int len, bool vec_ok, int sl, float (&v)[QK_K / LPB]) {
    constexpr int NV = QK_K / LPB;
    if (row == nullptr) {
#pragma unroll
        for (int i = 0; i < NV; ++i) v[i] = 0.0f;
    } else if (vec_ok && len == QK_K) {
#pragma unroll
        for (int i = 0; i < NV / 4; ++i) {
            const float4 a = MCU_ACT_LOAD((const float4 *)(row + NV * sl + 4 * i));
            v[4 * i] = a.x, v[4 * i + 1] = a.y, v[4 * i + 2] = a.z, v[4 * i + 3] = a.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < NV; ++i) v[i] = NV * sl + i < len ? MCU_ACT_LOAD(row + NV * sl + i) : 0.0f;
    }
}

template <int LPB>
__device__ __forceinline__ void pack_values_q8_k(const float (&v)[QK_K / LPB], bool valid, int lane, int8_t *q, float *d_out,
                                                 int16_t *bs32) {
    constexpr int NV = QK_K / LPB;
    const int sl = lane & (LPB - 1), grp = lane / LPB;
    float la = 0.0f, lv = 0.0f;  // first value of largest magnitude among this lane's
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const float a = fabsf(v[i]);
        if (a > la) {
            la = a;
            lv = v[i];
        }
    }
    float m = la;
#pragma unroll
    for (int o = LPB / 2; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    // the first occurrence in value order is in the lowest lane of the group that holds the maximum
    unsigned holders = __ballot_sync(0xffffffffu, la == m);
    if (LPB < 32) holders = (holders >> (grp * LPB)) & ((1u << (LPB & 31)) - 1u);
    const float max_val = __shfl_sync(0xffffffffu, lv, grp * LPB + __ffs(holders) - 1);
    const bool zero = !(m > 0.0f);
    const float iscale = zero ? 0.0f : __fdiv_rn(-127.0f, max_val);
    uint32_t w[NV / 4];
    int s = 0;
#pragma unroll
    for (int i = 0; i < NV / 4; ++i) {
        int qv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // round to nearest even by adding 1.5 * 2^23 (the reference's own trick; exact for |x| <= 127): two
            // full-rate instructions instead of a conversion on the quarter-rate pipe
            qv[j] = min(__float_as_int(__fadd_rn(__fmul_rn(iscale, v[4 * i + j]), 12582912.0f)) - 0x4B400000, 127);
            s += qv[j];
        }
        w[i] = (uint32_t)(qv[0] & 0xFF) | ((uint32_t)(qv[1] & 0xFF) << 8) | ((uint32_t)(qv[2] & 0xFF) << 16) |
            ((uint32_t)qv[3] << 24);
    }
    // sub-block sums: 32 values = 32 / NV lanes
    if (NV <= 16) s += __shfl_xor_sync(0xffffffffu, s, 1);
    if (NV <= 8) s += __shfl_xor_sync(0xffffffffu, s, 2);
    if (!valid) return;
    // value v0 = 64g + 32b + i lives at b*128 + g*32 + i; a lane's run never crosses a 32-value group
    const int v0 = NV * sl;
    int8_t *dst = q + ((v0 >> 5) & 1) * 128 + (v0 >> 6) * 32 + (v0 & 31);
    if (NV == 8) {
        *(uint2 *)dst = make_uint2(w[0], w[1]);
    } else {
#pragma unroll
        for (int i = 0; i < NV / 16; ++i) *(uint4 *)(dst + 16 * i) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
    }
    if (bs32 != nullptr) {  // sums of the 32-value sub-blocks, for callers that fold the Q4_K mins with them
        if (NV >= 32) {
            bs32[v0 >> 5] = (int16_t)s;  // NV == 32: the lane owns exactly one sub-block
        } else if ((sl & (32 / NV - 1)) == 0) {
            bs32[v0 >> 5] = (int16_t)s;
        }
    }
    if (sl == 0) *d_out = zero ? 0.0f : __fdiv_rn(1.0f, iscale);
}

// Q8_0 packer, matmul_quant_pack.c:23-62 with the scalar helpers of quantization/common/block.c (amax/127, roundf =
// half away from zero, fp16 stored scale).  Four lanes per 32-value block, eight values each.
__device__ __forceinline__ void load_values_q8_0(const float *row, int len, bool vec_ok, int sl, float (&v)[8]) {
    if (row == nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    } else if (vec_ok && len == Q8_0_VALUES) {
        const float4 a = MCU_ACT_LOAD((const float4 *)(row + 8 * sl)), b = MCU_ACT_LOAD((const float4 *)(row + 8 * sl + 4));
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 8 * sl + i < len ? MCU_ACT_LOAD(row + 8 * sl + i) : 0.0f;
    }
}

__device__ __forceinline__ void pack_values_q8_0(const float (&v)[8], bool valid, int sl, int8_t *q, float *d_out) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    float scale = __fdiv_rn(amax, 127.0f);
    if (scale < 1.17549435e-38f) scale = 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
    uint32_t w[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        int qv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) qv[j] = max(-127, min(127, (int)roundf(__fmul_rn(v[4 * i + j], inv))));
        w[i] = (uint32_t)(qv[0] & 0xFF) | ((uint32_t)(qv[1] & 0xFF) << 8) | ((uint32_t)(qv[2] & 0xFF) << 16) |
            ((uint32_t)qv[3] << 24);
    }
    if (!valid) return;
    *(uint2 *)(q + 8 * sl) = make_uint2(w[0], w[1]);
    if (sl == 0) *d_out = __half2float(__float2half_rn(scale));
}

}  // namespace mcu
