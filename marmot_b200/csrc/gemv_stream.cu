// Streaming decode-regime matmul for sm_100a (T <= 8 tokens).
//
// Persistent CTAs each own a contiguous range of weight rows.  A producer thread streams that range
// from HBM into a shared-memory ring with bulk asynchronous copies (cp.async.bulk, completion counted
// on mbarriers); the consumer warps quantize the activations into shared memory (same values as the
// reference's Q8_K / Q8_0 packers), then walk the ring, one weight row per warp: unpack scales and
// quants in registers, dp4a integer dots, per-block f32 scaling in the reference's operation order,
// shuffle reduction.
//
// The weight prefetch is issued before `griddepcontrol.wait`, and the single-token configuration
// keeps a CTA within half of an SM's registers, threads and shared memory: launched with programmatic
// stream serialization, the CTAs of GEMV n+1 become resident and pull their weights into shared
// memory while GEMV n is still computing (weights never depend on the previous kernel; the
// activations and the output buffer do, and are only touched after the wait).
//
// Every wait on an mbarrier is bounded: after SPIN_LIMIT failed polls the kernel records an error
// code in *err, stops consuming and returns.
#include "common.cuh"
#include "kernels.h"

#include <cstdlib>

namespace mcu {

constexpr int GS_MAX_STAGES = 8;
constexpr int GS_ACT_BLOCK = 272;  // 256 int8 + 16 pad: conflict-free 16-byte reads by the lane pairs
constexpr int GS_HEADER = 256;     // barriers + flags at the start of shared memory
constexpr uint32_t SPIN_LIMIT = 1u << 20;

struct GemvStreamParams {
    const uint8_t *W[2];
    float *out[2];
    const float *x;
    const float *bias;
    int *err;
    int ldx, ldo, K, nb, F;
    int row_bytes, rows_per_cta, rows_per_chunk;
    int act_bytes;     // shared memory reserved for the quantized activations (multiple of 128)
    int stages;        // ring depth, <= GS_MAX_STAGES
    int stage_stride;  // bytes between stage buffers (multiple of 128, includes over-read slack)
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; false after SPIN_LIMIT polls.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// unsigned bytes of a times signed bytes of b
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// N words starting at a 2-byte aligned shared-memory address (reads one aligned word beyond).
template <int N>
__device__ __forceinline__ void lds_words_align2(const uint8_t *p, uint32_t (&out)[N]) {
    const uint32_t a = smem_u32(p);
    const uint32_t *w = (const uint32_t *)(p - (a & 3u));
    const uint32_t sh = (a & 3u) * 8u;
    uint32_t prev = w[0];
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const uint32_t next = w[i + 1];
        out[i] = __funnelshift_r(prev, next, sh);
        prev = next;
    }
}

// ---------------------------------------------------------------------------------------------
// Activations -> shared memory.  Layouts:
//   K-quants: qs [T][nb][272] (value 64g+32b+i at b*128+g*32+i), d [T][nb] f32, bs32 [T][nb][8] int16
//             (sum of the quants of each 32-value sub-block = bsums[2j]+bsums[2j+1] of the Q8_K block)
//   Q8_0:     qs [T][nb*32], d [T][nb] f32 (value of the fp16-rounded scale)
// ---------------------------------------------------------------------------------------------
struct ActSmem {
    int8_t *qs;
    float *d;
    int16_t *bs32;
    int tstride;  // bytes between tokens in qs
};

template <bool KQ>
__device__ __forceinline__ ActSmem act_layout(uint8_t *base, int T, int nb) {
    ActSmem a;
    a.qs = (int8_t *)base;
    if (KQ) {
        a.tstride = nb * GS_ACT_BLOCK;
        a.d = (float *)(base + (size_t)T * a.tstride);
        // 8-byte vector reads of the sub-block sums: keep the array 16-byte aligned
        a.bs32 = (int16_t *)(base + (((size_t)T * a.tstride + (size_t)T * nb * 4 + 15) & ~(size_t)15));
    } else {
        a.tstride = (nb * Q8_0_VALUES + 15) & ~15;
        a.d = (float *)(base + (size_t)T * a.tstride);
        a.bs32 = nullptr;
    }
    return a;
}

__host__ __device__ inline int act_smem_bytes(bool kq, int T, int nb) {
    const int bytes = kq ? T * nb * (GS_ACT_BLOCK + 4 + 16) + 16 : T * (((nb * Q8_0_VALUES + 15) & ~15) + nb * 4);
    return (bytes + 127) & ~127;
}

// Q8_K packer for one (token, block) by one warp; matmul_quant_pack.c:106-142 of the reference.
// Lane l owns the eight consecutive values 8l .. 8l+7.  cvt.rni (round to nearest even) equals the
// reference's 1.5*2^23 rounding trick for |v| < 2^22, and |iscale*x| <= 127 here.
__device__ __forceinline__ void quantize_block_q8_k(const float *row, int len, bool vec_ok, int lane, int8_t *q,
                                                    float *d_out, int16_t *bs32) {
    float v[8];
    if (vec_ok && len == QK_K) {
        const float4 a = __ldg((const float4 *)(row + 8 * lane));
        const float4 b = __ldg((const float4 *)(row + 8 * lane + 4));
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 8 * lane + i < len ? __ldg(row + 8 * lane + i) : 0.0f;
    }
    float la = 0.0f, lv = 0.0f;  // first value of largest magnitude among this lane's eight
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float a = fabsf(v[i]);
        if (a > la) {
            la = a;
            lv = v[i];
        }
    }
    float m = la;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    // the first occurrence in value order is in the lowest lane that holds the maximum
    const unsigned holders = __ballot_sync(0xffffffffu, la == m);
    const float max_val = __shfl_sync(0xffffffffu, lv, __ffs(holders) - 1);
    const bool zero = !(m > 0.0f);
    const float iscale = zero ? 0.0f : __fdiv_rn(-127.0f, max_val);
    int qv[8];
    int s = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        qv[i] = min(__float2int_rn(__fmul_rn(iscale, v[i])), 127);
        s += qv[i];
    }
    const uint32_t w0 = (uint32_t)(qv[0] & 0xFF) | ((uint32_t)(qv[1] & 0xFF) << 8) | ((uint32_t)(qv[2] & 0xFF) << 16) |
        ((uint32_t)qv[3] << 24);
    const uint32_t w1 = (uint32_t)(qv[4] & 0xFF) | ((uint32_t)(qv[5] & 0xFF) << 8) | ((uint32_t)(qv[6] & 0xFF) << 16) |
        ((uint32_t)qv[7] << 24);
    // values 8l..8l+7: group g = l/8, half b = (l/4)&1, offset 8*(l&3) inside the 32
    *(uint2 *)(q + ((lane >> 2) & 1) * 128 + (lane >> 3) * 32 + (lane & 3) * 8) = make_uint2(w0, w1);
    // sub-block j = values 32j..32j+31 = lanes 4j..4j+3
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if ((lane & 3) == 0) bs32[lane >> 2] = (int16_t)s;
    if (lane == 0) *d_out = zero ? 0.0f : __fdiv_rn(1.0f, iscale);
}

// Q8_0 packer for one (token, block) by one warp; matmul_quant_pack.c:23-62 with the scalar helpers
// of quantization/common/block.c (amax/127, roundf = half away from zero, fp16 stored scale).
__device__ __forceinline__ void quantize_block_q8_0(const float *row, int len, int lane, int8_t *q, float *d_out) {
    const float v = lane < len ? __ldg(row + lane) : 0.0f;
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float scale = __fdiv_rn(amax, 127.0f);
    if (scale < 1.17549435e-38f) scale = 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
    int qv = (int)roundf(__fmul_rn(v, inv));
    qv = max(-127, min(127, qv));
    q[lane] = (int8_t)qv;
    if (lane == 0) *d_out = __half2float(__float2half_rn(scale));
}

// ---------------------------------------------------------------------------------------------
// Row dots from shared memory.  acc[t] gets the row's block terms owned by this lane.
// ---------------------------------------------------------------------------------------------

// Q4_K: two lanes per super-block; lane h owns sub-blocks 4h .. 4h+3 (qs bytes [64h, 64h+64)).
// High nibbles are used in place (byte & 0xF0 = 16*q): their dot is 16 times too large, which the
// exact arithmetic shift at the end undoes.
template <int T>
__device__ __forceinline__ void row_q4_k(const uint8_t *wrow, const ActSmem &a, int nb, int lane, float (&acc)[T]) {
    const int sub = lane >> 1, h = lane & 1;
    for (int b0 = 0; b0 < nb; b0 += 16) {
        const int blk = b0 + sub;
        const bool ok = blk < nb;
        int p[T], s[T];
        float ad[T];
#pragma unroll
        for (int t = 0; t < T; ++t) p[t] = 0, s[t] = 0, ad[t] = 0.0f;
        float d = 0.0f, dmin = 0.0f;
        if (ok) {
            const uint4 *bp = (const uint4 *)(wrow + (size_t)blk * Q4_K_BYTES);
            const uint4 hdr = bp[0];
            d = half_bits_to_float((uint16_t)(hdr.x & 0xFFFFu));
            dmin = half_bits_to_float((uint16_t)(hdr.x >> 16));
            // scales / mins of sub-blocks 4h..4h+3, one per byte (bit selection of get_scale_min_k4)
            const uint32_t sc4 =
                h == 0 ? (hdr.y & 0x3F3F3F3Fu) : ((hdr.w & 0x0F0F0F0Fu) | (((hdr.y >> 6) & 0x03030303u) << 4));
            const uint32_t mn4 =
                h == 0 ? (hdr.z & 0x3F3F3F3Fu) : (((hdr.w >> 4) & 0x0F0F0F0Fu) | (((hdr.z >> 6) & 0x03030303u) << 4));
            int phi[T];
#pragma unroll
            for (int t = 0; t < T; ++t) phi[t] = 0;
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                const uint4 q0 = bp[1 + 4 * h + 2 * g], q1 = bp[2 + 4 * h + 2 * g];
                const int gg = 2 * h + g;
                const int sc_lo = (int)((sc4 >> (16 * g)) & 0xFFu), sc_hi = (int)((sc4 >> (16 * g + 8)) & 0xFFu);
#pragma unroll
                for (int t = 0; t < T; ++t) {
                    const int8_t *qa = a.qs + (size_t)t * a.tstride + (size_t)blk * GS_ACT_BLOCK + gg * 32;
                    const int4 l0 = *(const int4 *)qa, l1 = *(const int4 *)(qa + 16);
                    const int4 h0 = *(const int4 *)(qa + 128), h1 = *(const int4 *)(qa + 144);
                    int dlo = __dp4a((int)(q0.x & 0x0F0F0F0Fu), l0.x, 0);
                    dlo = __dp4a((int)(q0.y & 0x0F0F0F0Fu), l0.y, dlo);
                    dlo = __dp4a((int)(q0.z & 0x0F0F0F0Fu), l0.z, dlo);
                    dlo = __dp4a((int)(q0.w & 0x0F0F0F0Fu), l0.w, dlo);
                    dlo = __dp4a((int)(q1.x & 0x0F0F0F0Fu), l1.x, dlo);
                    dlo = __dp4a((int)(q1.y & 0x0F0F0F0Fu), l1.y, dlo);
                    dlo = __dp4a((int)(q1.z & 0x0F0F0F0Fu), l1.z, dlo);
                    dlo = __dp4a((int)(q1.w & 0x0F0F0F0Fu), l1.w, dlo);
                    int dhi = dp4a_us(q0.x & 0xF0F0F0F0u, h0.x, 0);
                    dhi = dp4a_us(q0.y & 0xF0F0F0F0u, h0.y, dhi);
                    dhi = dp4a_us(q0.z & 0xF0F0F0F0u, h0.z, dhi);
                    dhi = dp4a_us(q0.w & 0xF0F0F0F0u, h0.w, dhi);
                    dhi = dp4a_us(q1.x & 0xF0F0F0F0u, h1.x, dhi);
                    dhi = dp4a_us(q1.y & 0xF0F0F0F0u, h1.y, dhi);
                    dhi = dp4a_us(q1.z & 0xF0F0F0F0u, h1.z, dhi);
                    dhi = dp4a_us(q1.w & 0xF0F0F0F0u, h1.w, dhi);
                    p[t] += sc_lo * dlo;
                    phi[t] += sc_hi * dhi;
                }
            }
#pragma unroll
            for (int t = 0; t < T; ++t) {
                p[t] += phi[t] >> 4;  // exact: every term is a multiple of 16
                const int2 bs = *(const int2 *)(a.bs32 + ((size_t)t * nb + blk) * 8 + 4 * h);
                s[t] = (int)(mn4 & 0xFFu) * (int)(int16_t)(bs.x & 0xFFFF) + (int)((mn4 >> 8) & 0xFFu) * (bs.x >> 16) +
                    (int)((mn4 >> 16) & 0xFFu) * (int)(int16_t)(bs.y & 0xFFFF) + (int)(mn4 >> 24) * (bs.y >> 16);
                ad[t] = a.d[t * nb + blk];
            }
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
            const int pp = p[t] + __shfl_xor_sync(0xffffffffu, p[t], 1);
            const int ss = s[t] + __shfl_xor_sync(0xffffffffu, s[t], 1);
            if (h == 0 && ok) {
                const float dd = __fmul_rn(ad[t], d), dm = __fmul_rn(ad[t], dmin);
                acc[t] = __fadd_rn(acc[t], __fsub_rn(__fmul_rn(dd, (float)pp), __fmul_rn(dm, (float)ss)));
            }
        }
    }
}

// Q6_K: two lanes per super-block; lane h owns the 128-value half h.
template <int T>
__device__ __forceinline__ void row_q6_k(const uint8_t *wrow, const ActSmem &a, int nb, int lane, float (&acc)[T]) {
    const int sub = lane >> 1, h = lane & 1;
    for (int b0 = 0; b0 < nb; b0 += 16) {
        const int blk = b0 + sub;
        const bool ok = blk < nb;
        int p[T];
        float ad[T];
#pragma unroll
        for (int t = 0; t < T; ++t) p[t] = 0, ad[t] = 0.0f;
        float d = 0.0f;
        if (ok) {
            const uint8_t *bp = wrow + (size_t)blk * Q6_K_BYTES;
            uint32_t qh[8], scw[2];
            lds_words_align2<8>(bp + 128 + 32 * h, qh);
            lds_words_align2<2>(bp + 192 + 8 * h, scw);
            d = half_bits_to_float(*(const uint16_t *)(bp + 208));
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t ql[8];
                lds_words_align2<8>(bp + 64 * h + 32 * (c & 1), ql);
                uint32_t qw[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t lo4 = (c & 2) ? ((ql[j] >> 4) & 0x0F0F0F0Fu) : (ql[j] & 0x0F0F0F0Fu);
                    const uint32_t h2 = (qh[j] >> (2 * c)) & 0x03030303u;
                    qw[j] = __vsub4(lo4 | (h2 << 4), 0x20202020u);
                }
                // int8 scales of the two 16-value groups: bytes 2c and 2c+1 of this half's eight
                const uint32_t sw = scw[c >> 1] >> (16 * (c & 1));
                const int sc0 = (int)(int8_t)(sw & 0xFFu), sc1 = (int)(int8_t)((sw >> 8) & 0xFFu);
#pragma unroll
                for (int t = 0; t < T; ++t) {
                    // values 128h + 32c + l live at (c&1)*128 + (2h + c/2)*32 + l
                    const int8_t *qa = a.qs + (size_t)t * a.tstride + (size_t)blk * GS_ACT_BLOCK + (c & 1) * 128 +
                        (2 * h + (c >> 1)) * 32;
                    const int4 a0 = *(const int4 *)qa, a1 = *(const int4 *)(qa + 16);
                    int s0 = __dp4a((int)qw[0], a0.x, 0);
                    s0 = __dp4a((int)qw[1], a0.y, s0);
                    s0 = __dp4a((int)qw[2], a0.z, s0);
                    s0 = __dp4a((int)qw[3], a0.w, s0);
                    int s1 = __dp4a((int)qw[4], a1.x, 0);
                    s1 = __dp4a((int)qw[5], a1.y, s1);
                    s1 = __dp4a((int)qw[6], a1.z, s1);
                    s1 = __dp4a((int)qw[7], a1.w, s1);
                    p[t] += sc0 * s0 + sc1 * s1;
                }
            }
#pragma unroll
            for (int t = 0; t < T; ++t) ad[t] = a.d[t * nb + blk];
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
            const int pp = p[t] + __shfl_xor_sync(0xffffffffu, p[t], 1);
            if (h == 0 && ok) acc[t] = __fadd_rn(acc[t], __fmul_rn(__fmul_rn(ad[t], d), (float)pp));
        }
    }
}

// Q8_0: one lane per 32-value block.
template <int T>
__device__ __forceinline__ void row_q8_0(const uint8_t *wrow, const ActSmem &a, int nb, int lane, float (&acc)[T]) {
    for (int blk = lane; blk < nb; blk += 32) {
        const uint8_t *bp = wrow + (size_t)blk * Q8_0_BYTES;
        const float d = half_bits_to_float(*(const uint16_t *)bp);
        uint32_t w[8];
        lds_words_align2<8>(bp + 2, w);
#pragma unroll
        for (int t = 0; t < T; ++t) {
            const int4 *qa = (const int4 *)(a.qs + (size_t)t * a.tstride + (size_t)blk * Q8_0_VALUES);
            const int4 a0 = qa[0], a1 = qa[1];
            int s = __dp4a((int)w[0], a0.x, 0);
            s = __dp4a((int)w[1], a0.y, s);
            s = __dp4a((int)w[2], a0.z, s);
            s = __dp4a((int)w[3], a0.w, s);
            s = __dp4a((int)w[4], a1.x, s);
            s = __dp4a((int)w[5], a1.y, s);
            s = __dp4a((int)w[6], a1.z, s);
            s = __dp4a((int)w[7], a1.w, s);
            const float ad = a.d[t * nb + blk];
            acc[t] = __fadd_rn(acc[t], __fmul_rn((float)s, __fmul_rn(d, ad)));
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The kernel.  NW consumer warps + one producer warp; grid = (CTAs, 1 or 2): blockIdx.y selects the
// weight matrix of a dual-output call.  MINB = 2 keeps the CTA within half of an SM.
// ---------------------------------------------------------------------------------------------
template <int KIND, int T, int NW, int MINB>
__global__ void __launch_bounds__((NW + 1) * 32, MINB) gemv_stream_kernel(const GemvStreamParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr bool KQ = KIND != KIND_Q8_0;
    uint64_t *full = (uint64_t *)smem;
    uint64_t *empty = full + GS_MAX_STAGES;
    int *abort_flag = (int *)(empty + GS_MAX_STAGES);
    uint8_t *act_base = smem + GS_HEADER;
    uint8_t *stage_base = act_base + p.act_bytes;
    const int S = p.stages;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint8_t *W = blockIdx.y == 0 ? p.W[0] : p.W[1];
    float *out = blockIdx.y == 0 ? p.out[0] : p.out[1];
    const int r0 = blockIdx.x * p.rows_per_cta;
    const int r1 = min(p.F, r0 + p.rows_per_cta);
    const int n_rows = max(0, r1 - r0);
    const int RC = p.rows_per_chunk;
    const int n_chunks = (n_rows + RC - 1) / RC;

    if (threadIdx.x == 0) {
        for (int i = 0; i < S; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], NW);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // Let the next kernel in the stream start its own weight prefetch as soon as it fits on the SMs.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == NW) {
        // ---------------- producer ----------------
        if (lane == 0) {
            for (int c = 0; c < n_chunks; ++c) {
                const int st = c % S, round = c / S;
                if (round > 0 && !mbar_wait(&empty[st], (uint32_t)((round - 1) & 1))) {
                    atomicExch(p.err, 1);
                    *(volatile int *)abort_flag = 1;
                    break;
                }
                const int rows = min(RC, n_rows - c * RC);
                const uint32_t bytes = (uint32_t)rows * (uint32_t)p.row_bytes;
                mbar_expect_tx(&full[st], bytes);
                bulk_g2s(stage_base + (size_t)st * p.stage_stride, W + ((size_t)r0 + (size_t)c * RC) * p.row_bytes, bytes,
                         &full[st]);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    // The activations (and the output buffer) may belong to the previous kernel until it has finished.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const ActSmem a = act_layout<KQ>(act_base, T, p.nb);
    {
        const int bv = KQ ? QK_K : Q8_0_VALUES;
        const int items = T * p.nb;
        const bool vec_ok = (((uintptr_t)p.x & 15) == 0) && ((p.ldx & 3) == 0);
        for (int it = warp; it < items; it += NW) {
            const int t = it / p.nb, blk = it - t * p.nb;
            const float *row = p.x + (size_t)t * p.ldx + (size_t)blk * bv;
            const int len = min(bv, p.K - blk * bv);
            if (KQ)
                quantize_block_q8_k(row, len, vec_ok, lane, a.qs + (size_t)t * a.tstride + (size_t)blk * GS_ACT_BLOCK,
                                    a.d + t * p.nb + blk, a.bs32 + ((size_t)t * p.nb + blk) * 8);
            else
                quantize_block_q8_0(row, len, lane, a.qs + (size_t)t * a.tstride + (size_t)blk * Q8_0_VALUES,
                                    a.d + t * p.nb + blk);
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");  // consumer warps only

    for (int c = 0; c < n_chunks; ++c) {
        const int st = c % S, round = c / S;
        if (!mbar_wait(&full[st], (uint32_t)(round & 1))) {
            if (lane == 0) atomicExch(p.err, 2);
            break;
        }
        if (*(volatile int *)abort_flag) break;
        const int rows = min(RC, n_rows - c * RC);
        const uint8_t *sbuf = stage_base + (size_t)st * p.stage_stride;
        // at most one row per warp and chunk (RC <= NW); the assignment rotates from chunk to chunk so that
        // short chunks still use every warp
        const int rl = (warp - (c * RC) % NW + NW) % NW;
        if (rl < rows) {
            float acc[T];
#pragma unroll
            for (int t = 0; t < T; ++t) acc[t] = 0.0f;
            const uint8_t *wrow = sbuf + (size_t)rl * p.row_bytes;
            if (KIND == KIND_Q4_K) row_q4_k<T>(wrow, a, p.nb, lane, acc);
            else if (KIND == KIND_Q6_K) row_q6_k<T>(wrow, a, p.nb, lane, acc);
            else row_q8_0<T>(wrow, a, p.nb, lane, acc);
            const int f = r0 + c * RC + rl;
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const float v = warp_sum(acc[t]);
                if (lane == 0) out[(size_t)t * p.ldo + f] = p.bias != nullptr ? __fadd_rn(v, p.bias[f]) : v;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
static int gcd_int(int a, int b) { return b == 0 ? a : gcd_int(b, a % b); }

constexpr int NW_SHORT = 14;  // single-token jobs: two CTAs per SM (this launch's and the next one's)
constexpr int NW_LONG = 16;

template <int KIND, int T, int NW, int MINB>
static cudaError_t launch_cfg(const GemvStreamParams &p, int grid_x, int grid_y, int smem_bytes, cudaStream_t s) {
    static int configured = 0;  // largest dynamic shared memory size opted in for this instantiation
    if (smem_bytes > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemv_stream_kernel<KIND, T, NW, MINB>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return e;
        // all of the SM's shared memory: CTAs of two consecutive launches must fit side by side
        e = cudaFuncSetAttribute(gemv_stream_kernel<KIND, T, NW, MINB>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        configured = smem_bytes;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid_x, (unsigned)grid_y, 1);
    cfg.blockDim = dim3((NW + 1) * 32, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const bool no_pdl = getenv("MARMOT_CUDA_NO_PDL") != nullptr;  // diagnostic switch
    cfg.numAttrs = no_pdl ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, gemv_stream_kernel<KIND, T, NW, MINB>, p);
}

template <int KIND>
static cudaError_t launch_k(int T, bool short_cfg, const GemvStreamParams &p, int gx, int gy, int smem, cudaStream_t s) {
    if (short_cfg) return launch_cfg<KIND, 1, NW_SHORT, 2>(p, gx, gy, smem, s);
    switch (T) {
    case 1: return launch_cfg<KIND, 1, NW_LONG, 1>(p, gx, gy, smem, s);
    case 2: return launch_cfg<KIND, 2, NW_LONG, 1>(p, gx, gy, smem, s);
    case 3: return launch_cfg<KIND, 3, NW_LONG, 1>(p, gx, gy, smem, s);
    case 4: return launch_cfg<KIND, 4, NW_LONG, 1>(p, gx, gy, smem, s);
    case 5: return launch_cfg<KIND, 5, NW_LONG, 1>(p, gx, gy, smem, s);
    case 6: return launch_cfg<KIND, 6, NW_LONG, 1>(p, gx, gy, smem, s);
    case 7: return launch_cfg<KIND, 7, NW_LONG, 1>(p, gx, gy, smem, s);
    default: return launch_cfg<KIND, 8, NW_LONG, 1>(p, gx, gy, smem, s);
    }
}

struct StreamPlan {
    bool ok;
    bool short_cfg;
    int unit, rows_per_cta, rows_per_chunk, gx, gy, stages, stage_stride, act_bytes, smem;
};

static StreamPlan plan_stream(int kind, const void *W, const void *W2, int T, int K, int F) {
    StreamPlan pl = {};
    if (T < 1 || T > GEMV_MAX_T || F < 1) return pl;
    if (((uintptr_t)W & 15) || ((uintptr_t)W2 & 15)) return pl;  // bulk copies need 16-byte aligned sources
    const int bv = block_values(kind), nb = (K + bv - 1) / bv;
    const long row_bytes = (long)nb * block_bytes(kind);
    if (row_bytes > 64 * 1024) return pl;
    pl.unit = 16 / gcd_int((int)(row_bytes % 16), 16);  // rows per 16-byte aligned group
    if (((long)F * row_bytes) & 15) return pl;           // the last chunk of the last CTA must also be a 16-byte multiple
    pl.act_bytes = act_smem_bytes(kind != KIND_Q8_0, T, nb);
    pl.gy = W2 != nullptr ? 2 : 1;
    const int sms = device_sm_count();
    const int ctas = max(1, sms / pl.gy);
    int rpc = (F + ctas - 1) / ctas;
    rpc = (rpc + pl.unit - 1) / pl.unit * pl.unit;

    // Single-token jobs whose per-CTA share fits in the ring: half-SM CTAs, everything prefetched at once.
    {
        const int nw = NW_SHORT;
        const int rc = (int)min((long)nw, (long)(40 * 1024) / row_bytes) / pl.unit * pl.unit;
        if (T == 1 && rc >= 1) {
            const int chunks = (rpc + rc - 1) / rc;
            const int stride = (int)((rc * row_bytes + 16 + 127) / 128 * 128);
            const int smem = GS_HEADER + pl.act_bytes + chunks * stride;
            if (chunks <= 3 && smem <= 110 * 1024) {
                pl.ok = true;
                pl.short_cfg = true;
                pl.rows_per_cta = rpc;
                pl.rows_per_chunk = rc;
                pl.stages = chunks;
                pl.stage_stride = stride;
                pl.smem = smem;
                pl.gx = (F + rpc - 1) / rpc;
                return pl;
            }
        }
    }
    // General case: one CTA per SM, sixteen consumer warps, as deep a ring as fits.
    {
        const int nw = NW_LONG;
        int rc = (int)min((long)nw, (long)(40 * 1024) / row_bytes) / pl.unit * pl.unit;
        if (rc < 1) {
            if (row_bytes * pl.unit > 64 * 1024 || pl.unit > nw) return pl;
            rc = pl.unit;
        }
        const int stride = (int)((rc * row_bytes + 16 + 127) / 128 * 128);
        const int budget = 200 * 1024 - GS_HEADER - pl.act_bytes;
        if (budget < 2 * stride) return pl;
        const int chunks = (rpc + rc - 1) / rc;
        int stages = min(GS_MAX_STAGES, budget / stride);
        stages = min(stages, max(2, chunks));
        pl.ok = true;
        pl.short_cfg = false;
        pl.rows_per_cta = rpc;
        pl.rows_per_chunk = rc;
        pl.stages = stages;
        pl.stage_stride = stride;
        pl.smem = GS_HEADER + pl.act_bytes + stages * stride;
        pl.gx = (F + rpc - 1) / rpc;
        return pl;
    }
}

bool gemv_stream_supported(int kind, const void *W, const void *W2, int T, int K, int F) {
    return plan_stream(kind, W, W2, T, K, F).ok;
}

cudaError_t launch_gemv_stream(int kind, const void *W, const void *W2, const float *x, int ldx, int T, int K, int F,
                               const float *bias, float *out, float *out2, int ldo, int *err_flag, cudaStream_t s) {
    const StreamPlan pl = plan_stream(kind, W, W2, T, K, F);
    if (!pl.ok) return cudaErrorInvalidValue;
    const int bv = block_values(kind), nb = (K + bv - 1) / bv;
    GemvStreamParams p;
    p.W[0] = (const uint8_t *)W;
    p.W[1] = (const uint8_t *)W2;
    p.out[0] = out;
    p.out[1] = out2;
    p.x = x;
    p.bias = bias;
    p.err = err_flag;
    p.ldx = ldx;
    p.ldo = ldo;
    p.K = K;
    p.nb = nb;
    p.F = F;
    p.row_bytes = nb * block_bytes(kind);
    p.rows_per_cta = pl.rows_per_cta;
    p.rows_per_chunk = pl.rows_per_chunk;
    p.act_bytes = pl.act_bytes;
    p.stages = pl.stages;
    p.stage_stride = pl.stage_stride;
    if (kind == KIND_Q4_K) return launch_k<KIND_Q4_K>(T, pl.short_cfg, p, pl.gx, pl.gy, pl.smem, s);
    if (kind == KIND_Q6_K) return launch_k<KIND_Q6_K>(T, pl.short_cfg, p, pl.gx, pl.gy, pl.smem, s);
    return launch_k<KIND_Q8_0>(T, pl.short_cfg, p, pl.gx, pl.gy, pl.smem, s);
}

}  // namespace mcu
