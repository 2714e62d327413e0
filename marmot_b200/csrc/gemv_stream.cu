// Streaming decode-regime matmul for sm_100a (T <= 8 tokens).
//
// One persistent CTA per SM owns a contiguous range of weight rows.  A producer thread streams that
// range from HBM into a shared-memory ring with bulk asynchronous copies (cp.async.bulk, completion
// counted on mbarriers); eight consumer warps quantize the activations into shared memory (same
// values as the reference's Q8_K / Q8_0 packers), then walk the ring: unpack scales and quants in
// registers, dp4a integer dots, per-block f32 scaling in the reference's operation order, shuffle
// reduction.  The weight prefetch is issued before `griddepcontrol.wait`, so with programmatic
// dependent launch the HBM stream of GEMV n+1 overlaps the tail of GEMV n (weights never depend
// on the previous kernel; the activations do).
//
// Every wait on an mbarrier is bounded: after SPIN_LIMIT failed polls the kernel records an error
// code in *err, stops consuming and returns.
#include "common.cuh"
#include "kernels.h"

namespace mcu {

constexpr int GS_WARPS = 8;                      // consumer warps per group; a group owns every GS_GROUPS-th chunk
constexpr int GS_GROUPS = 2;
constexpr int GS_CONSUMERS = GS_WARPS * GS_GROUPS;
constexpr int GS_THREADS = (GS_CONSUMERS + 1) * 32;  // + one producer warp
constexpr int GS_STAGES = 4;
constexpr int GS_STAGE_BYTES = 18432;            // eight Q4_K rows at K = 4096
constexpr int GS_STAGE_STRIDE = GS_STAGE_BYTES + 128;  // slack for the one-word over-read of unaligned rows
constexpr int GS_ACT_BLOCK = 272;                // 256 int8 + 16 pad: conflict-free 16-byte reads
constexpr uint32_t SPIN_LIMIT = 1u << 20;
static_assert(GS_STAGES % GS_GROUPS == 0, "a stage must always be consumed by the same warp group");

struct GemvStreamParams {
    const uint8_t *W[2];
    float *out[2];
    const float *x;
    const float *bias;
    int *err;
    int ldx, ldo, K, nb, F;
    int row_bytes, rows_per_cta, rows_per_chunk;
    int act_bytes;  // shared memory reserved for the quantized activations (multiple of 128)
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

__device__ __forceinline__ int dot8(const uint32_t (&w)[8], const int4 &a0, const int4 &a1) {
    int s = __dp4a((int)w[0], a0.x, 0);
    s = __dp4a((int)w[1], a0.y, s);
    s = __dp4a((int)w[2], a0.z, s);
    s = __dp4a((int)w[3], a0.w, s);
    s = __dp4a((int)w[4], a1.x, s);
    s = __dp4a((int)w[5], a1.y, s);
    s = __dp4a((int)w[6], a1.z, s);
    s = __dp4a((int)w[7], a1.w, s);
    return s;
}

__device__ __forceinline__ int nearest_int_rne(float v) {
    v = fminf(fmaxf(v, -4194303.0f), 4194303.0f);
    return (__float_as_int(__fadd_rn(v, 12582912.0f)) & 0x007fffff) - 0x00400000;
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
__device__ __forceinline__ void quantize_block_q8_k(const float *row, int len, int lane, int8_t *q, float *d_out,
                                                    int16_t *bs32) {
    float v[8];
    float best_abs = 0.0f, best_val = 0.0f;
    int best_idx = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int idx = lane + 32 * i;
        v[i] = idx < len ? __ldg(row + idx) : 0.0f;
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
    const bool zero = !(best_abs > 0.0f);
    const float iscale = zero ? 0.0f : __fdiv_rn(-127.0f, best_val);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int qv = zero ? 0 : min(nearest_int_rne(__fmul_rn(iscale, v[i])), 127);
        q[(i & 1) * 128 + (i >> 1) * 32 + lane] = (int8_t)qv;  // value 32*i + lane: g = i/2, b = i&1
        const int s = warp_sum(qv);                            // sub-block i = values 32i .. 32i+31
        if (lane == 0) bs32[i] = (int16_t)s;
    }
    if (lane == 0) *d_out = zero ? 0.0f : __fdiv_rn(1.0f, iscale);
}

// Q8_0 packer for one (token, block) by one warp; matmul_quant_pack.c:23-62 with the scalar helpers.
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
template <int T>
__device__ __forceinline__ void row_q4_k(const uint8_t *wrow, const ActSmem &a, int nb, int lane, float (&acc)[T]) {
    const int sub = lane >> 1, h = lane & 1;
    for (int b0 = 0; b0 < nb; b0 += 16) {
        const int blk = b0 + sub;
        const bool ok = blk < nb;
        uint4 hdr = make_uint4(0, 0, 0, 0);
        uint32_t lo[2][8], hi[2][8];
        if (ok) {
            const uint4 *bp = (const uint4 *)(wrow + (size_t)blk * Q4_K_BYTES);
            hdr = bp[0];
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                const uint4 q0 = bp[1 + 4 * h + 2 * g], q1 = bp[2 + 4 * h + 2 * g];
                const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    lo[g][j] = w[j] & 0x0F0F0F0Fu;
                    hi[g][j] = (w[j] >> 4) & 0x0F0F0F0Fu;
                }
            }
        } else {
#pragma unroll
            for (int g = 0; g < 2; ++g)
#pragma unroll
                for (int j = 0; j < 8; ++j) lo[g][j] = hi[g][j] = 0;
        }
        const float d = half_bits_to_float((uint16_t)(hdr.x & 0xFFFFu));
        const float dmin = half_bits_to_float((uint16_t)(hdr.x >> 16));
        // scales / mins of sub-blocks 4h..4h+3, one per byte (bit selection of get_scale_min_k4)
        const uint32_t sc4 = h == 0 ? (hdr.y & 0x3F3F3F3Fu) : ((hdr.w & 0x0F0F0F0Fu) | (((hdr.y >> 6) & 0x03030303u) << 4));
        const uint32_t mn4 = h == 0 ? (hdr.z & 0x3F3F3F3Fu)
                                    : (((hdr.w >> 4) & 0x0F0F0F0Fu) | (((hdr.z >> 6) & 0x03030303u) << 4));
#pragma unroll
        for (int t = 0; t < T; ++t) {
            int p = 0, s = 0;
            float ad = 0.0f;
            if (ok) {
                const int8_t *qa = a.qs + (size_t)t * a.tstride + (size_t)blk * GS_ACT_BLOCK;
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    const int gg = 2 * h + g;
                    const int4 *alo = (const int4 *)(qa + gg * 32);
                    const int4 *ahi = (const int4 *)(qa + 128 + gg * 32);
                    const int dlo = dot8(lo[g], alo[0], alo[1]);
                    const int dhi = dot8(hi[g], ahi[0], ahi[1]);
                    p += (int)((sc4 >> (16 * g)) & 0xFFu) * dlo + (int)((sc4 >> (16 * g + 8)) & 0xFFu) * dhi;
                }
                const int2 bs = *(const int2 *)(a.bs32 + ((size_t)t * nb + blk) * 8 + 4 * h);
                s = (int)(mn4 & 0xFFu) * (int)(int16_t)(bs.x & 0xFFFF) + (int)((mn4 >> 8) & 0xFFu) * (bs.x >> 16) +
                    (int)((mn4 >> 16) & 0xFFu) * (int)(int16_t)(bs.y & 0xFFFF) + (int)(mn4 >> 24) * (bs.y >> 16);
                ad = a.d[t * nb + blk];
            }
            p += __shfl_xor_sync(0xffffffffu, p, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            if (h == 0 && ok) {
                const float dd = __fmul_rn(ad, d), dm = __fmul_rn(ad, dmin);
                acc[t] = __fadd_rn(acc[t], __fsub_rn(__fmul_rn(dd, (float)p), __fmul_rn(dm, (float)s)));
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
        uint32_t qw[4][8];
        uint32_t scw[2] = {0, 0};
        float d = 0.0f;
        if (ok) {
            const uint8_t *bp = wrow + (size_t)blk * Q6_K_BYTES;
            uint32_t ql[16], qh[8];
            lds_words_align2<16>(bp + 64 * h, ql);
            lds_words_align2<8>(bp + 128 + 32 * h, qh);
            lds_words_align2<2>(bp + 192 + 8 * h, scw);
            d = half_bits_to_float(*(const uint16_t *)(bp + 208));
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t src = ql[(c & 1) * 8 + j];
                    const uint32_t lo4 = (c & 2) ? ((src >> 4) & 0x0F0F0F0Fu) : (src & 0x0F0F0F0Fu);
                    const uint32_t h2 = (qh[j] >> (2 * c)) & 0x03030303u;
                    qw[c][j] = __vsub4(lo4 | (h2 << 4), 0x20202020u);
                }
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int j = 0; j < 8; ++j) qw[c][j] = 0;
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
            int p = 0;
            float ad = 0.0f;
            if (ok) {
                const int8_t *qa = a.qs + (size_t)t * a.tstride + (size_t)blk * GS_ACT_BLOCK;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    // values 128h + 32c + l live at (c&1)*128 + (2h + c/2)*32 + l
                    const int4 *av = (const int4 *)(qa + (c & 1) * 128 + (2 * h + (c >> 1)) * 32);
                    const int4 a0 = av[0], a1 = av[1];
                    int s0 = __dp4a((int)qw[c][0], a0.x, 0);
                    s0 = __dp4a((int)qw[c][1], a0.y, s0);
                    s0 = __dp4a((int)qw[c][2], a0.z, s0);
                    s0 = __dp4a((int)qw[c][3], a0.w, s0);
                    int s1 = __dp4a((int)qw[c][4], a1.x, 0);
                    s1 = __dp4a((int)qw[c][5], a1.y, s1);
                    s1 = __dp4a((int)qw[c][6], a1.z, s1);
                    s1 = __dp4a((int)qw[c][7], a1.w, s1);
                    // int8 scales of the two 16-value groups: bytes 2c and 2c+1 of this half's eight
                    const uint32_t w = scw[c >> 1] >> (16 * (c & 1));
                    p += (int)(int8_t)(w & 0xFFu) * s0 + (int)(int8_t)((w >> 8) & 0xFFu) * s1;
                }
                ad = a.d[t * nb + blk];
            }
            p += __shfl_xor_sync(0xffffffffu, p, 1);
            if (h == 0 && ok) acc[t] = __fadd_rn(acc[t], __fmul_rn(__fmul_rn(ad, d), (float)p));
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
            const int s = dot8(w, qa[0], qa[1]);
            const float ad = a.d[t * nb + blk];
            acc[t] = __fadd_rn(acc[t], __fmul_rn((float)s, __fmul_rn(d, ad)));
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The kernel.  grid = (CTAs, 1 or 2): blockIdx.y selects the weight matrix of a dual-output call.
// ---------------------------------------------------------------------------------------------
template <int KIND, int T>
__global__ void __launch_bounds__(GS_THREADS, 1) gemv_stream_kernel(const GemvStreamParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr bool KQ = KIND != KIND_Q8_0;
    uint64_t *full = (uint64_t *)smem;
    uint64_t *empty = full + GS_STAGES;
    int *abort_flag = (int *)(empty + GS_STAGES);
    uint8_t *act_base = smem + 128;
    uint8_t *stage_base = act_base + p.act_bytes;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint8_t *W = p.W[blockIdx.y];
    float *out = p.out[blockIdx.y];
    const int r0 = blockIdx.x * p.rows_per_cta;
    const int r1 = min(p.F, r0 + p.rows_per_cta);
    const int n_rows = max(0, r1 - r0);
    const int RC = p.rows_per_chunk;
    const int n_chunks = (n_rows + RC - 1) / RC;

    if (threadIdx.x == 0) {
        for (int i = 0; i < GS_STAGES; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], GS_WARPS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // Let the next kernel in the stream start its own weight prefetch as soon as it fits on the SMs.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == GS_CONSUMERS) {
        // ---------------- producer ----------------
        if (lane == 0) {
            for (int c = 0; c < n_chunks; ++c) {
                const int st = c % GS_STAGES, round = c / GS_STAGES;
                if (round > 0 && !mbar_wait(&empty[st], (uint32_t)((round - 1) & 1))) {
                    atomicExch(p.err, 1);
                    *(volatile int *)abort_flag = 1;
                    break;
                }
                const int rows = min(RC, n_rows - c * RC);
                const uint32_t bytes = (uint32_t)rows * (uint32_t)p.row_bytes;
                mbar_expect_tx(&full[st], bytes);
                bulk_g2s(stage_base + (size_t)st * GS_STAGE_STRIDE, W + ((size_t)r0 + (size_t)c * RC) * p.row_bytes, bytes,
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
        for (int it = warp; it < items; it += GS_CONSUMERS) {
            const int t = it / p.nb, blk = it - t * p.nb;
            const float *row = p.x + (size_t)t * p.ldx + (size_t)blk * bv;
            const int len = min(bv, p.K - blk * bv);
            if (KQ)
                quantize_block_q8_k(row, len, lane, a.qs + (size_t)t * a.tstride + (size_t)blk * GS_ACT_BLOCK,
                                    a.d + t * p.nb + blk, a.bs32 + ((size_t)t * p.nb + blk) * 8);
            else
                quantize_block_q8_0(row, len, lane, a.qs + (size_t)t * a.tstride + (size_t)blk * Q8_0_VALUES,
                                    a.d + t * p.nb + blk);
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(GS_CONSUMERS * 32) : "memory");  // consumer warps only

    // Chunk c lives in stage c % GS_STAGES and is consumed by warp group c % GS_GROUPS (GS_STAGES is a
    // multiple of GS_GROUPS, so a stage always belongs to the same group): the groups work on
    // different chunks at the same time.
    const int group = warp / GS_WARPS, gwarp = warp % GS_WARPS;
    for (int c = group; c < n_chunks; c += GS_GROUPS) {
        const int st = c % GS_STAGES, round = c / GS_STAGES;
        if (!mbar_wait(&full[st], (uint32_t)(round & 1))) {
            if (lane == 0) atomicExch(p.err, 2);
            break;
        }
        if (*(volatile int *)abort_flag) break;
        const int rows = min(RC, n_rows - c * RC);
        const uint8_t *sbuf = stage_base + (size_t)st * GS_STAGE_STRIDE;
        // rotate the row -> warp assignment from chunk to chunk so that short chunks still use every warp
        const int first = (gwarp - ((c / GS_GROUPS) * RC) % GS_WARPS + GS_WARPS) % GS_WARPS;
        for (int rl = first; rl < rows; rl += GS_WARPS) {
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

template <int KIND, int T>
static cudaError_t launch_kt(const GemvStreamParams &p, int grid_x, int grid_y, int smem_bytes, cudaStream_t s) {
    static int configured = 0;  // largest dynamic shared memory size opted in for this instantiation
    if (smem_bytes > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemv_stream_kernel<KIND, T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             smem_bytes);
        if (e != cudaSuccess) return e;
        configured = smem_bytes;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid_x, (unsigned)grid_y, 1);
    cfg.blockDim = dim3(GS_THREADS, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemv_stream_kernel<KIND, T>, p);
}

template <int KIND>
static cudaError_t launch_k(int T, const GemvStreamParams &p, int gx, int gy, int smem, cudaStream_t s) {
    switch (T) {
    case 1: return launch_kt<KIND, 1>(p, gx, gy, smem, s);
    case 2: return launch_kt<KIND, 2>(p, gx, gy, smem, s);
    case 3: return launch_kt<KIND, 3>(p, gx, gy, smem, s);
    case 4: return launch_kt<KIND, 4>(p, gx, gy, smem, s);
    case 5: return launch_kt<KIND, 5>(p, gx, gy, smem, s);
    case 6: return launch_kt<KIND, 6>(p, gx, gy, smem, s);
    case 7: return launch_kt<KIND, 7>(p, gx, gy, smem, s);
    default: return launch_kt<KIND, 8>(p, gx, gy, smem, s);
    }
}

bool gemv_stream_supported(int kind, const void *W, const void *W2, int T, int K, int F) {
    if (T < 1 || T > GEMV_MAX_T || F < 1) return false;
    if (((uintptr_t)W & 15) || ((uintptr_t)W2 & 15)) return false;  // bulk copies need 16-byte aligned sources
    const int bv = block_values(kind), nb = (K + bv - 1) / bv;
    const long row_bytes = (long)nb * block_bytes(kind);
    const int unit = 16 / gcd_int((int)(row_bytes % 16), 16);  // rows per 16-byte aligned group
    if (row_bytes * unit > GS_STAGE_BYTES) return false;
    if (((long)F * row_bytes) & 15) return false;  // the last chunk of the last CTA must also be a 16-byte multiple
    const int act = act_smem_bytes(kind != KIND_Q8_0, T, nb);
    return 128 + act + GS_STAGES * GS_STAGE_STRIDE <= 200 * 1024;
}

cudaError_t launch_gemv_stream(int kind, const void *W, const void *W2, const float *x, int ldx, int T, int K, int F,
                               const float *bias, float *out, float *out2, int ldo, int *err_flag, cudaStream_t s) {
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
    const int unit = 16 / gcd_int(p.row_bytes % 16, 16);
    const int gy = W2 != nullptr ? 2 : 1;
    const int ctas = max(1, device_sm_count() / gy);
    int rows_per_cta = (F + ctas - 1) / ctas;
    rows_per_cta = (rows_per_cta + unit - 1) / unit * unit;
    const int gx = (F + rows_per_cta - 1) / rows_per_cta;
    int rc = GS_STAGE_BYTES / p.row_bytes;
    rc = max(unit, rc / unit * unit);
    rc = min(rc, max(unit, GS_WARPS / unit * unit));  // at most one row per warp per chunk
    p.rows_per_cta = rows_per_cta;
    p.rows_per_chunk = rc;
    p.act_bytes = act_smem_bytes(kind != KIND_Q8_0, T, nb);
    const int smem = 128 + p.act_bytes + GS_STAGES * GS_STAGE_STRIDE;
    if (kind == KIND_Q4_K) return launch_k<KIND_Q4_K>(T, p, gx, gy, smem, s);
    if (kind == KIND_Q6_K) return launch_k<KIND_Q6_K>(T, p, gx, gy, smem, s);
    return launch_k<KIND_Q8_0>(T, p, gx, gy, smem, s);
}

}  // namespace mcu
