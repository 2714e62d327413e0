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
#include "act_pack.cuh"
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
#ifdef MCU_TRACE
    int trace_slot;
#endif
};

// Diagnostic build only (-DMCU_TRACE): wall-clock stamps per launch, CTA and point.
#ifdef MCU_TRACE
constexpr int GS_TRACE_SLOTS = 64, GS_TRACE_CTAS = 160, GS_TRACE_POINTS = 24;
__device__ unsigned long long g_gs_trace[GS_TRACE_SLOTS][GS_TRACE_CTAS][GS_TRACE_POINTS];
#define GS_TRACE_POINT(pt)                                                                             \
    do {                                                                                               \
        unsigned long long t_;                                                                         \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                         \
        g_gs_trace[p.trace_slot % GS_TRACE_SLOTS][blockIdx.x % GS_TRACE_CTAS][pt] = t_;                \
    } while (0)
#define GS_TRACE_CLOCK(pt) g_gs_trace[p.trace_slot % GS_TRACE_SLOTS][blockIdx.x % GS_TRACE_CTAS][pt] = (unsigned long long)clock64()
__device__ int g_gs_trace_cur_slot;  // set by launch order; good enough for a one-stream lab run
#define GS_TRACE_CLOCK_AT(slot, pt)                                                                  \
    do {                                                                                               \
        if (threadIdx.x == 0) g_gs_trace[(slot) % GS_TRACE_SLOTS][blockIdx.x % GS_TRACE_CTAS][pt] = (unsigned long long)clock64(); \
    } while (0)
#else
#define GS_TRACE_POINT(pt) do { } while (0)
#define GS_TRACE_CLOCK(pt) do { } while (0)
#define GS_TRACE_CLOCK_AT(slot, pt) do { } while (0)
#endif

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

// All (token, block) pairs of the call by the consumer threads: groups of LPB lanes take blocks round robin; the
// values of a group's next block are requested before the current one is packed.
template <int LPB>
__device__ __forceinline__ void quantize_all_q8_k(const float *x, int ldx, int T, int K, int nb, const ActSmem &a, int tid,
                                                  int n_threads, int trace_slot = 0) {
    constexpr int NV = QK_K / LPB;
    const int lane = tid & 31, sl = lane & (LPB - 1);
    const int groups = n_threads / LPB, gid = tid / LPB;
    const int tasks = T * nb;
    const bool vec_ok = (((uintptr_t)x & 15) == 0) && ((ldx & 3) == 0);
    auto row_of = [&](int task, int &len) -> const float * {
        if (task >= tasks) {
            len = 0;
            return nullptr;
        }
        const int t = task / nb, blk = task - t * nb;
        len = min(QK_K, K - blk * QK_K);
        return x + (size_t)t * ldx + (size_t)blk * QK_K;
    };
    float cur[NV];
    int task = gid, len;
    const float *row = row_of(task, len);
    GS_TRACE_CLOCK_AT(trace_slot, 12);
    load_values_q8_k<LPB>(row, len, vec_ok, sl, cur);
#ifdef MCU_TRACE
    asm volatile("" ::"f"(cur[0]), "f"(cur[NV - 1]));  // the stamp below waits for the loads
    if (__float_as_uint(cur[0]) == 0x7fc12345u) return;
#endif
    GS_TRACE_CLOCK_AT(trace_slot, 13);
    for (int base = 0; base < tasks; base += groups) {
        const int t = task < tasks ? task / nb : 0, blk = task < tasks ? task - t * nb : 0;
        const bool valid = task < tasks;
        int8_t *q = a.qs + (size_t)t * a.tstride + (size_t)blk * GS_ACT_BLOCK;
        if (NV <= 16 && base + groups < tasks) {
            float nxt[NV];
            int nlen;
            const float *nrow = row_of(task + groups, nlen);
            load_values_q8_k<LPB>(nrow, nlen, vec_ok, sl, nxt);
            pack_values_q8_k<LPB>(cur, valid, lane, q, a.d + t * nb + blk, a.bs32 + ((size_t)t * nb + blk) * 8);
#pragma unroll
            for (int i = 0; i < NV; ++i) cur[i] = nxt[i];
        } else {
            pack_values_q8_k<LPB>(cur, valid, lane, q, a.d + t * nb + blk, a.bs32 + ((size_t)t * nb + blk) * 8);
            if (base + groups < tasks) {
                int nlen;
                const float *nrow = row_of(task + groups, nlen);
                load_values_q8_k<LPB>(nrow, nlen, vec_ok, sl, cur);
            }
        }
        task += groups;
    }
}

__device__ __forceinline__ void quantize_all_q8_0(const float *x, int ldx, int T, int K, int nb, const ActSmem &a, int tid,
                                                  int n_threads) {
    const int sl = tid & 3;
    const int groups = n_threads / 4, gid = tid / 4;
    const int tasks = T * nb;
    const bool vec_ok = (((uintptr_t)x & 15) == 0) && ((ldx & 3) == 0);
    auto row_of = [&](int task, int &len) -> const float * {
        if (task >= tasks) {
            len = 0;
            return nullptr;
        }
        const int t = task / nb, blk = task - t * nb;
        len = min(Q8_0_VALUES, K - blk * Q8_0_VALUES);
        return x + (size_t)t * ldx + (size_t)blk * Q8_0_VALUES;
    };
    float cur[8], nxt[8];
    int task = gid, len;
    const float *row = row_of(task, len);
    load_values_q8_0(row, len, vec_ok, sl, cur);
    for (int base = 0; base < tasks; base += groups) {
        const bool valid = task < tasks;
        const int t = valid ? task / nb : 0, blk = valid ? task - t * nb : 0;
        const bool more = base + groups < tasks;
        if (more) {
            int nlen;
            const float *nrow = row_of(task + groups, nlen);
            load_values_q8_0(nrow, nlen, vec_ok, sl, nxt);
        }
        pack_values_q8_0(cur, valid, sl, a.qs + (size_t)t * a.tstride + (size_t)blk * Q8_0_VALUES, a.d + t * nb + blk);
        if (more) {
#pragma unroll
            for (int i = 0; i < 8; ++i) cur[i] = nxt[i];
        }
        task += groups;
    }
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
// Two rows per warp at a time (one or two tokens).  A row of K = 4096 is a single pass of the loops above, so the
// cost of a row is its fixed part: header decode, shuffles, the final tree.  Taking two rows together shares the
// activation reads, doubles the independent work per lane and halves the shuffles: after a block, lane h of a pair
// keeps the block sum of row h and passes the other row's to its partner; mine[t] then holds partial sums of row
// (lane & 1), and one xor tree over 2, 4, 8, 16 finishes both rows.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void q4k_scales_of_half(const uint4 &hdr, int h, uint32_t &sc4, uint32_t &mn4) {
    sc4 = h == 0 ? (hdr.y & 0x3F3F3F3Fu) : ((hdr.w & 0x0F0F0F0Fu) | (((hdr.y >> 6) & 0x03030303u) << 4));
    mn4 = h == 0 ? (hdr.z & 0x3F3F3F3Fu) : (((hdr.w >> 4) & 0x0F0F0F0Fu) | (((hdr.z >> 6) & 0x03030303u) << 4));
}

template <int T>
__device__ __forceinline__ void rows2_q4_k(const uint8_t *w0, const uint8_t *w1, const ActSmem &a, int nb, int lane,
                                           float (&mine)[T]) {
    const int sub = lane >> 1, h = lane & 1;
    for (int b0 = 0; b0 < nb; b0 += 16) {
        const int blk = b0 + sub;
        const bool ok = blk < nb;
        int p[2][T], s[2][T];
        float ad[T];
#pragma unroll
        for (int t = 0; t < T; ++t) p[0][t] = p[1][t] = s[0][t] = s[1][t] = 0, ad[t] = 0.0f;
        float d = 0.0f, dmin = 0.0f;  // of the row this lane finishes (row h)
        if (ok) {
            const uint4 *bp[2] = {(const uint4 *)(w0 + (size_t)blk * Q4_K_BYTES), (const uint4 *)(w1 + (size_t)blk * Q4_K_BYTES)};
            const uint4 hdr0 = bp[0][0], hdr1 = bp[1][0];
            uint32_t sc4[2], mn4[2];
            q4k_scales_of_half(hdr0, h, sc4[0], mn4[0]);
            q4k_scales_of_half(hdr1, h, sc4[1], mn4[1]);
            const uint32_t dd_bits = h ? hdr1.x : hdr0.x;
            d = half_bits_to_float((uint16_t)(dd_bits & 0xFFFFu));
            dmin = half_bits_to_float((uint16_t)(dd_bits >> 16));
            int phi[2][T];
#pragma unroll
            for (int t = 0; t < T; ++t) phi[0][t] = phi[1][t] = 0;
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                uint4 q0[2], q1[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) q0[r] = bp[r][1 + 4 * h + 2 * g], q1[r] = bp[r][2 + 4 * h + 2 * g];
                const int gg = 2 * h + g;
#pragma unroll
                for (int t = 0; t < T; ++t) {
                    const int8_t *qa = a.qs + (size_t)t * a.tstride + (size_t)blk * GS_ACT_BLOCK + gg * 32;
                    const int4 l0 = *(const int4 *)qa, l1 = *(const int4 *)(qa + 16);
                    const int4 h0 = *(const int4 *)(qa + 128), h1 = *(const int4 *)(qa + 144);
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        const int sc_lo = (int)((sc4[r] >> (16 * g)) & 0xFFu), sc_hi = (int)((sc4[r] >> (16 * g + 8)) & 0xFFu);
                        int dlo = __dp4a((int)(q0[r].x & 0x0F0F0F0Fu), l0.x, 0);
                        int dlo2 = __dp4a((int)(q1[r].x & 0x0F0F0F0Fu), l1.x, 0);
                        dlo = __dp4a((int)(q0[r].y & 0x0F0F0F0Fu), l0.y, dlo);
                        dlo2 = __dp4a((int)(q1[r].y & 0x0F0F0F0Fu), l1.y, dlo2);
                        dlo = __dp4a((int)(q0[r].z & 0x0F0F0F0Fu), l0.z, dlo);
                        dlo2 = __dp4a((int)(q1[r].z & 0x0F0F0F0Fu), l1.z, dlo2);
                        dlo = __dp4a((int)(q0[r].w & 0x0F0F0F0Fu), l0.w, dlo);
                        dlo2 = __dp4a((int)(q1[r].w & 0x0F0F0F0Fu), l1.w, dlo2);
                        int dhi = dp4a_us(q0[r].x & 0xF0F0F0F0u, h0.x, 0);
                        int dhi2 = dp4a_us(q1[r].x & 0xF0F0F0F0u, h1.x, 0);
                        dhi = dp4a_us(q0[r].y & 0xF0F0F0F0u, h0.y, dhi);
                        dhi2 = dp4a_us(q1[r].y & 0xF0F0F0F0u, h1.y, dhi2);
                        dhi = dp4a_us(q0[r].z & 0xF0F0F0F0u, h0.z, dhi);
                        dhi2 = dp4a_us(q1[r].z & 0xF0F0F0F0u, h1.z, dhi2);
                        dhi = dp4a_us(q0[r].w & 0xF0F0F0F0u, h0.w, dhi);
                        dhi2 = dp4a_us(q1[r].w & 0xF0F0F0F0u, h1.w, dhi2);
                        p[r][t] += sc_lo * (dlo + dlo2);
                        phi[r][t] += sc_hi * (dhi + dhi2);
                    }
                }
            }
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const int2 bs = *(const int2 *)(a.bs32 + ((size_t)t * nb + blk) * 8 + 4 * h);
                const int b0s = (int)(int16_t)(bs.x & 0xFFFF), b1s = bs.x >> 16, b2s = (int)(int16_t)(bs.y & 0xFFFF), b3s = bs.y >> 16;
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    p[r][t] += phi[r][t] >> 4;  // exact: every term is a multiple of 16
                    s[r][t] = (int)(mn4[r] & 0xFFu) * b0s + (int)((mn4[r] >> 8) & 0xFFu) * b1s +
                        (int)((mn4[r] >> 16) & 0xFFu) * b2s + (int)(mn4[r] >> 24) * b3s;
                }
                ad[t] = a.d[t * nb + blk];
            }
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
            const int pp = (h ? p[1][t] : p[0][t]) + __shfl_xor_sync(0xffffffffu, h ? p[0][t] : p[1][t], 1);
            const int ss = (h ? s[1][t] : s[0][t]) + __shfl_xor_sync(0xffffffffu, h ? s[0][t] : s[1][t], 1);
            if (ok) {
                const float dd = __fmul_rn(ad[t], d), dm = __fmul_rn(ad[t], dmin);
                mine[t] = __fadd_rn(mine[t], __fsub_rn(__fmul_rn(dd, (float)pp), __fmul_rn(dm, (float)ss)));
            }
        }
    }
}

template <int T>
__device__ __forceinline__ void rows2_q6_k(const uint8_t *w0, const uint8_t *w1, const ActSmem &a, int nb, int lane,
                                           float (&mine)[T]) {
    const int sub = lane >> 1, h = lane & 1;
    for (int b0 = 0; b0 < nb; b0 += 16) {
        const int blk = b0 + sub;
        const bool ok = blk < nb;
        int p[2][T];
        float ad[T];
#pragma unroll
        for (int t = 0; t < T; ++t) p[0][t] = p[1][t] = 0, ad[t] = 0.0f;
        float d = 0.0f;
        if (ok) {
            const uint8_t *bp[2] = {w0 + (size_t)blk * Q6_K_BYTES, w1 + (size_t)blk * Q6_K_BYTES};
            uint32_t qh[2][8], scw[2][2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                lds_words_align2<8>(bp[r] + 128 + 32 * h, qh[r]);
                lds_words_align2<2>(bp[r] + 192 + 8 * h, scw[r]);
            }
            d = half_bits_to_float(*(const uint16_t *)(bp[h] + 208));
#pragma unroll
            for (int c = 0; c < 4; ++c) {
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    uint32_t ql[8];
                    lds_words_align2<8>(bp[r] + 64 * h + 32 * (c & 1), ql);
                    uint32_t qw[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint32_t lo4 = (c & 2) ? ((ql[j] >> 4) & 0x0F0F0F0Fu) : (ql[j] & 0x0F0F0F0Fu);
                        const uint32_t h2 = (qh[r][j] >> (2 * c)) & 0x03030303u;
                        qw[j] = __vsub4(lo4 | (h2 << 4), 0x20202020u);
                    }
                    const uint32_t sw = scw[r][c >> 1] >> (16 * (c & 1));
                    const int sc0 = (int)(int8_t)(sw & 0xFFu), sc1 = (int)(int8_t)((sw >> 8) & 0xFFu);
#pragma unroll
                    for (int t = 0; t < T; ++t) {
                        const int8_t *qa = a.qs + (size_t)t * a.tstride + (size_t)blk * GS_ACT_BLOCK + (c & 1) * 128 +
                            (2 * h + (c >> 1)) * 32;
                        const int4 a0 = *(const int4 *)qa, a1 = *(const int4 *)(qa + 16);
                        int s0 = __dp4a((int)qw[0], a0.x, 0);
                        int s1 = __dp4a((int)qw[4], a1.x, 0);
                        s0 = __dp4a((int)qw[1], a0.y, s0);
                        s1 = __dp4a((int)qw[5], a1.y, s1);
                        s0 = __dp4a((int)qw[2], a0.z, s0);
                        s1 = __dp4a((int)qw[6], a1.z, s1);
                        s0 = __dp4a((int)qw[3], a0.w, s0);
                        s1 = __dp4a((int)qw[7], a1.w, s1);
                        p[r][t] += sc0 * s0 + sc1 * s1;
                    }
                }
            }
#pragma unroll
            for (int t = 0; t < T; ++t) ad[t] = a.d[t * nb + blk];
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
            const int pp = (h ? p[1][t] : p[0][t]) + __shfl_xor_sync(0xffffffffu, h ? p[0][t] : p[1][t], 1);
            if (ok) mine[t] = __fadd_rn(mine[t], __fmul_rn(__fmul_rn(ad[t], d), (float)pp));
        }
    }
}

template <int T>
__device__ __forceinline__ void rows2_q8_0(const uint8_t *w0, const uint8_t *w1, const ActSmem &a, int nb, int lane,
                                           float (&mine)[T]) {
    float acc[2][T];
#pragma unroll
    for (int t = 0; t < T; ++t) acc[0][t] = acc[1][t] = 0.0f;
    for (int blk = lane; blk < nb; blk += 32) {
        const uint8_t *bp[2] = {w0 + (size_t)blk * Q8_0_BYTES, w1 + (size_t)blk * Q8_0_BYTES};
        uint32_t w[2][8];
        float d[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            d[r] = half_bits_to_float(*(const uint16_t *)bp[r]);
            lds_words_align2<8>(bp[r] + 2, w[r]);
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
            const int4 *qa = (const int4 *)(a.qs + (size_t)t * a.tstride + (size_t)blk * Q8_0_VALUES);
            const int4 a0 = qa[0], a1 = qa[1];
            const float ad = a.d[t * nb + blk];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                int s0 = __dp4a((int)w[r][0], a0.x, 0);
                int s1 = __dp4a((int)w[r][4], a1.x, 0);
                s0 = __dp4a((int)w[r][1], a0.y, s0);
                s1 = __dp4a((int)w[r][5], a1.y, s1);
                s0 = __dp4a((int)w[r][2], a0.z, s0);
                s1 = __dp4a((int)w[r][6], a1.z, s1);
                s0 = __dp4a((int)w[r][3], a0.w, s0);
                s1 = __dp4a((int)w[r][7], a1.w, s1);
                acc[r][t] = __fadd_rn(acc[r][t], __fmul_rn((float)(s0 + s1), __fmul_rn(d[r], ad)));
            }
        }
    }
    const int h = lane & 1;
#pragma unroll
    for (int t = 0; t < T; ++t)
        mine[t] = __fadd_rn(h ? acc[1][t] : acc[0][t], __shfl_xor_sync(0xffffffffu, h ? acc[0][t] : acc[1][t], 1));
}

// ---------------------------------------------------------------------------------------------
// The kernel.  TEAMS * TW consumer warps + one producer warp; grid = (CTAs, 1 or 2): blockIdx.y selects the weight
// matrix of a dual-output call.  A chunk of the ring holds at most TW rows, one per warp of a team.  With one or two
// tokens a team takes the chunks in pairs (two rows per warp at a time, see rows2_*) and the teams take the pairs in
// turn; with more tokens there is one team and it takes the chunks one by one.  MINB = 2 keeps the CTA within half
// of an SM.
// ---------------------------------------------------------------------------------------------
template <int KIND, int T, int TW, int TEAMS, int MINB>
__global__ void __launch_bounds__((TW * TEAMS + 1) * 32, MINB) gemv_stream_kernel(const GemvStreamParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr bool KQ = KIND != KIND_Q8_0;
    constexpr int NW = TW * TEAMS;
    // Row pairs pay where a row's fixed part dominates (Q4_K); the 2-byte aligned formats are bound by their 32-bit
    // shared-memory reads, which pairing does not reduce (measured: Q6_K 22 -> 27 us at T = 1, F = 28672).
    constexpr bool PAIRS = (KIND == KIND_Q4_K && T <= 2) || (KIND == KIND_Q8_0 && T == 2);
    static_assert(PAIRS || TEAMS == 1, "several teams only in the two-row form");
    uint64_t *full = (uint64_t *)smem;
    uint64_t *empty = full + GS_MAX_STAGES;
    int *abort_flag = (int *)(empty + GS_MAX_STAGES);
    uint8_t *act_base = smem + GS_HEADER;
    uint8_t *stage_base = act_base + p.act_bytes;
    const int S = p.stages;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) GS_TRACE_POINT(0);
    if (threadIdx.x == 0) GS_TRACE_CLOCK(9);
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
            mbar_init(&empty[i], TW);  // a chunk is read by the warps of one team
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // Let the next kernel in the stream start its own weight prefetch as soon as it fits on the SMs.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) GS_TRACE_POINT(1);

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
            GS_TRACE_POINT(6);
        }
        return;
    }

    // ---------------- consumers ----------------
    // The activations (and the output buffer) may belong to the previous kernel until it has finished.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) GS_TRACE_POINT(2);
    const ActSmem a = act_layout<KQ>(act_base, T, p.nb);
#ifdef MCU_TRACE
    const int TRACE_SLOT = p.trace_slot;
#else
    constexpr int TRACE_SLOT = 0;
#endif
    GS_TRACE_CLOCK_AT(TRACE_SLOT, 11);
    if (KQ) {
        // as many lanes per block as there are threads for: one round of loads when the blocks are few
        const int tasks = T * p.nb;
        if (tasks * 32 <= NW * 32) {
            quantize_all_q8_k<32>(p.x, p.ldx, T, p.K, p.nb, a, threadIdx.x, NW * 32, TRACE_SLOT);
        } else if (tasks * 16 <= NW * 32 || MINB > 1) {
            quantize_all_q8_k<16>(p.x, p.ldx, T, p.K, p.nb, a, threadIdx.x, NW * 32, TRACE_SLOT);
        } else {
            // 32 values per lane: only where a thread may use more than 64 registers
            if constexpr (MINB == 1) quantize_all_q8_k<8>(p.x, p.ldx, T, p.K, p.nb, a, threadIdx.x, NW * 32, TRACE_SLOT);
        }
    } else {
        quantize_all_q8_0(p.x, p.ldx, T, p.K, p.nb, a, threadIdx.x, NW * 32);
    }
    if (threadIdx.x == 0) GS_TRACE_POINT(8);
    GS_TRACE_CLOCK_AT(TRACE_SLOT, 14);
    asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");  // consumer warps only
    GS_TRACE_CLOCK_AT(TRACE_SLOT, 15);
    if (threadIdx.x == 0) GS_TRACE_POINT(3);

    if (PAIRS) {
        const int team = warp / TW, tw = warp - team * TW;
        const int n_pairs = (n_chunks + 1) / 2;
        for (int jp = team; jp < n_pairs; jp += TEAMS) {
            const int c0 = 2 * jp, c1 = c0 + 1;
            const bool two = c1 < n_chunks;
            const int st0 = c0 % S, st1 = c1 % S;
            bool ready = mbar_wait(&full[st0], (uint32_t)((c0 / S) & 1));
            if (ready && two) ready = mbar_wait(&full[st1], (uint32_t)((c1 / S) & 1));
            if (!ready) {
                if (lane == 0) atomicExch(p.err, 2);
                break;
            }
            if (*(volatile int *)abort_flag) break;
            if (threadIdx.x == 0 && jp < 2) GS_TRACE_POINT(4 + jp);
            if (jp == 0) GS_TRACE_CLOCK_AT(TRACE_SLOT, 16);
            const int rows0 = min(RC, n_rows - c0 * RC), rows1 = two ? min(RC, n_rows - c1 * RC) : 0;
            // at most one row per warp and chunk (RC <= TW); the assignment rotates from chunk to chunk so that
            // short chunks still use every warp
            const int rl0 = (tw - (c0 * RC) % TW + TW) % TW, rl1 = (tw - (c1 * RC) % TW + TW) % TW;
            const bool v0 = rl0 < rows0, v1 = rl1 < rows1;
            if (v0 || v1) {
                const uint8_t *wa = stage_base + (size_t)st0 * p.stage_stride + (size_t)rl0 * p.row_bytes;
                const uint8_t *wb = stage_base + (size_t)st1 * p.stage_stride + (size_t)rl1 * p.row_bytes;
                if (!v0) wa = wb;  // a lone row is computed twice and stored once
                if (!v1) wb = wa;
                float mine[T];
#pragma unroll
                for (int t = 0; t < T; ++t) mine[t] = 0.0f;
                if (KIND == KIND_Q4_K) rows2_q4_k<T>(wa, wb, a, p.nb, lane, mine);
                else if (KIND == KIND_Q6_K) rows2_q6_k<T>(wa, wb, a, p.nb, lane, mine);
                else rows2_q8_0<T>(wa, wb, a, p.nb, lane, mine);
#ifdef MCU_TRACE
                asm volatile("" ::"f"(mine[0]));
                if (__float_as_uint(mine[0]) == 0x7fc12345u) return;
#endif
                if (jp == 0) GS_TRACE_CLOCK_AT(TRACE_SLOT, 17);
                const int f = lane == 0 ? r0 + c0 * RC + rl0 : r0 + c1 * RC + rl1;
                const bool store = lane == 0 ? v0 : (lane == 1 && v1);
#pragma unroll
                for (int t = 0; t < T; ++t) {
                    float v = mine[t];  // partial sums of row (lane & 1)
                    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
                    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
                    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 8));
                    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 16));
                    if (store) out[(size_t)t * p.ldo + f] = p.bias != nullptr ? __fadd_rn(v, p.bias[f]) : v;
                }
            }
            __syncwarp();
            if (jp == 0) GS_TRACE_CLOCK_AT(TRACE_SLOT, 18);
            if (lane == 0) {
                mbar_arrive(&empty[st0]);
                if (two) mbar_arrive(&empty[st1]);
            }
        }
    } else {
        for (int c = 0; c < n_chunks; ++c) {
            const int st = c % S, round = c / S;
            if (!mbar_wait(&full[st], (uint32_t)(round & 1))) {
                if (lane == 0) atomicExch(p.err, 2);
                break;
            }
            if (*(volatile int *)abort_flag) break;
            if (threadIdx.x == 0 && c < 2) GS_TRACE_POINT(4 + c);
            const int rows = min(RC, n_rows - c * RC);
            const uint8_t *sbuf = stage_base + (size_t)st * p.stage_stride;
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
    if (threadIdx.x == 0) GS_TRACE_POINT(7);
    if (threadIdx.x == 0) GS_TRACE_CLOCK(10);
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
static int gcd_int(int a, int b) { return b == 0 ? a : gcd_int(b, a % b); }

constexpr int NW_SHORT = 14;  // single-token jobs: two CTAs per SM (this launch's and the next one's)
constexpr int NW_LONG = 16;

template <int KIND, int T, int TW, int TEAMS, int MINB>
static cudaError_t launch_cfg(const GemvStreamParams &p, int grid_x, int grid_y, int smem_bytes, cudaStream_t s) {
    static int configured = 0;  // largest dynamic shared memory size opted in for this instantiation
    if (smem_bytes > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemv_stream_kernel<KIND, T, TW, TEAMS, MINB>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return e;
        // all of the SM's shared memory: CTAs of two consecutive launches must fit side by side
        e = cudaFuncSetAttribute(gemv_stream_kernel<KIND, T, TW, TEAMS, MINB>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        configured = smem_bytes;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid_x, (unsigned)grid_y, 1);
    cfg.blockDim = dim3((TW * TEAMS + 1) * 32, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const bool no_pdl = getenv("MARMOT_CUDA_NO_PDL") != nullptr;  // diagnostic switch
    cfg.numAttrs = no_pdl ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, gemv_stream_kernel<KIND, T, TW, TEAMS, MINB>, p);
}

template <int KIND>
static cudaError_t launch_k(int T, bool short_cfg, const GemvStreamParams &p, int gx, int gy, int smem, cudaStream_t s) {
    if (short_cfg) return launch_cfg<KIND, 1, NW_SHORT, 1, 2>(p, gx, gy, smem, s);
    switch (T) {
    case 1: return launch_cfg<KIND, 1, NW_LONG, 1, 1>(p, gx, gy, smem, s);
    case 2: return launch_cfg<KIND, 2, NW_LONG, 1, 1>(p, gx, gy, smem, s);
    case 3: return launch_cfg<KIND, 3, NW_LONG, 1, 1>(p, gx, gy, smem, s);
    case 4: return launch_cfg<KIND, 4, NW_LONG, 1, 1>(p, gx, gy, smem, s);
    case 5: return launch_cfg<KIND, 5, NW_LONG, 1, 1>(p, gx, gy, smem, s);
    case 6: return launch_cfg<KIND, 6, NW_LONG, 1, 1>(p, gx, gy, smem, s);
    case 7: return launch_cfg<KIND, 7, NW_LONG, 1, 1>(p, gx, gy, smem, s);
    default: return launch_cfg<KIND, 8, NW_LONG, 1, 1>(p, gx, gy, smem, s);
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
#ifdef MCU_TRACE
    static int trace_next = 0;
    p.trace_slot = trace_next++;
#endif
    if (kind == KIND_Q4_K) return launch_k<KIND_Q4_K>(T, pl.short_cfg, p, pl.gx, pl.gy, pl.smem, s);
    if (kind == KIND_Q6_K) return launch_k<KIND_Q6_K>(T, pl.short_cfg, p, pl.gx, pl.gy, pl.smem, s);
    return launch_k<KIND_Q8_0>(T, pl.short_cfg, p, pl.gx, pl.gy, pl.smem, s);
}

}  // namespace mcu
