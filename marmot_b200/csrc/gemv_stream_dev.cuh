// Device-side building blocks of the streaming GEMV, shared by the kernels that stream packed weight rows through a
// shared-memory ring: mbarrier and bulk-copy helpers, the activation packers (plain and with a prologue), and the row
// dots on the packed blocks.  See gemv_stream.cu for the kernel that introduced them.
#pragma once

#include "act_pack.cuh"
#include "common.cuh"
#include "kernels.h"

#ifndef GS_TRACE_CLOCK_AT  // a diagnostic build of gemv_stream.cu defines these before including this file
#define GS_TRACE_POINT(pt) do { } while (0)
#define GS_TRACE_CLOCK(pt) do { } while (0)
#define GS_TRACE_CLOCK_AT(slot, pt) do { } while (0)
#endif

namespace mcu {

constexpr int GS_MAX_STAGES = 8;
constexpr int GS_ACT_BLOCK = 272;  // 256 int8 + 16 pad: conflict-free 16-byte reads by the lane pairs
constexpr int GS_HEADER = 1024;    // barriers, flags and the prologue's reduction scratch at the start of shared memory
constexpr int GS_RED_OFFSET = 256; // floats: inv[GEMV_MAX_T] then red[GEMV_MAX_T][16]
constexpr uint32_t SPIN_LIMIT = 1u << 20;
constexpr int KIND_MIXED = 0;      // template value: the block format is the job's (K-quants only)

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

// ---------------------------------------------------------------------------------------------
// Prologues: an elementwise step of the decoder layer applied to the activations on their way into the packer.
// ---------------------------------------------------------------------------------------------
// Per-token 1 / rms of x + aux over the K values (RMSNorm's statistic); CTA 0 also stores x + aux to x_out.
// red: GEMV_MAX_T * 16 floats of scratch, inv_s: GEMV_MAX_T floats; both in shared memory.  Ends with the consumer
// barrier, after which inv_s is valid.
// What the prologue helpers need of the launch parameters, passed by value: they are separate functions (the
// registers of the plain path stay as they are), and a reference to the parameter block would force a copy of it
// into local memory.
struct ProArgs {
    const float *x;
    int ldx, K, nb;
    GemvPrologue pro;
};

template <int T, int NTHREADS>
__device__ __noinline__ void pro_rms_stats(const ProArgs p, int tid, float *red, float *inv_s) {
    const GemvPrologue &g = p.pro;
    const int warp = tid >> 5, lane = tid & 31;
    const bool write_x = g.x_out != nullptr && blockIdx.x == 0;
    const bool vec = ((((uintptr_t)p.x | (uintptr_t)g.aux | (uintptr_t)g.x_out) & 15) == 0) &&
        (((p.ldx | g.ld_aux | g.ld_x_out | p.K) & 3) == 0);
    float s[T];
#pragma unroll
    for (int t = 0; t < T; ++t) s[t] = 0.0f;
    if (vec) {
        for (int i = tid * 4; i < p.K; i += NTHREADS * 4) {
#pragma unroll
            for (int t = 0; t < T; ++t) {
                float4 v = MCU_ACT_LOAD((const float4 *)(p.x + (size_t)t * p.ldx + i));
                if (g.aux != nullptr) {
                    const float4 d = MCU_ACT_LOAD((const float4 *)(g.aux + (size_t)t * g.ld_aux + i));
                    v.x = __fadd_rn(v.x, d.x), v.y = __fadd_rn(v.y, d.y), v.z = __fadd_rn(v.z, d.z), v.w = __fadd_rn(v.w, d.w);
                }
                if (write_x) *(float4 *)(g.x_out + (size_t)t * g.ld_x_out + i) = v;
                s[t] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        }
    } else {
        for (int i = tid; i < p.K; i += NTHREADS) {
#pragma unroll
            for (int t = 0; t < T; ++t) {
                float v = MCU_ACT_LOAD(p.x + (size_t)t * p.ldx + i);
                if (g.aux != nullptr) v = __fadd_rn(v, MCU_ACT_LOAD(g.aux + (size_t)t * g.ld_aux + i));
                if (write_x) g.x_out[(size_t)t * g.ld_x_out + i] = v;
                s[t] += v * v;
            }
        }
    }
#pragma unroll
    for (int t = 0; t < T; ++t) {
        const float w = warp_sum(s[t]);
        if (lane == 0) red[t * 16 + warp] = w;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NTHREADS) : "memory");
    if (tid < T) {
        float sum = 0.0f;
        for (int w = 0; w < NTHREADS / 32; ++w) sum += red[tid * 16 + w];
        inv_s[tid] = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)p.K), g.eps)))  /* = 1 / sqrt: both correctly rounded */;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NTHREADS) : "memory");
}

// NV consecutive values of token t from k0 on, through the prologue PRO (a template parameter so that the plain path
// keeps its registers); zeros past K.  vec: every pointer and stride involved allows 16-byte loads and K % 4 == 0.
template <int NV, int PRO>
__device__ __forceinline__ void load_values_pro(const ProArgs &p, bool vec, bool valid, int t, int k0, const float *inv_s,
                                                float (&v)[NV]) {
    const GemvPrologue &g = p.pro;
    const float *xr = p.x + (size_t)t * p.ldx;
    const float *ar = g.aux != nullptr ? g.aux + (size_t)t * g.ld_aux : nullptr;
    float b[NV], w[NV];
    if (vec) {
#pragma unroll
        for (int i = 0; i < NV / 4; ++i) {
            const int k = k0 + 4 * i;
            const bool in = valid && k < p.K;
            const float4 z = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            const float4 xv = in ? MCU_ACT_LOAD((const float4 *)(xr + k)) : z;
            const float4 av = in && ar != nullptr ? MCU_ACT_LOAD((const float4 *)(ar + k)) : z;
            const float4 wv = in && PRO == GEMV_PRO_ADD_RMSNORM && g.norm_w != nullptr ? MCU_ACT_LOAD((const float4 *)(g.norm_w + k)) : z;
            v[4 * i] = xv.x, v[4 * i + 1] = xv.y, v[4 * i + 2] = xv.z, v[4 * i + 3] = xv.w;
            b[4 * i] = av.x, b[4 * i + 1] = av.y, b[4 * i + 2] = av.z, b[4 * i + 3] = av.w;
            w[4 * i] = wv.x, w[4 * i + 1] = wv.y, w[4 * i + 2] = wv.z, w[4 * i + 3] = wv.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int k = k0 + i;
            const bool in = valid && k < p.K;
            v[i] = in ? MCU_ACT_LOAD(xr + k) : 0.0f;
            b[i] = in && ar != nullptr ? MCU_ACT_LOAD(ar + k) : 0.0f;
            w[i] = in && PRO == GEMV_PRO_ADD_RMSNORM && g.norm_w != nullptr ? MCU_ACT_LOAD(g.norm_w + k) : 0.0f;
        }
    }
    const float inv = PRO == GEMV_PRO_ADD_RMSNORM ? inv_s[t] : 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (PRO == GEMV_PRO_ADD_RMSNORM) {  // same operation order as the stand-alone add + rms_norm kernels
            float y = ar != nullptr ? __fadd_rn(v[i], b[i]) : v[i];
            y = __fmul_rn(y, inv);
            if (g.norm_w != nullptr) y = __fmul_rn(y, __fadd_rn(w[i], g.w_off));
            v[i] = y;
        } else {
            // silu(x) * aux with the fast exponential and division (relative error about 1e-6; the value is quantised
            // to eight bits two lines further on).  The IEEE forms cost 4.6 us per launch at K = 5632, measured.
            v[i] = __fmul_rn(__fdividef(v[i], __fadd_rn(1.0f, __expf(-v[i]))), b[i]);
        }
    }
}

__device__ __forceinline__ bool pro_vec_ok(const ProArgs &p) {
    const GemvPrologue &g = p.pro;
    return ((((uintptr_t)p.x | (uintptr_t)g.aux | (uintptr_t)g.norm_w) & 15) == 0) && (((p.ldx | g.ld_aux | p.K) & 3) == 0);
}

// The packers with a prologue: same lane layout as the plain ones, values transformed between the load and the packing.
template <int LPB, int PRO>
__device__ __noinline__ void quantize_all_q8_k_pro(const ProArgs p, int T, const ActSmem a, int tid, int n_threads,
                                                      const float *inv_s) {
    constexpr int NV = QK_K / LPB;
    const int lane = tid & 31, sl = lane & (LPB - 1);
    const int groups = n_threads / LPB, gid = tid / LPB;
    const int nb = p.nb, tasks = T * nb;
    const bool vec = pro_vec_ok(p);
    for (int base = 0; base < tasks; base += groups) {
        const int task = base + gid;
        const bool valid = task < tasks;
        const int t = valid ? task / nb : 0, blk = valid ? task - t * nb : 0;
        float v[NV];
        load_values_pro<NV, PRO>(p, vec, valid, t, blk * QK_K + NV * sl, inv_s, v);
        pack_values_q8_k<LPB>(v, valid, lane, a.qs + (size_t)t * a.tstride + (size_t)blk * GS_ACT_BLOCK, a.d + t * nb + blk,
                              a.bs32 + ((size_t)t * nb + blk) * 8);
    }
}

// add + RMSNorm + Q8_K packing in ONE trip to the activations, for calls whose (token, block) pairs all fit in one
// round of the thread groups: a group keeps its block's values in registers while the per-token sums of squares meet
// in shared memory (red[task], added up in block order by every thread, so all CTAs get the same bits).
template <int LPB, int NTHREADS>
__device__ __noinline__ void quantize_q8_k_addnorm_once(const ProArgs p, int T, const ActSmem a, int tid, float *red) {
    constexpr int NV = QK_K / LPB;
    const GemvPrologue &g = p.pro;
    const int lane = tid & 31, sl = lane & (LPB - 1);
    const int task = tid / LPB;
    const int nb = p.nb, tasks = T * nb;
    const bool valid = task < tasks;
    const int t = valid ? task / nb : 0, blk = valid ? task - t * nb : 0;
    const int k0 = blk * QK_K + NV * sl;
    const bool vec = pro_vec_ok(p) && (g.x_out == nullptr || ((((uintptr_t)g.x_out & 15) == 0) && ((g.ld_x_out & 3) == 0)));
    const bool write_x = g.x_out != nullptr && blockIdx.x == 0;
    const float *xr = p.x + (size_t)t * p.ldx;
    const float *ar = g.aux != nullptr ? g.aux + (size_t)t * g.ld_aux : nullptr;
    float v[NV], w[NV];
    if (vec) {
#pragma unroll
        for (int i = 0; i < NV / 4; ++i) {
            const int k = k0 + 4 * i;
            const bool in = valid && k < p.K;
            const float4 z = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            float4 xv = in ? MCU_ACT_LOAD((const float4 *)(xr + k)) : z;
            const float4 av = in && ar != nullptr ? MCU_ACT_LOAD((const float4 *)(ar + k)) : z;
            const float4 wv = in && g.norm_w != nullptr ? MCU_ACT_LOAD((const float4 *)(g.norm_w + k)) : z;
            if (ar != nullptr) xv.x = __fadd_rn(xv.x, av.x), xv.y = __fadd_rn(xv.y, av.y), xv.z = __fadd_rn(xv.z, av.z), xv.w = __fadd_rn(xv.w, av.w);
            if (write_x && in) *(float4 *)(g.x_out + (size_t)t * g.ld_x_out + k) = xv;
            v[4 * i] = xv.x, v[4 * i + 1] = xv.y, v[4 * i + 2] = xv.z, v[4 * i + 3] = xv.w;
            w[4 * i] = wv.x, w[4 * i + 1] = wv.y, w[4 * i + 2] = wv.z, w[4 * i + 3] = wv.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int k = k0 + i;
            const bool in = valid && k < p.K;
            float xv = in ? MCU_ACT_LOAD(xr + k) : 0.0f;
            if (in && ar != nullptr) xv = __fadd_rn(xv, MCU_ACT_LOAD(ar + k));
            if (write_x && in) g.x_out[(size_t)t * g.ld_x_out + k] = xv;
            v[i] = xv;
            w[i] = in && g.norm_w != nullptr ? MCU_ACT_LOAD(g.norm_w + k) : 0.0f;
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) ss += v[i] * v[i];
#pragma unroll
    for (int o = LPB / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (sl == 0 && valid) red[task] = ss;
    asm volatile("bar.sync 1, %0;" ::"n"(NTHREADS) : "memory");
    float sum = 0.0f;
    for (int b = 0; b < nb; ++b) sum += red[t * nb + b];
    const float inv = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)p.K), g.eps)))  /* = 1 / sqrt: both correctly rounded */;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        float y = __fmul_rn(v[i], inv);
        if (g.norm_w != nullptr) y = __fmul_rn(y, __fadd_rn(w[i], g.w_off));
        v[i] = y;
    }
    pack_values_q8_k<LPB>(v, valid, lane, a.qs + (size_t)t * a.tstride + (size_t)blk * GS_ACT_BLOCK, a.d + t * nb + blk,
                          a.bs32 + ((size_t)t * nb + blk) * 8);
}

template <int PRO>
__device__ __noinline__ void quantize_all_q8_0_pro(const ProArgs p, int T, const ActSmem a, int tid, int n_threads,
                                                      const float *inv_s) {
    const int sl = tid & 3;
    const int groups = n_threads / 4, gid = tid / 4;
    const int nb = p.nb, tasks = T * nb;
    const bool vec = pro_vec_ok(p);
    for (int base = 0; base < tasks; base += groups) {
        const int task = base + gid;
        const bool valid = task < tasks;
        const int t = valid ? task / nb : 0, blk = valid ? task - t * nb : 0;
        float v[8];
        load_values_pro<8, PRO>(p, vec, valid, t, blk * Q8_0_VALUES + 8 * sl, inv_s, v);
        pack_values_q8_0(v, valid, sl, a.qs + (size_t)t * a.tstride + (size_t)blk * Q8_0_VALUES, a.d + t * nb + blk);
    }
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
// SUBS = 8: each half of the warp works on a row of its own (wrow per lane, `lane` within the half), rows of <= 8 blocks.
template <int T, int SUBS = 16>
__device__ __forceinline__ void row_q4_k(const uint8_t *wrow, const ActSmem &a, int nb, int lane, float (&acc)[T]) {
    const int sub = lane >> 1, h = lane & 1;
    for (int b0 = 0; b0 < nb; b0 += SUBS) {
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

// Q6_K: two lanes per super-block; lane h owns the 128-value half h.  SUBS = 8: each half of the warp works on a row of
// its own (wrow is a per-lane value, `lane` the lane within the half), for rows of at most eight blocks.
template <int T, int SUBS = 16>
__device__ __forceinline__ void row_q6_k(const uint8_t *wrow, const ActSmem &a, int nb, int lane, float (&acc)[T]) {
    const int sub = lane >> 1, h = lane & 1;
    for (int b0 = 0; b0 < nb; b0 += SUBS) {
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

// SUBS = 8: the two halves of a warp work on a row pair each (w0 / w1 are per-lane values, `lane` the lane within the
// half), eight blocks per round -- for rows of at most eight blocks, where sixteen lanes would have nothing to do.
template <int T, int SUBS = 16>
__device__ __forceinline__ void rows2_q4_k(const uint8_t *w0, const uint8_t *w1, const ActSmem &a, int nb, int lane,
                                           float (&mine)[T]) {
    const int sub = lane >> 1, h = lane & 1;
    for (int b0 = 0; b0 < nb; b0 += SUBS) {
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

}  // namespace mcu
