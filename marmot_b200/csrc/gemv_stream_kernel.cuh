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
#pragma once
#include "common.cuh"
#include "kernels.h"

#include <cstdlib>

namespace mcu {

// One weight matrix of a launch: rows [0, F) dealt out to the CTAs [cta_begin, next job's cta_begin).
struct GemvJob {
    const uint8_t *W;
    float *out;
    const float *bias;
    int F, ldo, kind, row_bytes, rows_per_cta, rows_per_chunk, cta_begin;
};

struct GemvStreamParams {
    GemvJob job[GEMV_MAX_JOBS];
    int n_jobs;
    const float *x;
    int *err;
    int ldx, K, nb;
    int act_bytes;     // shared memory reserved for the quantized activations (multiple of 128)
    int stages;        // ring depth, <= GS_MAX_STAGES
    int stage_stride;  // bytes between stage buffers (multiple of 128, includes over-read slack)
    GemvPrologue pro;  // what happens to the activations before they are quantized
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

}  // namespace mcu

#include "gemv_stream_dev.cuh"  // after the stamp macros above, which its packers use in the diagnostic build

namespace mcu {

// ---------------------------------------------------------------------------------------------
// The kernel.  TW consumer warps + one producer warp; the CTAs [job.cta_begin, next job's cta_begin) work on one weight
// matrix of the launch.  A chunk of the ring holds at most TW rows, one per warp.  With one or two tokens (Q4_K, and
// Q8_0 at two) the warps take the chunks in pairs, two rows per warp at a time (see rows2_*); otherwise chunk by chunk.
// MINB = 2 keeps the CTA within half of an SM.  PRO is the launch's activation prologue (p.pro.op): a template
// parameter, because every prologue is tens of kilobytes of code and the kernels are short enough to feel their
// instruction fetches.  KIND is the block format of all the launch's matrices, or KIND_MIXED
// when Q4_K and Q6_K matrices share a launch (the CTA then branches on its job's format).
// ---------------------------------------------------------------------------------------------
template <int KIND, int T, int TW, int TEAMS, int MINB, int PRO>
__global__ void __launch_bounds__((TW * TEAMS + 1) * 32, MINB) gemv_stream_kernel(const GemvStreamParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    static_assert(TEAMS == 1, "one team of consumer warps");
    constexpr bool KQ = KIND != KIND_Q8_0;
    constexpr int NW = TW;
    uint64_t *full = (uint64_t *)smem;
    uint64_t *empty = full + GS_MAX_STAGES;
    int *abort_flag = (int *)(empty + GS_MAX_STAGES);
    float *inv_s = (float *)(smem + GS_RED_OFFSET);
    float *red = inv_s + GEMV_MAX_T;
    uint8_t *act_base = smem + GS_HEADER;
    uint8_t *stage_base = act_base + p.act_bytes;
    const int S = p.stages;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) GS_TRACE_POINT(0);
    if (threadIdx.x == 0) GS_TRACE_CLOCK(9);
    // this CTA's job: selects instead of an indexed read of the parameter block
    GemvJob job = p.job[0];
#pragma unroll
    for (int i = 1; i < GEMV_MAX_JOBS; ++i)
        if (i < p.n_jobs && (int)blockIdx.x >= p.job[i].cta_begin) job = p.job[i];
    const int kind = KIND == KIND_MIXED ? job.kind : KIND;
    // Row pairs pay where a row's fixed part dominates (Q4_K); the 2-byte aligned formats are bound by their 32-bit
    // shared-memory reads, which pairing does not reduce (measured: Q6_K 22 -> 27 us at T = 1, F = 28672).
    const bool pairs = (kind == KIND_Q4_K && T <= 2) || (kind == KIND_Q8_0 && T == 2);
    const uint8_t *W = job.W;
    float *out = job.out;
    const int r0 = ((int)blockIdx.x - job.cta_begin) * job.rows_per_cta;
    const int r1 = min(job.F, r0 + job.rows_per_cta);
    const int n_rows = max(0, r1 - r0);
    const int RC = job.rows_per_chunk;
    const int n_chunks = (n_rows + RC - 1) / RC;

    if (threadIdx.x == 0) {
        for (int i = 0; i < S; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], TW);
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
                const uint32_t bytes = (uint32_t)rows * (uint32_t)job.row_bytes;
                mbar_expect_tx(&full[st], bytes);
                bulk_g2s(stage_base + (size_t)st * p.stage_stride, W + ((size_t)r0 + (size_t)c * RC) * job.row_bytes, bytes,
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
    if constexpr (PRO == GEMV_PRO_NONE) {
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
    } else if constexpr (PRO == GEMV_PRO_ADD_RMSNORM) {
        const ProArgs pa{p.x, p.ldx, p.K, p.nb, p.pro};
        const int tasks = T * p.nb;
        if (KQ && tasks <= NW) {  // every (token, block) pair has a thread group: one trip to the activations
            quantize_q8_k_addnorm_once<32, NW * 32>(pa, T, a, threadIdx.x, red);
        } else if (KQ && tasks <= 2 * NW) {
            quantize_q8_k_addnorm_once<16, NW * 32>(pa, T, a, threadIdx.x, red);
        } else {
            pro_rms_stats<T, NW * 32>(pa, threadIdx.x, red, inv_s);
            if (KQ) quantize_all_q8_k_pro<16, GEMV_PRO_ADD_RMSNORM>(pa, T, a, threadIdx.x, NW * 32, inv_s);
            else quantize_all_q8_0_pro<GEMV_PRO_ADD_RMSNORM>(pa, T, a, threadIdx.x, NW * 32, inv_s);
        }
    } else {
        const ProArgs pa{p.x, p.ldx, p.K, p.nb, p.pro};
        if (KQ) {
            if (T * p.nb * 32 <= NW * 32) quantize_all_q8_k_pro<32, GEMV_PRO_SWIGLU>(pa, T, a, threadIdx.x, NW * 32, inv_s);
            else quantize_all_q8_k_pro<16, GEMV_PRO_SWIGLU>(pa, T, a, threadIdx.x, NW * 32, inv_s);
        } else {
            quantize_all_q8_0_pro<GEMV_PRO_SWIGLU>(pa, T, a, threadIdx.x, NW * 32, inv_s);
        }
    }
    if (threadIdx.x == 0) GS_TRACE_POINT(8);
    GS_TRACE_CLOCK_AT(TRACE_SLOT, 14);
    asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");  // consumer warps only
    GS_TRACE_CLOCK_AT(TRACE_SLOT, 15);
    if (threadIdx.x == 0) GS_TRACE_POINT(3);

    if (pairs) {
        const int tw = warp;
        const int n_pairs = (n_chunks + 1) / 2;
        for (int jp = 0; jp < n_pairs; ++jp) {
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
                const uint8_t *wa = stage_base + (size_t)st0 * p.stage_stride + (size_t)rl0 * job.row_bytes;
                const uint8_t *wb = stage_base + (size_t)st1 * p.stage_stride + (size_t)rl1 * job.row_bytes;
                if (!v0) wa = wb;  // a lone row is computed twice and stored once
                if (!v1) wb = wa;
                float mine[T];
#pragma unroll
                for (int t = 0; t < T; ++t) mine[t] = 0.0f;
                if (kind == KIND_Q4_K) {
                    if constexpr (KIND == KIND_Q4_K || KIND == KIND_MIXED) rows2_q4_k<T>(wa, wb, a, p.nb, lane, mine);
                } else if (kind == KIND_Q6_K) {
                    if constexpr (KIND == KIND_Q6_K) rows2_q6_k<T>(wa, wb, a, p.nb, lane, mine);
                } else {
                    if constexpr (KIND == KIND_Q8_0) rows2_q8_0<T>(wa, wb, a, p.nb, lane, mine);
                }
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
                    if (store) out[(size_t)t * job.ldo + f] = job.bias != nullptr ? __fadd_rn(v, job.bias[f]) : v;
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
                const uint8_t *wrow = sbuf + (size_t)rl * job.row_bytes;
                if (kind == KIND_Q4_K) {
                    if constexpr (KIND == KIND_Q4_K || KIND == KIND_MIXED) row_q4_k<T>(wrow, a, p.nb, lane, acc);
                } else if (kind == KIND_Q6_K) {
                    if constexpr (KIND == KIND_Q6_K || KIND == KIND_MIXED) row_q6_k<T>(wrow, a, p.nb, lane, acc);
                } else {
                    if constexpr (KIND == KIND_Q8_0) row_q8_0<T>(wrow, a, p.nb, lane, acc);
                }
                const int f = r0 + c * RC + rl;
#pragma unroll
                for (int t = 0; t < T; ++t) {
                    const float v = warp_sum(acc[t]);
                    if (lane == 0) out[(size_t)t * job.ldo + f] = job.bias != nullptr ? __fadd_rn(v, job.bias[f]) : v;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);
        }
    }
    if (threadIdx.x == 0) GS_TRACE_POINT(7);
    if (threadIdx.x == 0) GS_TRACE_CLOCK(10);
}

constexpr int NW_SHORT = 14;  // single-token jobs: two CTAs per SM (this launch's and the next one's)
constexpr int NW_LONG = 16;

template <int KIND, int T, int TW, int TEAMS, int MINB, int PRO>
static cudaError_t launch_cfg(const GemvStreamParams &p, int grid_x, int smem_bytes, cudaStream_t s) {
    static int configured = 0;  // largest dynamic shared memory size opted in for this instantiation
    if (smem_bytes > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemv_stream_kernel<KIND, T, TW, TEAMS, MINB, PRO>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return e;
        // all of the SM's shared memory: CTAs of two consecutive launches must fit side by side
        e = cudaFuncSetAttribute(gemv_stream_kernel<KIND, T, TW, TEAMS, MINB, PRO>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        configured = smem_bytes;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid_x, 1, 1);
    cfg.blockDim = dim3((TW * TEAMS + 1) * 32, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const bool no_pdl = getenv("MARMOT_CUDA_NO_PDL") != nullptr;  // diagnostic switch
    cfg.numAttrs = no_pdl ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, gemv_stream_kernel<KIND, T, TW, TEAMS, MINB, PRO>, p);
}

template <int KIND, int PRO>
static cudaError_t launch_k(int T, bool short_cfg, const GemvStreamParams &p, int gx, int smem, cudaStream_t s) {
    if (short_cfg) return launch_cfg<KIND, 1, NW_SHORT, 1, 2, PRO>(p, gx, smem, s);
    switch (T) {
    case 1: return launch_cfg<KIND, 1, NW_LONG, 1, 1, PRO>(p, gx, smem, s);
    case 2: return launch_cfg<KIND, 2, NW_LONG, 1, 1, PRO>(p, gx, smem, s);
    case 3: return launch_cfg<KIND, 3, NW_LONG, 1, 1, PRO>(p, gx, smem, s);
    case 4: return launch_cfg<KIND, 4, NW_LONG, 1, 1, PRO>(p, gx, smem, s);
    case 5: return launch_cfg<KIND, 5, NW_LONG, 1, 1, PRO>(p, gx, smem, s);
    case 6: return launch_cfg<KIND, 6, NW_LONG, 1, 1, PRO>(p, gx, smem, s);
    case 7: return launch_cfg<KIND, 7, NW_LONG, 1, 1, PRO>(p, gx, smem, s);
    default: return launch_cfg<KIND, 8, NW_LONG, 1, 1, PRO>(p, gx, smem, s);
    }
}

// All formats of one prologue: what a translation unit of the kernel family defines (one per prologue, so that they
// compile side by side).
template <int PRO>
static cudaError_t launch_all_kinds(int kind, int T, bool short_cfg, const GemvStreamParams &p, int gx, int smem, cudaStream_t s) {
    if (kind == KIND_Q4_K) return launch_k<KIND_Q4_K, PRO>(T, short_cfg, p, gx, smem, s);
    if (kind == KIND_Q6_K) return launch_k<KIND_Q6_K, PRO>(T, short_cfg, p, gx, smem, s);
    if (kind == KIND_Q8_0) return launch_k<KIND_Q8_0, PRO>(T, short_cfg, p, gx, smem, s);
    return launch_k<KIND_MIXED, PRO>(T, short_cfg, p, gx, smem, s);
}
cudaError_t launch_gemv_stream_plain(int kind, int T, bool short_cfg, const GemvStreamParams &p, int gx, int smem, cudaStream_t s);
cudaError_t launch_gemv_stream_addnorm(int kind, int T, bool short_cfg, const GemvStreamParams &p, int gx, int smem, cudaStream_t s);
cudaError_t launch_gemv_stream_swiglu(int kind, int T, bool short_cfg, const GemvStreamParams &p, int gx, int smem, cudaStream_t s);

}  // namespace mcu
