// One decode step of a Llama-family decoder (one token) as ONE persistent kernel.
//
// The five-launch layer (gemv_stream.cu with prologues, the decode attention of decoder.cu) is bound by what happens at
// every kernel boundary: the weight stream drains, the next kernel's consumers wait for the previous grid to retire,
// then load and pack their activations.  Here the CTAs stay resident for the whole step (cooperative launch, one CTA per
// SM) and walk a table of PHASES -- per layer: q/k/v, attention, o projection, gate/up, down; at the end the output
// projection -- separated by grid-wide barriers on a counter in global memory:
//   * the producer thread of a CTA runs through the CTA's weight chunks of ALL phases in order, limited only by free
//     ring slots, so HBM keeps streaming across the barriers and during the activation packing;
//   * the consumer warps do per phase what the streaming GEMV does per launch (prologue + packing of the activations,
//     row dots on the ring, stores), with the same device functions, hence the same bits;
//   * attention for the single token: one CTA per query head, in f32 on the f16 pool -- RoPE of the query head and of the
//     new K row from the step's table, the new K / V rows appended, every warp a running softmax state over its
//     32-position tiles (scores with one position per lane, P V with head_dim / 32 dimensions per lane), the states
//     merged through shared memory.  Made for the short contexts of single-sequence decoding: with thousands of
//     cached positions a few dozen SMs read the whole cache of a layer, and the five-launch layer is the faster one.
// What the phases cost is latency, not bandwidth, and the kernel is built around that: the phase descriptors travel
// through shared memory one phase ahead (read from global memory at the start of a phase their lines were dependent
// trips to L2), the next phase's norm weights are requested a phase ahead (used once per step, they come from HBM),
// nothing relies on L1 (with ~190 KB of shared memory configured it is a few tens of kilobytes: per-thread stack frames
// and re-read V rows went to L2 every time), gate and up are one gated job so that silu(gate) * up is formed where the
// two dot products meet, and rows of at most eight blocks are taken two pairs per warp.
// Every wait is bounded: a barrier or ring wait that runs out sets the error flag and an abort word that all CTAs
// poll, and the kernel returns.
#define MCU_ACT_LOAD(ptr) __ldcg(ptr)  // activations are written by other CTAs of this same launch
#include "gemv_stream_dev.cuh"

#include "../../include/marmot_cuda.h"

#include <cuda_fp16.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

namespace mcu {

#ifndef DS_TW_N
#define DS_TW_N 15
#endif
constexpr int DS_TW = DS_TW_N;                 // consumer warps
constexpr int DS_AW = DS_TW < 15 ? DS_TW : 15; // of them, the warps that take attention tiles (their states share the activation area)
constexpr int DS_THREADS = (DS_TW + 1) * 32;   // + the producer warp
constexpr int DS_MAX_JOBS = 3;
constexpr int DS_CHUNK_BYTES = 36 * 1024;                        // target size of a ring chunk (one or two rows per consumer warp)
constexpr int DS_STAGE_STRIDE = DS_CHUNK_BYTES + 1024;           // a chunk + over-read slack, multiple of 128
constexpr int DS_STAGES = 4;
constexpr int DS_HALF_NB = 8;                  // rows of at most this many blocks: each half of a warp takes its own (rows2_q4_k<1, 8>, row_q6_k<1, 8>)
constexpr int DS_ACT_BYTES = 20 * 1024;        // packed activations of one token: K up to 17408 values
constexpr int DS_ATTN_EXTRA_BYTES = 20 * 1024; // behind the activation area: with it the attention phase's queries and softmax states
constexpr uint32_t DS_SPIN_LIMIT = 1u << 22;        // polls of the grid barrier before a CTA gives up (seconds)

enum { DS_PHASE_GEMV = 0, DS_PHASE_ATTN = 1 };

// W2 != null: a gated pair (gate = W, up = W2, both Q4_K): the CTA streams its rows of both matrices, chunks
// alternating, a warp takes row r of both in one pass and stores silu(gate . x) * (up . x) -- the activation of the
// down projection, which then needs no prologue.
struct DsJob {
    const uint8_t *W, *W2;
    float *out;
    int F, kind, row_bytes, rows_per_cta, rows_per_chunk, cta_begin;
};
__device__ __forceinline__ int job_chunks(const DsJob &job, int n_rows) {
    const int n_rc = (n_rows + job.rows_per_chunk - 1) / job.rows_per_chunk;
    return job.W2 != nullptr ? 2 * n_rc : n_rc;
}

struct DsPhase {
    int type;
    int n_jobs;
    DsJob job[DS_MAX_JOBS];
    const float *x;  // activations of the token [K]
    int K, nb;
    GemvPrologue pro;
    int layer;       // attention: which layer of the pool
    const void *next_norm_w;  // the next phase's norm weights (used once per step, so they come from HBM): requested now
    int next_norm_bytes;
};

constexpr int DS_PH_WORDS = (int)(sizeof(DsPhase) / 4);
constexpr int DS_PH_STRIDE = (DS_PH_WORDS + 3) / 4 * 4;  // words between the two descriptor slots in shared memory
static_assert(sizeof(DsPhase) % 8 == 0 && DS_PH_WORDS <= DS_TW * 32, "a descriptor is copied by one word per consumer thread");

struct DsParams {
    const DsPhase *phases;
    int n_phases;
    uint32_t *sync;  // [0] arrivals of the grid barrier, [1] abort word (one aligned 8-byte word)
    int *err;
    // attention
    const uint32_t *meta;   // [4]: seq slot, position, kv slot, flags
    const uint32_t *table;  // [seqs][max_blocks]
    const float *q, *k_new, *v_new;
    __half *kv_k, *kv_v;
    const float2 *rope;     // [head_dim / 2] {cos, sin}
    float *att;             // [n_q_heads * head_dim]
    int n_q_heads, n_kv_heads, head_dim, max_blocks, n_layers, block_shift, neox;
    float scale;
    uint32_t spin_limit;         // polls of the grid barrier before a CTA gives up
    int skip_arrive_phase;       // test hook: CTA 1 does not arrive after this phase, so that the others' waits run out (-1: off)
    unsigned long long *stamps;  // nanosecond clock of CTA 0: [n_phases + 1] phase starts and the end, then per phase
                                 // {activations packed (matmul phases), phase work done}; or null
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// One thread per CTA: this CTA has finished a phase (the caller synchronised the CTA, so the release covers every
// warp's stores).
__device__ __forceinline__ void grid_arrive(uint32_t *sync) {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(sync) : "memory");
}
// Bounded wait until every CTA has finished phase `phase`; false on abort.  Arrivals and the abort word sit in one
// aligned 8-byte word, so one load per poll reads both.
__device__ __forceinline__ bool grid_wait(const DsParams &p, int phase) {
    const uint32_t want = (uint32_t)(phase + 1) * gridDim.x;
    for (uint32_t i = 0; i < p.spin_limit; ++i) {
        unsigned long long v;
        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p.sync) : "memory");
        if ((uint32_t)(v >> 32) != 0u) return false;
        if ((uint32_t)v >= want) return true;
    }
    atomicExch(p.err, 31);
    atomicExch(p.sync + 1, 1u);
    return false;
}

// ---------------------------------------------------------------------------------------------
// Attention of the one token for query head qh, by the consumer warps of one CTA.  `sm` overlays the activation area:
// the rotated and scaled query head [HD] (f32), the token's own K (rotated) and V rows as the pool stores them
// [2][HD] (f16), then one softmax state {m, l, acc[HD]} per warp.
//   1. RoPE of the query head and of the new K row; the CTA of a group's first query head also appends the new K and V
//      rows to the pool (the others use their own copy, so no CTA waits for another);
//   2. warp w takes the 32-position tiles w, w + W, ...: one position per lane for the scores (its K row in registers),
//      HD / 32 dimensions per lane for P V (the V rows in registers, sixteen at a time), a running maximum and sum;
//   3. warp 0 merges the warps' states in tile order.
// A single token's attention is a chain of latencies, not a stream: one query head per CTA and one tile per warp keep
// the chain short (K and V are read once per query head of the group, from L2), and nothing counts on L1 -- with
// this much shared memory configured it is a few tens of kilobytes.  Loops stay rolled where they can: every piece of
// code runs once per layer, so its size is part of what the step waits for.
// ---------------------------------------------------------------------------------------------
template <int HD>
__device__ __forceinline__ void attention_head(const DsParams &p, int layer, int qh, float *sm) {
    constexpr int HALF = HD / 2, DPL = HD / 32, NTH = DS_TW * 32, SW = HD + 2;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gsize = p.n_q_heads / p.n_kv_heads, h = qh / gsize;
    float *s_q = sm;
    __half *s_kn = (__half *)(sm + HD), *s_vn = s_kn + HD;
    float *s_state = sm + 2 * HD;
    const uint32_t seq = p.meta[0], new_pos = p.meta[1], kv_slot = p.meta[2], kv_len = new_pos + 1u;
    const size_t bs = (size_t)1 << p.block_shift;
    const size_t s3 = HD, s2 = bs * s3, s1 = (size_t)p.n_kv_heads * s2, s0 = (size_t)p.n_layers * s1;
    const size_t head_off = (size_t)layer * s1 + (size_t)h * s2;

    // ---- 1. rotations: threads [0, HALF) the query pairs, [64, 64 + HALF) the K pairs, [128, 128 + HD) the V values ----
    {
        const bool q_thread = tid < HALF, k_thread = tid >= 64 && tid < 64 + HALF, v_thread = tid >= 128 && tid < 128 + HD;
        const bool writer = qh == h * gsize;  // appends the rows to the pool
        const int i = q_thread ? tid : tid - 64;
        const int e = p.neox ? i : 2 * i, o = p.neox ? i + HALF : 2 * i + 1;
        float xe = 0.0f, xo = 0.0f, vx = 0.0f;
        float2 cs = make_float2(1.0f, 0.0f);
        if (q_thread || k_thread) {  // written by other CTAs in the previous phase
            const float *row = q_thread ? p.q + (size_t)qh * HD : p.k_new + (size_t)h * HD;
            xe = __ldcg(row + e);
            xo = __ldcg(row + o);
            cs = p.rope[i];
        }
        if (v_thread) vx = __ldcg(p.v_new + (size_t)h * HD + (tid - 128));
        const size_t dst = (size_t)(kv_slot >> p.block_shift) * s0 + head_off + (size_t)(kv_slot & (uint32_t)(bs - 1)) * s3;
        float re = __fsub_rn(__fmul_rn(xe, cs.x), __fmul_rn(xo, cs.y)), ro = __fadd_rn(__fmul_rn(xe, cs.y), __fmul_rn(xo, cs.x));
        if (q_thread) {
            if (p.scale != 1.0f) {
                re = __fmul_rn(re, p.scale);
                ro = __fmul_rn(ro, p.scale);
            }
            s_q[e] = re;
            s_q[o] = ro;
        }
        if (k_thread) {
            const __half ke = __float2half_rn(re), ko = __float2half_rn(ro);
            s_kn[e] = ke;
            s_kn[o] = ko;
            if (writer) {
                p.kv_k[dst + e] = ke;
                p.kv_k[dst + o] = ko;
            }
        }
        if (v_thread) {
            const __half vv = __float2half_rn(vx);
            s_vn[tid - 128] = vv;
            if (writer) p.kv_v[dst + (tid - 128)] = vv;
        }
    }
    const int n_tiles = (int)((kv_len + 31u) / 32u);
    auto block_of = [&](int tile) -> uint32_t {  // the pool block of this lane's position in the tile, or none
        const uint32_t pos = (uint32_t)tile * 32u + (uint32_t)lane;
        if (pos < kv_len && (pos >> p.block_shift) < (uint32_t)p.max_blocks) return p.table[(size_t)seq * p.max_blocks + (pos >> p.block_shift)];
        return 0xFFFFFFFFu;
    };
    uint32_t tb_next = warp < DS_AW && warp < n_tiles ? block_of(warp) : 0xFFFFFFFFu;  // in flight across the barrier
    asm volatile("bar.sync 1, %0;" ::"n"(NTH) : "memory");

    // ---- 2. tiles ----
    if (warp < DS_AW) {
        float m_run = -INFINITY, l_run = 0.0f, acc[DPL];
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[d] = 0.0f;
#pragma unroll 1
        for (int tile = warp; tile < n_tiles; tile += DS_AW) {
            const uint32_t k0 = (uint32_t)tile * 32u, pos = k0 + (uint32_t)lane;
            const uint32_t tb = tb_next;
            if (tile + DS_AW < n_tiles) tb_next = block_of(tile + DS_AW);
            const bool live = tb != 0xFFFFFFFFu;
            const size_t row_base = live ? (size_t)tb * s0 + head_off + (size_t)(pos & (uint32_t)(bs - 1)) * s3 : 0;
            const uint32_t live_mask = __ballot_sync(0xffffffffu, live);
            const int new_row = (new_pos >= k0 && new_pos < k0 + 32u) ? (int)(new_pos - k0) : -1;  // taken from shared memory
            constexpr int VR = HD == 64 ? 32 : 16;  // V rows in registers at a time
            uint32_t vraw[VR][DPL / 2];
            auto load_v = [&](int half) {
#pragma unroll
                for (int j = 0; j < VR; ++j) {
                    const int r = VR * half + j;
                    const unsigned long long rb = __shfl_sync(0xffffffffu, (unsigned long long)row_base, r);
#pragma unroll
                    for (int d = 0; d < DPL / 2; ++d) vraw[j][d] = 0u;
                    if (r == new_row) {
#pragma unroll
                        for (int d = 0; d < DPL / 2; ++d) vraw[j][d] = *(const uint32_t *)(s_vn + lane * DPL + 2 * d);
                    } else if ((live_mask >> r) & 1u) {
                        if constexpr (DPL == 2) {
                            vraw[j][0] = *(const uint32_t *)(p.kv_v + rb + lane * 2);
                        } else {
                            const uint2 t = *(const uint2 *)(p.kv_v + rb + lane * 4);
                            vraw[j][0] = t.x, vraw[j][1] = t.y;
                        }
                    }
                }
            };
            float w;
            {
                uint4 kraw[HD / 8];
#pragma unroll
                for (int c = 0; c < HD / 8; ++c) kraw[c] = make_uint4(0u, 0u, 0u, 0u);
                if (lane == new_row) {
#pragma unroll
                    for (int c = 0; c < HD / 8; ++c) kraw[c] = *(const uint4 *)(s_kn + 8 * c);
                } else if (live) {
#pragma unroll
                    for (int c = 0; c < HD / 8; ++c) kraw[c] = *(const uint4 *)(p.kv_k + row_base + 8 * c);
                }
                if constexpr (VR == 32) load_v(0);  // in flight with the K rows where the registers allow
                float sa = 0.0f, sb = 0.0f;
#pragma unroll
                for (int c = 0; c < HD / 8; ++c) {
                    const __half2 *h2 = (const __half2 *)&kraw[c];
                    const float4 qa = *(const float4 *)(s_q + 8 * c), qb = *(const float4 *)(s_q + 8 * c + 4);
                    const float2 k0f = __half22float2(h2[0]), k1f = __half22float2(h2[1]), k2f = __half22float2(h2[2]), k3f = __half22float2(h2[3]);
                    sa += qa.x * k0f.x + qa.y * k0f.y + qa.z * k1f.x + qa.w * k1f.y;
                    sb += qb.x * k2f.x + qb.y * k2f.y + qb.z * k3f.x + qb.w * k3f.y;
                }
                const float sc = sa + sb;
                float m = live ? sc : -INFINITY;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                const float m_new = fmaxf(m_run, m);  // finite: the token's own position is always there... in some tile
                float alpha = 1.0f;
                w = 0.0f;
                if (m_new != -INFINITY) {  // uniform
                    alpha = m_run == -INFINITY ? 0.0f : __expf(m_run - m_new);
                    w = live ? __expf(sc - m_new) : 0.0f;
                }
                float sum = w;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                l_run = l_run * alpha + sum;
#pragma unroll
                for (int d = 0; d < DPL; ++d) acc[d] *= alpha;
                m_run = m_new;
            }
            // O += P V, positions in order
#pragma unroll
            for (int half = 0; half < 32 / VR; ++half) {
                if constexpr (VR != 32) load_v(half);
#pragma unroll
                for (int j = 0; j < VR; ++j) {
                    const float wr = __shfl_sync(0xffffffffu, w, VR * half + j);  // zero for a position that is not there
#pragma unroll
                    for (int d = 0; d < DPL / 2; ++d) {
                        const float2 f = __half22float2(*(const __half2 *)&vraw[j][d]);
                        acc[2 * d] += wr * f.x;
                        acc[2 * d + 1] += wr * f.y;
                    }
                }
            }
        }
        float *st = s_state + (size_t)warp * SW;
        if (lane == 0) {
            st[0] = m_run;
            st[1] = l_run;
        }
#pragma unroll
        for (int d = 0; d < DPL; ++d) st[2 + lane * DPL + d] = acc[d];
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NTH) : "memory");

    // ---- 3. merge, in warp order ----
    if (warp == 0) {
        const int n_used = min(n_tiles, DS_AW);  // the warps that hold a state
        float M = -INFINITY;
        for (int t = 0; t < n_used; ++t) M = fmaxf(M, s_state[(size_t)t * SW]);
        float L = 0.0f, o[DPL];
#pragma unroll
        for (int d = 0; d < DPL; ++d) o[d] = 0.0f;
        if (M != -INFINITY) {
            for (int t = 0; t < n_used; ++t) {
                const float *st = s_state + (size_t)t * SW;
                const float mc = st[0];
                if (mc == -INFINITY) continue;
                const float e = __expf(mc - M);
                L += st[1] * e;
#pragma unroll
                for (int d = 0; d < DPL; ++d) o[d] += st[2 + lane * DPL + d] * e;
            }
        }
#pragma unroll
        for (int d = 0; d < DPL; ++d) p.att[(size_t)qh * HD + lane * DPL + d] = L > 0.0f ? __fdividef(o[d], L) : 0.0f;
    }
}

// ---------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ const DsJob &job_of(const DsPhase &ph, int cta) {
    int j = 0;
    for (int i = 1; i < ph.n_jobs; ++i)
        if (cta >= ph.job[i].cta_begin) j = i;
    return ph.job[j];
}

__global__ void __launch_bounds__(DS_THREADS, 1) decode_step_kernel(const DsParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = (uint64_t *)smem;
    uint64_t *empty = full + GS_MAX_STAGES;
    float *inv_s = (float *)(smem + GS_RED_OFFSET);
    float *red = inv_s + GEMV_MAX_T;
    uint8_t *act_base = smem + GS_HEADER;
    uint8_t *stage_base = act_base + DS_ACT_BYTES + DS_ATTN_EXTRA_BYTES;
    constexpr int S = DS_STAGES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, cta = blockIdx.x;
    (void)inv_s;

    if (threadIdx.x == 0) {
        for (int i = 0; i < S; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], DS_TW);  // every consumer warp releases every chunk
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == DS_TW) {
        // ---------------- producer: the weight chunks of all phases, in order ----------------
        if (lane == 0) {
            int cbase = 0;
            for (int ph_i = 0; ph_i < p.n_phases; ++ph_i) {
                const DsPhase &ph = p.phases[ph_i];
                if (ph.type != DS_PHASE_GEMV) continue;
                const DsJob &job = job_of(ph, cta);
                const int r0 = (cta - job.cta_begin) * job.rows_per_cta;
                const int n_rows = max(0, min(job.F, r0 + job.rows_per_cta) - r0);
                const int RC = job.rows_per_chunk, n_chunks = job_chunks(job, n_rows);
                const bool glu = job.W2 != nullptr;
                for (int c = 0; c < n_chunks; ++c) {
                    const int gc = cbase + c, st = gc % S, round = gc / S;
                    if (round > 0) {  // a free slot; gives up when the consumers have (abort word) or after its own limit
                        bool got = false;
                        for (uint32_t i = 0; i < SPIN_LIMIT && !got; ++i) {
                            got = mbar_try_wait(&empty[st], (uint32_t)((round - 1) & 1));
                            if (!got && (i & 255u) == 255u && *(volatile uint32_t *)(p.sync + 1) != 0u) return;
                        }
                        if (!got) {
                            atomicExch(p.err, 32);
                            atomicExch(p.sync + 1, 1u);
                            return;
                        }
                    }
                    const int k = glu ? c >> 1 : c;  // row chunk
                    const uint8_t *mat = glu && (c & 1) ? job.W2 : job.W;
                    const int rows = min(RC, n_rows - k * RC);
                    const uint32_t bytes = (uint32_t)rows * (uint32_t)job.row_bytes;
                    mbar_expect_tx(&full[st], bytes);
                    bulk_g2s(stage_base + (size_t)st * DS_STAGE_STRIDE, mat + ((size_t)r0 + (size_t)k * RC) * job.row_bytes, bytes, &full[st]);
                }
                cbase += n_chunks;
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    // The phase descriptors come through shared memory, the next one fetched while the current phase runs: read from
    // global memory at the start of a phase, its two or three lines were as many dependent trips to L2 (1.3 us).
    constexpr int NTH = DS_TW * 32;
    uint32_t *s_ph = (uint32_t *)(stage_base + (size_t)DS_STAGES * DS_STAGE_STRIDE);
    if (threadIdx.x < DS_PH_WORDS) s_ph[threadIdx.x] = __ldg((const uint32_t *)p.phases + threadIdx.x);
    asm volatile("bar.sync 1, %0;" ::"n"(NTH) : "memory");
    int cbase = 0;
    bool ok = true;
    for (int ph_i = 0; ph_i < p.n_phases && ok; ++ph_i) {
        const DsPhase &ph = *(const DsPhase *)(s_ph + (ph_i & 1) * DS_PH_STRIDE);
        if (ph_i > 0) {  // the previous phase's results, from every CTA
            if (threadIdx.x == 0) red[0] = grid_wait(p, ph_i - 1) ? 1.0f : 0.0f;
            asm volatile("bar.sync 1, %0;" ::"n"(NTH) : "memory");
            ok = red[0] != 0.0f;
            asm volatile("bar.sync 1, %0;" ::"n"(NTH) : "memory");
            if (!ok) break;
        }
        if (cta == 0 && threadIdx.x == 0 && p.stamps != nullptr) p.stamps[ph_i] = global_ns();
        uint32_t next_word = 0u;  // of the next descriptor; stored at the end of this phase
        const bool fetch_next = ph_i + 1 < p.n_phases && threadIdx.x < DS_PH_WORDS;
        if (fetch_next) next_word = __ldg((const uint32_t *)(p.phases + ph_i + 1) + threadIdx.x);
        if (cta == (ph_i % (int)gridDim.x) && (int)threadIdx.x * 128 < ph.next_norm_bytes)  // one CTA asks, a different one every phase
            asm volatile("prefetch.global.L2 [%0];" ::"l"((const char *)ph.next_norm_w + 128 * threadIdx.x));
        if (ph.type == DS_PHASE_ATTN) {
            if (cta < p.n_q_heads) {  // one CTA per query head; the others go straight to the barrier
                if (p.head_dim == 64) attention_head<64>(p, ph.layer, cta, (float *)act_base);
                else attention_head<128>(p, ph.layer, cta, (float *)act_base);
            }
        } else {
            const DsJob &job = job_of(ph, cta);
            const int kind = job.kind;
            const int r0 = (cta - job.cta_begin) * job.rows_per_cta;
            const int n_rows = max(0, min(job.F, r0 + job.rows_per_cta) - r0);
            const int RC = job.rows_per_chunk, n_chunks = job_chunks(job, n_rows);
            const ActSmem a = act_layout<true>(act_base, 1, ph.nb);
            // the activations, through the phase's prologue
            const ProArgs pa{ph.x, ph.K, ph.K, ph.nb, ph.pro};
            if (ph.pro.op == GEMV_PRO_ADD_RMSNORM) {
                if (ph.nb <= DS_TW) quantize_q8_k_addnorm_once<32, NTH>(pa, 1, a, threadIdx.x, red);
                else quantize_q8_k_addnorm_once<16, NTH>(pa, 1, a, threadIdx.x, red);
            } else if (ph.pro.op == GEMV_PRO_SWIGLU) {
                if (ph.nb <= DS_TW) quantize_all_q8_k_pro<32, GEMV_PRO_SWIGLU>(pa, 1, a, threadIdx.x, NTH, inv_s);
                else quantize_all_q8_k_pro<16, GEMV_PRO_SWIGLU>(pa, 1, a, threadIdx.x, NTH, inv_s);
            } else {
                if (ph.nb <= DS_TW) quantize_all_q8_k<32>(ph.x, ph.K, 1, ph.K, ph.nb, a, threadIdx.x, NTH);
                else quantize_all_q8_k<16>(ph.x, ph.K, 1, ph.K, ph.nb, a, threadIdx.x, NTH);
            }
            asm volatile("bar.sync 1, %0;" ::"n"(NTH) : "memory");
            if (cta == 0 && threadIdx.x == 0 && p.stamps != nullptr) p.stamps[p.n_phases + 1 + 2 * ph_i] = global_ns();
            if (kind == KIND_Q4_K) {
                // Chunks in pairs, a row of each per warp and pass (of a gated pair: the same row of gate and up); with
                // short rows each half of the warp takes such a pair.
                const bool glu = job.W2 != nullptr, halves = ph.nb <= DS_HALF_NB;
                const int half = halves ? lane >> 4 : 0, hl = halves ? lane & 15 : lane;
                // all rows in one pass of the warps: every chunk on its own, a row per (half-)warp, no pairs
                const bool single = !glu && n_rows <= DS_TW * (halves ? 2 : 1);
                for (int c0 = 0; c0 < n_chunks; c0 += single ? 1 : 2) {
                    const int c1 = c0 + 1, jp = c0 >> 1;
                    const bool two = !single && c1 < n_chunks;
                    const int g0 = cbase + c0, g1 = cbase + c1;
                    bool ready = mbar_wait(&full[g0 % S], (uint32_t)((g0 / S) & 1));
                    if (ready && two) ready = mbar_wait(&full[g1 % S], (uint32_t)((g1 / S) & 1));
                    if (!ready) {
                        if (lane == 0) {
                            atomicExch(p.err, 33);
                            atomicExch(p.sync + 1, 1u);
                        }
                        break;  // the abort word is set: every CTA leaves at its next grid wait
                    }
                    const int k0 = glu ? jp : c0, k1 = glu ? jp : c1;  // row chunks held by the two ring chunks
                    const int rows0 = min(RC, n_rows - k0 * RC), rows1 = two ? min(RC, n_rows - k1 * RC) : 0;
                    const int rl0 = (warp - (k0 * RC) % DS_TW + DS_TW) % DS_TW + DS_TW * half;
                    const int rl1 = (warp - (k1 * RC) % DS_TW + DS_TW) % DS_TW + DS_TW * half;
                    const bool v0 = rl0 < rows0, v1 = rl1 < rows1;
                    if (!two && !glu) {
                        // a lone chunk: one row per warp (or half of a warp) instead of a pair made of the row and itself
                        if (__any_sync(0xffffffffu, v0)) {
                            const uint8_t *wrow = stage_base + (size_t)(g0 % S) * DS_STAGE_STRIDE + (size_t)(v0 ? rl0 : 0) * job.row_bytes;
                            float acc[1] = {0.0f};
                            if (halves) row_q4_k<1, 8>(wrow, a, ph.nb, hl, acc);
                            else row_q4_k<1>(wrow, a, ph.nb, hl, acc);
                            float v = acc[0];
                            if (!halves) v += __shfl_xor_sync(0xffffffffu, v, 16);
                            v += __shfl_xor_sync(0xffffffffu, v, 8);
                            v += __shfl_xor_sync(0xffffffffu, v, 4);
                            v += __shfl_xor_sync(0xffffffffu, v, 2);
                            v += __shfl_xor_sync(0xffffffffu, v, 1);
                            if (hl == 0 && v0) job.out[r0 + k0 * RC + rl0] = v;
                        }
                    } else if (__any_sync(0xffffffffu, v0 || v1)) {
                        const uint8_t *base0 = stage_base + (size_t)(g0 % S) * DS_STAGE_STRIDE;
                        const uint8_t *base1 = two ? stage_base + (size_t)(g1 % S) * DS_STAGE_STRIDE : base0;
                        const uint8_t *wa = v0 ? base0 + (size_t)rl0 * job.row_bytes : (v1 ? base1 + (size_t)rl1 * job.row_bytes : base0);
                        const uint8_t *wb = v1 ? base1 + (size_t)rl1 * job.row_bytes : wa;
                        float mine[1] = {0.0f};
                        if (halves) rows2_q4_k<1, 8>(wa, wb, a, ph.nb, hl, mine);
                        else rows2_q4_k<1>(wa, wb, a, ph.nb, hl, mine);
                        float v = mine[0];
                        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
                        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
                        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 8));
                        if (!halves) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 16));
                        const float other = __shfl_down_sync(0xffffffffu, v, 1);  // at lane 0 of a (half) warp: the second row's
                        if (glu) {
                            if (hl == 0 && v0) job.out[r0 + k0 * RC + rl0] = __fmul_rn(__fdividef(v, __fadd_rn(1.0f, __expf(-v))), other);
                        } else {
                            if (hl == 0 && v0) job.out[r0 + k0 * RC + rl0] = v;
                            if (hl == 1 && v1) job.out[r0 + k1 * RC + rl1] = v;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(&empty[g0 % S]);
                        if (two) mbar_arrive(&empty[g1 % S]);
                    }
                }
            } else {
                // Q6_K: a row per warp and chunk; with short rows each half of the warp takes a row
                const bool halves = ph.nb <= DS_HALF_NB;
                const int half = halves ? lane >> 4 : 0, hl = halves ? lane & 15 : lane;
                for (int c = 0; c < n_chunks; ++c) {
                    const int gc = cbase + c, st = gc % S;
                    if (!mbar_wait(&full[st], (uint32_t)((gc / S) & 1))) {
                        if (lane == 0) {
                            atomicExch(p.err, 33);
                            atomicExch(p.sync + 1, 1u);
                        }
                        break;
                    }
                    const int rows = min(RC, n_rows - c * RC);
                    const int rl = (warp - (c * RC) % DS_TW + DS_TW) % DS_TW + DS_TW * half;
                    const bool valid = rl < rows;
                    if (__any_sync(0xffffffffu, valid)) {
                        const uint8_t *wrow = stage_base + (size_t)st * DS_STAGE_STRIDE + (size_t)(valid ? rl : 0) * job.row_bytes;
                        float acc[1] = {0.0f};
                        if (halves) row_q6_k<1, 8>(wrow, a, ph.nb, hl, acc);
                        else row_q6_k<1>(wrow, a, ph.nb, hl, acc);
                        float v = acc[0];  // the order of warp_sum (with halves, its first step would add zeros)
                        if (!halves) v += __shfl_xor_sync(0xffffffffu, v, 16);
                        v += __shfl_xor_sync(0xffffffffu, v, 8);
                        v += __shfl_xor_sync(0xffffffffu, v, 4);
                        v += __shfl_xor_sync(0xffffffffu, v, 2);
                        v += __shfl_xor_sync(0xffffffffu, v, 1);
                        if (hl == 0 && valid) job.out[r0 + c * RC + rl] = v;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[st]);
                }
            }
            cbase += n_chunks;
        }
        if (fetch_next) s_ph[((ph_i + 1) & 1) * DS_PH_STRIDE + threadIdx.x] = next_word;  // last read two phases ago
        // this CTA is through the phase; a warp that gave up has set the abort word, which every CTA reads in its next wait
        asm volatile("bar.sync 1, %0;" ::"n"(NTH) : "memory");
        if (cta == 0 && threadIdx.x == 0 && p.stamps != nullptr) p.stamps[p.n_phases + 2 + 2 * ph_i] = global_ns();
        if (threadIdx.x == 0 && !(ph_i == p.skip_arrive_phase && cta == 1)) grid_arrive(p.sync);
    }
    // the end of the step on CTA 0's clock (the counter is zeroed by the host before every launch)
    if (threadIdx.x == 0 && cta == 0 && ok && p.stamps != nullptr && grid_wait(p, p.n_phases - 1)) p.stamps[p.n_phases] = global_ns();
}

}  // namespace mcu

// ---------------------------------------------------------------------------------------------
// Host side: the plan (phase table on the device) and its launch
// ---------------------------------------------------------------------------------------------
using namespace mcu;

struct mcu_decode_plan {
    mcu_context_t *ctx = nullptr;
    DsParams params{};
    DsPhase *phases_dev = nullptr;
    uint32_t *sync_dev = nullptr;
    unsigned long long *stamps_dev = nullptr;
    int grid = 0, smem = 0;
};

#define DS_CUDA(expr)                                                                   \
    do {                                                                                \
        cudaError_t e__ = (expr);                                                       \
        if (e__ != cudaSuccess) {                                                       \
            char msg__[256];                                                            \
            snprintf(msg__, sizeof(msg__), "%s: %s", #expr, cudaGetErrorString(e__));   \
            return set_error(MCU_ERROR_INVALID_OPERATION, msg__);                       \
        }                                                                               \
    } while (0)

static int ds_gcd(int a, int b) { return b == 0 ? a : ds_gcd(b, a % b); }

// One matmul phase: the CTAs dealt to its jobs in proportion to their bytes, chunk sizes chosen for the ring.
static int ds_gemv_phase(DsPhase &ph, int sms, const float *x, int K, const GemvPrologue &pro, int n_jobs, const int *kinds,
                         const void *const *W, const int *F, float *const *out, const void *const *W2 = nullptr) {
    ph = DsPhase{};
    ph.type = DS_PHASE_GEMV;
    ph.n_jobs = n_jobs;
    ph.x = x;
    ph.K = K;
    ph.nb = (K + QK_K - 1) / QK_K;
    ph.pro = pro;
    if (act_smem_bytes(true, 1, ph.nb) > DS_ACT_BYTES) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "decode plan: rows too long");
    if (pro.op == GEMV_PRO_ADD_RMSNORM && ph.nb > 2 * DS_TW) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "decode plan: hidden size too large");
    double bytes[DS_MAX_JOBS], total = 0.0;
    int unit[DS_MAX_JOBS], rb[DS_MAX_JOBS];
    for (int j = 0; j < n_jobs; ++j) {
        if (kinds[j] != KIND_Q4_K && kinds[j] != KIND_Q6_K) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "decode plan: Q4_K / Q6_K weights only");
        if (((uintptr_t)W[j] & 15) || F[j] < 1) return set_error(MCU_ERROR_INVALID_ARGUMENT, "decode plan: weights must be 16-byte aligned");
        rb[j] = ph.nb * block_bytes(kinds[j]);
        unit[j] = 16 / ds_gcd(rb[j] % 16, 16);
        if (((long)F[j] * rb[j]) & 15) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "decode plan: weight matrix is not a whole number of 16-byte pieces");
        if ((long)unit[j] * rb[j] > DS_CHUNK_BYTES || unit[j] > DS_TW) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "decode plan: rows too long for the ring");
        const bool glu = W2 != nullptr && W2[j] != nullptr;
        if (glu && (kinds[j] != KIND_Q4_K || ((uintptr_t)W2[j] & 15))) return set_error(MCU_ERROR_INVALID_ARGUMENT, "decode plan: a gated pair is two aligned Q4_K matrices");
        bytes[j] = (double)F[j] * rb[j] * (glu ? 2.0 : 1.0);
        total += bytes[j];
    }
    if (sms < n_jobs) return set_error(MCU_ERROR_INVALID_OPERATION, "decode plan: fewer SMs than weight matrices");
    int ctas[DS_MAX_JOBS], given = 0;
    for (int j = 0; j < n_jobs; ++j) {
        ctas[j] = (int)((double)sms * bytes[j] / total);
        if (ctas[j] < 1) ctas[j] = 1;
        given += ctas[j];
    }
    while (given != sms) {  // hand out what rounding left (or take back), largest share per CTA first
        int best = -1;
        double best_v = 0.0;
        for (int j = 0; j < n_jobs; ++j) {
            if (given > sms && ctas[j] <= 1) continue;
            const double per = bytes[j] / ctas[j], v = given < sms ? per : -per;
            if (best < 0 || v > best_v) best = j, best_v = v;
        }
        if (best < 0) return set_error(MCU_ERROR_INVALID_OPERATION, "decode plan: cannot deal the CTAs");
        ctas[best] += given < sms ? 1 : -1;
        given += given < sms ? 1 : -1;
    }
    int begin = 0;
    for (int j = 0; j < n_jobs; ++j) {
        DsJob &g = ph.job[j];
        g.W = (const uint8_t *)W[j];
        g.W2 = W2 != nullptr ? (const uint8_t *)W2[j] : nullptr;
        g.out = out[j];
        g.F = F[j];
        g.kind = kinds[j];
        g.row_bytes = rb[j];
        int rpc = (F[j] + ctas[j] - 1) / ctas[j];
        g.rows_per_cta = (rpc + unit[j] - 1) / unit[j] * unit[j];
        int rc = DS_CHUNK_BYTES / rb[j];
        const int cap = ph.nb <= DS_HALF_NB ? 2 * DS_TW : DS_TW;  // rows a pass of the warps takes
        if (rc > cap) rc = cap;
        rc = rc / unit[j] * unit[j];
        g.rows_per_chunk = rc;
        g.cta_begin = begin;
        begin += ctas[j];  // every CTA of the grid belongs to a job, also those whose row range is empty
    }
    return MCU_SUCCESS;
}

extern "C" {

int mcu_decode_plan_create(mcu_context_t *ctx, const mcu_decode_plan_desc_t *d, mcu_decode_plan_t **out) {
    if (out == nullptr) return set_error(MCU_ERROR_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    if (ctx == nullptr) return set_error(MCU_ERROR_DEVICE_NOT_AVAILABLE, "CUDA context is not initialised");
    if (d == nullptr || d->layers == nullptr || d->n_layers == 0) return set_error(MCU_ERROR_INVALID_ARGUMENT, "decode plan: empty description");
    const void *ptrs[] = {d->x0, d->x1, d->q, d->k, d->v, d->att, d->proj, d->gate, d->up, d->logits, d->token_meta, d->block_table,
                          d->kv_k, d->kv_v, d->rope_table, d->out_norm, d->output};
    for (const void *p : ptrs)
        if (p == nullptr) return set_error(MCU_ERROR_INVALID_ARGUMENT, "decode plan: a buffer is missing");
    if (d->head_dim != 64 && d->head_dim != 128) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "decode plan: head_dim 64 or 128");
    if (d->n_kv_heads == 0 || d->n_q_heads % d->n_kv_heads != 0 || d->n_q_heads / d->n_kv_heads > 8)
        return set_error(MCU_ERROR_NOT_IMPLEMENTED, "decode plan: up to 8 query heads per KV head");
    if (d->kv_dtype != MCU_KV_F16) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "decode plan: float16 KV pool");
    if (d->block_size == 0 || (d->block_size & (d->block_size - 1)) != 0) return set_error(MCU_ERROR_INVALID_ARGUMENT, "decode plan: block_size must be a power of two");
    if (d->n_q_heads * d->head_dim != d->d || d->ffn == 0) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "decode plan: heads * head_dim must equal the hidden size");
    if (((uintptr_t)d->kv_k | (uintptr_t)d->kv_v | (uintptr_t)d->rope_table) & 15) return set_error(MCU_ERROR_INVALID_ARGUMENT, "decode plan: pools and RoPE table must be 16-byte aligned");
    DS_CUDA(cudaSetDevice(context_device(ctx)));
    const int sms = device_sm_count();
    if ((int)d->n_q_heads > sms) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "decode plan: more query heads than SMs");
    const int L = (int)d->n_layers, D = (int)d->d, FF = (int)d->ffn, HKV = (int)(d->n_kv_heads * d->head_dim);
    std::vector<DsPhase> phases;
    phases.reserve(5 * (size_t)L + 1);
    float *xs[2] = {d->x0, d->x1};
    int cur = 0;
    const float *pending = nullptr;
    auto add_norm = [&](const float *norm_w, bool store) {
        GemvPrologue g;
        g.op = GEMV_PRO_ADD_RMSNORM;
        g.aux = pending;
        g.ld_aux = D;
        g.norm_w = norm_w;
        g.eps = d->rms_eps;
        g.w_off = 0.0f;
        g.x_out = store && pending != nullptr ? xs[1 - cur] : nullptr;
        g.ld_x_out = D;
        return g;
    };
    for (int i = 0; i < L; ++i) {
        const mcu_decode_layer_t &lw = d->layers[i];
        {
            DsPhase ph;
            const int kinds[3] = {lw.kind_q, lw.kind_k, lw.kind_v};
            const void *W[3] = {lw.wq, lw.wk, lw.wv};
            const int F[3] = {D, HKV, HKV};
            float *o[3] = {d->q, d->k, d->v};
            const GemvPrologue g = add_norm(lw.attn_norm, true);
            if (int rc = ds_gemv_phase(ph, sms, xs[cur], D, g, 3, kinds, W, F, o)) return rc;
            phases.push_back(ph);
            if (pending != nullptr) cur = 1 - cur;
        }
        {
            DsPhase ph{};
            ph.type = DS_PHASE_ATTN;
            ph.layer = i;
            phases.push_back(ph);
        }
        {
            DsPhase ph;
            const int kinds[1] = {lw.kind_o};
            const void *W[1] = {lw.wo};
            const int F[1] = {D};
            float *o[1] = {d->proj};
            if (int rc = ds_gemv_phase(ph, sms, d->att, D, GemvPrologue{}, 1, kinds, W, F, o)) return rc;
            phases.push_back(ph);
            pending = d->proj;
        }
        const bool gated = lw.kind_gate == KIND_Q4_K && lw.kind_up == KIND_Q4_K;  // silu(gate) * up formed where the rows are
        if (gated) {
            DsPhase ph;
            const int kinds[1] = {KIND_Q4_K};
            const void *W[1] = {lw.gate}, *W2[1] = {lw.up};
            const int F[1] = {FF};
            float *o[1] = {d->gate};
            const GemvPrologue g = add_norm(lw.ffn_norm, true);
            if (int rc = ds_gemv_phase(ph, sms, xs[cur], D, g, 1, kinds, W, F, o, W2)) return rc;
            phases.push_back(ph);
            cur = 1 - cur;
        } else {
            DsPhase ph;
            const int kinds[2] = {lw.kind_gate, lw.kind_up};
            const void *W[2] = {lw.gate, lw.up};
            const int F[2] = {FF, FF};
            float *o[2] = {d->gate, d->up};
            const GemvPrologue g = add_norm(lw.ffn_norm, true);
            if (int rc = ds_gemv_phase(ph, sms, xs[cur], D, g, 2, kinds, W, F, o)) return rc;
            phases.push_back(ph);
            cur = 1 - cur;
        }
        {
            DsPhase ph;
            const int kinds[1] = {lw.kind_down};
            const void *W[1] = {lw.down};
            const int F[1] = {D};
            float *o[1] = {d->proj};
            GemvPrologue g;
            if (!gated) {
                g.op = GEMV_PRO_SWIGLU;
                g.aux = d->up;
                g.ld_aux = FF;
            }
            if (int rc = ds_gemv_phase(ph, sms, d->gate, FF, g, 1, kinds, W, F, o)) return rc;
            phases.push_back(ph);
            pending = d->proj;
        }
    }
    {
        DsPhase ph;
        const int kinds[1] = {d->kind_output};
        const void *W[1] = {d->output};
        const int F[1] = {(int)d->vocab};
        float *o[1] = {d->logits};
        const GemvPrologue g = add_norm(d->out_norm, false);
        if (int rc = ds_gemv_phase(ph, sms, xs[cur], D, g, 1, kinds, W, F, o)) return rc;
        phases.push_back(ph);
    }
    for (size_t i = 0; i + 1 < phases.size(); ++i) {
        const DsPhase &nx = phases[i + 1];
        if (nx.type == DS_PHASE_GEMV && nx.pro.op == GEMV_PRO_ADD_RMSNORM && nx.pro.norm_w != nullptr) {
            phases[i].next_norm_w = nx.pro.norm_w;
            phases[i].next_norm_bytes = nx.K * (int)sizeof(float);
        }
    }
    mcu_decode_plan *pl = new (std::nothrow) mcu_decode_plan;
    if (pl == nullptr) return set_error(MCU_ERROR_OUT_OF_MEMORY, "decode plan allocation failed");
    pl->ctx = ctx;
    pl->grid = sms;
    pl->smem = GS_HEADER + DS_ACT_BYTES + DS_ATTN_EXTRA_BYTES + DS_STAGES * DS_STAGE_STRIDE + 2 * DS_PH_STRIDE * (int)sizeof(uint32_t);
    const size_t sync_words = 2;
    cudaError_t e = cudaMalloc((void **)&pl->phases_dev, phases.size() * sizeof(DsPhase));
    if (e == cudaSuccess) e = cudaMalloc((void **)&pl->sync_dev, sync_words * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMalloc((void **)&pl->stamps_dev, (3 * phases.size() + 1) * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMemset(pl->stamps_dev, 0, (3 * phases.size() + 1) * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMemcpy(pl->phases_dev, phases.data(), phases.size() * sizeof(DsPhase), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemset(pl->sync_dev, 0, sync_words * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pl->smem);
    int per_sm = 0;
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel, DS_THREADS, pl->smem);
    if (e != cudaSuccess || per_sm < 1) {
        const int rc = set_error(MCU_ERROR_INVALID_OPERATION, e != cudaSuccess ? cudaGetErrorString(e) : "decode step kernel does not fit an SM");
        mcu_decode_plan_destroy(pl);
        return rc;
    }
    DsParams &p = pl->params;
    p.phases = pl->phases_dev;
    p.n_phases = (int)phases.size();
    p.sync = pl->sync_dev;
    p.err = context_err_flag(ctx);
    p.meta = d->token_meta;
    p.table = d->block_table;
    p.q = d->q;
    p.k_new = d->k;
    p.v_new = d->v;
    p.kv_k = (__half *)d->kv_k;
    p.kv_v = (__half *)d->kv_v;
    p.rope = (const float2 *)d->rope_table;
    p.att = d->att;
    p.n_q_heads = (int)d->n_q_heads;
    p.n_kv_heads = (int)d->n_kv_heads;
    p.head_dim = (int)d->head_dim;
    p.max_blocks = (int)d->max_blocks_per_seq;
    p.n_layers = (int)d->n_layers;
    p.block_shift = 0;
    while (((size_t)1 << p.block_shift) < d->block_size) ++p.block_shift;
    p.neox = d->rope_type == MCU_ROPE_NEOX ? 1 : 0;
    p.scale = d->attn_scale;
    p.stamps = pl->stamps_dev;
    // Test hooks (host-side fault injection: no kernel traps or spins without a bound): a short barrier limit, and one
    // CTA that skips one arrival so that the other CTAs' waits run out and the step ends with the error flag set.
    const char *lim = getenv("MARMOT_DECODE_PLAN_SPIN_LIMIT"), *skip = getenv("MARMOT_DECODE_PLAN_TEST_SKIP_ARRIVE");
    p.spin_limit = lim != nullptr && atoi(lim) > 0 ? (uint32_t)atoi(lim) : DS_SPIN_LIMIT;
    p.skip_arrive_phase = skip != nullptr ? atoi(skip) : -1;
    *out = pl;
    return MCU_SUCCESS;
}

int mcu_decode_plan_run(mcu_decode_plan_t *pl) {
    if (pl == nullptr) return set_error(MCU_ERROR_INVALID_ARGUMENT, "null plan");
    DS_CUDA(cudaSetDevice(context_device(pl->ctx)));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)pl->grid, 1, 1);
    cfg.blockDim = dim3(DS_THREADS, 1, 1);
    cfg.dynamicSmemBytes = (size_t)pl->smem;
    cfg.stream = (cudaStream_t)mcu_context_get_stream(pl->ctx);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident at once: they wait on one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // arrivals and abort word start from zero, also after a step that gave up
    DS_CUDA(cudaMemsetAsync(pl->sync_dev, 0, 2 * sizeof(uint32_t), cfg.stream));
    DS_CUDA(cudaLaunchKernelEx(&cfg, decode_step_kernel, pl->params));
    count_launches(1);
    return MCU_SUCCESS;
}

int mcu_decode_plan_phase_times(mcu_decode_plan_t *pl, unsigned long long *out, size_t capacity, size_t *n_out) {
    if (pl == nullptr || n_out == nullptr) return set_error(MCU_ERROR_INVALID_ARGUMENT, "null plan");
    const size_t n = 3 * (size_t)pl->params.n_phases + 1;
    *n_out = n;
    if (out == nullptr || capacity < n) return MCU_SUCCESS;  // the count alone
    DS_CUDA(cudaSetDevice(context_device(pl->ctx)));
    DS_CUDA(cudaStreamSynchronize((cudaStream_t)mcu_context_get_stream(pl->ctx)));
    DS_CUDA(cudaMemcpy(out, pl->stamps_dev, n * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    return MCU_SUCCESS;
}

void mcu_decode_plan_destroy(mcu_decode_plan_t *pl) {
    if (pl == nullptr) return;
    cudaSetDevice(context_device(pl->ctx));
    cudaStreamSynchronize((cudaStream_t)mcu_context_get_stream(pl->ctx));
    if (pl->phases_dev != nullptr) cudaFree(pl->phases_dev);
    if (pl->sync_dev != nullptr) cudaFree(pl->sync_dev);
    if (pl->stamps_dev != nullptr) cudaFree(pl->stamps_dev);
    delete pl;
}

}  // extern "C"
