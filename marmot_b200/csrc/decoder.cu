// Decoder operators around the quantized matmuls, f32 activations: RMSNorm (optional fused residual), RoPE, SwiGLU,
// add, paged attention with in-call KV append, quantized embedding gather, argmax.  Floating-point kernels: the
// results follow the reference CPU operators' formulas; sums that the reference accumulates sequentially are
// accumulated in parallel here (tolerances in the tests).
//   RMSNorm          src/backends/cpu/ops/normalization/scalar/normalization_scalar.c:780-791
//   RoPE             src/backends/cpu/ops/rope/rope_dispatch.c:343-375, frequencies src/core/helpers/rope.c:108-120
//   SwiGLU           src/backends/cpu/ops/elementwise/scalar/elementwise_f32_scalar.c:11-13,178
//   paged attention  src/backends/cpu/ops/paged_attention/paged_attention_ref.c:327-350 (KV append), :397-556
#include "../../include/marmot_cuda.h"

#include "common.cuh"
#include "kernels.h"

#include <climits>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cuda_fp16.h>

namespace mcu {

// Every kernel of this file is launched with programmatic stream serialization and starts by waiting for the
// kernel ahead of it (so nothing is read or written early), then lets the kernel behind it start its own launch:
// the launch latencies of a chain of small kernels overlap instead of adding up.
#define MCU_PDL_PROLOGUE()                                        \
    asm volatile("griddepcontrol.wait;" ::: "memory");            \
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory")

template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl_smem(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                   Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const bool no_pdl = getenv("MARMOT_CUDA_NO_PDL") != nullptr;  // diagnostic switch
    cfg.numAttrs = no_pdl ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t s, Args... args) {
    return launch_pdl_smem(kernel, grid, block, 0, s, args...);
}

// ---------------------------------------------------------------- RMSNorm
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ residual, const float *__restrict__ weight, int n,
               float eps, float weight_offset, float *__restrict__ out) {
    MCU_PDL_PROLOGUE();
    __shared__ float red[8];
    __shared__ float inv_s;
    const size_t row = blockIdx.x;
    const float *xr = x + row * n;
    const float *rr = residual != nullptr ? residual + row * n : nullptr;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = rr != nullptr ? __fadd_rn(xr[i], rr[i]) : xr[i];
        sum += v * v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        for (int i = 0; i < 8; ++i) s += red[i];
        inv_s = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(s, (float)n), eps)));
    }
    __syncthreads();
    const float inv = inv_s;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = rr != nullptr ? __fadd_rn(xr[i], rr[i]) : xr[i];
        float y = __fmul_rn(v, inv);
        if (weight != nullptr) y = __fmul_rn(y, __fadd_rn(weight[i], weight_offset));
        out[row * n + i] = y;
    }
}

// x_out = x + delta (the residual update), h_out = RMSNorm(x_out) * weight: the add and the rms_norm that follow every
// row-parallel projection, in one pass over the row.  x_out may alias x.
__global__ void __launch_bounds__(256)
add_rmsnorm_kernel(const float *x, const float *__restrict__ delta, const float *__restrict__ weight, int n, float eps,
                   float weight_offset, float *x_out, float *__restrict__ h_out) {
    MCU_PDL_PROLOGUE();
    __shared__ float red[8];
    __shared__ float inv_s;
    const size_t row = blockIdx.x;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = __fadd_rn(x[row * n + i], delta[row * n + i]);
        x_out[row * n + i] = v;
        sum += v * v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        for (int i = 0; i < 8; ++i) s += red[i];
        inv_s = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(s, (float)n), eps)));
    }
    __syncthreads();
    const float inv = inv_s;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float y = __fmul_rn(x_out[row * n + i], inv);  // this thread wrote that element above
        if (weight != nullptr) y = __fmul_rn(y, __fadd_rn(weight[i], weight_offset));
        h_out[row * n + i] = y;
    }
}

// ---------------------------------------------------------------- RoPE
constexpr int ROPE_MAX_PAIRS = 128;
struct RopeFreqs {
    float f[ROPE_MAX_PAIRS];  // computed on the host with the reference's formula (powf of the same libm)
};

// x [T][n_heads][head_dim] with row stride ldx; one position per token.
__global__ void rope_kernel(const float *__restrict__ x, size_t ldx, const int32_t *__restrict__ positions, int n_heads,
                            int head_dim, int neox, RopeFreqs freqs, float *__restrict__ out, size_t ldo) {
    MCU_PDL_PROLOGUE();
    const int t = blockIdx.x;
    const int half = head_dim >> 1;
    const float pos = (float)positions[t];
    for (int idx = threadIdx.x; idx < n_heads * half; idx += blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        float s, c;
        sincosf(__fmul_rn(pos, freqs.f[i]), &s, &c);
        const int e = neox ? i : 2 * i, o = neox ? i + half : 2 * i + 1;
        const float *xr = x + (size_t)t * ldx + (size_t)h * head_dim;
        float *yr = out + (size_t)t * ldo + (size_t)h * head_dim;
        const float xe = xr[e], xo = xr[o];
        yr[e] = __fsub_rn(__fmul_rn(xe, c), __fmul_rn(xo, s));
        yr[o] = __fadd_rn(__fmul_rn(xe, s), __fmul_rn(xo, c));
    }
}

// The same for the query and key projections of a token in one launch, in place.
__global__ void rope_qk_kernel(float *__restrict__ q, size_t ldq, int n_q_heads, float *__restrict__ k, size_t ldk,
                               int n_k_heads, const int32_t *__restrict__ positions, int head_dim, int neox,
                               RopeFreqs freqs) {
    MCU_PDL_PROLOGUE();
    const int t = blockIdx.x;
    const int half = head_dim >> 1;
    const float pos = (float)positions[t];
    for (int idx = threadIdx.x; idx < (n_q_heads + n_k_heads) * half; idx += blockDim.x) {
        const int hh = idx / half, i = idx - hh * half;
        float s, c;
        sincosf(__fmul_rn(pos, freqs.f[i]), &s, &c);
        const int e = neox ? i : 2 * i, o = neox ? i + half : 2 * i + 1;
        float *row = hh < n_q_heads ? q + (size_t)t * ldq + (size_t)hh * head_dim
                                    : k + (size_t)t * ldk + (size_t)(hh - n_q_heads) * head_dim;
        const float xe = row[e], xo = row[o];
        row[e] = __fsub_rn(__fmul_rn(xe, c), __fmul_rn(xo, s));
        row[o] = __fadd_rn(__fmul_rn(xe, s), __fmul_rn(xo, c));
    }
}

// {cos, sin} of position * frequency for every token and pair, once per decode step: the fused attention kernel of
// every layer rotates q and the new k with these (the same sincosf of the same product as rope_kernel).
__global__ void rope_table_kernel(const int32_t *__restrict__ positions, int half, RopeFreqs freqs, float2 *__restrict__ table) {
    MCU_PDL_PROLOGUE();
    const int t = blockIdx.x;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf(__fmul_rn(pos, freqs.f[i]), &s, &c);
        table[(size_t)t * half + i] = make_float2(c, s);
    }
}

// ---------------------------------------------------------------- elementwise
__global__ void swiglu_kernel(const float *__restrict__ a, const float *__restrict__ b, size_t n, float *__restrict__ out) {
    MCU_PDL_PROLOGUE();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __fmul_rn(__fdiv_rn(a[i], __fadd_rn(1.0f, expf(-a[i]))), b[i]);
}
__global__ void add_kernel(const float *__restrict__ a, const float *__restrict__ b, size_t n, float *__restrict__ out) {
    MCU_PDL_PROLOGUE();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __fadd_rn(a[i], b[i]);
}

// argmax over the last axis, first maximum wins.  grid (rows, slices): each CTA scans one slice of the row; with
// several slices the CTAs leave their candidates in `cand` and the one that draws the row's last ticket picks the
// winner (slices in ascending order, strict >, so the first maximum still wins) and puts the ticket back to zero.
struct ArgmaxCand {
    float v;
    int i;
};
__global__ void __launch_bounds__(256) argmax_kernel(const float *__restrict__ x, int n, int slice, ArgmaxCand *cand, int *tickets,
                                                     int32_t *__restrict__ out) {
    MCU_PDL_PROLOGUE();
    __shared__ float bv[8];
    __shared__ int bi[8];
    const int row = blockIdx.x, sp = blockIdx.y, nsp = gridDim.y;
    const float *xr = x + (size_t)row * n;
    const int lo = sp * slice, hi = min(n, lo + slice);
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {  // ascending i per thread: strict > keeps the first maximum
        const float v = xr[i];
        if (v > best || idx == 0x7fffffff) {
            best = v;
            idx = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (oi != 0x7fffffff && (idx == 0x7fffffff || ov > best || (ov == best && oi < idx))) {
            best = ov;
            idx = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        bv[threadIdx.x >> 5] = best;
        bi[threadIdx.x >> 5] = idx;
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    for (int w = 1; w < 8; ++w)
        if (bi[w] != 0x7fffffff && (bi[0] == 0x7fffffff || bv[w] > bv[0] || (bv[w] == bv[0] && bi[w] < bi[0]))) {
            bv[0] = bv[w];
            bi[0] = bi[w];
        }
    if (nsp == 1) {
        out[row] = bi[0] == 0x7fffffff ? 0 : bi[0];
        return;
    }
    ArgmaxCand *mine = cand + (size_t)row * nsp;
    mine[sp].v = bv[0];
    mine[sp].i = bi[0];
    __threadfence();
    const int drawn = atomicAdd(tickets + row, 1);
    if (drawn != nsp - 1) return;
    tickets[row] = 0;
    __threadfence();
    float wv = -INFINITY;
    int wi = 0x7fffffff;
    for (int c = 0; c < nsp; ++c) {
        const float v = __ldcg(&mine[c].v);
        const int i = __ldcg(&mine[c].i);
        if (i != 0x7fffffff && (wi == 0x7fffffff || v > wv)) {
            wv = v;
            wi = i;
        }
    }
    out[row] = wi == 0x7fffffff ? 0 : wi;
}

// ---------------------------------------------------------------- paged attention
struct PagedParams {
    const uint32_t *meta;   // [T][4]: seq_slot, pos, kv_slot, flags
    const uint32_t *table;  // [seqs][max_blocks]
    const float *q, *k_new, *v_new;
    void *kv_k, *kv_v;      // [blocks][layers][kv_heads][block_size][head_dim]
    float *out;
    int n_q_heads, n_kv_heads, max_blocks, n_layers, layer, block_shift;
    float scale;
};

__device__ __forceinline__ float kv_load(const float *p) { return *p; }
__device__ __forceinline__ float kv_load(const __half *p) { return __half2float(*p); }
__device__ __forceinline__ void kv_store(float *p, float v) { *p = v; }
__device__ __forceinline__ void kv_store(__half *p, float v) { *p = __float2half_rn(v); }

// K/V rows of the new tokens into the pool (f16 pools: round to nearest even, as the reference's NEON / F16C
// conversions).  grid (T, kv_heads), threads over head_dim.
template <typename KV>
__global__ void kv_append_kernel(PagedParams p, int head_dim) {
    MCU_PDL_PROLOGUE();
    const int t = blockIdx.x, h = blockIdx.y;
    const uint32_t kv_slot = p.meta[t * 4 + 2];
    const size_t bs = (size_t)1 << p.block_shift;
    const size_t s3 = head_dim, s2 = bs * s3, s1 = (size_t)p.n_kv_heads * s2, s0 = (size_t)p.n_layers * s1;
    const size_t base = (size_t)(kv_slot >> p.block_shift) * s0 + (size_t)p.layer * s1 + (size_t)h * s2 +
        (size_t)(kv_slot & (bs - 1)) * s3;
    const size_t src = ((size_t)t * p.n_kv_heads + h) * head_dim;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        kv_store((KV *)p.kv_k + base + d, p.k_new[src + d]);
        kv_store((KV *)p.kv_v + base + d, p.v_new[src + d]);
    }
}

// DPL consecutive pool elements -> f32 with 16-byte loads.
template <int DPL>
__device__ __forceinline__ void kv_load_vec(const float *p, float (&v)[DPL]) {
#pragma unroll
    for (int i = 0; i < DPL; i += 4) {
        const float4 t = *(const float4 *)(p + i);
        v[i] = t.x;
        v[i + 1] = t.y;
        v[i + 2] = t.z;
        v[i + 3] = t.w;
    }
}
template <int DPL>
__device__ __forceinline__ void kv_load_vec(const __half *p, float (&v)[DPL]) {
#pragma unroll
    for (int i = 0; i < DPL; i += 8) {
        const uint4 t = *(const uint4 *)(p + i);
        const __half2 *h2 = (const __half2 *)&t;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h2[j]);
            v[i + 2 * j] = f.x;
            v[i + 2 * j + 1] = f.y;
        }
    }
}

// Split-KV attention.  One CTA per (KV head, token, chunk of `chunk` positions), one warp per query head of the head's
// group.  The CTA stages tiles of 32 K rows and 32 V rows in shared memory with 16-byte loads spread over all its
// threads (every pool byte is fetched once per CTA, and a thread has several loads in flight), then every warp scores
// the tile for its query head: groups of 8 lanes take one row each, HD/8 dimensions per lane, online softmax per
// lane group.  The 4 group states of a warp are merged and written as one partial state {m, l, acc[HD]} per
// (token, query head, chunk); paged_attention_merge_kernel combines the chunks, so long contexts never serialise on
// one warp.
constexpr int PA_MAX_GROUP = 8;
constexpr int PA_TILE = 32;
template <typename KV, int HD>
__global__ void __launch_bounds__(32 * PA_MAX_GROUP) paged_attention_kernel(PagedParams p, int chunk, float *partial) {
    constexpr int DPL = HD / 8;                          // dimensions per lane
    constexpr int ROW_BYTES = HD * (int)sizeof(KV);
    constexpr int PIECES = ROW_BYTES / 16;               // 16-byte pieces per row
    constexpr int TILE_BYTES = PA_TILE * ROW_BYTES;
    constexpr int ACC_BYTES = PA_MAX_GROUP * 4 * HD * (int)sizeof(float);
    constexpr int SMEM_BYTES = 2 * TILE_BYTES > ACC_BYTES ? 2 * TILE_BYTES : ACC_BYTES;
    __shared__ __align__(16) uint8_t s_buf[SMEM_BYTES];  // K tile | V tile; reused for the group states at the end
    __shared__ float s_m[PA_MAX_GROUP][4], s_l[PA_MAX_GROUP][4];
    __shared__ int s_live[PA_TILE];
    MCU_PDL_PROLOGUE();
    const int h = blockIdx.x, t = blockIdx.y, c = blockIdx.z, n_chunks = gridDim.z;
    const uint32_t kv_len = p.meta[t * 4 + 1] + 1u;
    const uint32_t p0 = (uint32_t)c * (uint32_t)chunk;
    if (p0 >= kv_len) return;  // the merge kernel derives the number of live chunks from kv_len as well
    const uint32_t p1 = min(kv_len, p0 + (uint32_t)chunk);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane >> 3, l8 = lane & 7;
    const int gsize = p.n_q_heads / p.n_kv_heads;
    const int qh = h * gsize + warp;
    const uint32_t seq = p.meta[t * 4 + 0];
    const size_t bs = (size_t)1 << p.block_shift;
    const size_t s3 = HD, s2 = bs * s3, s1 = (size_t)p.n_kv_heads * s2, s0 = (size_t)p.n_layers * s1;
    const size_t head_off = (size_t)p.layer * s1 + (size_t)h * s2;
    const uint32_t *table = p.table + (size_t)seq * p.max_blocks;
    uint8_t *s_k = s_buf, *s_v = s_buf + TILE_BYTES;

    float qv[DPL], acc[DPL];
    const float *qrow = p.q + ((size_t)t * p.n_q_heads + qh) * HD + l8 * DPL;
#pragma unroll
    for (int d = 0; d < DPL; ++d) {
        qv[d] = p.scale != 1.0f ? __fmul_rn(qrow[d], p.scale) : qrow[d];
        acc[d] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    for (uint32_t t0 = p0; t0 < p1; t0 += PA_TILE) {
        // stage the tile
        for (int idx = threadIdx.x; idx < PA_TILE * PIECES; idx += blockDim.x) {
            const int r = idx / PIECES, pc = idx - r * PIECES;
            const uint32_t pos = t0 + (uint32_t)r;
            const uint32_t lb = pos >> p.block_shift;
            uint32_t tb = 0xFFFFFFFFu;
            if (pos < p1 && lb < (uint32_t)p.max_blocks) tb = table[lb];
            if (pc == 0) s_live[r] = tb != 0xFFFFFFFFu;
            if (tb != 0xFFFFFFFFu) {
                const size_t base = (size_t)tb * s0 + head_off + (size_t)(pos & (uint32_t)(bs - 1)) * s3;
                const uint4 kq = *((const uint4 *)((const KV *)p.kv_k + base) + pc);
                const uint4 vq = *((const uint4 *)((const KV *)p.kv_v + base) + pc);
                *((uint4 *)(s_k + r * ROW_BYTES) + pc) = kq;
                *((uint4 *)(s_v + r * ROW_BYTES) + pc) = vq;
            }
        }
        __syncthreads();
        // score the tile: lane group `sub` takes rows sub, sub+4, ...
#pragma unroll 2
        for (int r = sub; r < PA_TILE; r += 4) {
            if (!s_live[r]) continue;  // uniform over the lane group (and over the warps)
            float kf[DPL], vf[DPL];
            kv_load_vec<DPL>((const KV *)(s_k + r * ROW_BYTES) + l8 * DPL, kf);
            kv_load_vec<DPL>((const KV *)(s_v + r * ROW_BYTES) + l8 * DPL, vf);
            float dot = 0.0f;
#pragma unroll
            for (int d = 0; d < DPL; ++d) dot += qv[d] * kf[d];
            const uint32_t gmask = 0xFFu << (8 * sub);
            dot += __shfl_xor_sync(gmask, dot, 1);  // the eight lanes of a group decide alike
            dot += __shfl_xor_sync(gmask, dot, 2);
            dot += __shfl_xor_sync(gmask, dot, 4);
            const float m_new = fmaxf(m, dot);
            const float keep = m == -INFINITY ? 0.0f : expf(m - m_new);
            const float w = expf(dot - m_new);
            l = l * keep + w;
#pragma unroll
            for (int d = 0; d < DPL; ++d) acc[d] = acc[d] * keep + w * vf[d];
            m = m_new;
        }
        __syncthreads();
    }
    // merge the four lane-group states of this warp; the tile buffers are free now
    float (*s_acc)[4][HD] = (float (*)[4][HD])s_buf;
    if (l8 == 0) {
        s_m[warp][sub] = m;
        s_l[warp][sub] = l;
    }
#pragma unroll
    for (int d = 0; d < DPL; ++d) s_acc[warp][sub][l8 * DPL + d] = acc[d];
    __syncwarp();
    // partial state of this chunk: [token][query head][chunk][2 + HD]
    float *pr = partial + (((size_t)t * p.n_q_heads + qh) * n_chunks + c) * (HD + 2);
    float M = -INFINITY;
#pragma unroll
    for (int g = 0; g < 4; ++g) M = fmaxf(M, s_m[warp][g]);
    float e[4], L = 0.0f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        e[g] = (M == -INFINITY || s_m[warp][g] == -INFINITY) ? 0.0f : expf(s_m[warp][g] - M);
        L += s_l[warp][g] * e[g];
    }
    if (lane == 0) {
        pr[0] = M;
        pr[1] = L;
    }
    for (int d = lane; d < HD; d += 32) {
        float o = 0.0f;
#pragma unroll
        for (int g = 0; g < 4; ++g) o += s_acc[warp][g][d] * e[g];
        pr[2 + d] = o;
    }
}

// ---------------------------------------------------------------- f16-pool attention on the tensor cores
// The same split-KV scheme for f16 pools with the two products on mma.sync m16n8k16 (f16 in, f32 accumulate).
// One CTA per (KV head, token, chunk of 128 positions); each of its four warps owns one tile of 32 positions: it
// copies the tile's K and V rows into its own shared-memory slice with cp.async (16-byte pieces, XOR-swizzled by row
// so that ldmatrix reads are conflict-free), and meanwhile builds the A fragments of Q.  The M rows of the MMA are
// the query heads of the KV head's group (at most 8), so a K/V byte is read from HBM once for
// the whole group and scored by one instruction stream.
//   S = Q K^T : A = Q (heads x dims), B = K rows as they lie in the pool (ldmatrix, no transpose)
//   O = P V   : A = P straight from the S accumulators, B = V through ldmatrix.trans
// Q and P are split into an f16 head and an f16 tail (x = hi + lo): the heads go to rows 0..7 of A, the tails to rows
// 8..15 (the group has at most eight query heads), so ONE MMA gives both partial products; K and V are f16 already,
// so the products carry about 22 significant bits and the result stays within 1e-6 of f32 arithmetic.
// A warp sees exactly one tile, so its softmax needs no running rescale; the four warps' states are merged through
// shared memory in warp order and written as one partial state per (token, query head, chunk).
constexpr int PM_WARPS = 4;
constexpr int PM_TILE = 32;
constexpr int PM_CHUNK = PM_WARPS * PM_TILE;

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
// D += A B, all sixteen rows of A: rows 0..7 carry the f16 heads of the eight query heads' values, rows 8..15 their
// f16 tails, so one instruction yields both partial products (c[0..1] = head row g, c[2..3] = tail row g).
__device__ __forceinline__ void mma_hi_lo(float (&c)[4], uint32_t a_hi0, uint32_t a_lo0, uint32_t a_hi1, uint32_t a_lo1, uint32_t b0,
                                          uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a_hi0), "r"(a_lo0), "r"(a_hi1), "r"(a_lo1), "r"(b0), "r"(b1));
}
// (x, y) as an f16 pair plus the f16 pair of what that rounding lost.
__device__ __forceinline__ void split_half2(float x, float y, uint32_t &hi, uint32_t &lo) {
    const __half2 h = __floats2half2_rn(x, y);
    const float2 f = __half22float2(h);
    const __half2 t = __floats2half2_rn(x - f.x, y - f.y);
    hi = *(const uint32_t *)&h;
    lo = *(const uint32_t *)&t;
}

// FUSED (decode steps: at most one token per sequence in the call) folds the neighbours of the attention into the
// same launch.  RoPE: the query heads are rotated on their way into the A fragments, and the warp whose tile holds the
// token's own position rotates the new K row, converts K and V to f16 and puts them into its tile AND into the pool
// (no other CTA of the launch reads that pool row: every other position belongs to an earlier step).  Merge: a CTA
// that is alone on its token writes the output itself; otherwise each CTA writes its chunk state, takes a ticket, and
// the CTA that draws the last ticket of a (token, KV head) merges the chunk states in chunk order -- the arithmetic of
// paged_attention_merge_kernel, so both forms give the same bits.
struct FusedDecode {
    const float2 *rope;  // [T][HD / 2] {cos, sin} of position * frequency, from rope_table_kernel
    int *tickets;        // [T][kv_heads], zero between launches; null: the chunk states are merged by a kernel of its own
    int neox;
};

template <int HD, bool FUSED>
__global__ void __launch_bounds__(32 * PM_WARPS) paged_attention_mma_kernel(PagedParams p, float *partial, FusedDecode fd) {
    constexpr int ROWB = HD * 2;            // bytes of a K or V row
    constexpr int PIECES = ROWB / 16;       // 16-byte pieces per row
    constexpr int TILEB = PM_TILE * ROWB;
    constexpr int KS = HD / 16;             // k steps of Q K^T
    constexpr int NT = HD / 8;              // n tiles of P V
    extern __shared__ __align__(128) uint8_t pm_smem[];  // [warp][K tile | V tile]; reused for the warps' states
    __shared__ int s_last;
    MCU_PDL_PROLOGUE();
    const int h = blockIdx.x, t = blockIdx.y, c = blockIdx.z, n_chunks = gridDim.z;
    const uint32_t kv_len = p.meta[t * 4 + 1] + 1u;
    const uint32_t p0 = (uint32_t)c * PM_CHUNK;
    if (p0 >= kv_len) return;
    const uint32_t p1 = min(kv_len, p0 + (uint32_t)PM_CHUNK);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const int gsize = p.n_q_heads / p.n_kv_heads;
    const uint32_t seq = p.meta[t * 4 + 0];
    const size_t bs = (size_t)1 << p.block_shift;
    const size_t s3 = HD, s2 = bs * s3, s1 = (size_t)p.n_kv_heads * s2, s0 = (size_t)p.n_layers * s1;
    const size_t head_off = (size_t)p.layer * s1 + (size_t)h * s2;
    const uint32_t *table = p.table + (size_t)seq * p.max_blocks;
    const uint32_t sK = (uint32_t)__cvta_generic_to_shared(pm_smem) + (uint32_t)(warp * 2 * TILEB);
    const uint32_t sV = sK + TILEB;
    const uint32_t k0 = p0 + (uint32_t)(warp * PM_TILE);  // this warp's positions [k0, k0 + 32)
    const bool has_tile = k0 < p1;                        // uniform over the warp
    // FUSED: the token's own row (position kv_len - 1) comes from k_new / v_new, not from the pool
    const uint32_t new_pos = kv_len - 1u;
    const int new_row = FUSED && new_pos >= k0 && new_pos < k0 + PM_TILE ? (int)(new_pos - k0) : -1;
    // stage the tile: lane r looks up the pool block of position k0 + r, the warp copies two rows per step
    uint32_t live = 0;
    if (has_tile) {
        const uint32_t pos = k0 + (uint32_t)lane, lb = pos >> p.block_shift;
        uint32_t tb = 0xFFFFFFFFu;
        if (pos < p1 && lb < (uint32_t)p.max_blocks) tb = table[lb];
        live = __ballot_sync(0xffffffffu, tb != 0xFFFFFFFFu);
        const size_t row_base = tb != 0xFFFFFFFFu ? (size_t)tb * s0 + head_off + (size_t)(pos & (uint32_t)(bs - 1)) * s3 : 0;
#pragma unroll 4
        for (int idx = lane; idx < PM_TILE * PIECES; idx += 32) {
            const int r = idx / PIECES, pc = idx - r * PIECES;
            const unsigned long long base = __shfl_sync(0xffffffffu, (unsigned long long)row_base, r);
            const uint32_t off = (uint32_t)(r * ROWB + ((pc ^ (r & 7)) << 4));
            if (r == new_row) continue;  // written below
            if ((live >> r) & 1u) {
                cp_async16(sK + off, (const __half *)p.kv_k + base + pc * 8);
                cp_async16(sV + off, (const __half *)p.kv_v + base + pc * 8);
            } else {  // never scored, but 0 * garbage must not become NaN
                asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(sK + off), "r"(0u) : "memory");
                asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(sV + off), "r"(0u) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (FUSED && new_row >= 0) {
            // the new K row rotated, the new V row, both as f16: into this warp's tile and into the pool slot
            const int half = HD / 2, r = new_row;
            const float2 *rope = fd.rope + (size_t)t * half;
            const uint32_t kv_slot = p.meta[t * 4 + 2];
            const size_t dst = (size_t)(kv_slot >> p.block_shift) * s0 + head_off + (size_t)(kv_slot & (uint32_t)(bs - 1)) * s3;
            const float *krow = p.k_new + ((size_t)t * p.n_kv_heads + h) * HD;
            const float *vrow = p.v_new + ((size_t)t * p.n_kv_heads + h) * HD;
            uint8_t *tK = pm_smem + warp * 2 * TILEB, *tV = tK + TILEB;
            auto tile_off = [&](int d) { return r * ROWB + ((((d >> 3) ^ (r & 7))) << 4) + (d & 7) * 2; };
            for (int i = lane; i < half; i += 32) {
                const float cs = rope[i].x, sn = rope[i].y;
                const int e = fd.neox ? i : 2 * i, o = fd.neox ? i + half : 2 * i + 1;
                const float xe = krow[e], xo = krow[o];
                const __half ke = __float2half_rn(__fsub_rn(__fmul_rn(xe, cs), __fmul_rn(xo, sn)));
                const __half ko = __float2half_rn(__fadd_rn(__fmul_rn(xe, sn), __fmul_rn(xo, cs)));
                *(__half *)(tK + tile_off(e)) = ke;
                *(__half *)(tK + tile_off(o)) = ko;
                ((__half *)p.kv_k)[dst + e] = ke;
                ((__half *)p.kv_k)[dst + o] = ko;
            }
            for (int d = lane; d < HD; d += 32) {
                const __half vv = __float2half_rn(vrow[d]);
                *(__half *)(tV + tile_off(d)) = vv;
                ((__half *)p.kv_v)[dst + d] = vv;
            }
        }
    }

    // A fragments of Q (row g = query head g of the group): a0 = dims 16s + 2tq, +1; a2 = dims 16s + 8 + 2tq, +1.
    // FUSED: the values are rotated on the way (the partner of a dimension is its neighbour, or lies half a head
    // away with the NeoX pairing; either way this lane reads it itself).
    uint32_t qhi[KS][2], qlo[KS][2];
    {
        const bool head_ok = g < gsize;
        const float *qrow = p.q + ((size_t)t * p.n_q_heads + (size_t)h * gsize + (head_ok ? g : 0)) * HD;
        // All loads first, without a branch between them (a branch per pair would serialise sixteen trips to L2: measured,
        // +50 % on the whole kernel), then the rotation, then the split.
        float2 qv[KS][2];
#pragma unroll
        for (int s = 0; s < KS; ++s)
#pragma unroll
            for (int hk = 0; hk < 2; ++hk)
                qv[s][hk] = head_ok ? *(const float2 *)(qrow + 16 * s + 8 * hk + 2 * tq) : make_float2(0.0f, 0.0f);
        if (FUSED) {
            const float2 *rope = fd.rope + (size_t)t * (HD / 2);
            if (!fd.neox) {  // the pair (d, d + 1) is one float2
                float2 cs[KS][2];
#pragma unroll
                for (int s = 0; s < KS; ++s)
#pragma unroll
                    for (int hk = 0; hk < 2; ++hk) cs[s][hk] = __ldg(rope + ((16 * s + 8 * hk + 2 * tq) >> 1));
#pragma unroll
                for (int s = 0; s < KS; ++s)
#pragma unroll
                    for (int hk = 0; hk < 2; ++hk) {
                        const float x = qv[s][hk].x, y = qv[s][hk].y, c = cs[s][hk].x, sn = cs[s][hk].y;
                        qv[s][hk].x = __fsub_rn(__fmul_rn(x, c), __fmul_rn(y, sn));
                        qv[s][hk].y = __fadd_rn(__fmul_rn(x, sn), __fmul_rn(y, c));
                    }
            } else {  // the pairs (d, d +- HD/2): the partner of k step s is k step s +- KS/2 of this same lane
                float4 cs[KS / 2][2];  // {cos, sin} of the two pairs (d, d + 1) of the low half
#pragma unroll
                for (int s = 0; s < KS / 2; ++s)
#pragma unroll
                    for (int hk = 0; hk < 2; ++hk) cs[s][hk] = __ldg((const float4 *)(rope + 16 * s + 8 * hk + 2 * tq));
#pragma unroll
                for (int s = 0; s < KS / 2; ++s)
#pragma unroll
                    for (int hk = 0; hk < 2; ++hk) {
                        const float2 lo = qv[s][hk], hi = qv[s + KS / 2][hk];
                        const float4 c = cs[s][hk];
                        qv[s][hk].x = __fsub_rn(__fmul_rn(lo.x, c.x), __fmul_rn(hi.x, c.y));
                        qv[s][hk].y = __fsub_rn(__fmul_rn(lo.y, c.z), __fmul_rn(hi.y, c.w));
                        qv[s + KS / 2][hk].x = __fadd_rn(__fmul_rn(lo.x, c.y), __fmul_rn(hi.x, c.x));
                        qv[s + KS / 2][hk].y = __fadd_rn(__fmul_rn(lo.y, c.w), __fmul_rn(hi.y, c.z));
                    }
            }
        }
#pragma unroll
        for (int s = 0; s < KS; ++s)
#pragma unroll
            for (int hk = 0; hk < 2; ++hk) {
                float x = qv[s][hk].x, y = qv[s][hk].y;
                if (p.scale != 1.0f) {
                    x = __fmul_rn(x, p.scale);
                    y = __fmul_rn(y, p.scale);
                }
                split_half2(x, y, qhi[s][hk], qlo[s][hk]);
            }
    }

    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    float m = -INFINITY, l = 0.0f;
    if (has_tile) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
        // S[head g][key 8j + 2tq, +1] = sc[j][0..1] (f16 head of Q) + sc[j][2..3] (its tail).  Even and odd k steps
        // accumulate separately and the four key tiles alternate, so that consecutive MMAs never wait for one
        // another's accumulator.
        float sc[4][4], st[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) sc[j][e] = st[j][e] = 0.0f;
#pragma unroll
        for (int s = 0; s < KS; s += 2) {
            uint32_t b[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // matrices: (keys 8j.., piece 2s), (piece 2s+1), (piece 2s+2), (piece 2s+3)
                const int r = 8 * j + (lane & 7), pc = 2 * s + (lane >> 3);
                ldsm_x4(sK + (uint32_t)(r * ROWB + ((pc ^ (r & 7)) << 4)), b[j][0], b[j][1], b[j][2], b[j][3]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) mma_hi_lo(sc[j], qhi[s][0], qlo[s][0], qhi[s][1], qlo[s][1], b[j][0], b[j][1]);
#pragma unroll
            for (int j = 0; j < 4; ++j) mma_hi_lo(st[j], qhi[s + 1][0], qlo[s + 1][0], qhi[s + 1][1], qlo[s + 1][1], b[j][2], b[j][3]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            sc[j][0] = (sc[j][0] + st[j][0]) + (sc[j][2] + st[j][2]);
            sc[j][1] = (sc[j][1] + st[j][1]) + (sc[j][3] + st[j][3]);
        }
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                if (!((live >> (8 * j + 2 * tq + e)) & 1u)) sc[j][e] = -INFINITY;
                mx = fmaxf(mx, sc[j][e]);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        uint32_t phi[4], plo[4];
        float psum = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float w0 = mx == -INFINITY ? 0.0f : expf(sc[j][0] - mx);
            const float w1 = mx == -INFINITY ? 0.0f : expf(sc[j][1] - mx);
            psum += w0 + w1;
            split_half2(w0, w1, phi[j], plo[j]);
        }
        psum += __shfl_xor_sync(0xffffffffu, psum, 1);
        psum += __shfl_xor_sync(0xffffffffu, psum, 2);
        m = mx;
        l = psum;
        // O[head g][dim 8n + 2tq, +1] += P V, four dimension tiles at a time (independent accumulators back to back)
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int n = 0; n < NT; n += 4) {
                // matrices: (keys 16u.., piece n), (keys 16u+8.., piece n), (keys 16u.., piece n+1), (keys 16u+8.., piece n+1)
                const int mi = lane >> 3;
                const int r = 16 * u + 8 * (mi & 1) + (lane & 7);
                uint32_t b[2][4];
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) {
                    const int pc = n + 2 * h2 + (mi >> 1);
                    ldsm_x4_trans(sV + (uint32_t)(r * ROWB + ((pc ^ (r & 7)) << 4)), b[h2][0], b[h2][1], b[h2][2], b[h2][3]);
                }
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) {  // o[..][0..1] from the heads of P, o[..][2..3] from the tails
                    mma_hi_lo(o[n + 2 * h2], phi[2 * u], plo[2 * u], phi[2 * u + 1], plo[2 * u + 1], b[h2][0], b[h2][1]);
                    mma_hi_lo(o[n + 2 * h2 + 1], phi[2 * u], plo[2 * u], phi[2 * u + 1], plo[2 * u + 1], b[h2][2], b[h2][3]);
                }
            }
    }
    // merge the warps' states: the tile slices are free once every warp is past its MMAs
    __syncthreads();
    float *s_o = (float *)pm_smem;                                        // [warp][8 heads][HD]
    float *s_m = s_o + PM_WARPS * 8 * HD, *s_l = s_m + PM_WARPS * 8;      // [warp][8 heads]
    float *s_e = s_l + PM_WARPS * 8;                                      // weight of a warp's state in the chunk state
#pragma unroll
    for (int n = 0; n < NT; ++n)
        *(float2 *)(s_o + ((size_t)warp * 8 + g) * HD + 8 * n + 2 * tq) = make_float2(o[n][0] + o[n][2], o[n][1] + o[n][3]);
    if (tq == 0) {
        s_m[warp * 8 + g] = m;
        s_l[warp * 8 + g] = l;
    }
    __syncthreads();
    if (threadIdx.x < PM_WARPS * 8) {
        const int hh = threadIdx.x & 7;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < PM_WARPS; ++w) M = fmaxf(M, s_m[w * 8 + hh]);
        const float mw = s_m[threadIdx.x];
        s_e[threadIdx.x] = (M == -INFINITY || mw == -INFINITY) ? 0.0f : expf(mw - M);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < gsize * HD; idx += blockDim.x) {
        const int hh = idx / HD, d = idx - hh * HD;
        float L = 0.0f, O = 0.0f;
#pragma unroll
        for (int w = 0; w < PM_WARPS; ++w) {  // warp order: deterministic
            const float e = s_e[w * 8 + hh];
            L += s_l[w * 8 + hh] * e;
            O += s_o[((size_t)w * 8 + hh) * HD + d] * e;
        }
        if (FUSED && fd.tickets != nullptr && (kv_len <= (uint32_t)PM_CHUNK || n_chunks == 1)) {  // the only chunk of its token: this is the result
            p.out[((size_t)t * p.n_q_heads + (size_t)h * gsize + hh) * HD + d] = L > 0.0f ? O / L : 0.0f;
            continue;
        }
        float *pr = partial + (((size_t)t * p.n_q_heads + (size_t)h * gsize + hh) * n_chunks + c) * (HD + 2);
        if (d == 0) {
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < PM_WARPS; ++w) M = fmaxf(M, s_m[w * 8 + hh]);
            pr[0] = M;
            pr[1] = L;
        }
        pr[2 + d] = O;
    }
    if (!FUSED || kv_len <= (uint32_t)PM_CHUNK || n_chunks == 1 || fd.tickets == nullptr) return;
    // the last CTA of this (token, KV head) to finish merges the chunk states
    const int live_chunks = min(n_chunks, (int)((kv_len + (uint32_t)PM_CHUNK - 1u) / (uint32_t)PM_CHUNK));
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int *ticket = fd.tickets + (size_t)t * p.n_kv_heads + h;
        const int drawn = atomicAdd(ticket, 1);
        s_last = drawn == live_chunks - 1;
        if (s_last) *ticket = 0;  // every other CTA has drawn already: ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // The chunk states' maxima and sums first, all loads at once, into shared memory (the tile buffers are free); then
    // every (head, dimension) adds up its column with the loads of eight chunks in flight.  Same operations in the same
    // order as paged_attention_merge_kernel.
    float *s_cm = (float *)pm_smem;                 // [head][chunk] m, later the chunk's weight exp(m - M)
    float *s_cl = s_cm + 8 * live_chunks;           // [head][chunk] l
    float *s_M = s_cl + 8 * live_chunks;            // [head]
    __syncthreads();
    for (int idx = threadIdx.x; idx < gsize * live_chunks; idx += blockDim.x) {
        const int hh = idx / live_chunks, cc = idx - hh * live_chunks;
        const float *pr = partial + (((size_t)t * p.n_q_heads + h * gsize + hh) * n_chunks + cc) * (HD + 2);
        s_cm[hh * live_chunks + cc] = __ldcg(pr);
        s_cl[hh * live_chunks + cc] = __ldcg(pr + 1);
    }
    __syncthreads();
    if (threadIdx.x < gsize) {
        float M = -INFINITY;
        for (int cc = 0; cc < live_chunks; ++cc) M = fmaxf(M, s_cm[threadIdx.x * live_chunks + cc]);
        s_M[threadIdx.x] = M;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < gsize * live_chunks; idx += blockDim.x) {
        const int hh = idx / live_chunks;
        const float mc = s_cm[idx], M = s_M[hh];
        s_cm[idx] = (M == -INFINITY || mc == -INFINITY) ? 0.0f : expf(mc - M);  // weight 0: the merge kernel skips the chunk
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < gsize * HD; idx += blockDim.x) {
        const int hh = idx / HD, d = idx - hh * HD;
        const int qh = h * gsize + hh;
        const float *pr = partial + ((size_t)t * p.n_q_heads + qh) * n_chunks * (HD + 2) + 2 + d;
        const float *e = s_cm + hh * live_chunks, *lc = s_cl + hh * live_chunks;
        float L = 0.0f, o = 0.0f;
        int cc = 0;
        for (; cc + 8 <= live_chunks; cc += 8) {
            float vals[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) vals[u] = __ldcg(pr + (size_t)(cc + u) * (HD + 2));
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (e[cc + u] != 0.0f) {
                    L += lc[cc + u] * e[cc + u];
                    o += vals[u] * e[cc + u];
                }
        }
        for (; cc < live_chunks; ++cc)
            if (e[cc] != 0.0f) {
                L += lc[cc] * e[cc];
                o += __ldcg(pr + (size_t)cc * (HD + 2)) * e[cc];
            }
        p.out[((size_t)t * p.n_q_heads + qh) * HD + d] = L > 0.0f ? o / L : 0.0f;
    }
}

// out[t][qh][:] from the chunk states; grid (query heads, tokens), HD threads.  The chunks' maxima and sums go to shared
// memory first (one load per thread, all in flight together), then every thread adds up its column eight chunks at a
// time; chunk order throughout, so the result does not depend on how the work was cut.
template <int HD>
__global__ void paged_attention_merge_kernel(PagedParams p, int chunk, int n_chunks, const float *partial) {
    extern __shared__ float mg_s[];  // m [live], then weight exp(m - M) in place; l [live]
    MCU_PDL_PROLOGUE();
    const int qh = blockIdx.x, t = blockIdx.y, d = threadIdx.x;
    const uint32_t kv_len = p.meta[t * 4 + 1] + 1u;
    const int live = min(n_chunks, (int)((kv_len + (uint32_t)chunk - 1u) / (uint32_t)chunk));
    const float *pr = partial + ((size_t)t * p.n_q_heads + qh) * n_chunks * (HD + 2);
    float *s_e = mg_s, *s_l = mg_s + n_chunks;
    for (int c = d; c < live; c += HD) {
        s_e[c] = pr[(size_t)c * (HD + 2)];
        s_l[c] = pr[(size_t)c * (HD + 2) + 1];
    }
    __syncthreads();
    float M = -INFINITY;
    for (int c = 0; c < live; ++c) M = fmaxf(M, s_e[c]);
    __syncthreads();
    for (int c = d; c < live; c += HD) {
        const float mc = s_e[c];
        s_e[c] = (M == -INFINITY || mc == -INFINITY) ? 0.0f : expf(mc - M);  // 0: the chunk adds nothing
    }
    __syncthreads();
    float L = 0.0f, o = 0.0f;
    const float *col = pr + 2 + d;
    int c = 0;
    for (; c + 8 <= live; c += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = col[(size_t)(c + u) * (HD + 2)];
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (s_e[c + u] != 0.0f) {
                L += s_l[c + u] * s_e[c + u];
                o += v[u] * s_e[c + u];
            }
    }
    for (; c < live; ++c)
        if (s_e[c] != 0.0f) {
            L += s_l[c] * s_e[c];
            o += col[(size_t)c * (HD + 2)] * s_e[c];
        }
    p.out[((size_t)t * p.n_q_heads + qh) * HD + d] = L > 0.0f ? o / L : 0.0f;
}

}  // namespace mcu

using namespace mcu;

#define DEC_CUDA(expr)                                                                  \
    do {                                                                                \
        cudaError_t e__ = (expr);                                                       \
        if (e__ != cudaSuccess) {                                                       \
            char msg__[256];                                                            \
            snprintf(msg__, sizeof(msg__), "%s: %s", #expr, cudaGetErrorString(e__));   \
            return set_error(MCU_ERROR_INVALID_OPERATION, msg__);                       \
        }                                                                               \
    } while (0)

static int dec_begin(mcu_context_t *ctx, cudaStream_t *s) {
    if (ctx == nullptr) return set_error(MCU_ERROR_DEVICE_NOT_AVAILABLE, "CUDA context is not initialised");
    DEC_CUDA(cudaSetDevice(context_device(ctx)));
    *s = (cudaStream_t)mcu_context_get_stream(ctx);
    return MCU_SUCCESS;
}

extern "C" {

int mcu_rmsnorm(mcu_context_t *ctx, const float *x_dev, const float *residual_dev, const float *weight_dev, size_t rows,
                size_t n, float eps, float weight_offset, float *out_dev) {
    cudaStream_t s;
    if (int rc = dec_begin(ctx, &s)) return rc;
    if (rows == 0 || n == 0) return MCU_SUCCESS;
    if (x_dev == nullptr || out_dev == nullptr) return set_error(MCU_ERROR_INVALID_ARGUMENT, "null tensor data");
    if (n > (size_t)1 << 30 || rows > (size_t)1 << 30) return set_error(MCU_ERROR_INVALID_ARGUMENT, "dimension too large");
    DEC_CUDA(launch_pdl(rmsnorm_kernel, dim3((unsigned)rows), dim3(256), s, x_dev, residual_dev, weight_dev, (int)n, eps,
                        weight_offset, out_dev));
    count_launches(1);
    return MCU_SUCCESS;
}

int mcu_rope(mcu_context_t *ctx, const float *x_dev, size_t ldx, const int32_t *positions_dev, size_t T, size_t n_heads,
             size_t head_dim, float theta, float freq_scale, int rope_type, float *out_dev, size_t ldo) {
    cudaStream_t s;
    if (int rc = dec_begin(ctx, &s)) return rc;
    if (T == 0 || n_heads == 0) return MCU_SUCCESS;
    if (x_dev == nullptr || out_dev == nullptr || positions_dev == nullptr)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "null tensor data");
    if (head_dim % 2 != 0) return set_error(MCU_ERROR_DIMENSION_MISMATCH, "RoPE requires even dimension");
    if (head_dim / 2 > (size_t)ROPE_MAX_PAIRS) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "RoPE head_dim above 256");
    if (rope_type != MCU_ROPE_NORM && rope_type != MCU_ROPE_NEOX)
        return set_error(MCU_ERROR_NOT_IMPLEMENTED, "unknown RoPE type");
    if (ldx < n_heads * head_dim || ldo < n_heads * head_dim)
        return set_error(MCU_ERROR_DIMENSION_MISMATCH, "RoPE requires row strides >= feature dimension");
    RopeFreqs fr;
    for (size_t i = 0; i < head_dim / 2; ++i)
        fr.f[i] = powf(theta, -((float)(2 * i) / (float)head_dim)) * freq_scale;  // src/core/helpers/rope.c:111
    DEC_CUDA(launch_pdl(rope_kernel, dim3((unsigned)T), dim3(128), s, x_dev, ldx, positions_dev, (int)n_heads, (int)head_dim,
                        rope_type == MCU_ROPE_NEOX ? 1 : 0, fr, out_dev, ldo));
    count_launches(1);
    return MCU_SUCCESS;
}

int mcu_add_rmsnorm(mcu_context_t *ctx, const float *x_dev, const float *delta_dev, const float *weight_dev, size_t rows,
                    size_t n, float eps, float weight_offset, float *x_out_dev, float *h_out_dev) {
    cudaStream_t s;
    if (int rc = dec_begin(ctx, &s)) return rc;
    if (rows == 0 || n == 0) return MCU_SUCCESS;
    if (x_dev == nullptr || delta_dev == nullptr || x_out_dev == nullptr || h_out_dev == nullptr)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "null tensor data");
    if (n > (size_t)1 << 30 || rows > (size_t)1 << 30) return set_error(MCU_ERROR_INVALID_ARGUMENT, "dimension too large");
    DEC_CUDA(launch_pdl(add_rmsnorm_kernel, dim3((unsigned)rows), dim3(256), s, x_dev, delta_dev, weight_dev, (int)n, eps,
                        weight_offset, x_out_dev, h_out_dev));
    count_launches(1);
    return MCU_SUCCESS;
}

int mcu_rope_qk(mcu_context_t *ctx, float *q_dev, size_t ldq, size_t n_q_heads, float *k_dev, size_t ldk, size_t n_k_heads,
                const int32_t *positions_dev, size_t T, size_t head_dim, float theta, float freq_scale, int rope_type) {
    cudaStream_t s;
    if (int rc = dec_begin(ctx, &s)) return rc;
    if (T == 0 || n_q_heads + n_k_heads == 0) return MCU_SUCCESS;
    if (q_dev == nullptr || k_dev == nullptr || positions_dev == nullptr)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "null tensor data");
    if (head_dim % 2 != 0) return set_error(MCU_ERROR_DIMENSION_MISMATCH, "RoPE requires even dimension");
    if (head_dim / 2 > (size_t)ROPE_MAX_PAIRS) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "RoPE head_dim above 256");
    if (rope_type != MCU_ROPE_NORM && rope_type != MCU_ROPE_NEOX)
        return set_error(MCU_ERROR_NOT_IMPLEMENTED, "unknown RoPE type");
    if (ldq < n_q_heads * head_dim || ldk < n_k_heads * head_dim)
        return set_error(MCU_ERROR_DIMENSION_MISMATCH, "RoPE requires row strides >= feature dimension");
    RopeFreqs fr;
    for (size_t i = 0; i < head_dim / 2; ++i) fr.f[i] = powf(theta, -((float)(2 * i) / (float)head_dim)) * freq_scale;
    DEC_CUDA(launch_pdl(rope_qk_kernel, dim3((unsigned)T), dim3(128), s, q_dev, ldq, (int)n_q_heads, k_dev, ldk,
                        (int)n_k_heads, positions_dev, (int)head_dim, rope_type == MCU_ROPE_NEOX ? 1 : 0, fr));
    count_launches(1);
    return MCU_SUCCESS;
}

int mcu_swiglu(mcu_context_t *ctx, const float *gate_dev, const float *up_dev, size_t n, float *out_dev) {
    cudaStream_t s;
    if (int rc = dec_begin(ctx, &s)) return rc;
    if (n == 0) return MCU_SUCCESS;
    if (gate_dev == nullptr || up_dev == nullptr || out_dev == nullptr)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "null tensor data");
    DEC_CUDA(launch_pdl(swiglu_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), s, gate_dev, up_dev, n, out_dev));
    count_launches(1);
    return MCU_SUCCESS;
}

int mcu_add(mcu_context_t *ctx, const float *a_dev, const float *b_dev, size_t n, float *out_dev) {
    cudaStream_t s;
    if (int rc = dec_begin(ctx, &s)) return rc;
    if (n == 0) return MCU_SUCCESS;
    if (a_dev == nullptr || b_dev == nullptr || out_dev == nullptr)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "null tensor data");
    DEC_CUDA(launch_pdl(add_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), s, a_dev, b_dev, n, out_dev));
    count_launches(1);
    return MCU_SUCCESS;
}

int mcu_argmax(mcu_context_t *ctx, const float *x_dev, size_t rows, size_t n, int32_t *out_dev) {
    cudaStream_t s;
    if (int rc = dec_begin(ctx, &s)) return rc;
    if (rows == 0) return MCU_SUCCESS;
    if (x_dev == nullptr || out_dev == nullptr || n == 0) return set_error(MCU_ERROR_INVALID_ARGUMENT, "null tensor data");
    if (n > (size_t)INT_MAX || rows > 65535u * 1024u) return set_error(MCU_ERROR_INVALID_ARGUMENT, "dimension too large");
    // slices of at least 2048 values, as many CTAs as fill the device once
    size_t slices = (n + 2047) / 2048;
    const size_t want = ((size_t)device_sm_count() + rows - 1) / rows;
    if (slices > want) slices = want;
    if (slices > 64) slices = 64;
    if (slices < 1) slices = 1;
    const size_t slice = (n + slices - 1) / slices;
    slices = (n + slice - 1) / slice;
    void *cand = nullptr, *tickets = nullptr;
    if (slices > 1) {  // the attention's scratch areas: stream order keeps their users apart, and both leave the tickets at zero
        if (int rc = context_attention_scratch(ctx, rows * slices * sizeof(ArgmaxCand), &cand)) return rc;
        if (int rc = context_attention_tickets(ctx, rows * sizeof(int), &tickets)) return rc;
    }
    DEC_CUDA(launch_pdl(argmax_kernel, dim3((unsigned)rows, (unsigned)slices), dim3(256), s, x_dev, (int)n, (int)slice,
                        (ArgmaxCand *)cand, (int *)tickets, out_dev));
    count_launches(1);
    return MCU_SUCCESS;
}

int mcu_embedding_gather(mcu_context_t *ctx, int kind, const void *table_dev, size_t dim, const int32_t *ids_dev, size_t T,
                         float *out_dev) {
    cudaStream_t s;
    if (int rc = dec_begin(ctx, &s)) return rc;
    if (!kind_supported(kind)) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "quant kind has no CUDA kernel");
    if (T == 0 || dim == 0) return MCU_SUCCESS;
    if (table_dev == nullptr || ids_dev == nullptr || out_dev == nullptr)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "null tensor data");
    if (dim % 4) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "embedding width must be a multiple of 4");
    DEC_CUDA(launch_dequantize_rows(kind, table_dev, dim, mcu_row_bytes(kind, dim), ids_dev, T, out_dev, s));
    count_launches(1);
    return MCU_SUCCESS;
}

int mcu_paged_attention(mcu_context_t *ctx, const uint32_t *token_meta_dev, size_t T, const float *q_dev,
                        const float *k_new_dev, const float *v_new_dev, void *kv_k_dev, void *kv_v_dev, int kv_dtype,
                        const uint32_t *block_table_dev, size_t max_blocks_per_seq, size_t n_layers, size_t layer,
                        size_t n_q_heads, size_t n_kv_heads, size_t head_dim, size_t block_size, float scale,
                        float *out_dev) {
    cudaStream_t s;
    if (int rc = dec_begin(ctx, &s)) return rc;
    if (T == 0) return MCU_SUCCESS;
    if (token_meta_dev == nullptr || q_dev == nullptr || k_new_dev == nullptr || v_new_dev == nullptr ||
        kv_k_dev == nullptr || kv_v_dev == nullptr || block_table_dev == nullptr || out_dev == nullptr)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "paged_attention descriptor is incomplete");
    if (kv_dtype != MCU_KV_F32 && kv_dtype != MCU_KV_F16)
        return set_error(MCU_ERROR_UNSUPPORTED_DTYPE, "paged_attention KV pool must be FLOAT32 or FLOAT16");
    if (((uintptr_t)kv_k_dev | (uintptr_t)kv_v_dev) & 15)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "paged_attention KV pools must be 16-byte aligned");
    if ((uintptr_t)q_dev & 7) return set_error(MCU_ERROR_INVALID_ARGUMENT, "paged_attention q must be 8-byte aligned");
    if (head_dim != 64 && head_dim != 128)
        return set_error(MCU_ERROR_NOT_IMPLEMENTED, "paged_attention supports head_dim 64 and 128");
    if (block_size == 0 || (block_size & (block_size - 1)) != 0)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "paged_attention block_size must be a power of two");
    if (n_kv_heads == 0 || n_q_heads % n_kv_heads != 0 || layer >= n_layers)
        return set_error(MCU_ERROR_DIMENSION_MISMATCH, "paged_attention head / layer configuration invalid");
    PagedParams p;
    p.meta = token_meta_dev;
    p.table = block_table_dev;
    p.q = q_dev;
    p.k_new = k_new_dev;
    p.v_new = v_new_dev;
    p.kv_k = kv_k_dev;
    p.kv_v = kv_v_dev;
    p.out = out_dev;
    p.n_q_heads = (int)n_q_heads;
    p.n_kv_heads = (int)n_kv_heads;
    p.max_blocks = (int)max_blocks_per_seq;
    p.n_layers = (int)n_layers;
    p.layer = (int)layer;
    p.block_shift = 0;
    while (((size_t)1 << p.block_shift) < block_size) ++p.block_shift;
    p.scale = scale;
    if (n_q_heads / n_kv_heads > (size_t)PA_MAX_GROUP)
        return set_error(MCU_ERROR_NOT_IMPLEMENTED, "paged_attention supports up to 8 query heads per KV head");
    // chunk of positions per CTA: long enough to amortise the set-up, short enough that every SM gets several CTAs
    // even for one short sequence.  The context length lives in device memory, so the grid covers the longest
    // context the block table allows; CTAs beyond a token's length return at once.
    const size_t max_positions = max_blocks_per_seq * block_size;
    const bool mma_path = kv_dtype == MCU_KV_F16;  // f16 pools: tensor-core kernel, fixed 128-position chunks
    size_t chunk = mma_path ? (size_t)PM_CHUNK : 256;
    while (!mma_path && chunk > 32 &&
           n_kv_heads * T * ((max_positions + chunk - 1) / chunk) < 2 * (size_t)device_sm_count())
        chunk /= 2;
    const size_t n_chunks = (max_positions + chunk - 1) / chunk;
    if (n_chunks > 6000) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "paged_attention context bound too long");  // (the merge keeps two floats per chunk in shared memory)
    void *scratch = nullptr;
    if (int rc = context_attention_scratch(ctx, T * n_q_heads * n_chunks * (head_dim + 2) * sizeof(float), &scratch))
        return rc;
    float *partial = (float *)scratch;
    const dim3 ag((unsigned)T, (unsigned)n_kv_heads), qg((unsigned)n_kv_heads, (unsigned)T, (unsigned)n_chunks);
    const dim3 mg((unsigned)n_q_heads, (unsigned)T);
    const unsigned threads = 32u * (unsigned)(n_q_heads / n_kv_heads);
    const dim3 tb(threads);
    if (mma_path) {
        const size_t smem = (size_t)PM_WARPS * 2 * PM_TILE * head_dim * 2;  // >= the warps' merge states (8 heads each)
        if (head_dim == 64)
            DEC_CUDA(cudaFuncSetAttribute(paged_attention_mma_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        else
            DEC_CUDA(cudaFuncSetAttribute(paged_attention_mma_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        DEC_CUDA(launch_pdl(kv_append_kernel<__half>, ag, dim3(128), s, p, (int)head_dim));
        if (head_dim == 64)
            DEC_CUDA(launch_pdl_smem(paged_attention_mma_kernel<64, false>, qg, dim3(32 * PM_WARPS), smem, s, p, partial, FusedDecode{}));
        else
            DEC_CUDA(launch_pdl_smem(paged_attention_mma_kernel<128, false>, qg, dim3(32 * PM_WARPS), smem, s, p, partial, FusedDecode{}));
    } else {
        DEC_CUDA(launch_pdl(kv_append_kernel<float>, ag, dim3(128), s, p, (int)head_dim));
        if (head_dim == 64) DEC_CUDA(launch_pdl(paged_attention_kernel<float, 64>, qg, tb, s, p, (int)chunk, partial));
        else DEC_CUDA(launch_pdl(paged_attention_kernel<float, 128>, qg, tb, s, p, (int)chunk, partial));
    }
    if (head_dim == 64)
        DEC_CUDA(launch_pdl_smem(paged_attention_merge_kernel<64>, mg, dim3(64), 2 * n_chunks * sizeof(float), s, p, (int)chunk, (int)n_chunks, (const float *)partial));
    else
        DEC_CUDA(launch_pdl_smem(paged_attention_merge_kernel<128>, mg, dim3(128), 2 * n_chunks * sizeof(float), s, p, (int)chunk, (int)n_chunks, (const float *)partial));
    count_launches(3);
    return MCU_SUCCESS;
}


int mcu_rope_table(mcu_context_t *ctx, const int32_t *positions_dev, size_t T, size_t head_dim, float theta, float freq_scale,
                   float *table_dev) {
    cudaStream_t s;
    if (int rc = dec_begin(ctx, &s)) return rc;
    if (T == 0) return MCU_SUCCESS;
    if (positions_dev == nullptr || table_dev == nullptr) return set_error(MCU_ERROR_INVALID_ARGUMENT, "null tensor data");
    if (head_dim % 2 != 0 || head_dim / 2 > (size_t)ROPE_MAX_PAIRS || ((uintptr_t)table_dev & 7))
        return set_error(MCU_ERROR_DIMENSION_MISMATCH, "RoPE table: even head_dim up to 256, 8-byte aligned table");
    RopeFreqs fr = {};
    for (size_t i = 0; i < head_dim / 2; ++i)
        fr.f[i] = powf(theta, -((float)(2 * i) / (float)head_dim)) * freq_scale;  // src/core/helpers/rope.c:111
    DEC_CUDA(launch_pdl(rope_table_kernel, dim3((unsigned)T), dim3(64), s, positions_dev, (int)(head_dim / 2), fr, (float2 *)table_dev));
    count_launches(1);
    return MCU_SUCCESS;
}

int mcu_paged_attention_decode(mcu_context_t *ctx, const uint32_t *token_meta_dev, size_t T, float *q_dev, float *k_new_dev,
                               const float *v_new_dev, void *kv_k_dev, void *kv_v_dev, int kv_dtype,
                               const uint32_t *block_table_dev, size_t max_blocks_per_seq, size_t n_layers, size_t layer,
                               size_t n_q_heads, size_t n_kv_heads, size_t head_dim, size_t block_size, float scale,
                               const int32_t *positions_dev, float rope_theta, float rope_freq_scale, int rope_type,
                               const float *rope_table_dev, float *out_dev) {
    cudaStream_t s;
    if (int rc = dec_begin(ctx, &s)) return rc;
    if (T == 0) return MCU_SUCCESS;
    // (the merge at the end of the fused kernel keeps two floats per query head and chunk in shared memory)
    const bool fused = kv_dtype == MCU_KV_F16 && (head_dim == 64 || head_dim == 128) && n_kv_heads != 0 &&
        n_q_heads % n_kv_heads == 0 && n_q_heads / n_kv_heads <= (size_t)PA_MAX_GROUP &&
        (max_blocks_per_seq * block_size + PM_CHUNK - 1) / PM_CHUNK <= 1024;
    if (!fused) {  // the three stand-alone steps; they check their own arguments
        if (int rc = mcu_rope_qk(ctx, q_dev, n_q_heads * head_dim, n_q_heads, k_new_dev, n_kv_heads * head_dim, n_kv_heads,
                                 positions_dev, T, head_dim, rope_theta, rope_freq_scale, rope_type))
            return rc;
        return mcu_paged_attention(ctx, token_meta_dev, T, q_dev, k_new_dev, v_new_dev, kv_k_dev, kv_v_dev, kv_dtype,
                                   block_table_dev, max_blocks_per_seq, n_layers, layer, n_q_heads, n_kv_heads, head_dim,
                                   block_size, scale, out_dev);
    }
    if (token_meta_dev == nullptr || q_dev == nullptr || k_new_dev == nullptr || v_new_dev == nullptr || kv_k_dev == nullptr ||
        kv_v_dev == nullptr || block_table_dev == nullptr || out_dev == nullptr || positions_dev == nullptr)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "paged_attention descriptor is incomplete");
    if (((uintptr_t)kv_k_dev | (uintptr_t)kv_v_dev) & 15)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "paged_attention KV pools must be 16-byte aligned");
    if (block_size == 0 || (block_size & (block_size - 1)) != 0)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "paged_attention block_size must be a power of two");
    if (layer >= n_layers) return set_error(MCU_ERROR_DIMENSION_MISMATCH, "paged_attention head / layer configuration invalid");
    if (((uintptr_t)q_dev & 7) || ((uintptr_t)rope_table_dev & 15))
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "paged_attention q must be 8-byte aligned, the RoPE table 16-byte aligned");
    if (rope_type != MCU_ROPE_NORM && rope_type != MCU_ROPE_NEOX) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "unknown RoPE type");
    PagedParams p;
    p.meta = token_meta_dev;
    p.table = block_table_dev;
    p.q = q_dev;
    p.k_new = k_new_dev;
    p.v_new = v_new_dev;
    p.kv_k = kv_k_dev;
    p.kv_v = kv_v_dev;
    p.out = out_dev;
    p.n_q_heads = (int)n_q_heads;
    p.n_kv_heads = (int)n_kv_heads;
    p.max_blocks = (int)max_blocks_per_seq;
    p.n_layers = (int)n_layers;
    p.layer = (int)layer;
    p.block_shift = 0;
    while (((size_t)1 << p.block_shift) < block_size) ++p.block_shift;
    p.scale = scale;
    const size_t max_positions = max_blocks_per_seq * block_size;
    const size_t n_chunks = (max_positions + PM_CHUNK - 1) / PM_CHUNK;
    if (n_chunks > 6000) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "paged_attention context bound too long");  // (the merge keeps two floats per chunk in shared memory)
    // Few CTAs: the step is a chain of latencies, and the last CTA of a token merging in place saves a launch.  Many
    // CTAs: the fence and the ticket keep every CTA (and its shared memory) alive for a round trip to L2 longer, which
    // at 64 sequences x 8 KV heads x ~17 chunks cost 25 % of the kernel (measured); a merge kernel is cheaper there.
    const bool ticket_merge = n_kv_heads * T * n_chunks <= 4 * (size_t)device_sm_count();
    void *scratch = nullptr, *tickets = nullptr;
    if (int rc = context_attention_scratch(ctx, T * n_q_heads * n_chunks * (head_dim + 2) * sizeof(float), &scratch)) return rc;
    if (ticket_merge)
        if (int rc = context_attention_tickets(ctx, T * n_kv_heads * sizeof(int), &tickets)) return rc;
    if (rope_table_dev == nullptr) {  // no table from the caller: make one for this call (one more launch)
        void *tab = nullptr;
        if (int rc = context_rope_table(ctx, T * (head_dim / 2) * 2 * sizeof(float), &tab)) return rc;
        if (int rc = mcu_rope_table(ctx, positions_dev, T, head_dim, rope_theta, rope_freq_scale, (float *)tab)) return rc;
        rope_table_dev = (const float *)tab;
    }
    FusedDecode fd;
    fd.rope = (const float2 *)rope_table_dev;
    fd.tickets = (int *)tickets;
    fd.neox = rope_type == MCU_ROPE_NEOX ? 1 : 0;
    const dim3 qg((unsigned)n_kv_heads, (unsigned)T, (unsigned)n_chunks);
    const size_t smem = (size_t)PM_WARPS * 2 * PM_TILE * head_dim * 2;
    if (head_dim == 64) {
        DEC_CUDA(cudaFuncSetAttribute(paged_attention_mma_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        DEC_CUDA(launch_pdl_smem(paged_attention_mma_kernel<64, true>, qg, dim3(32 * PM_WARPS), smem, s, p, (float *)scratch, fd));
    } else {
        DEC_CUDA(cudaFuncSetAttribute(paged_attention_mma_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        DEC_CUDA(launch_pdl_smem(paged_attention_mma_kernel<128, true>, qg, dim3(32 * PM_WARPS), smem, s, p, (float *)scratch, fd));
    }
    count_launches(1);
    if (!ticket_merge) {
        const dim3 mg((unsigned)n_q_heads, (unsigned)T);
        if (head_dim == 64)
            DEC_CUDA(launch_pdl_smem(paged_attention_merge_kernel<64>, mg, dim3(64), 2 * n_chunks * sizeof(float), s, p, (int)PM_CHUNK, (int)n_chunks, (const float *)scratch));
        else
            DEC_CUDA(launch_pdl_smem(paged_attention_merge_kernel<128>, mg, dim3(128), 2 * n_chunks * sizeof(float), s, p, (int)PM_CHUNK, (int)n_chunks, (const float *)scratch));
        count_launches(1);
    }
    return MCU_SUCCESS;
}

}  // extern "C"
