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

#include <cmath>
#include <cstdio>
#include <cuda_fp16.h>

namespace mcu {

// ---------------------------------------------------------------- RMSNorm
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ residual, const float *__restrict__ weight, int n,
               float eps, float weight_offset, float *__restrict__ out) {
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

// ---------------------------------------------------------------- RoPE
constexpr int ROPE_MAX_PAIRS = 128;
struct RopeFreqs {
    float f[ROPE_MAX_PAIRS];  // computed on the host with the reference's formula (powf of the same libm)
};

// x [T][n_heads][head_dim] with row stride ldx; one position per token.
__global__ void rope_kernel(const float *__restrict__ x, size_t ldx, const int32_t *__restrict__ positions, int n_heads,
                            int head_dim, int neox, RopeFreqs freqs, float *__restrict__ out, size_t ldo) {
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

// ---------------------------------------------------------------- elementwise
__global__ void swiglu_kernel(const float *__restrict__ a, const float *__restrict__ b, size_t n, float *__restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __fmul_rn(__fdiv_rn(a[i], __fadd_rn(1.0f, expf(-a[i]))), b[i]);
}
__global__ void add_kernel(const float *__restrict__ a, const float *__restrict__ b, size_t n, float *__restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __fadd_rn(a[i], b[i]);
}

// argmax over the last axis, first maximum wins; one CTA per row
__global__ void __launch_bounds__(256) argmax_kernel(const float *__restrict__ x, int n, int32_t *__restrict__ out) {
    __shared__ float bv[8];
    __shared__ int bi[8];
    const float *xr = x + (size_t)blockIdx.x * n;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {  // ascending i per thread: strict > keeps the first maximum
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
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (bi[w] != 0x7fffffff && (bi[0] == 0x7fffffff || bv[w] > bv[0] || (bv[w] == bv[0] && bi[w] < bi[0]))) {
                bv[0] = bv[w];
                bi[0] = bi[w];
            }
        out[blockIdx.x] = bi[0] == 0x7fffffff ? 0 : bi[0];
    }
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

// out[t][qh][:] from the chunk states; grid (query heads, tokens), HD threads.
template <int HD>
__global__ void paged_attention_merge_kernel(PagedParams p, int chunk, int n_chunks, const float *partial) {
    const int qh = blockIdx.x, t = blockIdx.y, d = threadIdx.x;
    const uint32_t kv_len = p.meta[t * 4 + 1] + 1u;
    const int live = min(n_chunks, (int)((kv_len + (uint32_t)chunk - 1u) / (uint32_t)chunk));
    const float *pr = partial + ((size_t)t * p.n_q_heads + qh) * n_chunks * (HD + 2);
    float M = -INFINITY;
    for (int c = 0; c < live; ++c) M = fmaxf(M, pr[(size_t)c * (HD + 2)]);
    float L = 0.0f, o = 0.0f;
    if (M != -INFINITY) {
        for (int c = 0; c < live; ++c) {
            const float mc = pr[(size_t)c * (HD + 2)];
            if (mc == -INFINITY) continue;
            const float e = expf(mc - M);
            L += pr[(size_t)c * (HD + 2) + 1] * e;
            o += pr[(size_t)c * (HD + 2) + 2 + d] * e;
        }
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
    rmsnorm_kernel<<<(unsigned)rows, 256, 0, s>>>(x_dev, residual_dev, weight_dev, (int)n, eps, weight_offset, out_dev);
    DEC_CUDA(cudaGetLastError());
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
    rope_kernel<<<(unsigned)T, 128, 0, s>>>(x_dev, ldx, positions_dev, (int)n_heads, (int)head_dim,
                                            rope_type == MCU_ROPE_NEOX ? 1 : 0, fr, out_dev, ldo);
    DEC_CUDA(cudaGetLastError());
    count_launches(1);
    return MCU_SUCCESS;
}

int mcu_swiglu(mcu_context_t *ctx, const float *gate_dev, const float *up_dev, size_t n, float *out_dev) {
    cudaStream_t s;
    if (int rc = dec_begin(ctx, &s)) return rc;
    if (n == 0) return MCU_SUCCESS;
    if (gate_dev == nullptr || up_dev == nullptr || out_dev == nullptr)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "null tensor data");
    swiglu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(gate_dev, up_dev, n, out_dev);
    DEC_CUDA(cudaGetLastError());
    count_launches(1);
    return MCU_SUCCESS;
}

int mcu_add(mcu_context_t *ctx, const float *a_dev, const float *b_dev, size_t n, float *out_dev) {
    cudaStream_t s;
    if (int rc = dec_begin(ctx, &s)) return rc;
    if (n == 0) return MCU_SUCCESS;
    if (a_dev == nullptr || b_dev == nullptr || out_dev == nullptr)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "null tensor data");
    add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a_dev, b_dev, n, out_dev);
    DEC_CUDA(cudaGetLastError());
    count_launches(1);
    return MCU_SUCCESS;
}

int mcu_argmax(mcu_context_t *ctx, const float *x_dev, size_t rows, size_t n, int32_t *out_dev) {
    cudaStream_t s;
    if (int rc = dec_begin(ctx, &s)) return rc;
    if (rows == 0) return MCU_SUCCESS;
    if (x_dev == nullptr || out_dev == nullptr || n == 0) return set_error(MCU_ERROR_INVALID_ARGUMENT, "null tensor data");
    argmax_kernel<<<(unsigned)rows, 256, 0, s>>>(x_dev, (int)n, out_dev);
    DEC_CUDA(cudaGetLastError());
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
    size_t chunk = 256;
    while (chunk > 32 && n_kv_heads * T * ((max_positions + chunk - 1) / chunk) < 2 * (size_t)device_sm_count()) chunk /= 2;
    const size_t n_chunks = (max_positions + chunk - 1) / chunk;
    if (n_chunks > 65535) return set_error(MCU_ERROR_NOT_IMPLEMENTED, "paged_attention context bound too long");
    void *scratch = nullptr;
    if (int rc = context_attention_scratch(ctx, T * n_q_heads * n_chunks * (head_dim + 2) * sizeof(float), &scratch))
        return rc;
    float *partial = (float *)scratch;
    const dim3 ag((unsigned)T, (unsigned)n_kv_heads), qg((unsigned)n_kv_heads, (unsigned)T, (unsigned)n_chunks);
    const dim3 mg((unsigned)n_q_heads, (unsigned)T);
    const unsigned threads = 32u * (unsigned)(n_q_heads / n_kv_heads);
    if (kv_dtype == MCU_KV_F16) {
        kv_append_kernel<__half><<<ag, 128, 0, s>>>(p, (int)head_dim);
        if (head_dim == 64) paged_attention_kernel<__half, 64><<<qg, threads, 0, s>>>(p, (int)chunk, partial);
        else paged_attention_kernel<__half, 128><<<qg, threads, 0, s>>>(p, (int)chunk, partial);
    } else {
        kv_append_kernel<float><<<ag, 128, 0, s>>>(p, (int)head_dim);
        if (head_dim == 64) paged_attention_kernel<float, 64><<<qg, threads, 0, s>>>(p, (int)chunk, partial);
        else paged_attention_kernel<float, 128><<<qg, threads, 0, s>>>(p, (int)chunk, partial);
    }
    if (head_dim == 64) paged_attention_merge_kernel<64><<<mg, 64, 0, s>>>(p, (int)chunk, (int)n_chunks, partial);
    else paged_attention_merge_kernel<128><<<mg, 128, 0, s>>>(p, (int)chunk, (int)n_chunks, partial);
    DEC_CUDA(cudaGetLastError());
    count_launches(3);
    return MCU_SUCCESS;
}

}  // extern "C"
