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

// One CTA per (query head, token): 4 warps, every group of 8 lanes walks its own positions (16 positions per CTA
// iteration) holding HD/8 dimensions per lane; online softmax per group, the 16 group states merged at the end.
template <typename KV, int HD>
__global__ void __launch_bounds__(128) paged_attention_kernel(PagedParams p) {
    constexpr int DPL = HD / 8;  // dimensions per lane
    __shared__ float s_acc[16][HD];
    __shared__ float s_m[16], s_l[16];
    const int qh = blockIdx.x, t = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane >> 3, l8 = lane & 7;
    const int group = warp * 4 + sub;
    const uint32_t seq = p.meta[t * 4 + 0], kv_len = p.meta[t * 4 + 1] + 1u;
    const int h = qh / (p.n_q_heads / p.n_kv_heads);
    const size_t bs = (size_t)1 << p.block_shift;
    const size_t s3 = HD, s2 = bs * s3, s1 = (size_t)p.n_kv_heads * s2, s0 = (size_t)p.n_layers * s1;
    const size_t head_off = (size_t)p.layer * s1 + (size_t)h * s2;

    float qv[DPL], acc[DPL];
    const float *qrow = p.q + ((size_t)t * p.n_q_heads + qh) * HD + l8 * DPL;
#pragma unroll
    for (int d = 0; d < DPL; ++d) {
        qv[d] = p.scale != 1.0f ? __fmul_rn(qrow[d], p.scale) : qrow[d];
        acc[d] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    const uint32_t gmask = 0xFFu << (8 * sub);
    for (uint32_t pos = (uint32_t)group; pos < kv_len; pos += 16u) {
        const uint32_t lb = pos >> p.block_shift;
        if (lb >= (uint32_t)p.max_blocks) break;
        const uint32_t tb = p.table[(size_t)seq * p.max_blocks + lb];
        if (tb == 0xFFFFFFFFu) continue;
        const size_t base = (size_t)tb * s0 + head_off + (size_t)(pos & (uint32_t)(bs - 1)) * s3 + l8 * DPL;
        const KV *kr = (const KV *)p.kv_k + base, *vr = (const KV *)p.kv_v + base;
        float dot = 0.0f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) dot += qv[d] * kv_load(kr + d);
        dot += __shfl_xor_sync(gmask, dot, 1);  // the eight lanes of a group share their trip count, groups do not
        dot += __shfl_xor_sync(gmask, dot, 2);
        dot += __shfl_xor_sync(gmask, dot, 4);
        const float m_new = fmaxf(m, dot);
        const float keep = m == -INFINITY ? 0.0f : expf(m - m_new);
        const float w = expf(dot - m_new);
        l = l * keep + w;
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[d] = acc[d] * keep + w * kv_load(vr + d);
        m = m_new;
    }
    // the loop is not warp-uniform (groups run out of positions at different times): reconverge before shuffles end
    __syncwarp();
    if (l8 == 0) {
        s_m[group] = m;
        s_l[group] = l;
    }
#pragma unroll
    for (int d = 0; d < DPL; ++d) s_acc[group][l8 * DPL + d] = acc[d];
    __syncthreads();
    float *orow = p.out + ((size_t)t * p.n_q_heads + qh) * HD;
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float M = -INFINITY;
#pragma unroll
        for (int g = 0; g < 16; ++g) M = fmaxf(M, s_m[g]);
        float L = 0.0f, o = 0.0f;
        if (M != -INFINITY) {
#pragma unroll
            for (int g = 0; g < 16; ++g) {
                if (s_m[g] == -INFINITY) continue;
                const float e = expf(s_m[g] - M);
                L += s_l[g] * e;
                o += s_acc[g][d] * e;
            }
        }
        orow[d] = L > 0.0f ? o / L : 0.0f;
    }
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
    const dim3 ag((unsigned)T, (unsigned)n_kv_heads), qg((unsigned)n_q_heads, (unsigned)T);
    if (kv_dtype == MCU_KV_F16) {
        kv_append_kernel<__half><<<ag, 128, 0, s>>>(p, (int)head_dim);
        if (head_dim == 64) paged_attention_kernel<__half, 64><<<qg, 128, 0, s>>>(p);
        else paged_attention_kernel<__half, 128><<<qg, 128, 0, s>>>(p);
    } else {
        kv_append_kernel<float><<<ag, 128, 0, s>>>(p, (int)head_dim);
        if (head_dim == 64) paged_attention_kernel<float, 64><<<qg, 128, 0, s>>>(p);
        else paged_attention_kernel<float, 128><<<qg, 128, 0, s>>>(p);
    }
    DEC_CUDA(cudaGetLastError());
    count_launches(2);
    return MCU_SUCCESS;
}

}  // extern "C"
