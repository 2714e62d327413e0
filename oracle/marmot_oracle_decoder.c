/*
 * CPU oracle for the decoder operators around the quantized matmuls (RMSNorm, RoPE, SwiGLU, paged attention,
 * quantized embedding gather, argmax).  TEST INFRASTRUCTURE ONLY, like marmot_oracle.c: a plain-C restatement of
 * the reference CPU backend's scalar code paths, f32 activations, -ffp-contract=off.  Each function names the
 * reference file:line it follows; tests pin it against the reference library itself.
 */
#include "marmot_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* rmsnorm_f32_scalar_range, src/backends/cpu/ops/normalization/scalar/normalization_scalar.c:780-791:
 * v = x (+ residual); mean of v^2 accumulated in order; inv = 1/sqrtf(mean + eps); out = v*inv*(w + offset). */
void mo_rmsnorm_f32(
    const float *x, const float *residual, const float *weight, size_t rows, size_t n, float eps, float weight_offset,
    float *out
) {
    for (size_t r = 0; r < rows; ++r) {
        const float *xr = x + r * n;
        const float *rr = residual != NULL ? residual + r * n : NULL;
        float sum = 0.0f;
        for (size_t i = 0; i < n; ++i) {
            const float v = rr != NULL ? xr[i] + rr[i] : xr[i];
            sum += v * v;
        }
        const float inv = 1.0f / sqrtf(sum / (float)n + eps);
        for (size_t i = 0; i < n; ++i) {
            const float v = rr != NULL ? xr[i] + rr[i] : xr[i];
            float y = v * inv;
            if (weight != NULL) y *= weight[i] + weight_offset;
            out[r * n + i] = y;
        }
    }
}

/* RoPE without frequency scaling extensions: frequencies powf(theta, -2i/dim) * freq_scale
 * (src/core/helpers/rope.c:108-120), angle = (float)pos * freq, pairs (2i, 2i+1) for the NORM type and
 * (i, i + dim/2) for NEOX (src/backends/cpu/ops/rope/rope_dispatch.c:343-375).  One position per row. */
void mo_rope_f32(
    const float *x, const int32_t *positions, size_t rows, size_t dim, float theta, float freq_scale, int neox,
    float *out
) {
    const size_t half = dim / 2;
    float *freqs = (float *)malloc(sizeof(float) * (half > 0 ? half : 1));
    for (size_t i = 0; i < half; ++i) freqs[i] = powf(theta, -((float)(2 * i) / (float)dim)) * freq_scale;
    for (size_t r = 0; r < rows; ++r) {
        const float pos = (float)positions[r];
        const float *xr = x + r * dim;
        float *yr = out + r * dim;
        for (size_t i = 0; i < half; ++i) {
            const float angle = pos * freqs[i];
            const float s = sinf(angle), c = cosf(angle);
            const size_t e = neox ? i : 2 * i, o = neox ? i + half : 2 * i + 1;
            const float xe = xr[e], xo = xr[o];
            yr[e] = xe * c - xo * s;
            yr[o] = xe * s + xo * c;
        }
    }
    free(freqs);
}

/* swiglu(a, b) = silu(a) * b with silu(x) = x / (1 + expf(-x)), the formula of the elementwise operator
 * (src/backends/cpu/ops/elementwise, same as moe_ops.c:318-320). */
void mo_swiglu_f32(const float *a, const float *b, size_t n, float *out) {
    for (size_t i = 0; i < n; ++i) out[i] = (a[i] / (1.0f + expf(-a[i]))) * b[i];
}

static float mo_half_to_float(uint16_t h) {
    _Float16 v;
    memcpy(&v, &h, sizeof(v));
    return (float)v;
}
/* f32 -> f16.  The reference's NEON and F16C builds convert with round-to-nearest-even (vcvt_f16_f32,
 * _mm256_cvtps_ph, src/backends/cpu/ops/convert/dtype_convert.c:22-36); its scalar build (and the scalar tail of the
 * vector builds) truncates the mantissa (marmot_f32_to_f16_ref, src/utils/dtype_ref.c:14-51).  truncate != 0
 * reproduces the latter, which is what a scalar-flavour reference library built with gcc does. */
static uint16_t mo_float_to_half(float f, int truncate) {
    if (!truncate) {
        const _Float16 v = (_Float16)f; /* round to nearest even */
        uint16_t h;
        memcpy(&h, &v, sizeof(h));
        return h;
    }
    uint32_t b;
    memcpy(&b, &f, sizeof(b));
    const uint32_t sign = (b >> 16) & 0x8000u, exponent = (b >> 23) & 0xFFu;
    uint32_t mantissa = b & 0x7FFFFFu;
    if (exponent == 0xFFu) return (uint16_t)(sign | 0x7C00u | (mantissa != 0 ? (mantissa >> 13) : 0u));
    const int32_t e = (int32_t)exponent - 127 + 15;
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        mantissa = (mantissa | 0x800000u) >> (1 - e);
        return (uint16_t)(sign | (mantissa >> 13));
    }
    if (e >= 0x1F) return (uint16_t)(sign | 0x7C00u);
    return (uint16_t)(sign | ((uint32_t)e << 10) | (mantissa >> 13));
}

/* Paged attention, f32 activations, f32 or f16 pool (kv_is_half).  Follows paged_attention_ref.c: first every token's
 * K/V rows go into the pool at kv_slot (:327-350), then per token and query head an online-softmax pass over the
 * positions 0..pos of the token's sequence in blocks of block_n rows (:397-556, block_n from :31-50, scalar
 * helpers scalar/paged_attention_scalar.c).  token_meta [T][4] = {seq_slot, pos, kv_slot, flags}; pool layout
 * [blocks][layers][kv_heads][block_size][head_dim]; block_table [seqs][max_blocks] with 0xFFFFFFFF = no block. */
int mo_paged_attention_f32(
    const uint32_t *token_meta, size_t T, const float *q, const float *k_new, const float *v_new, void *kv_k,
    void *kv_v, int kv_is_half, int kv_truncate, const uint32_t *block_table, size_t max_blocks_per_seq, size_t n_layers, size_t layer,
    size_t n_q_heads, size_t n_kv_heads, size_t head_dim, size_t block_size, float scale, float *out
) {
    uint32_t shift = 0;
    while (((size_t)1 << shift) < block_size) ++shift;
    if (((size_t)1 << shift) != block_size || n_kv_heads == 0 || n_q_heads % n_kv_heads) return -1;
    const uint32_t mask = (uint32_t)block_size - 1u;
    const size_t s3 = head_dim, s2 = block_size * s3, s1 = n_kv_heads * s2, s0 = n_layers * s1;
    const size_t group = n_q_heads / n_kv_heads;
    for (size_t t = 0; t < T; ++t) {
        const uint32_t kv_slot = token_meta[t * 4 + 2];
        const size_t base = (size_t)(kv_slot >> shift) * s0 + layer * s1 + (size_t)(kv_slot & mask) * s3;
        for (size_t h = 0; h < n_kv_heads; ++h)
            for (size_t d = 0; d < head_dim; ++d) {
                const float kvv = k_new[(t * n_kv_heads + h) * head_dim + d], vvv = v_new[(t * n_kv_heads + h) * head_dim + d];
                if (kv_is_half) {
                    ((uint16_t *)kv_k)[base + h * s2 + d] = mo_float_to_half(kvv, kv_truncate);
                    ((uint16_t *)kv_v)[base + h * s2 + d] = mo_float_to_half(vvv, kv_truncate);
                } else {
                    ((float *)kv_k)[base + h * s2 + d] = kvv;
                    ((float *)kv_v)[base + h * s2 + d] = vvv;
                }
            }
    }
    size_t block_n = (64 * 1024) / (2 * head_dim * sizeof(float));
    if (block_n < 32) block_n = 32;
    if (block_n > 256) block_n = 256;
    float *kb = (float *)malloc(sizeof(float) * block_n * head_dim * 2 + sizeof(float) * (block_n + 2 * head_dim));
    float *vb = kb + block_n * head_dim, *scores = vb + block_n * head_dim, *qv = scores + block_n, *ov = qv + head_dim;
    for (size_t t = 0; t < T; ++t) {
        const uint32_t seq = token_meta[t * 4 + 0], kv_len = token_meta[t * 4 + 1] + 1u;
        for (size_t qh = 0; qh < n_q_heads; ++qh) {
            const size_t h = qh / group;
            for (size_t d = 0; d < head_dim; ++d) qv[d] = q[(t * n_q_heads + qh) * head_dim + d];
            if (scale != 1.0f)
                for (size_t d = 0; d < head_dim; ++d) qv[d] *= scale;
            memset(ov, 0, sizeof(float) * head_dim);
            float max_score = -INFINITY, sum = 0.0f;
            int any = 0;
            for (uint32_t k0 = 0; k0 < kv_len; k0 += (uint32_t)block_n) {
                uint32_t k1 = k0 + (uint32_t)block_n;
                if (k1 > kv_len) k1 = kv_len;
                size_t cnt = 0;
                for (uint32_t p = k0; p < k1; ++p) {
                    const uint32_t lb = p >> shift;
                    if (lb >= max_blocks_per_seq) break;
                    const uint32_t tb = block_table[(size_t)seq * max_blocks_per_seq + lb];
                    if (tb == 0xFFFFFFFFu) continue;
                    const size_t base = (size_t)tb * s0 + layer * s1 + h * s2 + (size_t)(p & mask) * s3;
                    for (size_t d = 0; d < head_dim; ++d) {
                        kb[cnt * head_dim + d] = kv_is_half ? mo_half_to_float(((const uint16_t *)kv_k)[base + d]) : ((const float *)kv_k)[base + d];
                        vb[cnt * head_dim + d] = kv_is_half ? mo_half_to_float(((const uint16_t *)kv_v)[base + d]) : ((const float *)kv_v)[base + d];
                    }
                    ++cnt;
                }
                if (cnt == 0) continue;
                float row_max = -INFINITY;
                for (size_t j = 0; j < cnt; ++j) {
                    float dot = 0.0f;
                    for (size_t d = 0; d < head_dim; ++d) dot += qv[d] * kb[j * head_dim + d];
                    scores[j] = dot;
                    if (dot > row_max) row_max = dot;
                }
                const float next_max = max_score > row_max ? max_score : row_max;
                const float exp_prev = max_score == -INFINITY ? 0.0f : expf(max_score - next_max);
                if (exp_prev != 1.0f)
                    for (size_t d = 0; d < head_dim; ++d) ov[d] *= exp_prev;
                float block_sum = 0.0f;
                for (size_t j = 0; j < cnt; ++j) {
                    const float w = expf(scores[j] - next_max);
                    block_sum += w;
                    for (size_t d = 0; d < head_dim; ++d) ov[d] += w * vb[j * head_dim + d];
                }
                sum = sum * exp_prev + block_sum;
                max_score = next_max;
                any = 1;
            }
            float *orow = out + (t * n_q_heads + qh) * head_dim;
            if (!any) {
                memset(orow, 0, sizeof(float) * head_dim);
                continue;
            }
            const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
            for (size_t d = 0; d < head_dim; ++d) orow[d] = inv != 1.0f ? ov[d] * inv : ov[d];
        }
    }
    free(kb);
    return 0;
}

/* Embedding gather from a block-quantized table: row ids[t] dequantised to f32 (the dequantizers of
 * marmot_oracle.c, bit-exact with the reference's). */
int mo_embedding_gather(int kind, const void *table, size_t dim, const int32_t *ids, size_t T, float *out) {
    const size_t rb = mo_row_bytes(kind, dim);
    for (size_t t = 0; t < T; ++t) {
        const int rc = mo_dequantize(kind, (const uint8_t *)table + (size_t)ids[t] * rb, dim, out + t * dim);
        if (rc != 0) return rc;
    }
    return 0;
}

/* argmax over the last axis, first maximum wins (the reduction's tie rule). */
void mo_argmax_f32(const float *x, size_t rows, size_t n, int32_t *out) {
    for (size_t r = 0; r < rows; ++r) {
        size_t best = 0;
        for (size_t i = 1; i < n; ++i)
            if (x[r * n + i] > x[r * n + best]) best = i;
        out[r] = (int32_t)best;
    }
}
