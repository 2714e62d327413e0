/*
 * CPU oracle for the quantized GGUF matmul path of darekhta/marmot.
 *
 * TEST INFRASTRUCTURE ONLY: the shipped CUDA library never links or calls this
 * file.  Plain-C restatement of what the reference CPU backend computes in its
 * scalar flavour; compile with -ffp-contract=off so every product and sum is
 * an individually rounded IEEE binary32 operation, as in the reference build.
 *
 * Parity of this restatement is pinned twice: against the reference's own
 * llama.cpp-generated golden vectors (tests/backend/golden_matmul_llama.h,
 * golden_vec_dot_llama.h, golden_quant_llama.h in the reference tree) and
 * bit-for-bit against the reference library built from its sources.
 */
#include "marmot_oracle.h"

#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#define QK_K 256
#define Q8_0_VALUES 32
#define KC_BLOCKS 64 /* CPU_QUANT_KC_BLOCKS, matmul_quant_internal.h:11-21 */

/* ---- block layouts (include/marmot/quant_block.h:48-52,91-97,111-117,121-126) ---- */
#pragma pack(push, 1)
typedef struct { uint16_t d; int8_t qs[32]; } blk_q8_0;
typedef struct { uint16_t d; uint16_t dmin; uint8_t scales[12]; uint8_t qs[128]; } blk_q4_k;
typedef struct { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; uint16_t d; } blk_q6_k;
typedef struct { float d; int8_t qs[256]; int16_t bsums[16]; } blk_q8_k;
#pragma pack(pop)
_Static_assert(sizeof(blk_q8_0) == 34, "q8_0");
_Static_assert(sizeof(blk_q4_k) == 144, "q4_k");
_Static_assert(sizeof(blk_q6_k) == 210, "q6_k");
_Static_assert(sizeof(blk_q8_k) == 292, "q8_k");

/* fp16 <-> f32: the reference widens/narrows through native _Float16 (cpu_backend_internal.h:584-600). */
static inline float h2f(uint16_t bits) {
    _Float16 h;
    memcpy(&h, &bits, 2);
    return (float)h;
}
static inline uint16_t f2h(float v) {
    _Float16 h = (_Float16)v;
    uint16_t bits;
    memcpy(&bits, &h, 2);
    return bits;
}

size_t mo_block_values(int kind) {
    return kind == MO_KIND_Q8_0 ? Q8_0_VALUES : (kind == MO_KIND_Q4_K || kind == MO_KIND_Q6_K) ? QK_K : 0;
}
size_t mo_block_bytes(int kind) {
    switch (kind) {
    case MO_KIND_Q8_0: return MO_Q8_0_BLOCK_BYTES;
    case MO_KIND_Q4_K: return MO_Q4_K_BLOCK_BYTES;
    case MO_KIND_Q6_K: return MO_Q6_K_BLOCK_BYTES;
    default: return 0;
    }
}
size_t mo_row_bytes(int kind, size_t K) {
    const size_t bv = mo_block_values(kind);
    return bv == 0 ? 0 : ((K + bv - 1) / bv) * mo_block_bytes(kind);
}

/* 6-bit (scale, min) pair j of a Q4_K block: get_scale_min_k4, kquant_common.h:29-37 */
static inline void k4_scale_min(int j, const uint8_t *q, uint8_t *sc, uint8_t *mn) {
    if (j < 4) {
        *sc = q[j] & 63;
        *mn = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* ---- dequantizers ---- */

/* q4_k_dequantize_block, src/backends/cpu/quantization/formats/q4k_gguf.c:133-166:
 * d1 = d*sc; m1 = dmin*m; out = d1*q - m1  (three roundings). */
static void deq_q4_k(const blk_q4_k *b, size_t n, float *out) {
    const float d = h2f(b->d), dmin = h2f(b->dmin);
    const uint8_t *q = b->qs;
    size_t w = 0;
    for (int g = 0; g < 4 && w < n; ++g) {
        uint8_t sc, mn;
        k4_scale_min(2 * g, b->scales, &sc, &mn);
        const float d1 = d * (float)sc, m1 = dmin * (float)mn;
        k4_scale_min(2 * g + 1, b->scales, &sc, &mn);
        const float d2 = d * (float)sc, m2 = dmin * (float)mn;
        for (int l = 0; l < 32 && w < n; ++l, ++w) out[w] = d1 * (float)(q[l] & 0xF) - m1;
        for (int l = 0; l < 32 && w < n; ++l, ++w) out[w] = d2 * (float)(q[l] >> 4) - m2;
        q += 32;
    }
}

/* q6_k_dequantize_block, q6k_gguf.c:63-99: out = (d*sc)*q, q in [-32,31]. */
static void deq_q6_k(const blk_q6_k *b, size_t n, float *out) {
    const float d = h2f(b->d);
    const uint8_t *ql = b->ql, *qh = b->qh;
    const int8_t *sc = b->scales;
    for (size_t base = 0; base < QK_K && base < n; base += 128) {
        for (int l = 0; l < 32; ++l) {
            const int is = l / 16;
            const int8_t q1 = (int8_t)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
            const int8_t q2 = (int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
            const int8_t q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            const int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            if (base + l < n) out[base + l] = d * (float)sc[is + 0] * (float)q1;
            if (base + l + 32 < n) out[base + l + 32] = d * (float)sc[is + 2] * (float)q2;
            if (base + l + 64 < n) out[base + l + 64] = d * (float)sc[is + 4] * (float)q3;
            if (base + l + 96 < n) out[base + l + 96] = d * (float)sc[is + 6] * (float)q4;
        }
        ql += 64;
        qh += 32;
        sc += 8;
    }
}

/* q8_0_dequantize_block, q8_gguf.c:110-114,189-200: out = (float)q * d. */
static void deq_q8_0(const blk_q8_0 *b, size_t n, float *out) {
    const float d = h2f(b->d);
    for (size_t i = 0; i < n && i < Q8_0_VALUES; ++i) out[i] = (float)b->qs[i] * d;
}

/* Row loop of cpu_dequantize_blockwise, quantization/ops/quantize_core.c:267-331. */
int mo_dequantize(int kind, const void *blocks, size_t n_values, float *out) {
    const size_t bv = mo_block_values(kind), bb = mo_block_bytes(kind);
    if (bv == 0 || blocks == NULL || out == NULL) return -1;
    const uint8_t *p = (const uint8_t *)blocks;
    for (size_t off = 0; off < n_values; off += bv, p += bb) {
        const size_t n = n_values - off < bv ? n_values - off : bv;
        if (kind == MO_KIND_Q4_K) deq_q4_k((const blk_q4_k *)p, n, out + off);
        else if (kind == MO_KIND_Q6_K) deq_q6_k((const blk_q6_k *)p, n, out + off);
        else deq_q8_0((const blk_q8_0 *)p, n, out + off);
    }
    return 0;
}

/* ---- activation packers ---- */

/* cpu_quant_matmul_nearest_int, matmul_quant_pack.c:11-21: round-to-nearest-even via the 1.5*2^23 trick. */
static inline int nearest_int(float v) {
    if (v > 4194303.0f) v = 4194303.0f;
    else if (v < -4194303.0f) v = -4194303.0f;
    const float shifted = v + 12582912.0f;
    int bits;
    memcpy(&bits, &shifted, 4);
    return (bits & 0x007fffff) - 0x00400000;
}

/* cpu_quant_matmul_pack_q8_k_block + cpu_matmul_quant_pack_q8_k_f32, matmul_quant_pack.c:106-169. */
void mo_pack_q8_k_f32(const float *x, size_t K, void *dst_blocks) {
    blk_q8_k *dst = (blk_q8_k *)dst_blocks;
    const size_t nb = (K + QK_K - 1) / QK_K;
    float buf[QK_K];
    for (size_t b = 0; b < nb; ++b) {
        const size_t start = b * QK_K;
        const size_t len = K - start < QK_K ? K - start : QK_K;
        memcpy(buf, x + start, len * sizeof(float));
        if (len < QK_K) memset(buf + len, 0, (QK_K - len) * sizeof(float));

        float max_val = 0.0f, abs_max = 0.0f;
        for (int i = 0; i < QK_K; ++i) {
            const float ax = fabsf(buf[i]);
            if (ax > abs_max) {
                abs_max = ax;
                max_val = buf[i];
            }
        }
        blk_q8_k *o = &dst[b];
        if (abs_max <= 0.0f) {
            memset(o, 0, sizeof(*o));
            continue;
        }
        const float iscale = -127.0f / max_val;
        for (int i = 0; i < QK_K; ++i) {
            int v = nearest_int(iscale * buf[i]);
            if (v > 127) v = 127;
            o->qs[i] = (int8_t)v;
        }
        for (int j = 0; j < QK_K / 16; ++j) {
            int s = 0;
            for (int i = 0; i < 16; ++i) s += o->qs[j * 16 + i];
            o->bsums[j] = (int16_t)s;
        }
        o->d = 1.0f / iscale;
    }
}

/* cpu_matmul_quant_pack_q8_0_f32, matmul_quant_pack.c:23-62, with the scalar
 * helpers max_abs_scalar / quantize_q8_0_scalar (quantization/common/block.c:175-183,221-232):
 * scale = amax/127 (1 when below FLT_MIN); q = roundf(x * (1/scale)) clamped; stored scale is fp16. */
void mo_pack_q8_0_f32(const float *x, size_t K, void *dst_blocks) {
    blk_q8_0 *dst = (blk_q8_0 *)dst_blocks;
    const size_t nb = (K + Q8_0_VALUES - 1) / Q8_0_VALUES;
    for (size_t b = 0; b < nb; ++b) {
        const size_t start = b * Q8_0_VALUES;
        const size_t len = K - start < Q8_0_VALUES ? K - start : Q8_0_VALUES;
        float amax = 0.0f;
        for (size_t i = 0; i < len; ++i) {
            const float ax = fabsf(x[start + i]);
            if (ax > amax) amax = ax;
        }
        float scale = amax / 127.0f;
        if (scale < FLT_MIN) scale = 1.0f;
        const float inv = 1.0f / scale;
        blk_q8_0 *o = &dst[b];
        memset(o, 0, sizeof(*o));
        o->d = f2h(scale);
        for (size_t i = 0; i < len; ++i) {
            int q = (int)roundf(x[start + i] * inv);
            if (q < -127) q = -127;
            else if (q > 127) q = 127;
            o->qs[i] = (int8_t)q;
        }
    }
}

/* ---- row dots ---- */

/* cpu_vec_dot_q4_k_q8_k, ops/matmul/quantized/vec_dot_impl.h:688-732 (helpers :541-563). */
float mo_vec_dot_q4_k_q8_k(const void *wv, const void *av, size_t nb) {
    const blk_q4_k *w = (const blk_q4_k *)wv;
    const blk_q8_k *a = (const blk_q8_k *)av;
    float total = 0.0f;
    for (size_t b = 0; b < nb; ++b) {
        uint8_t sc[8], mn[8];
        for (int j = 0; j < 8; ++j) k4_scale_min(j, w[b].scales, &sc[j], &mn[j]);
        int32_t sumi = 0;
        for (int j = 0; j < 16; ++j) sumi += (int32_t)a[b].bsums[j] * (int32_t)mn[j / 2];
        int32_t block_sum = 0;
        for (int sg = 0; sg < 8; ++sg) {
            const uint8_t *q4 = w[b].qs + (sg / 2) * 32;
            const int8_t *q8 = a[b].qs + sg * 32;
            int32_t dot = 0;
            for (int l = 0; l < 32; ++l) {
                const int32_t wq = (sg & 1) ? (q4[l] >> 4) : (q4[l] & 0xF);
                dot += wq * (int32_t)q8[l];
            }
            block_sum += (int32_t)sc[sg] * dot;
        }
        const float d = a[b].d * h2f(w[b].d);
        const float dm = a[b].d * h2f(w[b].dmin);
        total += d * (float)block_sum - dm * (float)sumi;
    }
    return total;
}

/* cpu_vec_dot_q6_k_q8_k, vec_dot_impl.h:783-828. */
float mo_vec_dot_q6_k_q8_k(const void *wv, const void *av, size_t nb) {
    const blk_q6_k *w = (const blk_q6_k *)wv;
    const blk_q8_k *a = (const blk_q8_k *)av;
    float total = 0.0f;
    for (size_t b = 0; b < nb; ++b) {
        const int8_t *q8 = a[b].qs;
        int32_t block_sum = 0;
        for (int sg = 0; sg < 16; ++sg) {
            const int g32 = sg / 2, half = g32 / 4, gih = g32 & 3, part = sg & 1;
            const uint8_t *ql = w[b].ql + half * 64 + ((gih & 1) ? 32 : 0) + part * 16;
            const uint8_t *qh = w[b].qh + half * 32 + part * 16;
            const int shift = gih * 2;
            int32_t dot = 0;
            for (int l = 0; l < 16; ++l) {
                const uint8_t lo = gih >= 2 ? (ql[l] >> 4) : (ql[l] & 0xF);
                const uint8_t hi = (qh[l] >> shift) & 3;
                const int8_t q = (int8_t)((lo | (hi << 4)) - 32);
                dot += (int32_t)q * (int32_t)q8[l];
            }
            block_sum += (int32_t)w[b].scales[sg] * dot;
            q8 += 16;
        }
        const float d = a[b].d * h2f(w[b].d);
        total += d * (float)block_sum;
    }
    return total;
}

/* cpu_vec_dot_q8_0_q8_0, vec_dot_impl.h:452-479. */
float mo_vec_dot_q8_0_q8_0(const void *wv, const void *av, size_t nb) {
    const blk_q8_0 *w = (const blk_q8_0 *)wv;
    const blk_q8_0 *a = (const blk_q8_0 *)av;
    float total = 0.0f;
    for (size_t b = 0; b < nb; ++b) {
        int32_t s = 0;
        for (int i = 0; i < Q8_0_VALUES; ++i) s += (int32_t)w[b].qs[i] * (int32_t)a[b].qs[i];
        const float scale = h2f(w[b].d) * h2f(a[b].d);
        total += (float)s * scale;
    }
    return total;
}

/* ---- matmul driver ---- */

typedef float (*dot_fn)(const void *, const void *, size_t);

/*
 * cpu_matmul_quantized_impl (matmul_quant_dispatch.c:373-591) for f32 input:
 * every token row is packed to Q8_K (K-quants) or Q8_0 (legacy formats), then
 * each output is the sum over 64-block K chunks of the row dot
 * (cpu_quant_matmul_compute_rows, matmul_quant_compute.c:1032-1112; Q8_0 with
 * two or more tokens goes through ..._q8_0_blocked_generic, :412-466, same
 * sums).  Bias epilogue: out += bias (ops/matmul/matmul_epilogue.c).
 * The result does not depend on the thread count: one thread owns an output.
 */
int mo_linear(
    int kind, const float *x, size_t ldx, const void *W, size_t T, size_t K, size_t F, const float *bias, float *out,
    size_t ldo, int n_threads
) {
    const size_t bv = mo_block_values(kind), bb = mo_block_bytes(kind);
    if (bv == 0 || x == NULL || W == NULL || out == NULL) return -1;
    const size_t nb = (K + bv - 1) / bv;
    const int k_quant = kind != MO_KIND_Q8_0;
    const size_t abytes = k_quant ? sizeof(blk_q8_k) : sizeof(blk_q8_0);
    const dot_fn dot = kind == MO_KIND_Q4_K ? mo_vec_dot_q4_k_q8_k
        : kind == MO_KIND_Q6_K             ? mo_vec_dot_q6_k_q8_k
                                           : mo_vec_dot_q8_0_q8_0;
    uint8_t *act = (uint8_t *)malloc(T * nb * abytes + 1);
    if (act == NULL) return -2;
    for (size_t t = 0; t < T; ++t) {
        if (k_quant) mo_pack_q8_k_f32(x + t * ldx, K, act + t * nb * abytes);
        else mo_pack_q8_0_f32(x + t * ldx, K, act + t * nb * abytes);
    }
    const uint8_t *wb = (const uint8_t *)W;
    (void)n_threads;
#pragma omp parallel for schedule(static) num_threads(n_threads > 0 ? n_threads : 1)
    for (long f = 0; f < (long)F; ++f) {
        const uint8_t *row = wb + (size_t)f * nb * bb;
        for (size_t t = 0; t < T; ++t) {
            const uint8_t *arow = act + t * nb * abytes;
            float acc = 0.0f;
            for (size_t kb = 0; kb < nb; kb += KC_BLOCKS) {
                const size_t chunk = nb - kb < KC_BLOCKS ? nb - kb : KC_BLOCKS;
                acc += dot(row + kb * bb, arow + kb * abytes, chunk);
            }
            if (bias != NULL) acc += bias[f];
            out[t * ldo + (size_t)f] = acc;
        }
    }
    free(act);
    return 0;
}

/*
 * The f16-activation form (matmul_quant_dispatch.c:449-470 -> cpu_quant_matmul_dispatch_fp16_tile): no activation
 * packing; every output is ONE running f32 sum over the row, total += w_val * (float)x[k], in k order, with the
 * weight value formed as in cpu_vec_dot_q4_k_f16 (vec_dot_impl.h:973-1023), cpu_vec_dot_q8_0_f16 (:419-447) and
 * cpu_vec_dot_q6_k_f16 (:1082-1127).  The Q6_K function does NOT read the block as the dequantizer does: value idx of
 * a block takes the scale sc[idx / 128], the nibble idx of ql counted linearly (even idx low, odd idx high) and the
 * two bits (idx % 4) of qh[idx / 4].  The reference's golden output (g_matmul_q6_k_output_from_f16) pins that reading,
 * so it is restated as it stands.  Bias: out += bias.
 */
static float dot_f16_q4_k(const blk_q4_k *w, const uint16_t *x, size_t nb, size_t K) {
    float total = 0.0f;
    for (size_t b = 0; b < nb; ++b) {
        const uint8_t *q = w[b].qs;
        const float d = h2f(w[b].d), dmin = h2f(w[b].dmin);
        const uint16_t *a = x + b * QK_K;
        const size_t len = K - b * QK_K < QK_K ? K - b * QK_K : QK_K;
        size_t at = 0;
        for (int g = 0; g < 4 && at < len; ++g) {
            uint8_t sc, mn;
            k4_scale_min(2 * g, w[b].scales, &sc, &mn);
            const float d1 = d * (float)sc, m1 = dmin * (float)mn;
            k4_scale_min(2 * g + 1, w[b].scales, &sc, &mn);
            const float d2 = d * (float)sc, m2 = dmin * (float)mn;
            for (int l = 0; l < 32 && at < len; ++l, ++at) {
                const float wv = d1 * (float)(q[l] & 0xF) - m1;
                total += wv * h2f(a[at]);
            }
            for (int l = 0; l < 32 && at < len; ++l, ++at) {
                const float wv = d2 * (float)(q[l] >> 4) - m2;
                total += wv * h2f(a[at]);
            }
            q += 32;
        }
    }
    return total;
}
static float dot_f16_q6_k(const blk_q6_k *w, const uint16_t *x, size_t nb, size_t K) {
    float total = 0.0f;
    for (size_t b = 0; b < nb; ++b) {
        const float d = h2f(w[b].d);
        const uint16_t *a = x + b * QK_K;
        const size_t len = K - b * QK_K < QK_K ? K - b * QK_K : QK_K;
        for (size_t idx = 0; idx < len; ++idx) {
            const float scale = d * (float)w[b].scales[idx / 128];
            const uint8_t lo = (idx % 2 == 0) ? (uint8_t)(w[b].ql[idx / 2] & 0xF) : (uint8_t)(w[b].ql[idx / 2] >> 4);
            const uint8_t hi = (uint8_t)((w[b].qh[idx / 4] >> ((idx % 4) * 2)) & 0x3);
            const int8_t sq = (int8_t)((int8_t)(lo | (hi << 4)) - 32);
            const float wv = scale * (float)sq;
            total += wv * h2f(a[idx]);
        }
    }
    return total;
}
static float dot_f16_q8_0(const blk_q8_0 *w, const uint16_t *x, size_t nb, size_t K) {
    float total = 0.0f;
    for (size_t b = 0; b < nb; ++b) {
        const float sw = h2f(w[b].d);
        const uint16_t *a = x + b * Q8_0_VALUES;
        const size_t len = K - b * Q8_0_VALUES < Q8_0_VALUES ? K - b * Q8_0_VALUES : Q8_0_VALUES;
        for (size_t i = 0; i < len; ++i) total += ((float)w[b].qs[i]) * sw * h2f(a[i]);
    }
    return total;
}
int mo_linear_f16(
    int kind, const uint16_t *x, size_t ldx, const void *W, size_t T, size_t K, size_t F, const float *bias, float *out,
    size_t ldo
) {
    const size_t bv = mo_block_values(kind), bb = mo_block_bytes(kind);
    if (bv == 0 || x == NULL || W == NULL || out == NULL) return -1;
    const size_t nb = (K + bv - 1) / bv;
    const uint8_t *wb = (const uint8_t *)W;
    for (size_t f = 0; f < F; ++f) {
        const uint8_t *row = wb + f * nb * bb;
        for (size_t t = 0; t < T; ++t) {
            const uint16_t *xr = x + t * ldx;
            float acc = kind == MO_KIND_Q4_K ? dot_f16_q4_k((const blk_q4_k *)row, xr, nb, K)
                : kind == MO_KIND_Q6_K     ? dot_f16_q6_k((const blk_q6_k *)row, xr, nb, K)
                                           : dot_f16_q8_0((const blk_q8_0 *)row, xr, nb, K);
            if (bias != NULL) acc += bias[f];
            out[t * ldo + f] = acc;
        }
    }
    return 0;
}

/* ---- MoE ---- */

/* cpu_topk_impl, ops/moe/moe_ops.c:789-889: insertion top-k, equal values keep the lower column first. */
void mo_topk(const float *x, size_t rows, size_t cols, size_t ldx, size_t k, float *values, int32_t *indices) {
    for (size_t r = 0; r < rows; ++r) {
        float *bv = values + r * k;
        int32_t *bi = indices + r * k;
        for (size_t i = 0; i < k; ++i) {
            bv[i] = -FLT_MAX;
            bi[i] = -1;
        }
        for (size_t c = 0; c < cols; ++c) {
            const float v = x[r * ldx + c];
            size_t pos = k;
            for (size_t i = 0; i < k; ++i) {
                if (v > bv[i] || (v == bv[i] && (int32_t)c < bi[i])) {
                    pos = i;
                    break;
                }
            }
            if (pos == k) continue;
            for (size_t i = k - 1; i > pos; --i) {
                bv[i] = bv[i - 1];
                bi[i] = bi[i - 1];
            }
            bv[pos] = v;
            bi[pos] = (int32_t)c;
        }
    }
}

static inline float silu(float x) { return x / (1.0f + expf(-x)); }                     /* moe_ops.c:318-320 */
static inline float gelu(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f)); } /* moe_ops.c:322-324 */

/*
 * cpu_moe_execute_grouped, moe_ops.c:891-1049: histogram -> exclusive prefix ->
 * stable scatter of (token, weight*norm) -> gather hidden rows -> per expert
 * gate/up (dual-output matmul == two singles, matmul_quant_dispatch.c:593-856),
 * act(gate)*up, down matmul -> out[token] += w * down[route] in route order
 * (expert-major, token order inside an expert).  The small-batch decode variant
 * (:622-787) differs only in visiting experts in first-appearance order, which
 * changes the result only through the order of the per-token additions; this
 * oracle uses that order when T <= 4 and routes <= 64, as the reference does.
 */
int mo_moe_experts(
    int gate_kind, int up_kind, int down_kind, const float *hidden, size_t T, size_t H, size_t FF, size_t E,
    const void *gate, const void *up, const void *down, const int32_t *topk_ids, const float *topk_weights, size_t k,
    int ffn_type, float weights_scale, int policy, float *out, int n_threads
) {
    const size_t routes = T * k;
    for (size_t i = 0; i < routes; ++i)
        if (topk_ids[i] < 0 || (size_t)topk_ids[i] >= E) return -1;

    size_t *counts = (size_t *)calloc(E, sizeof(size_t));
    size_t *offsets = (size_t *)calloc(E + 1, sizeof(size_t));
    size_t *cursor = (size_t *)calloc(E, sizeof(size_t));
    size_t *order = (size_t *)calloc(E, sizeof(size_t));
    uint32_t *sorted_tok = (uint32_t *)malloc((routes + 1) * sizeof(uint32_t));
    float *sorted_w = (float *)malloc((routes + 1) * sizeof(float));
    float *route_hidden = (float *)malloc((routes * H + 1) * sizeof(float));
    float *route_down = (float *)malloc((routes * H + 1) * sizeof(float));
    float *gate_out = (float *)malloc((routes * FF + 1) * sizeof(float));
    float *up_out = (float *)malloc((routes * FF + 1) * sizeof(float));
    int rc = 0;
    if (!counts || !offsets || !cursor || !order || !sorted_tok || !sorted_w || !route_hidden || !route_down ||
        !gate_out || !up_out) {
        rc = -2;
        goto done;
    }

    for (size_t i = 0; i < routes; ++i) counts[topk_ids[i]]++;
    /* visiting order of the experts (affects only the per-token addition order) */
    size_t n_order = 0;
    const int decode = T <= 4 && routes <= 64; /* kCpuMoeDecodeMaxTokens / MaxRoutes, moe_ops.c:22-23,417-424 */
    if (decode) {
        for (size_t i = 0; i < routes; ++i) {
            const size_t e = (size_t)topk_ids[i];
            size_t j = 0;
            for (; j < n_order; ++j)
                if (order[j] == e) break;
            if (j == n_order) order[n_order++] = e;
        }
    } else {
        for (size_t e = 0; e < E; ++e)
            if (counts[e] != 0) order[n_order++] = e;
    }
    size_t prefix = 0;
    for (size_t j = 0; j < n_order; ++j) {
        offsets[order[j]] = prefix;
        cursor[order[j]] = prefix;
        prefix += counts[order[j]];
    }

    for (size_t t = 0; t < T; ++t) {
        float norm = weights_scale;
        if (policy == MO_ROUTER_POLICY_RENORMALIZE_SELECTED) {
            float s = 0.0f;
            for (size_t j = 0; j < k; ++j) s += topk_weights[t * k + j];
            norm = s > FLT_MIN ? weights_scale / s : 0.0f;
        }
        for (size_t j = 0; j < k; ++j) {
            const size_t e = (size_t)topk_ids[t * k + j];
            const size_t pos = cursor[e]++;
            sorted_tok[pos] = (uint32_t)t;
            sorted_w[pos] = topk_weights[t * k + j] * norm;
        }
    }
    for (size_t r = 0; r < routes; ++r)
        memcpy(route_hidden + r * H, hidden + (size_t)sorted_tok[r] * H, H * sizeof(float));
    memset(out, 0, T * H * sizeof(float));

    const uint8_t *gp = (const uint8_t *)gate, *upp = (const uint8_t *)up, *dp = (const uint8_t *)down;
    const size_t gate_slice = FF * mo_row_bytes(gate_kind, H);
    const size_t up_slice = FF * mo_row_bytes(up_kind, H);
    const size_t down_slice = H * mo_row_bytes(down_kind, FF);
    for (size_t j = 0; j < n_order && rc == 0; ++j) {
        const size_t e = order[j], cnt = counts[e], off = offsets[e];
        if (cnt == 0) continue;
        rc |= mo_linear(gate_kind, route_hidden + off * H, H, gp + e * gate_slice, cnt, H, FF, NULL,
                        gate_out + off * FF, FF, n_threads);
        rc |= mo_linear(up_kind, route_hidden + off * H, H, upp + e * up_slice, cnt, H, FF, NULL, up_out + off * FF,
                        FF, n_threads);
        for (size_t i = 0; i < cnt * FF; ++i) {
            const float g = gate_out[off * FF + i];
            const float a = ffn_type == MO_FFN_GEGLU ? gelu(g) : silu(g);
            gate_out[off * FF + i] = a * up_out[off * FF + i];
        }
        rc |= mo_linear(down_kind, gate_out + off * FF, FF, dp + e * down_slice, cnt, FF, H, NULL,
                        route_down + off * H, H, n_threads);
    }
    if (rc == 0) {
        for (size_t r = 0; r < routes; ++r) {
            const float w = sorted_w[r];
            const float *src = route_down + r * H;
            float *dst = out + (size_t)sorted_tok[r] * H;
            for (size_t c = 0; c < H; ++c) dst[c] += w * src[c];
        }
    }
done:
    free(counts); free(offsets); free(cursor); free(order); free(sorted_tok); free(sorted_w);
    free(route_hidden); free(route_down); free(gate_out); free(up_out);
    return rc;
}
