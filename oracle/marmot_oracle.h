/*
 * CPU oracle for the quantized GGUF matmul path of darekhta/marmot.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the arithmetic
 * the reference CPU backend performs (scalar flavour, no FMA contraction); the
 * shipped library never links, loads or calls it.  Every function names the
 * reference file:line whose operation order it follows.  The restatement is
 * pinned against the reference's own golden vectors (llama.cpp-generated
 * matmul / vec_dot / quantizer fixtures) and against the reference library
 * itself built from its sources; see tests/test_oracle_*.py.
 *
 * Dimension letters: T = tokens (rows of the activation), K = reduction
 * length, F = output features (rows of the weight matrix).
 */
#ifndef MARMOT_ORACLE_H
#define MARMOT_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    MO_KIND_Q8_0 = 5,  /* numeric values of marmot_quant_kind_t, include/marmot/types.h:373-387 */
    MO_KIND_Q4_K = 9,
    MO_KIND_Q6_K = 11,
};

enum {
    MO_Q8_0_BLOCK_BYTES = 34,
    MO_Q4_K_BLOCK_BYTES = 144,
    MO_Q6_K_BLOCK_BYTES = 210,
    MO_Q8_K_BLOCK_BYTES = 292,
};

enum { /* marmot_router_weight_policy_t, include/marmot/types.h:288-293 */
    MO_ROUTER_POLICY_SOFTMAX_SELECTED = 0,
    MO_ROUTER_POLICY_SOFTMAX_SELECTED_SCALED = 1,
    MO_ROUTER_POLICY_RENORMALIZE_SELECTED = 2,
};

enum { MO_FFN_SWIGLU = 0, MO_FFN_GELU = 1, MO_FFN_GEGLU = 2 }; /* marmot_ffn_type_t, types.h:281-286 */

size_t mo_block_values(int kind);
size_t mo_block_bytes(int kind);
size_t mo_row_bytes(int kind, size_t K);

/* block -> f32, bit-exact with the reference dequantizers */
int mo_dequantize(int kind, const void *blocks, size_t n_values, float *out);

/* f32 activations -> Q8_K / Q8_0 blocks (the matmul driver's packers) */
void mo_pack_q8_k_f32(const float *x, size_t K, void *dst_blocks);
void mo_pack_q8_0_f32(const float *x, size_t K, void *dst_blocks);

/* one weight row . one packed activation row */
float mo_vec_dot_q4_k_q8_k(const void *w, const void *a, size_t n_blocks);
float mo_vec_dot_q6_k_q8_k(const void *w, const void *a, size_t n_blocks);
float mo_vec_dot_q8_0_q8_0(const void *w, const void *a, size_t n_blocks);

/*
 * out[T,F] = x[T,K] . W[F,K]^T (+ bias[F]) for f32 activations; ldx / ldo are
 * row strides in elements.
 */
int mo_linear(
    int kind, const float *x, size_t ldx, const void *W, size_t T, size_t K, size_t F, const float *bias, float *out,
    size_t ldo, int n_threads
);
/* f16 activations, no packing: one running f32 sum per output (cpu_vec_dot_*_f16, vec_dot_impl.h) */
int mo_linear_f16(
    int kind, const uint16_t *x, size_t ldx, const void *W, size_t T, size_t K, size_t F, const float *bias, float *out,
    size_t ldo
);

/* top-k per row, ties -> lower index */
void mo_topk(const float *x, size_t rows, size_t cols, size_t ldx, size_t k, float *values, int32_t *indices);

/*
 * MoE expert FFN.  gate/up: E contiguous [FF, H] quantized matrices, down: E
 * contiguous [H, FF]; out[T,H] f32.
 */
int mo_moe_experts(
    int gate_kind, int up_kind, int down_kind, const float *hidden, size_t T, size_t H, size_t FF, size_t E,
    const void *gate, const void *up, const void *down, const int32_t *topk_ids, const float *topk_weights, size_t k,
    int ffn_type, float weights_scale, int policy, float *out, int n_threads
);

/* ---- decoder operators around the matmuls (marmot_oracle_decoder.c) ---- */
void mo_rmsnorm_f32(const float *x, const float *residual, const float *weight, size_t rows, size_t n, float eps,
                    float weight_offset, float *out);
void mo_rope_f32(const float *x, const int32_t *positions, size_t rows, size_t dim, float theta, float freq_scale,
                 int neox, float *out);
void mo_swiglu_f32(const float *a, const float *b, size_t n, float *out);
int mo_paged_attention_f32(const uint32_t *token_meta, size_t T, const float *q, const float *k_new, const float *v_new,
                           void *kv_k, void *kv_v, int kv_is_half, int kv_truncate, const uint32_t *block_table,
                           size_t max_blocks_per_seq, size_t n_layers, size_t layer, size_t n_q_heads,
                           size_t n_kv_heads, size_t head_dim, size_t block_size, float scale, float *out);
int mo_embedding_gather(int kind, const void *table, size_t dim, const int32_t *ids, size_t T, float *out);
void mo_argmax_f32(const float *x, size_t rows, size_t n, int32_t *out);

#ifdef __cplusplus
}
#endif
#endif
