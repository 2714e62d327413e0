/*
 * libmarmot_cuda: hand-written sm_100a kernels for marmot's quantized GGUF matmul path behind a
 * thin C ABI.  Plain pointers and sizes only; no marmot, torch or C++ types cross this boundary.
 *
 * This is the layer the reference's generated CUDA dispatch entries call.  In the reference the
 * same position is held by the CPU backend's implementation functions named by the kernel-DSL
 * `.def` files (IMPL_FUNCTION), which the generated `*_exec` wrappers invoke; each declaration
 * below cites the reference function it stands in for (paths relative to the reference tree).
 *
 * Conventions
 *   - T = tokens (rows of the activation), K = reduction length, F = output features.  The
 *     reference calls these N, K, M (include/marmot/ops/matmul.h:11).
 *   - `kind` is the numeric marmot_quant_kind_t (include/marmot/types.h:373-387):
 *     Q8_0 = 5, Q4_K = 9, Q6_K = 11.  Weights are raw GGUF blocks, row-major [F][ceil(K/bv)].
 *   - Return value: 0 on success, otherwise the negative marmot_error_t code
 *     (include/marmot/types.h:210-220).  A message is kept per thread, see
 *     mcu_last_error_message().
 *   - Functions taking `*_dev` pointers expect device memory and only enqueue work on the
 *     context's stream; functions with `_host` in the name take host memory, copy in and out on
 *     that stream and return after the result is in host memory.
 *   - Quantized weights are model constants: a matmul starts streaming them before the kernel
 *     enqueued ahead of it on the stream has finished (programmatic dependent launch; only the
 *     activations, bias and output wait for it).  Weights produced by a kernel on the same stream
 *     must therefore be complete (stream or event synchronised) before the first matmul that reads
 *     them is enqueued; weights brought in by mcu_memcpy_to_device or cudaMemcpy* need nothing.
 *   - There is no CPU fallback: every entry point fails with MCU_ERROR_DEVICE_NOT_AVAILABLE when
 *     no CUDA device can be used.
 */
#ifndef MARMOT_CUDA_H
#define MARMOT_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    MCU_SUCCESS = 0,
    MCU_ERROR_INVALID_ARGUMENT = -1,
    MCU_ERROR_OUT_OF_MEMORY = -2,
    MCU_ERROR_DEVICE_NOT_AVAILABLE = -3,
    MCU_ERROR_BACKEND_INIT_FAILED = -4,
    MCU_ERROR_INVALID_OPERATION = -5,
    MCU_ERROR_UNSUPPORTED_DTYPE = -6,
    MCU_ERROR_DIMENSION_MISMATCH = -7,
    MCU_ERROR_NOT_IMPLEMENTED = -8,
};

enum { MCU_KIND_Q8_0 = 5, MCU_KIND_Q4_K = 9, MCU_KIND_Q6_K = 11 };

/* marmot_router_weight_policy_t / marmot_ffn_type_t values (include/marmot/types.h:281-293) */
enum { MCU_ROUTER_SOFTMAX_SELECTED = 0, MCU_ROUTER_SOFTMAX_SELECTED_SCALED = 1, MCU_ROUTER_RENORMALIZE_SELECTED = 2 };
enum { MCU_FFN_SWIGLU = 0, MCU_FFN_GELU = 1, MCU_FFN_GEGLU = 2 };

/* Regime override for mcu_linear*: the analogue of the reference's MARMOT_METAL_FORCE_{MV,MM}
 * switches (src/backends/metal/ops/matmul_quant_dispatch.mm:41). */
enum {
    MCU_REGIME_AUTO = 0,
    MCU_REGIME_GEMV = 1,       /* decode kernels for every T (tokens processed eight at a time) */
    MCU_REGIME_GEMM = 2,       /* tensor-core kernel for every T */
    MCU_REGIME_GEMV_PLAIN = 3, /* decode kernels without the shared-memory streaming variant */
    MCU_REGIME_I8MMA = 4,      /* integer tensor-core kernel wherever it applies (2..64 tokens, Q4_K / Q6_K) */
};

typedef struct mcu_context mcu_context_t;

/* ---- context: the device half of marmot_device_ops (include/marmot/device.h:43-66);
 *      stands in for cpu_init / cpu_destroy / cpu_synchronize
 *      (src/backends/cpu/runtime/runtime.c:1409-1443, src/backends/cpu/dispatch/device_ops.c:12-30). ---- */
/* What marmot_cuda_detect_default_caps fills marmot_device_caps_t from (include/marmot/device_caps.h:14-71; the reference
 * reserves backend.cuda.{sm_count, shared_mem_kb, compute_capability} there).  MCU_ERROR_DEVICE_NOT_AVAILABLE when the
 * process sees no such device. */
typedef struct mcu_device_caps {
    int sm_count;
    int compute_capability;  /* 100 for sm_100 */
    int shared_mem_kb;       /* per SM */
    int l2_cache_kb;
    int sm_clock_mhz;
    float mem_bw_gbps;       /* nominal: 2 x memory clock x bus width */
    size_t total_mem_bytes;
    int copy_engines;
} mcu_device_caps_t;
int mcu_device_caps(int device, mcu_device_caps_t *out);

int mcu_context_create(int device, mcu_context_t **out);
void mcu_context_destroy(mcu_context_t *ctx);
/* Use a stream owned by the caller (cudaStream_t passed as void*); NULL restores the context's own
 * non-blocking stream.  To run on the legacy default stream pass cudaStreamLegacy ((void*)0x1). */
int mcu_context_set_stream(mcu_context_t *ctx, void *cuda_stream);
void *mcu_context_get_stream(mcu_context_t *ctx);
int mcu_context_set_regime(mcu_context_t *ctx, int regime);

/* ---- CUDA-graph capture: what graph_batch_begin / graph_batch_end of the device-ops vtable bracket
 *      (include/marmot/device.h:59-60, called around a bytecode program by src/core/context/context.c:260-286).
 *      Every call between begin and end is recorded on the context's stream instead of run; mcu_graph_launch replays
 *      the whole sequence with one launch (a decode step of a few hundred small kernels is bound by launch latency
 *      otherwise).  Run the sequence once before capturing: workspace cannot grow during a capture, and the entry
 *      points that wait for the device (mcu_linear_host, mcu_vec_dot_host, mcu_moe_experts, mcu_synchronize) refuse
 *      to be captured.  The recorded pointers are the ones passed during capture: update inputs in place. ---- */
typedef struct mcu_graph mcu_graph_t;
int mcu_graph_capture_begin(mcu_context_t *ctx);
int mcu_graph_capture_end(mcu_context_t *ctx, mcu_graph_t **out_graph); /* out_graph NULL: discard the capture */
int mcu_graph_launch(mcu_graph_t *graph);
void mcu_graph_destroy(mcu_graph_t *graph);
int mcu_synchronize(mcu_context_t *ctx);
const char *mcu_last_error_message(void);
/* Number of kernels this context has launched so far. */
uint64_t mcu_kernel_launch_count(const mcu_context_t *ctx);

/* ---- device memory: alloc / free / memcpy slots of marmot_device_ops (include/marmot/device.h:47-56) ---- */
int mcu_malloc(mcu_context_t *ctx, size_t bytes, void **out_dev);
int mcu_free(mcu_context_t *ctx, void *dev);
/* mcu_memcpy_to_device returns when src_host may be reused; the copy itself is ordered on the context's stream before
 * everything enqueued after it (copies of up to 64 KB go through page-locked slots of the context and do not wait for
 * the device; larger ones do).  mcu_memcpy_to_host returns with the bytes in dst_host. */
int mcu_memcpy_to_device(mcu_context_t *ctx, void *dst_dev, const void *src_host, size_t bytes);
int mcu_memcpy_to_host(mcu_context_t *ctx, void *dst_host, const void *src_dev, size_t bytes);

size_t mcu_row_bytes(int kind, size_t K);

/* ---- dequantize: cpu_dequantize_{q4_k,q6_k,q8_0}
 *      (src/backends/cpu/quantization/formats/q4k_gguf.c:133-166, q6k_gguf.c:63-99,
 *       q8_gguf.c:110-114,189-200; row loop quantization/ops/quantize_core.c:267-331). Bit-exact. ---- */
int mcu_dequantize(mcu_context_t *ctx, int kind, const void *blocks_dev, size_t n_values, float *out_dev);

/* ---- activation packers: cpu_matmul_quant_pack_q8_k_f32 / cpu_matmul_quant_pack_q8_0_f32
 *      (src/backends/cpu/ops/matmul/quantized/matmul_quant_pack.c:106-169, :23-62). Bit-exact values in a
 *      structure-of-arrays layout: qs[T][kp] int8 (kp = K rounded up to the block size; within each
 *      256-value Q8_K block the value 64g+32b+i is stored at b*128+g*32+i), d[T][nb] f32,
 *      bsums[T][nb*16] int16 (Q8_K only, may be NULL for Q8_0). ---- */
int mcu_quantize_activations(
    mcu_context_t *ctx, int weight_kind, const float *x_dev, size_t ldx, size_t T, size_t K, int8_t *qs_dev,
    float *d_dev, int16_t *bsums_dev
);

/* ---- quantized row dot: cpu_vec_dot (src/backends/cpu/ops/vec_dot/vec_dot.c:6-65, the public marmot_vec_dot),
 *      the building block the reference's own golden vectors pin (tests/backend/golden_vec_dot_llama.h).
 *      One weight row of num_blocks GGUF blocks times one PRE-QUANTIZED activation row given as the reference's
 *      block structs (Q8_K blocks of 292 bytes {f32 d, int8 qs[256], int16 bsums[16]} for the K-quants,
 *      Q8_0 blocks of 34 bytes for Q8_0), both in host memory as in the reference API; the integer dots and the
 *      per-block f32 terms are those of the decode kernels. ---- */
int mcu_vec_dot_host(
    mcu_context_t *ctx, int weight_kind, const void *weights_host, const void *activations_host, size_t num_blocks,
    float *result_host
);

/* ---- quantized linear: cpu_matmul_quantized_{q4_k,q6_k,q8_0} -> cpu_matmul_quantized_impl
 *      (src/backends/cpu/ops/matmul/quantized/matmul_quant_dispatch.c:373-591,905-960) with the bias epilogue of
 *      cpu_matmul_apply_epilogue (src/backends/cpu/ops/matmul/matmul_epilogue.c).
 *      out[t*ldo + f] = sum_k x[t*ldx + k] * W[f][k] (+ bias[f]); f32 in, f32 out. ---- */
int mcu_linear(
    mcu_context_t *ctx, int kind, const float *x_dev, size_t ldx, const void *w_dev, size_t T, size_t K, size_t F,
    const float *bias_dev, float *out_dev, size_t ldo
);

/* ---- FLOAT16 activations: the branch of cpu_matmul_quantized_impl taken for f16 inputs
 *      (matmul_quant_dispatch.c:449-470): no activation packing, out[t][f] = sum_k w(f, k) * (float)x[t][k] in f32 with
 *      w formed as cpu_vec_dot_{q4_k,q6_k,q8_0}_f16 form it (vec_dot_impl.h:419-447,973-1023,1082-1127; the Q6_K
 *      function reads the block linearly, not as the dequantizer does, and its golden output pins that).
 *      x_f16_dev: IEEE half bits; out_dtype MCU_OUT_F32 (float *out_dev) or MCU_OUT_F16 (half bits, no bias). ---- */
enum { MCU_OUT_F32 = 0, MCU_OUT_F16 = 1 };
int mcu_linear_f16(
    mcu_context_t *ctx, int kind, const uint16_t *x_f16_dev, size_t ldx, const void *w_dev, size_t T, size_t K, size_t F,
    const float *bias_dev, void *out_dev, size_t ldo, int out_dtype
);

/* ---- two weights, one activation read: cpu_matmul_quantized_dual_output
 *      (matmul_quant_dispatch.c:593-856); gate/up of the FFN and of MoE experts. ---- */
int mcu_linear_dual(
    mcu_context_t *ctx, int kind, const float *x_dev, size_t ldx, const void *w_a_dev, const void *w_b_dev, size_t T,
    size_t K, size_t F, float *out_a_dev, float *out_b_dev, size_t ldo
);

/* ---- several weights, one activation read, optionally through one of the decoder layer's elementwise steps:
 *      marmot_matmul_qkv_shared_input with separate wq / wk / wv (include/marmot/ops/matmul.h:74-122,
 *      src/backends/cpu/ops/matmul/qkv/matmul_qkv.c) generalised to 1..4 weights that may differ in kind and F, plus
 *      the step that produces the activations in the GGUF graph (src/graph/gguf/graph_builder.cpp:1454-2400):
 *        MCU_PROLOGUE_ADD_RMSNORM  x' = x + aux (aux may be NULL); the weights multiply
 *                                  rms_norm(x') * (norm_weight + weight_offset); x' is stored to x_out when that is
 *                                  set.  x_out must not overlap x or aux.
 *        MCU_PROLOGUE_SWIGLU       the weights multiply silu(x) * aux (x = gate, aux = up projection)
 *      Up to 8 tokens with every weight on the streaming path this is ONE launch -- except for 5 to 8 tokens over 24 MB
 *      or more of Q4_K / Q6_K weights, where the integer-MMA kernel behind a stand-alone prologue kernel is faster than
 *      the one launch; more than 16 tokens: the prologue rides in the tensor-core path's activation staging; otherwise the
 *      prologue runs as its stand-alone kernel (which needs contiguous rows: ldx = ld_aux = ld_x_out = K) followed by
 *      the matmuls. ---- */
enum { MCU_PROLOGUE_NONE = 0, MCU_PROLOGUE_ADD_RMSNORM = 1, MCU_PROLOGUE_SWIGLU = 2 };
#define MCU_LINEAR_MAX_JOBS 4
typedef struct mcu_linear_job {
    int kind;
    const void *w_dev;
    size_t F;
    const float *bias_dev; /* may be NULL */
    float *out_dev;
    size_t ldo;
} mcu_linear_job_t;
typedef struct mcu_prologue {
    int op;
    const float *aux_dev;
    size_t ld_aux;
    const float *norm_weight_dev; /* may be NULL: plain normalisation */
    float eps, weight_offset;
    float *x_out_dev; /* may be NULL */
    size_t ld_x_out;
} mcu_prologue_t;
int mcu_linear_multi(
    mcu_context_t *ctx, const float *x_dev, size_t ldx, size_t T, size_t K, const mcu_prologue_t *prologue,
    const mcu_linear_job_t *jobs, size_t n_jobs
);

/* Same as mcu_linear with host activations / bias / output; weights stay device resident (made so once
 * with mcu_malloc + mcu_memcpy_to_device, the residency contract of marmot_tensor_to_device,
 * src/core/tensor/transfer.c:22). */
int mcu_linear_host(
    mcu_context_t *ctx, int kind, const float *x_host, size_t ldx, const void *w_dev, size_t T, size_t K, size_t F,
    const float *bias_host, float *out_host, size_t ldo
);

/* ---- mcu_linear without any allocation.  No counterpart in the reference: it exists for callers of this
 *      library that cannot call cudaMalloc at the time they need a matmul, for example code running after a
 *      serving engine or a caching allocator has reserved all of the device memory (a further cudaMalloc
 *      would fail), or a latency-critical thread that cannot afford the device-wide synchronisation a
 *      cudaMalloc / cudaFree implies.  Same arithmetic as mcu_linear's decode kernels (f32 activations packed to
 *      Q8_K / Q8_0, integer dots, per-block f32 scaling), limited to T <= MCU_STATIC_SCRATCH_MAX_T tokens and
 *      K <= MCU_STATIC_SCRATCH_MAX_K; larger sizes are rejected with MCU_ERROR_INVALID_ARGUMENT.
 *      The packed activations go to a fixed 160 KiB array inside the library's device image (each GPU that
 *      loads the library holds it until the process exits).  The call takes no context and performs no
 *      cudaMalloc, cudaFree or other allocating call; it enqueues two kernels on `cuda_stream` (a cudaStream_t,
 *      NULL = default stream) of the current device.  The first call on each device looks up the array's
 *      device address (cudaGetSymbolAddress); make that first call outside of any stream capture.  With lazy
 *      module loading that first call is also when the driver loads the two kernels and the array onto the
 *      device, which may itself take device memory: make it early, before the rest of the device memory is
 *      reserved, so that later calls are certain to need nothing.
 *      All calls share the one array and it keeps the last call's contents.  Nothing in it needs clearing
 *      (each call rewrites every byte it later reads), but two calls that overlap on the GPU, e.g. on
 *      different streams, race on it: serialise them. ---- */
#define MCU_STATIC_SCRATCH_MAX_T 8
#define MCU_STATIC_SCRATCH_MAX_K 16384
int mcu_linear_static_scratch(
    void *cuda_stream, int kind, const float *x_dev, size_t ldx, const void *w_dev, size_t T, size_t K, size_t F,
    const float *bias_dev, float *out_dev, size_t ldo
);

/* ---- top-k over the last axis, ties to the lower index: cpu_topk_impl
 *      (src/backends/cpu/ops/moe/moe_ops.c:789-889). ---- */
int mcu_topk(
    mcu_context_t *ctx, const float *x_dev, size_t rows, size_t cols, size_t ldx, size_t k, float *values_dev,
    int32_t *indices_dev
);

/* ---- MoE expert FFN: cpu_moe_experts_impl -> cpu_moe_execute_grouped / cpu_moe_execute_decode
 *      (src/backends/cpu/ops/moe/moe_ops.c:1069-1178, 891-1049, 622-787).
 *      hidden [T][H] f32; gate/up: E contiguous [FF][H] quantized matrices; down: E contiguous [H][FF];
 *      topk_ids [T][k] int32, topk_weights [T][k] f32; out [T][H] f32.
 *      With T * k >= 256 (gate and up of one kind, weight rows a multiple of 16 bytes) the call reads nothing back: it is
 *      asynchronous, may be recorded by mcu_graph_capture_begin/end, and an expert id outside [0, E) is reported by the
 *      next mcu_synchronize as MCU_ERROR_INVALID_ARGUMENT.  Smaller batches read the group sizes back (one stream
 *      synchronisation), report a bad id from the call itself and refuse to be captured. ---- */
int mcu_moe_experts(
    mcu_context_t *ctx, int gate_kind, int up_kind, int down_kind, const float *hidden_dev, size_t T, size_t H,
    size_t FF, size_t E, const void *gate_dev, const void *up_dev, const void *down_dev, const int32_t *topk_ids_dev,
    const float *topk_weights_dev, size_t k, int ffn_type, float weights_scale, int router_weight_policy,
    float *out_dev
);

/* ---- decoder operators around the matmuls (f32 activations), the callers of the hot path in a decode step:
 *      marmot_rmsnorm (src/backends/cpu/ops/normalization/scalar/normalization_scalar.c:780-833),
 *      marmot_rope (src/backends/cpu/ops/rope/rope_dispatch.c:144-382; no YaRN / long-rope scaling),
 *      marmot_swiglu / marmot_add (src/backends/cpu/ops/elementwise/scalar/elementwise_f32_scalar.c),
 *      marmot_paged_attention (include/marmot/ops/paged_attention.h:32-56,
 *      src/backends/cpu/ops/paged_attention/paged_attention_ref.c:599-1082),
 *      marmot_embedding_gather on a block-quantized table, marmot_reduce_argmax over the last axis. ---- */
enum { MCU_ROPE_NORM = 0, MCU_ROPE_NEOX = 1 }; /* marmot_rope_type_t, include/marmot/types.h:263-267 */
enum { MCU_KV_F32 = 0, MCU_KV_F16 = 1 };       /* dtype of the paged KV pool */

/* out = (x [+ residual]) * rsqrt(mean((x [+ residual])^2) + eps) * (weight + weight_offset); residual and weight may
 * be NULL; rows x n contiguous. */
int mcu_rmsnorm(
    mcu_context_t *ctx, const float *x_dev, const float *residual_dev, const float *weight_dev, size_t rows, size_t n,
    float eps, float weight_offset, float *out_dev
);
/* x [T][n_heads][head_dim] with row stride ldx (floats), one int32 position per token; pairs (2i, 2i+1) for
 * MCU_ROPE_NORM, (i, i + head_dim/2) for MCU_ROPE_NEOX; angle = pos * theta^(-2i/head_dim) * freq_scale. */
int mcu_rope(
    mcu_context_t *ctx, const float *x_dev, size_t ldx, const int32_t *positions_dev, size_t T, size_t n_heads,
    size_t head_dim, float theta, float freq_scale, int rope_type, float *out_dev, size_t ldo
);
/* Two reference operators in one launch each (same arithmetic as the separate calls):
 *   mcu_add_rmsnorm  x_out = x + delta, h_out = rmsnorm(x_out) * (weight + offset)   (marmot_add, then marmot_rmsnorm);
 *   mcu_rope_qk      mcu_rope in place on the query and the key projection of the same tokens. */
int mcu_add_rmsnorm(
    mcu_context_t *ctx, const float *x_dev, const float *delta_dev, const float *weight_dev, size_t rows, size_t n,
    float eps, float weight_offset, float *x_out_dev, float *h_out_dev
);
int mcu_rope_qk(
    mcu_context_t *ctx, float *q_dev, size_t ldq, size_t n_q_heads, float *k_dev, size_t ldk, size_t n_k_heads,
    const int32_t *positions_dev, size_t T, size_t head_dim, float theta, float freq_scale, int rope_type
);
int mcu_swiglu(mcu_context_t *ctx, const float *gate_dev, const float *up_dev, size_t n, float *out_dev);
int mcu_add(mcu_context_t *ctx, const float *a_dev, const float *b_dev, size_t n, float *out_dev);
int mcu_argmax(mcu_context_t *ctx, const float *x_dev, size_t rows, size_t n, int32_t *out_dev);
/* out [T][dim] = dequantised rows ids[t] of a quantized [rows][dim] table (bit-exact with mcu_dequantize). */
int mcu_embedding_gather(
    mcu_context_t *ctx, int kind, const void *table_dev, size_t dim, const int32_t *ids_dev, size_t T, float *out_dev
);
/* Paged attention for T tokens (decode steps and prefill chunks alike).  token_meta [T][4] u32 = {seq_slot, pos, kv_slot,
 * flags}; q/out [T][n_q_heads][head_dim], k_new/v_new [T][n_kv_heads][head_dim], contiguous; the KV pool
 * [blocks][n_layers][n_kv_heads][block_size][head_dim] (f32 or f16) first receives the new rows at kv_slot
 * (block = kv_slot / block_size; f16 pools round to nearest even like the reference's NEON / F16C conversions), then
 * every token attends to positions 0..pos of its sequence through block_table [seqs][max_blocks_per_seq]
 * (0xFFFFFFFF = no block).  head_dim 64 or 128. */
int mcu_paged_attention(
    mcu_context_t *ctx, const uint32_t *token_meta_dev, size_t T, const float *q_dev, const float *k_new_dev,
    const float *v_new_dev, void *kv_k_dev, void *kv_v_dev, int kv_dtype, const uint32_t *block_table_dev,
    size_t max_blocks_per_seq, size_t n_layers, size_t layer, size_t n_q_heads, size_t n_kv_heads, size_t head_dim,
    size_t block_size, float scale, float *out_dev
);
/* The decode step's form of the same: RoPE of q and k_new (marmot_rope, or the rope_params of marmot_matmul_qkv,
 * include/marmot/ops/matmul.h:83-95), the append, the attention and the merge of the context chunks as ONE launch.
 * q_dev and k_new_dev hold the projections BEFORE RoPE; they may be rotated in place (callers must not reuse them).
 * rope_table_dev [T][head_dim/2][2] = {cos, sin} of position * frequency from mcu_rope_table, made once per step and
 * shared by all layers; NULL makes the call compute one itself (one more launch).
 * Precondition: at most one token per sequence in the call (a token's own K/V row is taken from k_new / v_new, every
 * other position from the pool, so rows appended by the same call are not seen by the call's other tokens); prefill
 * chunks use mcu_rope_qk + mcu_paged_attention.  f16 pools run fused; f32 pools run the stand-alone kernels. */
int mcu_rope_table(
    mcu_context_t *ctx, const int32_t *positions_dev, size_t T, size_t head_dim, float theta, float freq_scale,
    float *table_dev
);
int mcu_paged_attention_decode(
    mcu_context_t *ctx, const uint32_t *token_meta_dev, size_t T, float *q_dev, float *k_new_dev, const float *v_new_dev,
    void *kv_k_dev, void *kv_v_dev, int kv_dtype, const uint32_t *block_table_dev, size_t max_blocks_per_seq,
    size_t n_layers, size_t layer, size_t n_q_heads, size_t n_kv_heads, size_t head_dim, size_t block_size, float scale,
    const int32_t *positions_dev, float rope_theta, float rope_freq_scale, int rope_type, const float *rope_table_dev,
    float *out_dev
);

/* ---- GGUF model files: the reading half of the reference's loader (src/graph/gguf/loader.cpp) and the uploads of
 *      a tensor-parallel rank.  The file is memory-mapped and indexed once; payloads go to the device straight out of
 *      the mapping: whole tensors and row ranges (column-parallel shards) as one copy, a K range of every row
 *      (row-parallel shards: a run of blocks per row) as one strided 2-D copy into a packed [rows][K shard] matrix.
 *      GGUF versions 2 and 3; dims[0] is the innermost (K) extent as in the file. ---- */
typedef struct mcu_gguf mcu_gguf_t;
typedef struct mcu_gguf_tensor_info {
    const char *name;      /* owned by the handle */
    uint32_t ggml_type;    /* 0 F32, 1 F16, 8 Q8_0, 12 Q4_K, 14 Q6_K, ... */
    int kind;              /* MCU_KIND_* for the three block formats with kernels, else -1 */
    uint32_t n_dims;
    uint64_t dims[4];
    size_t nbytes;         /* 0 when the type's layout is unknown to this library */
    const void *data;      /* host pointer into the mapping */
} mcu_gguf_tensor_info_t;
int mcu_gguf_open(const char *path, mcu_gguf_t **out);
void mcu_gguf_close(mcu_gguf_t *g);
size_t mcu_gguf_tensor_count(const mcu_gguf_t *g);
int mcu_gguf_find_tensor(const mcu_gguf_t *g, const char *name); /* index, or -1 */
int mcu_gguf_tensor_info(const mcu_gguf_t *g, size_t index, mcu_gguf_tensor_info_t *out);
/* metadata by key: integers (any width, bool; arrays answer with their length), floats, strings */
int mcu_gguf_meta_u64(const mcu_gguf_t *g, const char *key, uint64_t *out);
int mcu_gguf_meta_f64(const mcu_gguf_t *g, const char *key, double *out);
int mcu_gguf_meta_str(const mcu_gguf_t *g, const char *key, const char **out, size_t *out_len);
/* rows [row_lo, row_hi) x values [k_lo, k_hi) of tensor `index` -> dst_dev, packed; asynchronous on the context's stream
 * (the mapping must stay open until the stream has passed the copy) */
int mcu_gguf_upload(
    mcu_context_t *ctx, const mcu_gguf_t *g, size_t index, size_t row_lo, size_t row_hi, size_t k_lo, size_t k_hi,
    void *dst_dev
);

/* ---- one decode step (one token) of a Llama-family decoder as ONE persistent kernel.  The op sequence of
 *      src/graph/gguf/graph_builder.cpp:1454-2400 for a single token -- per layer: add + rms_norm, q/k/v, rope, paged
 *      attention with KV append, o projection, add + rms_norm, gate/up, swiglu, down; then add + rms_norm and the output
 *      projection -- with the CTAs resident for the whole step (cooperative launch), grid-wide barriers between the
 *      dependent phases and the weight stream running across them.  The plan fixes every pointer: the caller puts the
 *      embedded token into x0, the token's {seq slot, position, kv slot, flags} into token_meta and the {cos, sin} table of
 *      its position (mcu_rope_table) into rope_table, runs the plan, and finds the logits in `logits`.  Q4_K / Q6_K
 *      weights, float16 KV pool, head_dim 64 or 128; the matmul arithmetic is that of mcu_linear_multi (same device
 *      functions), the attention is f32 on the f16 pool.  Bounded waits: a barrier that runs out sets the error reported by
 *      mcu_synchronize.  The launch can be recorded into a CUDA graph. ---- */
typedef struct mcu_decode_layer {
    int kind_q, kind_k, kind_v, kind_o, kind_gate, kind_up, kind_down;
    const void *wq, *wk, *wv, *wo, *gate, *up, *down;
    const float *attn_norm, *ffn_norm;
} mcu_decode_layer_t;
typedef struct mcu_decode_plan_desc {
    size_t n_layers, d, ffn, n_q_heads, n_kv_heads, head_dim, vocab;
    float rms_eps, attn_scale;
    int rope_type;
    const mcu_decode_layer_t *layers; /* host array [n_layers] */
    const float *out_norm;
    int kind_output;
    const void *output;
    float *x0, *x1;                           /* residual stream, two buffers [d] */
    float *q, *k, *v, *att, *proj, *gate, *up; /* scratch: [d], [kv], [kv], [d], [d], [ffn], [ffn] */
    float *logits;                            /* [vocab] */
    const uint32_t *token_meta;               /* [4] */
    const uint32_t *block_table;
    size_t max_blocks_per_seq;
    void *kv_k, *kv_v;
    int kv_dtype;
    size_t block_size;
    const float *rope_table; /* [head_dim / 2][2] */
} mcu_decode_plan_desc_t;
typedef struct mcu_decode_plan mcu_decode_plan_t;
int mcu_decode_plan_create(mcu_context_t *ctx, const mcu_decode_plan_desc_t *desc, mcu_decode_plan_t **out_plan);
int mcu_decode_plan_run(mcu_decode_plan_t *plan);
/* Timeline of the last run, the device's nanosecond clock as CTA 0 saw it: at the start of every phase (per layer:
 * q/k/v, attention, o projection, gate/up, down; then the output projection) and at the end (n_phases + 1 values),
 * then per phase two more: activations packed (matmul phases; 0 otherwise) and phase work done, before the grid
 * barrier.  3 * n_phases + 1 values.  Waits for the stream.  With out == NULL or capacity too small only *n_out is
 * set. */
int mcu_decode_plan_phase_times(mcu_decode_plan_t *plan, unsigned long long *out, size_t capacity, size_t *n_out);
void mcu_decode_plan_destroy(mcu_decode_plan_t *plan);

/* ---- paged KV-cache pool: marmot_kv_pool_* (include/marmot/inference/kv_pool.h:65-101, implementation
 *      src/inference/kv_pool/kv_pool.cpp).  Same bookkeeping, decision for decision (slot and block order, reference
 *      counts and copy on write for shared prefixes, retained blocks, swap with the exchange path, error codes); the K
 *      and V pools [blocks][layers][kv_heads][block_size][head_dim] and the block table [max_seqs][max_blocks_per_seq]
 *      u32 live in device memory (what mcu_paged_attention reads), swap blocks in page-locked host memory, and every
 *      table edit, clone and swap is an asynchronous copy on the context's stream: kernels enqueued after a call see
 *      its effect, and nothing waits for the device.  kv_slot = (block_id << log2(block_size)) | offset, as in the
 *      reference.  A pool created with ctx == NULL keeps books only (no storage), for admission planning.
 *      FP8 pools (per-block scales) are not covered: MCU_ERROR_UNSUPPORTED_DTYPE. ---- */
#define MCU_BLOCK_ID_INVALID 0xFFFFFFFFu
enum { MCU_KV_POOL_FLAG_NONE = 0, MCU_KV_POOL_FLAG_DETERMINISTIC_ALLOC = 1 };
typedef struct mcu_kv_pool mcu_kv_pool_t;
typedef struct mcu_kv_pool_options {
    uint64_t flags;
    size_t max_seqs, max_seq_len, block_size;
    size_t num_blocks, num_swap_blocks, num_layers, num_kv_heads, head_dim;
    int kv_dtype; /* MCU_KV_F32 / MCU_KV_F16 */
} mcu_kv_pool_options_t;
typedef struct mcu_kv_append_plan {
    uint32_t seq;
    size_t token_count;
    uint64_t cookie;
} mcu_kv_append_plan_t;
typedef struct mcu_kv_prefix_plan {
    uint32_t seq;
    size_t num_blocks, prefix_len;
    uint64_t cookie;
} mcu_kv_prefix_plan_t;
int mcu_kv_pool_options_init(mcu_kv_pool_options_t *opts);
int mcu_kv_pool_create(mcu_context_t *ctx, const mcu_kv_pool_options_t *opts, mcu_kv_pool_t **out_pool);
void mcu_kv_pool_destroy(mcu_kv_pool_t *pool);
int mcu_kv_pool_acquire_seq(mcu_kv_pool_t *pool, uint32_t *out_seq);
int mcu_kv_pool_release_seq(mcu_kv_pool_t *pool, uint32_t seq);
int mcu_kv_pool_prepare_append(
    mcu_kv_pool_t *pool, uint32_t seq, size_t token_count, mcu_kv_append_plan_t *out_plan, uint32_t *out_slots,
    size_t *out_start_pos
);
int mcu_kv_pool_commit_append(mcu_kv_pool_t *pool, const mcu_kv_append_plan_t *plan);
void mcu_kv_pool_abort_append(mcu_kv_pool_t *pool, const mcu_kv_append_plan_t *plan);
int mcu_kv_pool_prepare_prefix_attach(
    mcu_kv_pool_t *pool, uint32_t seq, const uint32_t *block_ids, size_t num_blocks, size_t prefix_len,
    mcu_kv_prefix_plan_t *out_plan
);
int mcu_kv_pool_commit_prefix_attach(mcu_kv_pool_t *pool, const mcu_kv_prefix_plan_t *plan);
void mcu_kv_pool_abort_prefix_attach(mcu_kv_pool_t *pool, const mcu_kv_prefix_plan_t *plan);
/* device pointers of the K pool, the V pool and the block table (marmot_kv_pool_get_tensors); NULL for a books-only pool */
int mcu_kv_pool_get_pointers(
    mcu_kv_pool_t *pool, void **out_k_dev, void **out_v_dev, uint32_t **out_block_table_dev, size_t *out_max_blocks_per_seq
);
size_t mcu_kv_pool_free_block_count(mcu_kv_pool_t *pool);
size_t mcu_kv_pool_total_block_count(mcu_kv_pool_t *pool);
size_t mcu_kv_pool_seq_len(mcu_kv_pool_t *pool, uint32_t seq);
uint32_t mcu_kv_pool_block_id(mcu_kv_pool_t *pool, uint32_t seq, size_t logical_block);
uint32_t mcu_kv_pool_block_generation(mcu_kv_pool_t *pool, uint32_t block_id);
void mcu_kv_pool_set_block_retained(mcu_kv_pool_t *pool, uint32_t block_id, int retained);
int mcu_kv_pool_swap_out_seq(mcu_kv_pool_t *pool, uint32_t seq);
int mcu_kv_pool_swap_in_seq(mcu_kv_pool_t *pool, uint32_t seq);
int mcu_kv_pool_is_seq_swapped(mcu_kv_pool_t *pool, uint32_t seq, int *out_swapped);

/* ---- tensor / expert parallelism over the GPUs of one box.  No reference counterpart: the reference runs on
 *      one device (include/marmot/device.h:72-80) and only reserves placeholders for sharding
 *      (include/marmot/graph/kernel_selection.h:18-23). ---- */

/* MoE expert FFN of the experts [expert_begin, expert_begin + expert_count) only: gate/up/down hold those
 * experts' matrices, topk_ids still name experts of the whole model (0..E-1), router weights are normalised
 * over all selected experts, and routes to other experts add nothing to out.  Summing the outputs of ranks
 * that partition the experts gives mcu_moe_experts' result. */
int mcu_moe_experts_local(
    mcu_context_t *ctx, int gate_kind, int up_kind, int down_kind, const float *hidden_dev, size_t T, size_t H,
    size_t FF, size_t E, size_t expert_begin, size_t expert_count, const void *gate_dev, const void *up_dev,
    const void *down_dev, const int32_t *topk_ids_dev, const float *topk_weights_dev, size_t k, int ffn_type,
    float weights_scale, int router_weight_policy, float *out_dev
);

/* The intermediate results of the context's last mcu_moe_experts / mcu_moe_experts_local call, for checking the
 * operator stage by stage: device pointers into the context's workspace, valid until the next MoE call on the
 * context (synchronize first).  Rows are in sorted-route order (expert-major, then route order): sorted_tok[r] is the
 * token of sorted route r, offsets[e] .. offsets[e+1] are expert e's rows.  gate_out holds the gate projection where
 * the GLU is applied by the consumer of the down projection (T * k >= 256), act(gate) * up otherwise. */
typedef struct mcu_moe_buffers {
    const int32_t *offsets;     /* [E + 1] */
    const int32_t *sorted_tok;  /* [routes] */
    const float *sorted_w;      /* [routes] normalised router weights */
    const int32_t *route_pos;   /* [T * k] sorted position of every route, -1 for a rejected expert id */
    const float *gate_out;      /* [routes][FF] */
    const float *up_out;        /* [routes][FF] */
    const float *route_down;    /* [routes][H] */
    size_t routes, experts;
    int grouped;                /* 1 when the grouped launches ran (gate_out is then the plain gate projection) */
} mcu_moe_buffers_t;
int mcu_moe_last_buffers(mcu_context_t *ctx, mcu_moe_buffers_t *out);

/* Peer communicator: a staging buffer per rank, mapped into the other ranks (one process per GPU, CUDA IPC),
 * and a one-shot all-reduce(sum) kernel over peer loads with a fixed summation order (rank 0 first), so all
 * ranks obtain bit-identical results.  Set-up: every rank creates a communicator, exports its 64-byte handle,
 * the host exchanges the handles (any transport), every rank connects with the array of all handles in rank
 * order.  All ranks must issue the same sequence of all-reduces.  A peer that does not arrive within two
 * seconds makes the kernel give up: the next mcu_synchronize reports the error, nothing hangs.
 * Destroy only after all ranks have synchronised (a barrier on the host). */
typedef struct mcu_peer_comm mcu_peer_comm_t;
#define MCU_PEER_HANDLE_BYTES 64
int mcu_peer_comm_create(mcu_context_t *ctx, int rank, int world, size_t max_bytes, mcu_peer_comm_t **out);
int mcu_peer_comm_export(mcu_peer_comm_t *comm, void *handle_out /* MCU_PEER_HANDLE_BYTES */);
int mcu_peer_comm_connect(mcu_peer_comm_t *comm, const void *all_handles /* world x MCU_PEER_HANDLE_BYTES */);
/* Device buffer (max_bytes) that the NEXT mcu_peer_allreduce sums across ranks: write the partial result here. */
void *mcu_peer_comm_staging(mcu_peer_comm_t *comm);
int mcu_peer_allreduce(mcu_peer_comm_t *comm, size_t n_floats, float *out_dev);
void mcu_peer_comm_destroy(mcu_peer_comm_t *comm);

/* Expert-parallel form over a connected peer communicator: rank q holds the matrices of the experts
 * [expert_bounds[q], expert_bounds[q + 1]) (host array of world + 1 entries, 0 first, E last); hidden, topk_ids and
 * topk_weights are the same on every rank (replicated router).  Each rank runs its experts' grouped matmuls on the
 * routes that name them; the routed rows then go back to the owners of their tokens (rank q owns tokens
 * [q * ceil(T / world), ...)), which combine them in sorted-route order exactly as mcu_moe_experts does, and the
 * token slices are gathered: out [T][H] on every rank, bit for bit mcu_moe_experts' result.  All peer traffic is
 * plain loads from the peers' staging slots, which must hold (T * k + T) * H floats; waits are bounded.
 * MCU_ERROR_NOT_IMPLEMENTED when the shape does not take the grouped path (fewer than 256 routes, mixed gate / up
 * kinds, ...): use mcu_moe_experts_local and an all-reduce then.  Every rank must make the same call. */
size_t mcu_peer_comm_capacity(mcu_peer_comm_t *comm);
int mcu_peer_comm_rank(mcu_peer_comm_t *comm);
int mcu_peer_comm_world(mcu_peer_comm_t *comm);
int mcu_moe_experts_ep(
    mcu_context_t *ctx, mcu_peer_comm_t *comm, int gate_kind, int up_kind, int down_kind, const float *hidden_dev, size_t T,
    size_t H, size_t FF, size_t E, const int32_t *expert_bounds, const void *gate_dev, const void *up_dev,
    const void *down_dev, const int32_t *topk_ids_dev, const float *topk_weights_dev, size_t k, int ffn_type,
    float weights_scale, int router_weight_policy, float *out_dev
);
/* The exchange alone: the routed rows [T * k][H] (sorted-route order) are in the communicator's staging slot. */
int mcu_peer_moe_combine(
    mcu_peer_comm_t *comm, const int32_t *route_pos_dev, const float *sorted_w_dev, const int32_t *offsets_dev,
    const int32_t *bad_id_count_dev, const int32_t *expert_bounds, size_t T, size_t k, size_t H, float *out_dev
);


/* Row-parallel quantized linear: this rank's K-slice of the weights times its K-slice of the activations, written
 * straight into the staging buffer, then the all-reduce; out [T][F] contiguous.
 * Two forms, chosen per communicator with mcu_peer_comm_set_fused (every rank must choose the same):
 *   0 (default)  the matmul kernel followed by the all-reduce kernel on the same stream;
 *   1            for 8 < T <= 64 and TMA-capable weights ONE kernel: the matmul's epilogue publishes each finished
 *                tile (one flag per rank and tile), waits (bounded) for the same tile of the other ranks, pulls their
 *                tiles with peer loads and adds in rank order; other shapes fall back to form 0.
 * Measured on 2 GPUs at T = 64 the two-kernel form is the faster one (25 vs 32 us for a 4096x2048 shard), which
 * is why it is the default. */
int mcu_peer_comm_set_fused(mcu_peer_comm_t *comm, int enabled);
/* One staging slot instead of two alternating ones: every collective then ends with a "finished reading" exchange, and a
 * captured CUDA graph may hold any number of collectives (with two slots: an even number).  Costs one more flag round trip
 * per collective; synchronizes the context's stream; every rank must choose the same. */
int mcu_peer_comm_set_one_slot(mcu_peer_comm_t *comm, int enabled);
int mcu_linear_allreduce(
    mcu_context_t *ctx, mcu_peer_comm_t *comm, int kind, const float *x_dev, size_t ldx, const void *w_dev, size_t T,
    size_t K, size_t F, float *out_dev
);

#ifdef __cplusplus
}
#endif
#endif
