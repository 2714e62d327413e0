// Internal launcher declarations shared by the translation units of libmarmot_cuda.so.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace mcu {

// Device buffers holding quantized activations (structure of arrays).
struct ActBuffers {
    int8_t *qs;      // [T][kp]
    float *d;        // [T][nb]
    int16_t *bsums;  // [T][nb*16], Q8_K only
};

// f32 activations -> Q8_K (K-quant weights) or Q8_0 (Q8_0 weights); xh (optional) receives the
// dequantised activations d*q as fp16, row stride kp.
cudaError_t launch_quantize_act(int kind, const float *x, int ldx, int T, int K, const ActBuffers &a, __half *xh,
                                cudaStream_t s);

// fp16 operands of the tensor-core matmul from the quantized activations: xh[t][k] = d*q*2^-e_t (row stride kp),
// rowscale[t] = 2^e_t.  k_order: the order of the K values inside a row, matching how the matmul that reads it
// extracts packed weights: ACT_ORDER_NATURAL; ACT_ORDER_QUAD stores every four consecutive values as (0, 2, 1, 3)
// (gemm_tma); ACT_ORDER_FRAG16 stores every sixteen values v = 4t + j at position 8(j & 1) + 2t + (j >> 1), the k
// labelling of the mma.sync fragments of gemm_warp.
constexpr int ACT_ORDER_NATURAL = 0, ACT_ORDER_QUAD = 1, ACT_ORDER_FRAG16 = 2;
cudaError_t launch_half_acts(int kind, const ActBuffers &a, int T, int K, int k_order, __half *xh, float *rowscale,
                             cudaStream_t s);

// The two steps above in one kernel (one CTA per token, the quantized row kept in shared memory) when the int8
// values are not needed in global memory; usable while act_half_fused_smem() fits the default 48 KB.
size_t act_half_fused_smem(int kind, int K);
cudaError_t launch_act_half_fused(int kind, const float *x, int ldx, int T, int K, int k_order, __half *xh,
                                  float *rowscale, cudaStream_t s);
// Where the staging kernel takes its rows from, for callers that would otherwise run a gather or a GLU pass first:
// row t comes from x + row_index[t] * ldx when row_index is set; with x2 set the value is act(x) * x2 (glu 1 = SiLU,
// 2 = GELU, rounded like the MoE GLU kernel); rows outside [*row_lo, *row_hi) (device-resident) are skipped.
// With norm set the row is first x + add (add may be null; the sum goes to x_out when that is set, which may be x
// itself: a CTA owns its row) and the values are rms_norm(row) * (norm_w + w_off), the operations and their order
// those of the stand-alone add + RMSNorm kernel.
struct ActSource {
    const float *x2 = nullptr;
    int glu = 0;
    const int32_t *row_index = nullptr;
    const int *row_lo = nullptr, *row_hi = nullptr;
    int norm = 0;
    const float *add = nullptr, *norm_w = nullptr;
    float eps = 0.0f, w_off = 0.0f;
    float *x_out = nullptr;
};
cudaError_t launch_act_half_fused_from(int kind, const float *x, int ldx, const ActSource &src, int T, int K, int k_order,
                                       __half *xh, float *rowscale, cudaStream_t s);

// blocks -> f32 (bit-exact with the reference dequantizers)
cudaError_t launch_dequantize(int kind, const void *blocks, size_t n_values, float *out, cudaStream_t s);
// rows row_ids[0..n_rows) of a quantized [rows][dim] table -> f32 [n_rows][dim] (embedding gather)
cudaError_t launch_dequantize_rows(int kind, const void *table, size_t dim, size_t row_bytes, const int32_t *row_ids,
                                   size_t n_rows, float *out, cudaStream_t s);

// Decode-regime matmul, T <= GEMV_MAX_T tokens: out[t*ldo + f] = dot(W[f], act[t]) (+ bias[f]).
// W2/out2 non-null computes a second weight matrix of the same shape from the same activations.
constexpr int GEMV_MAX_T = 8;
cudaError_t launch_gemv(int kind, const void *W, const void *W2, const ActBuffers &a, int T, int K, int F,
                        const float *bias, float *out, float *out2, int ldo, cudaStream_t s);

// Streaming variant of the decode-regime matmul: activation quantisation fused in, weights streamed through
// shared memory with bulk asynchronous copies, launched with programmatic stream serialization.  One launch serves up
// to GEMV_MAX_JOBS weight matrices that read the same activations (q / k / v, gate / up): the CTAs are dealt out in
// proportion to the matrices' bytes.  Before they are quantized the activations can go through one of the decoder
// layer's elementwise steps, so that step needs no launch of its own:
//   GEMV_PRO_ADD_RMSNORM  x' = x + aux (aux may be null), h = x' / rms(x') * (norm_w + w_off); the matrices multiply h;
//                         x' is also written to x_out when that is set (x_out must not alias x: other CTAs still read it)
//   GEMV_PRO_SWIGLU       the matrices multiply silu(x) * aux
// *err_flag (device int) receives a non-zero code if a bounded device-side wait ran out.
constexpr int GEMV_MAX_JOBS = 4;
enum { GEMV_PRO_NONE = 0, GEMV_PRO_ADD_RMSNORM = 1, GEMV_PRO_SWIGLU = 2 };
struct GemvPrologue {
    int op = GEMV_PRO_NONE;
    const float *aux = nullptr;
    int ld_aux = 0;
    const float *norm_w = nullptr;
    float eps = 0.0f, w_off = 0.0f;
    float *x_out = nullptr;
    int ld_x_out = 0;
};
struct GemvJobSpec {
    int kind;
    const void *W;
    int F;
    const float *bias;
    float *out;
    int ldo;
};
bool gemv_stream_jobs_supported(const GemvJobSpec *jobs, int n_jobs, int T, int K, const GemvPrologue &pro);
cudaError_t launch_gemv_stream_jobs(const GemvJobSpec *jobs, int n_jobs, const float *x, int ldx, int T, int K,
                                    const GemvPrologue &pro, int *err_flag, cudaStream_t s);
// one matrix, or two of the same shape (W2 / out2), no prologue
bool gemv_stream_supported(int kind, const void *W, const void *W2, int T, int K, int F);
cudaError_t launch_gemv_stream(int kind, const void *W, const void *W2, const float *x, int ldx, int T, int K, int F,
                               const float *bias, float *out, float *out2, int ldo, int *err_flag, cudaStream_t s);

// f16 activations, no packing: every weight value formed in f32, products and sums in f32; f32 or f16 out
// (exactly one of out32 / out16 set).  See linear_f16.cu for the Q6_K reading.
cudaError_t launch_linear_f16(int kind, const void *W, const __half *x, size_t ldx, int T, int K, int F, const float *bias,
                              float *out32, __half *out16, size_t ldo, cudaStream_t s);

// Few-token regime (2 <= T <= 64) on integer tensor-core instructions: activations packed to Q8_K by a first launch,
// exact int32 sub-block dots (mma.sync s8), f32 scaling per block; Q4_K and Q6_K, rows a multiple of 16 bytes.
// The caller provides the workspace (sizes from gemm_i8_workspace_bytes); `tickets` must be zero before the first
// launch and is left zero.
bool gemm_i8_supported(int kind, const void *W, const void *W2, int T, int K, int F);
void gemm_i8_workspace_bytes(int T, int K, int F, bool dual, size_t *qs_bytes, size_t *dT_bytes, size_t *partial_bytes,
                             size_t *ticket_bytes);
cudaError_t launch_gemm_i8(int kind, const void *W, const void *W2, const float *x, int ldx, int T, int K, int F,
                           const float *bias, float *out, float *out2, int ldo, int8_t *qs, float *dT, float *partial,
                           int *tickets, int *err_flag, cudaStream_t s);

// Prefill / batched regime on the tcgen05 tensor cores: weights dequantised to fp16 tiles in shared
// memory, activations given as fp16 (d*q of the quantized activations, row stride ldxh), f32
// accumulation in tensor memory.
bool gemm_tc_supported(int kind, int T, int K, int F);
cudaError_t launch_gemm_tc(int kind, const void *W, const void *W2, const __half *xh, const float *rowscale, int ldxh,
                           int T, int K, int F, const float *bias, float *out, float *out2, int ldo, int *err_flag,
                           cudaStream_t s, int *launches);

// Row-parallel matmul fused with its all-reduce over peer memory (gemm_tma, T <= 64, full 128-row tiles): every CTA
// that holds a finished output tile stores it into this rank's peer-visible staging buffer, releases one flag per
// rank and tile, waits (bounded) for the same tile of all ranks, pulls their tiles with plain peer loads and adds
// them in rank order.  world == 0 means "not fused".
constexpr int PEER_FUSE_MAX_WORLD = 8;
constexpr int PEER_FUSE_MAX_TILES = 128;
struct PeerFuse {
    float *slots[PEER_FUSE_MAX_WORLD];     // rank d's staging buffer for this parity, as mapped in this process
    uint32_t *flags[PEER_FUSE_MAX_WORLD];  // rank d's flags for this parity: [world][PEER_FUSE_MAX_TILES]
    uint32_t *ctr;                         // this rank's {epoch of the last finished collective, ticket}
    size_t slot_floats;                    // capacity of a staging buffer
    int rank, world;
    uint32_t parity_of_next;               // parity the host expects for the next epoch (consistency check)
};

// TMA-fed variant of the tensor-core matmul (packed weight slabs and activation tiles arrive by
// cp.async.bulk.tensor); needs 16-byte aligned weights whose rows are 16-byte multiples.
bool gemm_tma_supported(int kind, const void *W, const void *W2, int T, int K, int F);
// Split-K workspace: `partial` needs gemm_tma_workspace_bytes() bytes (0: no split for this shape), `counters`
// GEMM_TMA_MAX_TILE_COUNTERS zero-initialised ints that the kernel leaves zero again.
constexpr int GEMM_TMA_MAX_TILE_COUNTERS = 4096;
size_t gemm_tma_workspace_bytes(int kind, int T, int K, int F);
cudaError_t launch_gemm_tma(int kind, const void *W, const void *W2, const __half *xh, const float *rowscale, int ldxh,
                            int T, int K, int F, const float *bias, float *out, float *out2, int ldo, float *partial,
                            int *counters, int *err_flag, cudaStream_t s, int *launches,
                            const PeerFuse *fuse = nullptr);
// Register-operand variant for 8 < T <= 64 tokens on Q4_K / Q6_K (mma.sync fragments built straight from the packed
// words, nothing dequantised to shared memory); activations in ACT_ORDER_FRAG16; same workspace contract.
bool gemm_warp_supported(int kind, const void *W, const void *W2, int T, int K, int F);
size_t gemm_warp_workspace_bytes(int kind, int T, int K, int F, bool dual);
cudaError_t launch_gemm_warp(int kind, const void *W, const void *W2, const __half *xh, const float *rowscale, int ldxh,
                             int T, int K, int F, const float *bias, float *out, float *out2, int ldo, float *partial,
                             int *counters, int *err_flag, cudaStream_t s);
// Grouped form (MoE experts): one launch for n_groups matmuls over a stacked weight matrix [n_groups * F, K]; group g
// owns group_counts[g] rows of xh / rowscale / out starting at row group_offsets[g] (device arrays: no host read-back).
bool gemm_tma_grouped_supported(int kind, const void *W, int K, int F);
cudaError_t launch_gemm_tma_grouped(int kind, const void *W, int n_groups, const __half *xh, const float *rowscale,
                                    int ldxh, int total_rows, int K, int F, const int *group_counts,
                                    const int *group_offsets, float *out, int ldo, int *err_flag, cudaStream_t s);
// Can launch_gemm_tma fuse the all-reduce for this shape (same answer on every rank: it depends on T and F only)?
bool gemm_tma_can_fuse(int kind, int T, int F);

int device_sm_count();

// Record the calling thread's error message (read back by mcu_last_error_message) and return `code`.
int set_error(int code, const char *message);
void count_launches(int n);

}  // namespace mcu

// Accessors of the opaque context for the other translation units.
struct mcu_context;
namespace mcu {
int context_device(const mcu_context *ctx);
int *context_err_flag(mcu_context *ctx);
// workspace of the context for the split-KV attention partials (grows on demand)
int context_attention_scratch(mcu_context *ctx, size_t bytes, void **out);
int context_attention_tickets(mcu_context *ctx, size_t bytes, void **out);  // zero-filled counters
int context_rope_table(mcu_context *ctx, size_t bytes, void **out);
// mcu_linear with the all-reduce fused into the matmul's epilogue; MCU_ERROR_NOT_IMPLEMENTED when the shape or the
// weights do not allow it (the caller then runs the matmul and the all-reduce kernel separately).
int linear_fused_allreduce(mcu_context *ctx, int kind, const float *x, size_t ldx, const void *w, size_t T, size_t K,
                           size_t F, float *out, const PeerFuse &fuse);
}  // namespace mcu
