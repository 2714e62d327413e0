// Declarations of the CUDA backend's host layer (cuda_backend.c) for marmot's generated dispatch sources: the
// functions the `.def` files under kernels/ and the CUDA entry of scripts/codegen/backend_config.py name.
#pragma once

#include "marmot/device.h"
#include "marmot/error.h"
#include "marmot/ops/paged_attention.h"
#include "marmot/ops_types.h"
#include "marmot/quant_traits.h"
#include "marmot/tensor.h"
#include "marmot/types.h"

#ifdef __cplusplus
extern "C" {
#endif

const marmot_device_ops_t *marmot_get_cuda_ops(void);

marmot_error_t cuda_matmul_quantized_any(
    const void *device_ctx, const marmot_tensor_t *input, const marmot_tensor_t *weight,
    const marmot_matmul_epilogue_t *epilogue, marmot_tensor_t *out
);
marmot_error_t cuda_matmul_quantized_q4_k(
    const void *device_ctx, const marmot_tensor_t *input, const marmot_tensor_t *weight,
    const marmot_matmul_epilogue_t *epilogue, marmot_tensor_t *out
);
marmot_error_t cuda_matmul_quantized_q6_k(
    const void *device_ctx, const marmot_tensor_t *input, const marmot_tensor_t *weight,
    const marmot_matmul_epilogue_t *epilogue, marmot_tensor_t *out
);
marmot_error_t cuda_matmul_quantized_q8_0(
    const void *device_ctx, const marmot_tensor_t *input, const marmot_tensor_t *weight,
    const marmot_matmul_epilogue_t *epilogue, marmot_tensor_t *out
);
marmot_error_t cuda_matmul_quantized_dual_output(
    const void *device_ctx, const marmot_tensor_t *input, const marmot_tensor_t *weight_a,
    const marmot_tensor_t *weight_b, marmot_tensor_t *out_a, marmot_tensor_t *out_b
);
marmot_error_t cuda_topk_impl(const void *device_ctx, const marmot_topk_desc_t *desc);
marmot_error_t cuda_moe_experts_impl(const void *device_ctx, const marmot_moe_experts_desc_t *desc);
marmot_error_t cuda_dequantize_dispatch(
    const void *device_ctx, marmot_quant_kind_t kind, marmot_quant_layout_t layout, const marmot_tensor_t *input,
    marmot_tensor_t *output
);
marmot_error_t cuda_dequantize_q4_k(const void *device_ctx, const marmot_tensor_t *input, marmot_tensor_t *output);
marmot_error_t cuda_dequantize_q6_k(const void *device_ctx, const marmot_tensor_t *input, marmot_tensor_t *output);
marmot_error_t cuda_dequantize_q8_0(const void *device_ctx, const marmot_tensor_t *input, marmot_tensor_t *output);
marmot_error_t cuda_vec_dot(const void *device_ctx, const marmot_vec_dot_descriptor_t *desc, float *result);

// decoder operators around the matmuls (FLOAT32)
marmot_error_t cuda_rmsnorm_impl(const void *device_ctx, const marmot_rmsnorm_desc_t *desc);
marmot_error_t cuda_rmsnorm_gemma_impl(const void *device_ctx, const marmot_rmsnorm_desc_t *desc);
marmot_error_t cuda_rope(
    const void *device_ctx, const marmot_tensor_t *x, const marmot_rope_params_t *params, marmot_tensor_t *out
);
marmot_error_t cuda_elementwise_binary_impl(
    const void *device_ctx, marmot_device_binary_op_t op, const marmot_tensor_t *a, const marmot_tensor_t *b,
    marmot_tensor_t *out
);
marmot_error_t cuda_embedding_gather(const void *device_ctx, const marmot_embedding_gather_desc_t *desc);
marmot_error_t cuda_paged_attention_impl(const void *device_ctx, const marmot_paged_attention_desc_t *desc);

#ifdef __cplusplus
}
#endif
