// Checks of the kernel-query / preferences / capabilities entry points of the C23 host layer, compiled by
// tests/test_host_query_cpu.py against marmot's headers (tests only).  Prints one line per failed check and
// exits with the number of failures.
#include "marmot/device_caps.h"
#include "marmot/graph/kernel_selection.h"
#include "marmot/graph/op_signature.h"

#include "core/dispatch/kernel_query.h"

#include <stdio.h>
#include <string.h>

marmot_kernel_selection_t marmot_cuda_query_kernel(const marmot_op_signature_t *sig, const marmot_device_caps_t *caps);
marmot_device_caps_t marmot_cuda_detect_default_caps(void);
bool marmot_cuda_default_preferences(const marmot_device_caps_t *caps, marmot_backend_preferences_t *out);

static int failures = 0;
#define CHECK(cond)                                                   \
    do {                                                              \
        if (!(cond)) {                                                \
            printf("FAILED line %d: %s\n", __LINE__, #cond);          \
            ++failures;                                               \
        }                                                             \
    } while (0)

static marmot_op_signature_t linear_sig(marmot_qscheme_id_t q, size_t T, size_t K, size_t F) {
    marmot_op_signature_t s;
    memset(&s, 0, sizeof(s));
    s.op_id = MARMOT_OP_LINEAR;
    s.matmul_layout = MARMOT_MATMUL_LAYOUT_NT;
    s.input_dtype = MARMOT_DTYPE_FLOAT32;
    s.output_dtype = MARMOT_DTYPE_FLOAT32;
    s.accum_dtype = MARMOT_DTYPE_FLOAT32;
    s.qscheme_id = q;
    s.weight_layout = MARMOT_WEIGHT_LAYOUT_SEPARATE;
    s.stride_mode = MARMOT_STRIDE_MODE_CONTIGUOUS;
    s.dims.matmul.N = T;
    s.dims.matmul.K = K;
    s.dims.matmul.M = F;
    return s;
}

int main(int argc, char **argv) {
    const bool expect_device = argc > 1 && strcmp(argv[1], "device") == 0;
    marmot_device_caps_t caps;
    memset(&caps, 0, sizeof(caps));
    caps.backend.cuda.compute_capability = 100;
    caps.backend.cuda.sm_count = 148;
    caps.mem_bw_gbps = 6500.0f;
    caps.peak_flops_tflops_fp16 = 1600.0f;
    caps.launch_overhead_us = 4.0f;

    // the three block formats with kernels, decode and prefill shapes
    const marmot_qscheme_id_t kinds[3] = {MARMOT_QSCHEME_Q4_K, MARMOT_QSCHEME_Q6_K, MARMOT_QSCHEME_Q8_0};
    marmot_kernel_id_t ids[3];
    for (int i = 0; i < 3; ++i) {
        marmot_op_signature_t s = linear_sig(kinds[i], 1, 4096, 4096);
        marmot_kernel_selection_t sel = marmot_cuda_query_kernel(&s, &caps);
        CHECK(sel.supported && sel.fallback_reason == nullptr);
        CHECK((int)sel.kernel_id >= (int)MARMOT_KERNEL_COUNT);
        CHECK(sel.op_index != MARMOT_KERNEL_OP_INDEX_INVALID);
        CHECK(sel.est_comm_us == 0.0 && sel.shardable_axes == 0 && sel.device_affinity == 0);
        ids[i] = sel.kernel_id;
        s.op_id = MARMOT_OP_MATMUL;
        CHECK(marmot_cuda_query_kernel(&s, &caps).kernel_id == sel.kernel_id);
        s.epilogue_flags = MARMOT_EPILOGUE_BIAS;
        CHECK(marmot_cuda_query_kernel(&s, &caps).supported);
    }
    CHECK(ids[0] != ids[1] && ids[1] != ids[2]);
    {
        // the C1 GEMV is bandwidth bound (9.4 MB at 6.5 TB/s + a launch), the C2 GEMM tensor bound (60 GFLOP at 1.6 PFLOP/s)
        marmot_op_signature_t c1 = linear_sig(MARMOT_QSCHEME_Q4_K, 1, 4096, 4096);
        marmot_op_signature_t c2 = linear_sig(MARMOT_QSCHEME_Q8_0, 512, 4096, 14336);
        const double t1 = marmot_cuda_query_kernel(&c1, &caps).estimated_us, t2 = marmot_cuda_query_kernel(&c2, &caps).estimated_us;
        CHECK(t1 > 5.0 && t1 < 6.0);
        CHECK(t2 > 40.0 && t2 < 45.0);
        marmot_op_signature_t mid = linear_sig(MARMOT_QSCHEME_Q4_K, 64, 4096, 4096);
        CHECK(marmot_cuda_query_kernel(&mid, &caps).est_workspace_mb > 0.0);
        CHECK(marmot_cuda_query_kernel(&c1, &caps).est_workspace_mb < 0.1);
    }
    // what has no CUDA kernel is refused at query time, with a reason
    {
        marmot_op_signature_t s = linear_sig(MARMOT_QSCHEME_Q4_K, 1, 4096, 4096);
        s.input_dtype = MARMOT_DTYPE_FLOAT16;  // FLOAT16 activations are served (f32 or f16 out) ...
        CHECK(marmot_cuda_query_kernel(&s, &caps).supported);
        s.output_dtype = MARMOT_DTYPE_FLOAT16;
        CHECK(marmot_cuda_query_kernel(&s, &caps).supported);
        s.input_dtype = MARMOT_DTYPE_FLOAT32;  // ... FLOAT32 activations with a FLOAT16 output are not
        marmot_kernel_selection_t sel = marmot_cuda_query_kernel(&s, &caps);
        CHECK(!sel.supported && sel.fallback_reason != nullptr && sel.kernel_id == MARMOT_KERNEL_INVALID);
        s = linear_sig(MARMOT_QSCHEME_NONE, 1, 4096, 4096);
        CHECK(!marmot_cuda_query_kernel(&s, &caps).supported);
        s = linear_sig(MARMOT_QSCHEME_Q4_K, 1, 4096, 4096);
        s.epilogue_flags = MARMOT_EPILOGUE_BIAS | MARMOT_EPILOGUE_ACTIVATION;
        CHECK(!marmot_cuda_query_kernel(&s, &caps).supported);
        s = linear_sig(MARMOT_QSCHEME_Q4_K, 1, 4096, 4096);
        s.variant_flags = 1u << 14;  // residual-add fusion
        CHECK(!marmot_cuda_query_kernel(&s, &caps).supported);
        s = linear_sig(MARMOT_QSCHEME_Q4_K, 1, 4096, 4096);
        s.matmul_layout = MARMOT_MATMUL_LAYOUT_NN;
        CHECK(!marmot_cuda_query_kernel(&s, &caps).supported);
        s = linear_sig(MARMOT_QSCHEME_Q4_K, 1, 4096, 4096);
        s.op_id = MARMOT_OP_SOFTMAX;
        CHECK(!marmot_cuda_query_kernel(&s, &caps).supported);
        marmot_device_caps_t old = caps;
        old.backend.cuda.compute_capability = 90;
        s = linear_sig(MARMOT_QSCHEME_Q4_K, 1, 4096, 4096);
        CHECK(!marmot_cuda_query_kernel(&s, &old).supported);
        CHECK(!marmot_cuda_query_kernel(nullptr, &caps).supported && !marmot_cuda_query_kernel(&s, nullptr).supported);
    }
    // the other operators of the decode step
    {
        const marmot_op_id_t ops[] = {MARMOT_OP_MOE_EXPERTS, MARMOT_OP_TOPK,       MARMOT_OP_DEQUANTIZE,
                                      MARMOT_OP_EMBEDDING,   MARMOT_OP_RMS_NORM,   MARMOT_OP_RMS_NORM_GEMMA,
                                      MARMOT_OP_ROPE,        MARMOT_OP_ADD,        MARMOT_OP_SWIGLU,
                                      MARMOT_OP_PAGED_ATTENTION};
        for (size_t i = 0; i < sizeof(ops) / sizeof(ops[0]); ++i) {
            marmot_op_signature_t s;
            memset(&s, 0, sizeof(s));
            s.op_id = ops[i];
            s.input_dtype = s.output_dtype = s.weight_dtype = MARMOT_DTYPE_FLOAT32;
            s.qscheme_id = MARMOT_QSCHEME_Q4_K;
            CHECK(marmot_cuda_query_kernel(&s, &caps).supported);
        }
        marmot_op_signature_t s;
        memset(&s, 0, sizeof(s));
        // an operator the host layer has no implementation function for is not advertised
        s.op_id = MARMOT_OP_REDUCTION_ARGMAX;
        s.input_dtype = s.output_dtype = MARMOT_DTYPE_FLOAT32;
        CHECK(!marmot_cuda_query_kernel(&s, &caps).supported);
        memset(&s, 0, sizeof(s));
        s.op_id = MARMOT_OP_PAGED_ATTENTION;
        s.input_dtype = s.output_dtype = MARMOT_DTYPE_FLOAT32;
        s.weight_dtype = MARMOT_DTYPE_FLOAT16;
        const marmot_kernel_id_t f16_pool = marmot_cuda_query_kernel(&s, &caps).kernel_id;
        s.weight_dtype = MARMOT_DTYPE_FLOAT32;
        CHECK(marmot_cuda_query_kernel(&s, &caps).kernel_id != f16_pool);
        s.weight_dtype = MARMOT_DTYPE_INT32;
        CHECK(!marmot_cuda_query_kernel(&s, &caps).supported);
    }
    // preferences: everything on the GPU, no fused variants, raw blocks
    {
        marmot_backend_preferences_t prefs;
        memset(&prefs, 0xff, sizeof(prefs));
        CHECK(marmot_cuda_default_preferences(&caps, &prefs));
        CHECK(prefs.routing_policy == MARMOT_ROUTING_ALWAYS_GPU);
        CHECK(prefs.policy.variant_flags_mask == 0 && !prefs.policy.matmul_prefer_packed_weights);
        CHECK(prefs.policy.embedding_quant_output_dtype == MARMOT_DTYPE_FLOAT32);
        CHECK(!marmot_cuda_default_preferences(&caps, nullptr));
    }
    // capabilities of the device, or all zeros without one (then nothing is supported)
    {
        marmot_device_caps_t det = marmot_cuda_detect_default_caps();
        marmot_op_signature_t s = linear_sig(MARMOT_QSCHEME_Q4_K, 1, 4096, 4096);
        if (expect_device) {
            CHECK(det.backend.cuda.compute_capability / 10 == 10 && det.backend.cuda.sm_count >= 100);
            CHECK(det.mem_bw_gbps > 4000.0f && det.has_tensor_cores && det.simd_width == 32);
            CHECK(marmot_cuda_query_kernel(&s, &det).supported);
        } else if (det.backend.cuda.compute_capability == 0) {
            CHECK(det.num_compute_units == 0 && !marmot_cuda_query_kernel(&s, &det).supported);
        }
    }
    printf("%d failures\n", failures);
    return failures;
}
