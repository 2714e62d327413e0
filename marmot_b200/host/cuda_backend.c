// marmot CUDA backend, host side (C23): the device-ops vtable and the implementation functions the
// generated CUDA dispatch entries call, written against marmot's own headers.  Every function here is
// a thin adapter from marmot tensors to the plain-pointer C ABI of libmarmot_cuda (marmot_cuda.h); no
// arithmetic happens on the host.
//
// Reference counterparts (paths in the marmot tree):
//   marmot_get_cuda_ops            <- marmot_get_cpu_ops, src/backends/cpu/dispatch/device_ops.c:12-30
//   cuda_matmul_quantized_*        <- cpu_matmul_quantized_{q4_k,q6_k,q8_0}, matmul_quant_dispatch.c:905-960
//   cuda_matmul_quantized_dual_output <- cpu_matmul_quantized_dual_output, matmul_quant_dispatch.c:593-856
//   cuda_moe_experts_impl          <- cpu_moe_experts_impl, src/backends/cpu/ops/moe/moe_ops.c:1069-1178
//   cuda_topk_impl                 <- cpu_topk_impl, moe_ops.c:789-889
//   cuda_dequantize_*              <- cpu_dequantize_*, src/backends/cpu/quantization/formats/*.c
//   cuda_vec_dot                   <- cpu_vec_dot, src/backends/cpu/ops/vec_dot/vec_dot.c:6-65
//   marmot_cuda_query_kernel, marmot_cuda_detect_default_caps, marmot_cuda_default_preferences
//                                  <- the externs of src/core/dispatch/kernel_query.c:10-17
//
// Residency: marmot tensors own host memory and are identified by their host pointer.  The backend keeps a
// map host range -> device mirror.  `memcpy_to_device(p, p, n)` means "make [p, p+n) resident / refresh it"
// and `memcpy_from_device(p, p, n)` "make the host copy current" (src/core/tensor/transfer.c:22,49-51).
// Interior pointers (views into a larger allocation, e.g. one expert of a stacked MoE weight) resolve to
// an offset inside the mirror of the enclosing range.
#include "marmot/device.h"
#include "marmot/error.h"
#include "marmot/ops/paged_attention.h"
#include "marmot/ops_types.h"
#include "marmot/tensor.h"
#include "marmot/types.h"

#include "marmot/device_caps.h"
#include "marmot/graph/kernel_selection.h"
#include "marmot/graph/op_signature.h"

#include "core/dispatch/kernel_query.h"
#include "core/helpers/matmul.h"

#include "marmot_cuda.h"

#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    uintptr_t host;  // start of the host range
    size_t bytes;
    void *dev;
    bool dirty;  // an operator wrote the device copy and the host copy has not been refreshed since
} cuda_mirror_t;

typedef struct cuda_ctx {
    mcu_context_t *mcu;
    pthread_mutex_t mu;
    cuda_mirror_t *mirrors;  // sorted by host address, ranges never overlap
    size_t n_mirrors, cap_mirrors;
    size_t bytes_resident;
    // graph_batch_begin / graph_batch_end (include/marmot/device.h:57-60)
    int batch_depth;
    bool batch_capture;    // MARMOT_CUDA_GRAPH_BATCH=capture: a batch is recorded into a CUDA graph and launched at its end
    bool capture_open;
} cuda_ctx_t;

static marmot_error_t cuda_fail(int rc) {
    marmot_set_error((marmot_error_t)rc, mcu_last_error_message());
    return (marmot_error_t)rc;
}

// ---- residency map ------------------------------------------------------------------------------------

// index of the first mirror whose end lies beyond `addr`
static size_t mirror_lower_bound(const cuda_ctx_t *c, uintptr_t addr) {
    size_t lo = 0, hi = c->n_mirrors;
    while (lo < hi) {
        const size_t mid = (lo + hi) / 2;
        if (c->mirrors[mid].host + c->mirrors[mid].bytes <= addr) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}

// mirror that fully contains [addr, addr + bytes), or nullptr
static cuda_mirror_t *mirror_find(cuda_ctx_t *c, uintptr_t addr, size_t bytes) {
    const size_t i = mirror_lower_bound(c, addr);
    if (i == c->n_mirrors) return nullptr;
    cuda_mirror_t *m = &c->mirrors[i];
    if (m->host <= addr && addr + bytes <= m->host + m->bytes) return m;
    return nullptr;
}

// Drops the mirrors that overlap [addr, addr + bytes).  With `write_back` a mirror whose device copy is the current
// one is first copied to its host range (a larger operand is about to replace it and will be uploaded from there);
// without, the host memory itself is going away.
static void mirror_drop_overlapping(cuda_ctx_t *c, uintptr_t addr, size_t bytes, bool write_back) {
    size_t i = mirror_lower_bound(c, addr);
    while (i < c->n_mirrors && c->mirrors[i].host < addr + bytes) {
        if (write_back && c->mirrors[i].dirty)
            (void)mcu_memcpy_to_host(c->mcu, (void *)c->mirrors[i].host, c->mirrors[i].dev, c->mirrors[i].bytes);
        mcu_free(c->mcu, c->mirrors[i].dev);
        c->bytes_resident -= c->mirrors[i].bytes;
        memmove(&c->mirrors[i], &c->mirrors[i + 1], (c->n_mirrors - i - 1) * sizeof(cuda_mirror_t));
        c->n_mirrors--;
    }
}

// Device address of host range [addr, addr+bytes); allocates a mirror when none covers it (ranges that only
// partly overlap an older mirror replace it).
static marmot_error_t mirror_get(cuda_ctx_t *c, const void *host, size_t bytes, bool *created, void **dev_out) {
    const uintptr_t addr = (uintptr_t)host;
    *created = false;
    cuda_mirror_t *m = mirror_find(c, addr, bytes);
    if (m != nullptr) {
        *dev_out = (uint8_t *)m->dev + (addr - m->host);
        return MARMOT_SUCCESS;
    }
    if (c->capture_open) {
        marmot_set_error(MARMOT_ERROR_INVALID_OPERATION,
                         "CUDA graph batch: an operand is not resident; make tensors resident (marmot_tensor_to_device) "
                         "and run the program once before a captured batch");
        return MARMOT_ERROR_INVALID_OPERATION;
    }
    mirror_drop_overlapping(c, addr, bytes, true);
    if (c->n_mirrors == c->cap_mirrors) {
        const size_t cap = c->cap_mirrors == 0 ? 64 : c->cap_mirrors * 2;
        cuda_mirror_t *grown = realloc(c->mirrors, cap * sizeof(cuda_mirror_t));
        if (grown == nullptr) {
            marmot_set_error(MARMOT_ERROR_OUT_OF_MEMORY, "CUDA residency map allocation failed");
            return MARMOT_ERROR_OUT_OF_MEMORY;
        }
        c->mirrors = grown;
        c->cap_mirrors = cap;
    }
    void *dev = nullptr;
    const int rc = mcu_malloc(c->mcu, bytes, &dev);
    if (rc != 0) return cuda_fail(rc);
    const size_t at = mirror_lower_bound(c, addr);
    memmove(&c->mirrors[at + 1], &c->mirrors[at], (c->n_mirrors - at) * sizeof(cuda_mirror_t));
    c->mirrors[at] = (cuda_mirror_t){.host = addr, .bytes = bytes, .dev = dev, .dirty = false};
    c->n_mirrors++;
    c->bytes_resident += bytes;
    *created = true;
    *dev_out = dev;
    return MARMOT_SUCCESS;
}

// ---- tensors <-> mirrors ----------------------------------------------------------------------------------

static size_t tensor_bytes(const marmot_tensor_t *t) {
    const size_t logical = marmot_tensor_size_bytes(t);
    return logical != 0 ? logical : t->capacity_bytes;
}

// Read-only operand: resident and up to date on the device.
static marmot_error_t resident_ro(cuda_ctx_t *c, const marmot_tensor_t *t, size_t bytes, const void **dev) {
    bool created = false;
    void *d = nullptr;
    marmot_error_t st = mirror_get(c, t->data, bytes, &created, &d);
    if (st != MARMOT_SUCCESS) return st;
    if (created || t->memory_location != MARMOT_MEMORY_DEVICE) {
        if (c->capture_open) {
            marmot_set_error(MARMOT_ERROR_INVALID_OPERATION, "CUDA graph batch: an operand's host copy is newer than its "
                                                             "device copy; upload it before the batch");
            return MARMOT_ERROR_INVALID_OPERATION;
        }
        const int rc = mcu_memcpy_to_device(c->mcu, d, t->data, bytes);
        if (rc != 0) return cuda_fail(rc);
        // the two copies are now equal; like the CPU backend's pack caches this bookkeeping is not part of the
        // tensor's logical value
        marmot_tensor_t *mt = (marmot_tensor_t *)t;
        mt->memory_location = MARMOT_MEMORY_DEVICE;
        mt->needs_sync = false;
    }
    *dev = d;
    return MARMOT_SUCCESS;
}

// Output operand: a mirror to write into; the device copy becomes the current one.
static marmot_error_t resident_rw(cuda_ctx_t *c, marmot_tensor_t *t, size_t bytes, void **dev) {
    bool created = false;
    marmot_error_t st = mirror_get(c, t->data, bytes, &created, dev);
    if (st != MARMOT_SUCCESS) return st;
    cuda_mirror_t *m = mirror_find(c, (uintptr_t)t->data, bytes);
    if (m != nullptr) m->dirty = true;
    t->memory_location = MARMOT_MEMORY_DEVICE;
    t->needs_sync = true;  // marmot_tensor_to_host() will fetch it (src/core/tensor/transfer.c:36-62)
    return MARMOT_SUCCESS;
}

// ---- device-ops vtable (include/marmot/device.h:43-66) ------------------------------------------------------

static marmot_error_t cuda_init(void **device_ctx) {
    if (device_ctx == nullptr) return MARMOT_ERROR_INVALID_ARGUMENT;
    cuda_ctx_t *c = calloc(1, sizeof(*c));
    if (c == nullptr) {
        marmot_set_error(MARMOT_ERROR_OUT_OF_MEMORY, "CUDA context allocation failed");
        return MARMOT_ERROR_OUT_OF_MEMORY;
    }
    int device = 0;
    const char *env = getenv("MARMOT_CUDA_DEVICE");
    if (env != nullptr) device = atoi(env);
    const int rc = mcu_context_create(device, &c->mcu);
    if (rc != 0) {
        free(c);
        return cuda_fail(rc);
    }
    pthread_mutex_init(&c->mu, nullptr);
    const char *batch = getenv("MARMOT_CUDA_GRAPH_BATCH");
    c->batch_capture = batch != nullptr && strcmp(batch, "capture") == 0;
    *device_ctx = c;
    return MARMOT_SUCCESS;
}

static void cuda_destroy(const void *device_ctx) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (c == nullptr) return;
    if (c->capture_open) {  // a batch that was never ended: drop the recording before anything else touches the stream
        (void)mcu_graph_capture_end(c->mcu, nullptr);
        c->capture_open = false;
    }
    mcu_synchronize(c->mcu);
    for (size_t i = 0; i < c->n_mirrors; ++i) mcu_free(c->mcu, c->mirrors[i].dev);
    free(c->mirrors);
    mcu_context_destroy(c->mcu);
    pthread_mutex_destroy(&c->mu);
    free(c);
}

static marmot_error_t cuda_configure(const void *device_ctx, const marmot_context_t *ctx) {
    (void)ctx;
    return device_ctx != nullptr ? MARMOT_SUCCESS : MARMOT_ERROR_DEVICE_NOT_AVAILABLE;
}

static marmot_error_t cuda_alloc(const void *device_ctx, size_t size, void **ptr) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (c == nullptr) return MARMOT_ERROR_DEVICE_NOT_AVAILABLE;
    const int rc = mcu_malloc(c->mcu, size, ptr);
    return rc == 0 ? MARMOT_SUCCESS : cuda_fail(rc);
}

static void cuda_free(const void *device_ctx, void *ptr) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (c != nullptr) mcu_free(c->mcu, ptr);
}

// dst is the identity (host address) of the tensor storage; src holds the bytes (often the same pointer)
static marmot_error_t cuda_memcpy_to_device(const void *device_ctx, void *dst, const void *src, size_t size) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (c == nullptr) return MARMOT_ERROR_DEVICE_NOT_AVAILABLE;
    if (size == 0) return MARMOT_SUCCESS;
    pthread_mutex_lock(&c->mu);
    bool created = false;
    void *d = nullptr;
    marmot_error_t st = mirror_get(c, dst, size, &created, &d);
    if (st == MARMOT_SUCCESS) {
        const int rc = mcu_memcpy_to_device(c->mcu, d, src, size);
        if (rc != 0) st = cuda_fail(rc);
        cuda_mirror_t *m = mirror_find(c, (uintptr_t)dst, size);
        if (rc == 0 && m != nullptr && (uintptr_t)dst == m->host && size == m->bytes) m->dirty = false;
    }
    pthread_mutex_unlock(&c->mu);
    return st;
}

static marmot_error_t cuda_memcpy_from_device(const void *device_ctx, void *dst, const void *src, size_t size) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (c == nullptr) return MARMOT_ERROR_DEVICE_NOT_AVAILABLE;
    if (size == 0) return MARMOT_SUCCESS;
    pthread_mutex_lock(&c->mu);
    marmot_error_t st = MARMOT_SUCCESS;
    cuda_mirror_t *m = mirror_find(c, (uintptr_t)src, size);
    if (m != nullptr) {
        const int rc = mcu_memcpy_to_host(c->mcu, dst, (const uint8_t *)m->dev + ((uintptr_t)src - m->host), size);
        if (rc != 0) st = cuda_fail(rc);
        else if (dst == src && (uintptr_t)src == m->host && size == m->bytes) m->dirty = false;
    } else {
        const int rc = mcu_synchronize(c->mcu);  // nothing resident for this range: the host copy is the only one
        if (rc != 0) st = cuda_fail(rc);
    }
    pthread_mutex_unlock(&c->mu);
    return st;
}

static marmot_error_t cuda_synchronize(const void *device_ctx) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (c == nullptr) return MARMOT_ERROR_DEVICE_NOT_AVAILABLE;
    const int rc = mcu_synchronize(c->mcu);
    return rc == 0 ? MARMOT_SUCCESS : cuda_fail(rc);
}

static marmot_error_t cuda_allocator_usage(const void *device_ctx, marmot_allocator_usage_t *usage) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (c == nullptr || usage == nullptr) return MARMOT_ERROR_INVALID_ARGUMENT;
    memset(usage, 0, sizeof(*usage));
    usage->current_bytes = c->bytes_resident;
    usage->active_allocations = c->n_mirrors;
    return MARMOT_SUCCESS;
}

static void cuda_on_host_range_freed(void *device_ctx, const void *start, size_t length) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (c == nullptr || start == nullptr) return;
    pthread_mutex_lock(&c->mu);
    mirror_drop_overlapping(c, (uintptr_t)start, length > 0 ? length : 1, false);
    pthread_mutex_unlock(&c->mu);
}

static void cuda_on_host_ptr_freed(void *device_ctx, const void *ptr) { cuda_on_host_range_freed(device_ctx, ptr, 1); }

// Graph batching (include/marmot/device.h:57-60; the graph executor brackets every bytecode program with these,
// src/graph/graph_executor.cpp:770,932).  Operators already only enqueue work on the context's stream, so by default
// a batch needs nothing at its start; at its end a failed program (commit == false) waits for the device so that
// whatever was enqueued has finished - and a device-side error has surfaced - before the caller reuses the tensors.
// With MARMOT_CUDA_GRAPH_BATCH=capture the outermost batch is recorded into a CUDA graph instead (mcu_graph_capture_*)
// and launched once at its end: every operand must then be resident and the workspace warm (run the program once
// unbatched first), since uploads and allocations cannot be recorded; an operator that needs either fails the batch.
static marmot_error_t cuda_graph_batch_begin(void *device_ctx) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (c == nullptr) return MARMOT_ERROR_DEVICE_NOT_AVAILABLE;
    pthread_mutex_lock(&c->mu);
    marmot_error_t st = MARMOT_SUCCESS;
    if (c->batch_depth == 0 && c->batch_capture) {
        const int rc = mcu_graph_capture_begin(c->mcu);
        if (rc != 0) st = cuda_fail(rc);
        else c->capture_open = true;
    }
    if (st == MARMOT_SUCCESS) c->batch_depth++;
    pthread_mutex_unlock(&c->mu);
    return st;
}

static marmot_error_t cuda_graph_batch_end(void *device_ctx, bool commit) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (c == nullptr) return MARMOT_ERROR_DEVICE_NOT_AVAILABLE;
    pthread_mutex_lock(&c->mu);
    marmot_error_t st = MARMOT_SUCCESS;
    if (c->batch_depth <= 0) {
        marmot_set_error(MARMOT_ERROR_INVALID_OPERATION, "graph_batch_end without graph_batch_begin");
        st = MARMOT_ERROR_INVALID_OPERATION;
    } else if (--c->batch_depth == 0) {
        if (c->capture_open) {
            c->capture_open = false;
            mcu_graph_t *graph = nullptr;
            int rc = mcu_graph_capture_end(c->mcu, commit ? &graph : nullptr);
            if (rc == 0 && graph != nullptr) {
                rc = mcu_graph_launch(graph);
                const int rc_sync = mcu_synchronize(c->mcu);  // the graph must not be destroyed while it runs
                if (rc == 0) rc = rc_sync;
                mcu_graph_destroy(graph);
            }
            if (rc != 0) st = cuda_fail(rc);
        } else if (!commit) {
            const int rc = mcu_synchronize(c->mcu);
            if (rc != 0) st = cuda_fail(rc);
        }
    }
    pthread_mutex_unlock(&c->mu);
    return st;
}

static const marmot_device_ops_t g_cuda_ops = {
    .init = cuda_init,
    .destroy = cuda_destroy,
    .configure = cuda_configure,
    .alloc = cuda_alloc,
    .free = cuda_free,
    .memcpy_to_device = cuda_memcpy_to_device,
    .memcpy_from_device = cuda_memcpy_from_device,
    .synchronize = cuda_synchronize,
    .allocator_usage = cuda_allocator_usage,
    .graph_batch_begin = cuda_graph_batch_begin,
    .graph_batch_end = cuda_graph_batch_end,
    .on_host_ptr_freed = cuda_on_host_ptr_freed,
    .on_host_range_freed = cuda_on_host_range_freed,
};

const marmot_device_ops_t *marmot_get_cuda_ops(void) { return &g_cuda_ops; }

// ---- operator implementations ---------------------------------------------------------------------------------

static int mcu_kind_of(marmot_quant_kind_t kind) {
    switch (kind) {
    case MARMOT_QUANT_KIND_Q4_K: return MCU_KIND_Q4_K;
    case MARMOT_QUANT_KIND_Q6_K: return MCU_KIND_Q6_K;
    case MARMOT_QUANT_KIND_Q8_0: return MCU_KIND_Q8_0;
    default: return -1;
    }
}

static marmot_error_t cuda_matmul_quantized(
    const void *device_ctx, const marmot_tensor_t *input, const marmot_tensor_t *weight_a,
    const marmot_tensor_t *weight_b, const marmot_matmul_epilogue_t *epilogue, marmot_tensor_t *out_a,
    marmot_tensor_t *out_b, marmot_quant_kind_t expect_kind
) {
    if (input == nullptr || weight_a == nullptr || out_a == nullptr) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "Tensor argument must not be null");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (c == nullptr) {
        marmot_set_error(MARMOT_ERROR_DEVICE_NOT_AVAILABLE, "CUDA context is not initialised");
        return MARMOT_ERROR_DEVICE_NOT_AVAILABLE;
    }
    marmot_matmul_dims_t dims = {0};
    marmot_matmul_activation_profile_t profile = {0};
    const marmot_quant_kind_traits_t *traits = nullptr;
    marmot_error_t st = marmot_matmul_validate_quantized(input, weight_a, out_a, &dims, &profile, &traits);
    if (st != MARMOT_SUCCESS) return st;
    if (weight_a->quant_kind != expect_kind || mcu_kind_of(weight_a->quant_kind) < 0) {
        marmot_set_error(MARMOT_ERROR_NOT_IMPLEMENTED, "CUDA quantized matmul: unsupported quant kind");
        return MARMOT_ERROR_NOT_IMPLEMENTED;
    }
    // FLOAT32 in and out: activations packed on the device (mcu_linear).  FLOAT16 in: the reference's unpacked f32
    // arithmetic (mcu_linear_f16), FLOAT32 or FLOAT16 out, one weight.
    const bool half_in = profile.input_is_fp16;
    if (!(profile.input_is_fp32 && profile.output_is_fp32) &&
        !(half_in && (profile.output_is_fp32 || profile.output_is_fp16) && weight_b == nullptr)) {
        marmot_set_error(MARMOT_ERROR_UNSUPPORTED_DTYPE,
                         "CUDA quantized matmul takes FLOAT32 in and out, or FLOAT16 in with FLOAT32 / FLOAT16 out");
        return MARMOT_ERROR_UNSUPPORTED_DTYPE;
    }
    const size_t in_elem = half_in ? 2 : 4, out_elem = profile.output_is_fp16 ? 2 : 4;
    if (input->shape.strides[1] != 1 || out_a->shape.strides[1] != 1) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "CUDA quantized matmul needs unit inner strides");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    const int kind = mcu_kind_of(weight_a->quant_kind);
    const size_t T = dims.N, K = dims.K, F = dims.M;
    const size_t ldx = input->shape.strides[0], ldo = out_a->shape.strides[0];
    if (weight_b != nullptr) {
        if (out_b == nullptr || weight_b->quant_kind != weight_a->quant_kind || weight_b->shape.shape[0] != F ||
            weight_b->shape.shape[1] != K || out_b->shape.strides[0] != ldo) {
            marmot_set_error(MARMOT_ERROR_DIMENSION_MISMATCH, "dual-output matmul operands do not match");
            return MARMOT_ERROR_DIMENSION_MISMATCH;
        }
    }
    const size_t w_bytes = F * mcu_row_bytes(kind, K);
    pthread_mutex_lock(&c->mu);
    const void *x = nullptr, *wa = nullptr, *wb = nullptr, *bias = nullptr;
    void *ya = nullptr, *yb = nullptr;
    st = resident_ro(c, input, ((T - 1) * ldx + K) * in_elem, &x);
    if (st == MARMOT_SUCCESS) st = resident_ro(c, weight_a, w_bytes, &wa);
    if (st == MARMOT_SUCCESS && weight_b != nullptr) st = resident_ro(c, weight_b, w_bytes, &wb);
    if (st == MARMOT_SUCCESS && epilogue != nullptr && epilogue->bias != nullptr) {
        if (epilogue->bias->dtype != MARMOT_DTYPE_FLOAT32 || marmot_tensor_num_elements(epilogue->bias) != F) {
            marmot_set_error(MARMOT_ERROR_UNSUPPORTED_DTYPE, "CUDA matmul bias must be FLOAT32 [features]");
            st = MARMOT_ERROR_UNSUPPORTED_DTYPE;
        } else {
            st = resident_ro(c, epilogue->bias, F * sizeof(float), &bias);
        }
    }
    if (st == MARMOT_SUCCESS) st = resident_rw(c, out_a, ((T - 1) * ldo + F) * out_elem, &ya);
    if (st == MARMOT_SUCCESS && out_b != nullptr) st = resident_rw(c, out_b, ((T - 1) * ldo + F) * sizeof(float), &yb);
    if (st == MARMOT_SUCCESS) {
        const int rc = half_in ? mcu_linear_f16(c->mcu, kind, x, ldx, wa, T, K, F, bias, ya, ldo,
                                                profile.output_is_fp16 ? MCU_OUT_F16 : MCU_OUT_F32)
            : weight_b == nullptr ? mcu_linear(c->mcu, kind, x, ldx, wa, T, K, F, bias, ya, ldo)
                                  : mcu_linear_dual(c->mcu, kind, x, ldx, wa, wb, T, K, F, ya, yb, ldo);
        if (rc != 0) st = cuda_fail(rc);
    }
    pthread_mutex_unlock(&c->mu);
    return st;
}

marmot_error_t cuda_matmul_quantized_q4_k(
    const void *device_ctx, const marmot_tensor_t *input, const marmot_tensor_t *weight,
    const marmot_matmul_epilogue_t *epilogue, marmot_tensor_t *out
) {
    return cuda_matmul_quantized(device_ctx, input, weight, nullptr, epilogue, out, nullptr, MARMOT_QUANT_KIND_Q4_K);
}

marmot_error_t cuda_matmul_quantized_q6_k(
    const void *device_ctx, const marmot_tensor_t *input, const marmot_tensor_t *weight,
    const marmot_matmul_epilogue_t *epilogue, marmot_tensor_t *out
) {
    return cuda_matmul_quantized(device_ctx, input, weight, nullptr, epilogue, out, nullptr, MARMOT_QUANT_KIND_Q6_K);
}

marmot_error_t cuda_matmul_quantized_q8_0(
    const void *device_ctx, const marmot_tensor_t *input, const marmot_tensor_t *weight,
    const marmot_matmul_epilogue_t *epilogue, marmot_tensor_t *out
) {
    return cuda_matmul_quantized(device_ctx, input, weight, nullptr, epilogue, out, nullptr, MARMOT_QUANT_KIND_Q8_0);
}

// The handler the generated `marmot_cuda_matmul_*_exec` wrappers call (scripts/codegen/templates/backend_dispatch.j2
// routes every quantized matmul entry of a backend to its one `matmul_quantized` handler): the block format comes
// from the weight tensor.
marmot_error_t cuda_matmul_quantized_any(
    const void *device_ctx, const marmot_tensor_t *input, const marmot_tensor_t *weight,
    const marmot_matmul_epilogue_t *epilogue, marmot_tensor_t *out
) {
    if (weight == nullptr) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "Tensor argument must not be null");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    return cuda_matmul_quantized(device_ctx, input, weight, nullptr, epilogue, out, nullptr, weight->quant_kind);
}

marmot_error_t cuda_matmul_quantized_dual_output(
    const void *device_ctx, const marmot_tensor_t *input, const marmot_tensor_t *weight_a,
    const marmot_tensor_t *weight_b, marmot_tensor_t *out_a, marmot_tensor_t *out_b
) {
    if (weight_a == nullptr || weight_b == nullptr || out_b == nullptr) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "Tensor argument must not be null");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    return cuda_matmul_quantized(device_ctx, input, weight_a, weight_b, nullptr, out_a, out_b, weight_a->quant_kind);
}

// Replaces cpu_topk_impl (src/backends/cpu/ops/moe/moe_ops.c:789-889): the same checks in the same order,
// FLOAT32 values only.
marmot_error_t cuda_topk_impl(const void *device_ctx, const marmot_topk_desc_t *desc) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (desc == nullptr || desc->x == nullptr || desc->values_out == nullptr || desc->indices_out == nullptr) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "TopK descriptor is incomplete");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    if (desc->x->dtype != MARMOT_DTYPE_FLOAT32 || desc->values_out->dtype != MARMOT_DTYPE_FLOAT32 ||
        desc->indices_out->dtype != MARMOT_DTYPE_INT32) {
        marmot_set_error(MARMOT_ERROR_UNSUPPORTED_DTYPE, "CUDA TopK supports FLOAT32 values and INT32 indices only");
        return MARMOT_ERROR_UNSUPPORTED_DTYPE;
    }
    if (desc->x->shape.ndim != 2 || desc->values_out->shape.ndim != 2 || desc->indices_out->shape.ndim != 2) {
        marmot_set_error(MARMOT_ERROR_DIMENSION_MISMATCH, "TopK expects 2D tensors");
        return MARMOT_ERROR_DIMENSION_MISMATCH;
    }
    if (desc->axis != 1 && desc->axis != -1) {
        marmot_set_error(MARMOT_ERROR_NOT_IMPLEMENTED, "TopK currently supports only the last axis");
        return MARMOT_ERROR_NOT_IMPLEMENTED;
    }
    const size_t rows = desc->x->shape.shape[0], cols = desc->x->shape.shape[1], k = desc->k;
    if (k == 0 || k > cols || desc->values_out->shape.shape[0] != rows || desc->indices_out->shape.shape[0] != rows ||
        desc->values_out->shape.shape[1] != k || desc->indices_out->shape.shape[1] != k) {
        marmot_set_error(MARMOT_ERROR_DIMENSION_MISMATCH, "TopK shapes do not match");
        return MARMOT_ERROR_DIMENSION_MISMATCH;
    }
    if (desc->values_out->shape.strides[0] != k || desc->indices_out->shape.strides[0] != k) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "CUDA TopK needs contiguous outputs");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    if (c == nullptr) {
        marmot_set_error(MARMOT_ERROR_DEVICE_NOT_AVAILABLE, "CUDA context is not initialised");
        return MARMOT_ERROR_DEVICE_NOT_AVAILABLE;
    }
    const size_t ldx = desc->x->shape.strides[0];
    pthread_mutex_lock(&c->mu);
    const void *x = nullptr;
    void *vals = nullptr, *idx = nullptr;
    marmot_error_t st = resident_ro(c, desc->x, ((rows - 1) * ldx + cols) * sizeof(float), &x);
    if (st == MARMOT_SUCCESS) st = resident_rw(c, desc->values_out, rows * k * sizeof(float), &vals);
    if (st == MARMOT_SUCCESS) st = resident_rw(c, desc->indices_out, rows * k * sizeof(int32_t), &idx);
    if (st == MARMOT_SUCCESS) {
        const int rc = mcu_topk(c->mcu, x, rows, cols, ldx, k, vals, idx);
        if (rc != 0) st = cuda_fail(rc);
    }
    pthread_mutex_unlock(&c->mu);
    return st;
}

// Replaces cpu_moe_experts_impl (src/backends/cpu/ops/moe/moe_ops.c:1069-1178) for quantized experts with FLOAT32
// activations. Expert tensors are [in, out, experts] in GGUF order (shape[0] innermost), as the reference reads
// them (moe_ops.c:897-898).
marmot_error_t cuda_moe_experts_impl(const void *device_ctx, const marmot_moe_experts_desc_t *desc) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (desc == nullptr || desc->hidden_states == nullptr || desc->gate_exps == nullptr || desc->up_exps == nullptr ||
        desc->down_exps == nullptr || desc->topk_ids == nullptr || desc->topk_weights == nullptr ||
        desc->out == nullptr) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "MoE descriptor is incomplete");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    const int gk = mcu_kind_of(desc->gate_exps->quant_kind), uk = mcu_kind_of(desc->up_exps->quant_kind),
              dk = mcu_kind_of(desc->down_exps->quant_kind);
    if (gk < 0 || uk < 0 || dk < 0) {
        marmot_set_error(MARMOT_ERROR_NOT_IMPLEMENTED, "CUDA MoE experts needs Q4_K, Q6_K or Q8_0 expert weights");
        return MARMOT_ERROR_NOT_IMPLEMENTED;
    }
    if (desc->hidden_states->dtype != MARMOT_DTYPE_FLOAT32 || desc->topk_weights->dtype != MARMOT_DTYPE_FLOAT32 ||
        desc->out->dtype != MARMOT_DTYPE_FLOAT32 || desc->topk_ids->dtype != MARMOT_DTYPE_INT32) {
        marmot_set_error(
            MARMOT_ERROR_UNSUPPORTED_DTYPE,
            "CUDA MoE experts supports FLOAT32 activations with FLOAT32 router weights and INT32 expert ids"
        );
        return MARMOT_ERROR_UNSUPPORTED_DTYPE;
    }
    const marmot_tensor_t *h = desc->hidden_states;
    if (h->shape.ndim != 2 || desc->out->shape.ndim != 2 || desc->topk_ids->shape.ndim != 2 ||
        desc->topk_weights->shape.ndim != 2 || desc->gate_exps->shape.ndim != 3 || desc->up_exps->shape.ndim != 3 ||
        desc->down_exps->shape.ndim != 3) {
        marmot_set_error(MARMOT_ERROR_DIMENSION_MISMATCH, "MoE tensors have the wrong rank");
        return MARMOT_ERROR_DIMENSION_MISMATCH;
    }
    const size_t T = h->shape.shape[0], H = h->shape.shape[1];
    const size_t FF = desc->gate_exps->shape.shape[1], E = desc->gate_exps->shape.shape[2];
    const size_t k = desc->topk_ids->shape.shape[1];
    const size_t *us = desc->up_exps->shape.shape, *ds = desc->down_exps->shape.shape;
    if (desc->gate_exps->shape.shape[0] != H || us[0] != H || us[1] != FF || us[2] != E || ds[0] != FF || ds[1] != H ||
        ds[2] != E || desc->out->shape.shape[0] != T || desc->out->shape.shape[1] != H ||
        desc->topk_ids->shape.shape[0] != T || desc->topk_weights->shape.shape[0] != T ||
        desc->topk_weights->shape.shape[1] != k) {
        marmot_set_error(MARMOT_ERROR_DIMENSION_MISMATCH, "MoE tensor shapes do not match");
        return MARMOT_ERROR_DIMENSION_MISMATCH;
    }
    if (h->shape.strides[0] != H || desc->out->shape.strides[0] != H || desc->topk_ids->shape.strides[0] != k ||
        desc->topk_weights->shape.strides[0] != k) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "CUDA MoE experts needs contiguous activations");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    if (c == nullptr) {
        marmot_set_error(MARMOT_ERROR_DEVICE_NOT_AVAILABLE, "CUDA context is not initialised");
        return MARMOT_ERROR_DEVICE_NOT_AVAILABLE;
    }
    pthread_mutex_lock(&c->mu);
    const void *hid = nullptr, *gate = nullptr, *up = nullptr, *down = nullptr, *ids = nullptr, *wts = nullptr;
    void *out = nullptr;
    marmot_error_t st = resident_ro(c, h, T * H * sizeof(float), &hid);
    if (st == MARMOT_SUCCESS) st = resident_ro(c, desc->gate_exps, E * FF * mcu_row_bytes(gk, H), &gate);
    if (st == MARMOT_SUCCESS) st = resident_ro(c, desc->up_exps, E * FF * mcu_row_bytes(uk, H), &up);
    if (st == MARMOT_SUCCESS) st = resident_ro(c, desc->down_exps, E * H * mcu_row_bytes(dk, FF), &down);
    if (st == MARMOT_SUCCESS) st = resident_ro(c, desc->topk_ids, T * k * sizeof(int32_t), &ids);
    if (st == MARMOT_SUCCESS) st = resident_ro(c, desc->topk_weights, T * k * sizeof(float), &wts);
    if (st == MARMOT_SUCCESS) st = resident_rw(c, desc->out, T * H * sizeof(float), &out);
    if (st == MARMOT_SUCCESS) {
        const int rc = mcu_moe_experts(
            c->mcu, gk, uk, dk, hid, T, H, FF, E, gate, up, down, ids, wts, k, (int)desc->ffn_type,
            desc->weights_scale, (int)desc->router_weight_policy, out
        );
        if (rc != 0) st = cuda_fail(rc);
    }
    pthread_mutex_unlock(&c->mu);
    return st;
}

// Replaces cpu_dequantize_{q4_k,q6_k,q8_0} -> cpu_dequantize_blockwise
// (src/backends/cpu/quantization/ops/quantize_core.c:268-330): rows are padded to whole blocks in the input.
static marmot_error_t
cuda_dequantize_blockwise(const void *device_ctx, int kind, const marmot_tensor_t *input, marmot_tensor_t *output) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (input == nullptr || output == nullptr) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "Null tensor pointer");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    if (input->dtype != MARMOT_DTYPE_UINT8 && input->dtype != MARMOT_DTYPE_INT8) {
        marmot_set_error(MARMOT_ERROR_UNSUPPORTED_DTYPE, "Block dequantization expects UINT8 or INT8 input buffer");
        return MARMOT_ERROR_UNSUPPORTED_DTYPE;
    }
    if (output->dtype != MARMOT_DTYPE_FLOAT32) {
        marmot_set_error(MARMOT_ERROR_UNSUPPORTED_DTYPE, "Block dequantization requires FLOAT32 output");
        return MARMOT_ERROR_UNSUPPORTED_DTYPE;
    }
    const size_t total = marmot_tensor_num_elements(output);
    const size_t rows = output->shape.ndim == 2 ? output->shape.shape[0] : 1;
    const size_t row = output->shape.ndim == 2 ? output->shape.shape[1] : total;
    const size_t row_bytes = mcu_row_bytes(kind, row);
    if (rows * row_bytes > tensor_bytes(input)) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "Quantized input buffer too small");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    if (c == nullptr) {
        marmot_set_error(MARMOT_ERROR_DEVICE_NOT_AVAILABLE, "CUDA context is not initialised");
        return MARMOT_ERROR_DEVICE_NOT_AVAILABLE;
    }
    const size_t block = kind == MCU_KIND_Q8_0 ? 32 : 256;
    pthread_mutex_lock(&c->mu);
    const void *src = nullptr;
    void *dst = nullptr;
    marmot_error_t st = resident_ro(c, input, rows * row_bytes, &src);
    if (st == MARMOT_SUCCESS) st = resident_rw(c, output, total * sizeof(float), &dst);
    if (st == MARMOT_SUCCESS) {
        int rc = 0;
        if (row % block == 0) {
            rc = mcu_dequantize(c->mcu, kind, src, total, dst);
        } else {
            for (size_t r = 0; r < rows && rc == 0; ++r)
                rc = mcu_dequantize(c->mcu, kind, (const uint8_t *)src + r * row_bytes, row, (float *)dst + r * row);
        }
        if (rc != 0) st = cuda_fail(rc);
    }
    pthread_mutex_unlock(&c->mu);
    return st;
}

marmot_error_t cuda_dequantize_q4_k(const void *device_ctx, const marmot_tensor_t *input, marmot_tensor_t *output) {
    return cuda_dequantize_blockwise(device_ctx, MCU_KIND_Q4_K, input, output);
}

marmot_error_t cuda_dequantize_q6_k(const void *device_ctx, const marmot_tensor_t *input, marmot_tensor_t *output) {
    return cuda_dequantize_blockwise(device_ctx, MCU_KIND_Q6_K, input, output);
}

marmot_error_t cuda_dequantize_q8_0(const void *device_ctx, const marmot_tensor_t *input, marmot_tensor_t *output) {
    return cuda_dequantize_blockwise(device_ctx, MCU_KIND_Q8_0, input, output);
}

// The unified dequantize handler of the generated dispatch (the same shape as metal_dequantize_dispatch).
marmot_error_t cuda_dequantize_dispatch(
    const void *device_ctx, marmot_quant_kind_t kind, marmot_quant_layout_t layout, const marmot_tensor_t *input,
    marmot_tensor_t *output
) {
    (void)layout;
    const int k = mcu_kind_of(kind);
    if (k < 0) {
        marmot_set_error(MARMOT_ERROR_NOT_IMPLEMENTED, "CUDA dequantize: block format has no kernel (Q4_K, Q6_K, Q8_0 do)");
        return MARMOT_ERROR_NOT_IMPLEMENTED;
    }
    return cuda_dequantize_blockwise(device_ctx, k, input, output);
}

// ---- quantized row dot (the public marmot_vec_dot; host pointers, as in the reference) ----------------
// num_blocks counts 32-value blocks in the descriptor's convention for Q8_0 activations and 256-value super-blocks for
// Q8_K ones, exactly what cpu_vec_dot hands to its dot kernels (src/backends/cpu/ops/vec_dot/vec_dot.c:52-62).
marmot_error_t cuda_vec_dot(const void *device_ctx, const marmot_vec_dot_descriptor_t *desc, float *result) {
    if (desc == nullptr || result == nullptr) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "cuda_vec_dot: null descriptor or result");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    if (desc->weights == nullptr || desc->activations == nullptr || desc->num_blocks == 0) {
        *result = 0.0f;
        return MARMOT_SUCCESS;
    }
    if (device_ctx == nullptr) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "cuda_vec_dot: null device context");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    const int kind = mcu_kind_of(desc->weight_kind);
    if (kind < 0) {
        marmot_set_error(MARMOT_ERROR_NOT_IMPLEMENTED, "cuda_vec_dot: unsupported quantization kind");
        return MARMOT_ERROR_NOT_IMPLEMENTED;
    }
    if (desc->layout != MARMOT_QUANT_LAYOUT_GGUF) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "cuda_vec_dot: quantization layout mismatch");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    const marmot_quant_kind_t expected = kind == MCU_KIND_Q8_0 ? MARMOT_QUANT_KIND_Q8_0 : MARMOT_QUANT_KIND_Q8_K;
    if (desc->activation_kind != expected) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "cuda_vec_dot: activation kind mismatch");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    const int rc = mcu_vec_dot_host(c->mcu, kind, desc->weights, desc->activations, desc->num_blocks, result);
    return rc == 0 ? MARMOT_SUCCESS : cuda_fail(rc);
}

// ---- decoder operators around the matmuls ---------------------------------------------------------------------
// Adapters from marmot's descriptors to the C ABI's decoder kernels (mcu_rmsnorm, mcu_rope, mcu_swiglu, mcu_add,
// mcu_embedding_gather, mcu_paged_attention).  FLOAT32 activations, the shapes the graph builder emits for a
// Llama-family layer (src/graph/gguf/graph_builder.cpp:1454-2400); anything else is refused, never computed on
// the host.  Reference counterparts: cpu_rmsnorm_impl / cpu_rmsnorm_gemma_impl
// (src/backends/cpu/ops/normalization/normalization.c:240-246), cpu_rope (ops/rope/rope_dispatch.c:144-382),
// cpu_elementwise_binary_impl (ops/elementwise), cpu_embedding_gather (ops/embedding), cpu_paged_attention_impl
// (ops/paged_attention/paged_attention_ref.c).

static bool cuda_is_dense_f32(const marmot_tensor_t *t) {
    if (t == nullptr || t->dtype != MARMOT_DTYPE_FLOAT32 || t->shape.ndim == 0) return false;
    size_t expect = 1;
    for (size_t i = t->shape.ndim; i-- > 0;) {
        if (t->shape.shape[i] != 1 && t->shape.strides[i] != expect) return false;
        expect *= t->shape.shape[i];
    }
    return true;
}

static marmot_error_t cuda_rmsnorm_common(const void *device_ctx, const marmot_rmsnorm_desc_t *desc, float weight_offset) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (c == nullptr) {
        marmot_set_error(MARMOT_ERROR_DEVICE_NOT_AVAILABLE, "CUDA context is not initialised");
        return MARMOT_ERROR_DEVICE_NOT_AVAILABLE;
    }
    if (desc == nullptr || desc->x == nullptr || desc->out == nullptr) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "RMSNorm descriptor is incomplete");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    const marmot_tensor_t *x = desc->x;
    if (!cuda_is_dense_f32(x) || !cuda_is_dense_f32(desc->out) || (desc->residual != nullptr && !cuda_is_dense_f32(desc->residual)) ||
        (desc->weight != nullptr && desc->weight->dtype != MARMOT_DTYPE_FLOAT32)) {
        marmot_set_error(MARMOT_ERROR_UNSUPPORTED_DTYPE, "CUDA RMSNorm takes dense FLOAT32 tensors");
        return MARMOT_ERROR_UNSUPPORTED_DTYPE;
    }
    const size_t n = x->shape.shape[x->shape.ndim - 1], total = marmot_tensor_num_elements(x);
    if (n == 0 || marmot_tensor_num_elements(desc->out) != total ||
        (desc->residual != nullptr && marmot_tensor_num_elements(desc->residual) != total) ||
        (desc->weight != nullptr && marmot_tensor_num_elements(desc->weight) != n)) {
        marmot_set_error(MARMOT_ERROR_DIMENSION_MISMATCH, "RMSNorm shapes do not match");
        return MARMOT_ERROR_DIMENSION_MISMATCH;
    }
    pthread_mutex_lock(&c->mu);
    const void *xd = nullptr, *rd = nullptr, *wd = nullptr;
    void *od = nullptr;
    marmot_error_t st = resident_ro(c, x, total * sizeof(float), &xd);
    if (st == MARMOT_SUCCESS && desc->residual != nullptr) st = resident_ro(c, desc->residual, total * sizeof(float), &rd);
    if (st == MARMOT_SUCCESS && desc->weight != nullptr) st = resident_ro(c, desc->weight, n * sizeof(float), &wd);
    if (st == MARMOT_SUCCESS) st = resident_rw(c, desc->out, total * sizeof(float), &od);
    if (st == MARMOT_SUCCESS) {
        const int rc = mcu_rmsnorm(c->mcu, xd, rd, wd, total / n, n, desc->eps, weight_offset, od);
        if (rc != 0) st = cuda_fail(rc);
    }
    pthread_mutex_unlock(&c->mu);
    return st;
}

marmot_error_t cuda_rmsnorm_impl(const void *device_ctx, const marmot_rmsnorm_desc_t *desc) {
    return cuda_rmsnorm_common(device_ctx, desc, 0.0f);
}

marmot_error_t cuda_rmsnorm_gemma_impl(const void *device_ctx, const marmot_rmsnorm_desc_t *desc) {
    return cuda_rmsnorm_common(device_ctx, desc, 1.0f);
}

// x [..., rows, dim]: every row is one head of one token and is rotated with the position of its row
// (the graph reshapes q / k to [tokens * heads, head_dim] and repeats the positions, like the reference's callers).
marmot_error_t cuda_rope(const void *device_ctx, const marmot_tensor_t *x, const marmot_rope_params_t *params, marmot_tensor_t *out) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (c == nullptr) {
        marmot_set_error(MARMOT_ERROR_DEVICE_NOT_AVAILABLE, "CUDA context is not initialised");
        return MARMOT_ERROR_DEVICE_NOT_AVAILABLE;
    }
    if (params == nullptr || params->positions == nullptr || x == nullptr || out == nullptr) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "RoPE needs input, output and a positions tensor");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    if (!cuda_is_dense_f32(x) || !cuda_is_dense_f32(out) || params->positions->dtype != MARMOT_DTYPE_INT32) {
        marmot_set_error(MARMOT_ERROR_UNSUPPORTED_DTYPE, "CUDA RoPE takes dense FLOAT32 tensors and INT32 positions");
        return MARMOT_ERROR_UNSUPPORTED_DTYPE;
    }
    if (params->scaling_type != MARMOT_ROPE_SCALING_NONE && params->scaling_type != MARMOT_ROPE_SCALING_LINEAR) {
        marmot_set_error(MARMOT_ERROR_NOT_IMPLEMENTED, "CUDA RoPE covers plain and linearly scaled frequencies only");
        return MARMOT_ERROR_NOT_IMPLEMENTED;
    }
    if (params->rope_type != MARMOT_ROPE_TYPE_NORM && params->rope_type != MARMOT_ROPE_TYPE_NEOX) {
        marmot_set_error(MARMOT_ERROR_NOT_IMPLEMENTED, "CUDA RoPE covers the NORM and NEOX pairings");
        return MARMOT_ERROR_NOT_IMPLEMENTED;
    }
    if (x->shape.ndim < 2) {
        marmot_set_error(MARMOT_ERROR_DIMENSION_MISMATCH, "RoPE requires at least 2D tensor");
        return MARMOT_ERROR_DIMENSION_MISMATCH;
    }
    const size_t dim = x->shape.shape[x->shape.ndim - 1], total = marmot_tensor_num_elements(x);
    if (dim == 0 || dim % 2 != 0 || total == 0 || marmot_tensor_num_elements(out) != total ||
        marmot_tensor_num_elements(params->positions) != total / dim) {
        marmot_set_error(MARMOT_ERROR_DIMENSION_MISMATCH, "RoPE shapes do not match");
        return MARMOT_ERROR_DIMENSION_MISMATCH;
    }
    const size_t rows = total / dim;
    const float freq_scale = params->scaling_type == MARMOT_ROPE_SCALING_LINEAR ? params->freq_scale : 1.0f;
    pthread_mutex_lock(&c->mu);
    const void *xd = nullptr, *pd = nullptr;
    void *od = nullptr;
    marmot_error_t st = resident_ro(c, x, total * sizeof(float), &xd);
    if (st == MARMOT_SUCCESS) st = resident_ro(c, params->positions, rows * sizeof(int32_t), &pd);
    if (st == MARMOT_SUCCESS) st = resident_rw(c, out, total * sizeof(float), &od);
    if (st == MARMOT_SUCCESS) {
        const int rc = mcu_rope(c->mcu, xd, dim, pd, rows, 1, dim, params->theta, freq_scale,
                                params->rope_type == MARMOT_ROPE_TYPE_NEOX ? MCU_ROPE_NEOX : MCU_ROPE_NORM, od, dim);
        if (rc != 0) st = cuda_fail(rc);
    }
    pthread_mutex_unlock(&c->mu);
    return st;
}

// add and swiglu (silu(a) * b) on dense FLOAT32 tensors of equal size.
marmot_error_t cuda_elementwise_binary_impl(
    const void *device_ctx, marmot_device_binary_op_t op, const marmot_tensor_t *a, const marmot_tensor_t *b,
    marmot_tensor_t *out
) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (c == nullptr) {
        marmot_set_error(MARMOT_ERROR_DEVICE_NOT_AVAILABLE, "CUDA context is not initialised");
        return MARMOT_ERROR_DEVICE_NOT_AVAILABLE;
    }
    if (op != MARMOT_DEVICE_BINARY_ADD && op != MARMOT_DEVICE_BINARY_SWIGLU) {
        marmot_set_error(MARMOT_ERROR_NOT_IMPLEMENTED, "CUDA elementwise kernels: add and swiglu");
        return MARMOT_ERROR_NOT_IMPLEMENTED;
    }
    if (a == nullptr || b == nullptr || out == nullptr) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "Null tensor pointer");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    if (!cuda_is_dense_f32(a) || !cuda_is_dense_f32(b) || !cuda_is_dense_f32(out)) {
        marmot_set_error(MARMOT_ERROR_UNSUPPORTED_DTYPE, "CUDA elementwise kernels take dense FLOAT32 tensors");
        return MARMOT_ERROR_UNSUPPORTED_DTYPE;
    }
    const size_t n = marmot_tensor_num_elements(a);
    if (marmot_tensor_num_elements(b) != n || marmot_tensor_num_elements(out) != n) {
        marmot_set_error(MARMOT_ERROR_DIMENSION_MISMATCH, "elementwise operands must have equal sizes (no broadcasting)");
        return MARMOT_ERROR_DIMENSION_MISMATCH;
    }
    if (n == 0) return MARMOT_SUCCESS;
    pthread_mutex_lock(&c->mu);
    const void *ad = nullptr, *bd = nullptr;
    void *od = nullptr;
    marmot_error_t st = resident_ro(c, a, n * sizeof(float), &ad);
    if (st == MARMOT_SUCCESS) st = resident_ro(c, b, n * sizeof(float), &bd);
    if (st == MARMOT_SUCCESS) st = resident_rw(c, out, n * sizeof(float), &od);
    if (st == MARMOT_SUCCESS) {
        const int rc = op == MARMOT_DEVICE_BINARY_ADD ? mcu_add(c->mcu, ad, bd, n, od) : mcu_swiglu(c->mcu, ad, bd, n, od);
        if (rc != 0) st = cuda_fail(rc);
    }
    pthread_mutex_unlock(&c->mu);
    return st;
}

// Rows of a quantized table -> FLOAT32 (bit-exact with the dequantizers); INT32 token ids.
marmot_error_t cuda_embedding_gather(const void *device_ctx, const marmot_embedding_gather_desc_t *desc) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (c == nullptr) {
        marmot_set_error(MARMOT_ERROR_DEVICE_NOT_AVAILABLE, "CUDA context is not initialised");
        return MARMOT_ERROR_DEVICE_NOT_AVAILABLE;
    }
    if (desc == nullptr || desc->weights == nullptr || desc->token_ids == nullptr || desc->out == nullptr) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "Embedding descriptor is incomplete");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    const marmot_tensor_t *w = desc->weights;
    const int kind = mcu_kind_of(w->quant_kind);
    if (kind < 0 || w->shape.ndim != 2) {
        marmot_set_error(MARMOT_ERROR_NOT_IMPLEMENTED, "CUDA embedding gather covers 2D Q4_K, Q6_K and Q8_0 tables");
        return MARMOT_ERROR_NOT_IMPLEMENTED;
    }
    if (desc->token_ids->dtype != MARMOT_DTYPE_INT32 || !cuda_is_dense_f32(desc->out) ||
        (desc->dtype_out != MARMOT_DTYPE_FLOAT32 && desc->dtype_out != MARMOT_DTYPE_COUNT)) {
        marmot_set_error(MARMOT_ERROR_UNSUPPORTED_DTYPE, "CUDA embedding gather takes INT32 ids and writes FLOAT32");
        return MARMOT_ERROR_UNSUPPORTED_DTYPE;
    }
    if (desc->scale != 1.0f && desc->scale != 0.0f) {
        marmot_set_error(MARMOT_ERROR_NOT_IMPLEMENTED, "CUDA embedding gather does not scale its output");
        return MARMOT_ERROR_NOT_IMPLEMENTED;
    }
    const size_t vocab = w->shape.shape[0], dim = w->shape.shape[1], T = marmot_tensor_num_elements(desc->token_ids);
    if (marmot_tensor_num_elements(desc->out) != T * dim) {
        marmot_set_error(MARMOT_ERROR_DIMENSION_MISMATCH, "Embedding output shape does not match");
        return MARMOT_ERROR_DIMENSION_MISMATCH;
    }
    if (T == 0) return MARMOT_SUCCESS;
    if (desc->bounds_check || desc->padding_id >= 0) {
        // ids are host-visible when the caller asks for checks: reject what the kernel would read out of range
        const int32_t *ids = (const int32_t *)desc->token_ids->data;
        for (size_t i = 0; i < T; ++i) {
            if (ids[i] < 0 || (size_t)ids[i] >= vocab || ids[i] == desc->padding_id) {
                marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "Embedding token id out of range (padding ids are not supported on CUDA)");
                return MARMOT_ERROR_INVALID_ARGUMENT;
            }
        }
    }
    pthread_mutex_lock(&c->mu);
    const void *wd = nullptr, *id = nullptr;
    void *od = nullptr;
    marmot_error_t st = resident_ro(c, w, vocab * mcu_row_bytes(kind, dim), &wd);
    if (st == MARMOT_SUCCESS) st = resident_ro(c, desc->token_ids, T * sizeof(int32_t), &id);
    if (st == MARMOT_SUCCESS) st = resident_rw(c, desc->out, T * dim * sizeof(float), &od);
    if (st == MARMOT_SUCCESS) {
        const int rc = mcu_embedding_gather(c->mcu, kind, wd, dim, id, T, od);
        if (rc != 0) st = cuda_fail(rc);
    }
    pthread_mutex_unlock(&c->mu);
    return st;
}

// Contract of include/marmot/ops/paged_attention.h:13-56; FLOAT32 q / k / v, FLOAT32 or FLOAT16 pools, no FP8 scales.
marmot_error_t cuda_paged_attention_impl(const void *device_ctx, const marmot_paged_attention_desc_t *desc) {
    cuda_ctx_t *c = (cuda_ctx_t *)device_ctx;
    if (c == nullptr) {
        marmot_set_error(MARMOT_ERROR_DEVICE_NOT_AVAILABLE, "CUDA context is not initialised");
        return MARMOT_ERROR_DEVICE_NOT_AVAILABLE;
    }
    if (desc == nullptr || desc->token_meta == nullptr || desc->q == nullptr || desc->k_new == nullptr || desc->v_new == nullptr ||
        desc->kv_k == nullptr || desc->kv_v == nullptr || desc->block_table == nullptr || desc->out == nullptr) {
        marmot_set_error(MARMOT_ERROR_INVALID_ARGUMENT, "Paged attention descriptor is incomplete");
        return MARMOT_ERROR_INVALID_ARGUMENT;
    }
    if (desc->pnext != nullptr) {
        marmot_set_error(MARMOT_ERROR_NOT_IMPLEMENTED, "CUDA paged attention has no FP8 pools with per-block scales");
        return MARMOT_ERROR_NOT_IMPLEMENTED;
    }
    const marmot_dtype_t kv_dt = desc->kv_k->dtype;
    if (!cuda_is_dense_f32(desc->q) || !cuda_is_dense_f32(desc->k_new) || !cuda_is_dense_f32(desc->v_new) ||
        !cuda_is_dense_f32(desc->out) || (kv_dt != MARMOT_DTYPE_FLOAT32 && kv_dt != MARMOT_DTYPE_FLOAT16) ||
        desc->kv_v->dtype != kv_dt || desc->token_meta->dtype != MARMOT_DTYPE_UINT32 ||
        desc->block_table->dtype != MARMOT_DTYPE_UINT32) {
        marmot_set_error(MARMOT_ERROR_UNSUPPORTED_DTYPE, "CUDA paged attention: FLOAT32 q/k/v, FLOAT32 or FLOAT16 pools, UINT32 tables");
        return MARMOT_ERROR_UNSUPPORTED_DTYPE;
    }
    const size_t T = desc->token_count, hq = desc->num_q_heads, hkv = desc->num_kv_heads, hd = desc->head_dim, bs = desc->block_size;
    if (desc->kv_k->shape.ndim != 5 || desc->block_table->shape.ndim != 2 || desc->token_meta->shape.ndim != 2 ||
        desc->token_meta->shape.shape[0] < T || desc->token_meta->shape.shape[1] != 4 ||
        marmot_tensor_num_elements(desc->q) < T * hq * hd || marmot_tensor_num_elements(desc->k_new) < T * hkv * hd ||
        marmot_tensor_num_elements(desc->v_new) < T * hkv * hd || marmot_tensor_num_elements(desc->out) < T * hq * hd ||
        desc->kv_k->shape.shape[2] != hkv || desc->kv_k->shape.shape[3] != bs || desc->kv_k->shape.shape[4] != hd ||
        desc->layer_idx >= desc->kv_k->shape.shape[1]) {
        marmot_set_error(MARMOT_ERROR_DIMENSION_MISMATCH, "Paged attention shapes do not match");
        return MARMOT_ERROR_DIMENSION_MISMATCH;
    }
    if (T == 0) return MARMOT_SUCCESS;
    const size_t pool_bytes = marmot_tensor_num_elements(desc->kv_k) * (kv_dt == MARMOT_DTYPE_FLOAT16 ? 2 : 4);
    pthread_mutex_lock(&c->mu);
    const void *md = nullptr, *qd = nullptr, *kd = nullptr, *vd = nullptr, *td = nullptr;
    void *pk = nullptr, *pv = nullptr, *od = nullptr;
    marmot_error_t st = resident_ro(c, desc->token_meta, T * 4 * sizeof(uint32_t), &md);
    if (st == MARMOT_SUCCESS) st = resident_ro(c, desc->q, T * hq * hd * sizeof(float), &qd);
    if (st == MARMOT_SUCCESS) st = resident_ro(c, desc->k_new, T * hkv * hd * sizeof(float), &kd);
    if (st == MARMOT_SUCCESS) st = resident_ro(c, desc->v_new, T * hkv * hd * sizeof(float), &vd);
    if (st == MARMOT_SUCCESS) st = resident_ro(c, desc->block_table, marmot_tensor_num_elements(desc->block_table) * sizeof(uint32_t), &td);
    // the pools are read and written: current on the device first, then the device copy becomes the newer one
    const void *tmp = nullptr;
    if (st == MARMOT_SUCCESS) st = resident_ro(c, desc->kv_k, pool_bytes, &tmp);
    if (st == MARMOT_SUCCESS) st = resident_rw(c, (marmot_tensor_t *)desc->kv_k, pool_bytes, &pk);
    if (st == MARMOT_SUCCESS) st = resident_ro(c, desc->kv_v, pool_bytes, &tmp);
    if (st == MARMOT_SUCCESS) st = resident_rw(c, (marmot_tensor_t *)desc->kv_v, pool_bytes, &pv);
    if (st == MARMOT_SUCCESS) st = resident_rw(c, desc->out, T * hq * hd * sizeof(float), &od);
    if (st == MARMOT_SUCCESS) {
        const int rc = mcu_paged_attention(c->mcu, md, T, qd, kd, vd, pk, pv, kv_dt == MARMOT_DTYPE_FLOAT16 ? MCU_KV_F16 : MCU_KV_F32,
                                           td, desc->block_table->shape.shape[1], desc->kv_k->shape.shape[1], desc->layer_idx, hq,
                                           hkv, hd, bs, desc->scale, od);
        if (rc != 0) st = cuda_fail(rc);
    }
    pthread_mutex_unlock(&c->mu);
    return st;
}

// ---- kernel query, capabilities, preferences ----------------------------------------------------------
// Reference counterparts: marmot_cpu_query_kernel / marmot_metal_query_kernel (generated, called from
// src/core/dispatch/kernel_query.c:35-52), marmot_metal_detect_default_caps and marmot_*_default_preferences
// (kernel_query.c:88-132, src/backends/cpu/runtime/runtime.c:1388-1407).  A signature without a CUDA kernel is
// answered with supported = false here, at query time: nothing is ever computed on the host instead
// (src/core/dispatch/dispatch_execute.c:214-233 would otherwise look for an unfused fallback).
//
#if !defined(MARMOT_CUDA_GENERATED_QUERY)
// Inside a marmot build the query is GENERATED from kernels/*.def by scripts/codegen/gen_kernels.py (build_marmot.py
// compiles this file with MARMOT_CUDA_GENERATED_QUERY); the function below serves the stand-alone host library, which
// is built against an unmodified marmot whose enumeration has no CUDA entries: its kernel ids continue marmot's
// generated enumeration (include/marmot/traits_ids.gen.h) and it answers for the same operators as the .def files.
enum {
    CUDA_KERNEL_MATMUL_Q4_K_F32_NT = MARMOT_KERNEL_COUNT,
    CUDA_KERNEL_MATMUL_Q6_K_F32_NT,
    CUDA_KERNEL_MATMUL_Q8_0_F32_NT,
    CUDA_KERNEL_MOE_EXPERTS_Q4_K,
    CUDA_KERNEL_MOE_EXPERTS_Q6_K,
    CUDA_KERNEL_MOE_EXPERTS_Q8_0,
    CUDA_KERNEL_TOPK_F32,
    CUDA_KERNEL_DEQUANTIZE_Q4_K,
    CUDA_KERNEL_DEQUANTIZE_Q6_K,
    CUDA_KERNEL_DEQUANTIZE_Q8_0,
    CUDA_KERNEL_EMBEDDING_Q4_K,
    CUDA_KERNEL_EMBEDDING_Q6_K,
    CUDA_KERNEL_EMBEDDING_Q8_0,
    CUDA_KERNEL_RMS_NORM_F32,
    CUDA_KERNEL_RMS_NORM_GEMMA_F32,
    CUDA_KERNEL_ROPE_F32,
    CUDA_KERNEL_ADD_F32,
    CUDA_KERNEL_SWIGLU_F32,
    CUDA_KERNEL_PAGED_ATTENTION_F32_KV_F32,
    CUDA_KERNEL_PAGED_ATTENTION_F32_KV_F16,
    CUDA_KERNEL_END,
};

static marmot_kernel_selection_t cuda_unsupported(const char *reason) {
    return (marmot_kernel_selection_t){
        .supported = false,
        .kernel_id = MARMOT_KERNEL_INVALID,
        .op_index = MARMOT_KERNEL_OP_INDEX_INVALID,
        .fallback_reason = reason,
    };
}

// bytes moved / bandwidth + flops / tensor rate + a launch: the same shape of estimate the other backends give the
// graph scheduler; est_comm_us / shardable_axes / device_affinity stay 0 as everywhere in the reference
// (include/marmot/graph/kernel_selection.h:18-23).
static marmot_kernel_selection_t
cuda_supported(int kernel, const marmot_device_caps_t *caps, double bytes, double flops, double workspace_bytes) {
    const double bw = caps->mem_bw_gbps > 0.0f ? caps->mem_bw_gbps : 6500.0;            // GB/s
    const double tf = caps->peak_flops_tflops_fp16 > 0.0f ? caps->peak_flops_tflops_fp16 : 1600.0;
    const double launch = caps->launch_overhead_us > 0.0f ? caps->launch_overhead_us : 4.0;
    const double t_mem = bytes / (bw * 1e3), t_math = flops / (tf * 1e6);  // microseconds
    return (marmot_kernel_selection_t){
        .supported = true,
        .kernel_id = (marmot_kernel_id_t)kernel,
        .op_index = (uint16_t)(kernel - (int)MARMOT_KERNEL_COUNT),
        .estimated_us = launch + (t_mem > t_math ? t_mem : t_math),
        .est_workspace_mb = workspace_bytes / (1024.0 * 1024.0),
        .confidence = 0.8f,
        .fallback_reason = nullptr,
    };
}

static int cuda_kind_slot(marmot_qscheme_id_t q) {  // 0 / 1 / 2 for the three block formats with kernels, else -1
    switch (q) {
    case MARMOT_QSCHEME_Q4_K:
        return 0;
    case MARMOT_QSCHEME_Q6_K:
        return 1;
    case MARMOT_QSCHEME_Q8_0:
        return 2;
    default:
        return -1;
    }
}

static double cuda_bits_per_weight(int slot) { return slot == 0 ? 4.5 : slot == 1 ? 6.5625 : 8.5; }

marmot_kernel_selection_t marmot_cuda_query_kernel(const marmot_op_signature_t *sig, const marmot_device_caps_t *caps) {
    if (sig == nullptr || caps == nullptr) return cuda_unsupported("Invalid kernel query arguments");
    if (caps->backend.cuda.compute_capability / 10 != 10)
        return cuda_unsupported("CUDA kernels are built for sm_100a only");
    if (sig->variant_flags != 0) return cuda_unsupported("no fused variants on CUDA");
    const bool f32_io = sig->input_dtype == MARMOT_DTYPE_FLOAT32 && sig->output_dtype == MARMOT_DTYPE_FLOAT32;
    const int slot = cuda_kind_slot(sig->qscheme_id);
    switch (sig->op_id) {
    case MARMOT_OP_MATMUL:
    case MARMOT_OP_LINEAR: {
        if (slot < 0) return cuda_unsupported("CUDA matmul covers Q4_K, Q6_K and Q8_0 weights");
        const bool f16_in = sig->input_dtype == MARMOT_DTYPE_FLOAT16 &&
            (sig->output_dtype == MARMOT_DTYPE_FLOAT32 || sig->output_dtype == MARMOT_DTYPE_FLOAT16);
        if (!f32_io && !f16_in)
            return cuda_unsupported("CUDA quantized matmul takes FLOAT32 in and out, or FLOAT16 in with FLOAT32 / FLOAT16 out");
        if (sig->matmul_layout != MARMOT_MATMUL_LAYOUT_NT) return cuda_unsupported("CUDA quantized matmul is NT only");
        if (sig->weight_layout != MARMOT_WEIGHT_LAYOUT_SEPARATE) return cuda_unsupported("packed weight layouts are CPU caches");
        if ((sig->epilogue_flags & ~(uint32_t)MARMOT_EPILOGUE_BIAS) != 0 || sig->activation != MARMOT_DEVICE_UNARY_IDENTITY)
            return cuda_unsupported("CUDA matmul epilogue is bias only");
        if (sig->stride_mode == MARMOT_STRIDE_MODE_STRIDED) return cuda_unsupported("inner stride must be 1");
        const double T = (double)sig->dims.matmul.N, K = (double)sig->dims.matmul.K, F = (double)sig->dims.matmul.M;
        const double bytes = F * K * cuda_bits_per_weight(slot) / 8.0 + 4.0 * T * (K + F);
        // split-K partial tiles of the few-token tensor-core path (at most sixteen splits)
        const double ws = (T > 8 && T <= 64) ? 16.0 * T * F * 4.0 : 0.0;
        return cuda_supported(CUDA_KERNEL_MATMUL_Q4_K_F32_NT + slot, caps, bytes, 2.0 * T * K * F, ws + 2.0 * T * K);
    }
    case MARMOT_OP_MOE_EXPERTS:
        if (slot < 0) return cuda_unsupported("CUDA MoE experts cover Q4_K, Q6_K and Q8_0 weights");
        if (!f32_io) return cuda_unsupported("CUDA MoE experts take FLOAT32 activations");
        return cuda_supported(CUDA_KERNEL_MOE_EXPERTS_Q4_K + slot, caps, 0.0, 0.0, 0.0);
    case MARMOT_OP_TOPK:
        if (sig->input_dtype != MARMOT_DTYPE_FLOAT32) return cuda_unsupported("CUDA top-k is FLOAT32");
        return cuda_supported(CUDA_KERNEL_TOPK_F32, caps, 0.0, 0.0, 0.0);
    case MARMOT_OP_DEQUANTIZE:
        if (slot < 0 || sig->output_dtype != MARMOT_DTYPE_FLOAT32)
            return cuda_unsupported("CUDA dequantize covers Q4_K, Q6_K and Q8_0 to FLOAT32");
        return cuda_supported(CUDA_KERNEL_DEQUANTIZE_Q4_K + slot, caps, 4.0 * sig->dims.elementwise.n_elems, 0.0, 0.0);
    case MARMOT_OP_EMBEDDING:
        if (slot < 0 || sig->output_dtype != MARMOT_DTYPE_FLOAT32)
            return cuda_unsupported("CUDA embedding gather covers Q4_K, Q6_K and Q8_0 tables to FLOAT32");
        return cuda_supported(CUDA_KERNEL_EMBEDDING_Q4_K + slot, caps, 0.0, 0.0, 0.0);
    case MARMOT_OP_RMS_NORM:
    case MARMOT_OP_RMS_NORM_GEMMA:
        if (!f32_io) return cuda_unsupported("CUDA RMSNorm is FLOAT32");
        return cuda_supported(sig->op_id == MARMOT_OP_RMS_NORM ? CUDA_KERNEL_RMS_NORM_F32 : CUDA_KERNEL_RMS_NORM_GEMMA_F32,
                              caps, 8.0 * sig->dims.layernorm.n * sig->dims.layernorm.d, 0.0, 0.0);
    case MARMOT_OP_ROPE:
        if (!f32_io) return cuda_unsupported("CUDA RoPE is FLOAT32");
        return cuda_supported(CUDA_KERNEL_ROPE_F32, caps, 0.0, 0.0, 0.0);
    case MARMOT_OP_ADD:
    case MARMOT_OP_SWIGLU:
        if (!f32_io) return cuda_unsupported("CUDA elementwise kernels are FLOAT32");
        if (sig->stride_mode != MARMOT_STRIDE_MODE_ANY && sig->stride_mode != MARMOT_STRIDE_MODE_CONTIGUOUS)
            return cuda_unsupported("CUDA elementwise kernels take contiguous tensors");
        return cuda_supported(sig->op_id == MARMOT_OP_ADD ? CUDA_KERNEL_ADD_F32 : CUDA_KERNEL_SWIGLU_F32, caps,
                              12.0 * sig->dims.elementwise.n_elems, 0.0, 0.0);
    case MARMOT_OP_PAGED_ATTENTION:
        if (!f32_io) return cuda_unsupported("CUDA paged attention takes FLOAT32 q/k/v");
        if (sig->weight_dtype == MARMOT_DTYPE_FLOAT16)
            return cuda_supported(CUDA_KERNEL_PAGED_ATTENTION_F32_KV_F16, caps, 0.0, 0.0, 0.0);
        if (sig->weight_dtype == MARMOT_DTYPE_FLOAT32)
            return cuda_supported(CUDA_KERNEL_PAGED_ATTENTION_F32_KV_F32, caps, 0.0, 0.0, 0.0);
        return cuda_unsupported("CUDA paged attention KV pool must be FLOAT32 or FLOAT16");
    default:
        return cuda_unsupported("no CUDA kernel for this operator");
    }
}

#endif  // !MARMOT_CUDA_GENERATED_QUERY

marmot_device_caps_t marmot_cuda_detect_default_caps(void) {
    marmot_device_caps_t caps;
    memset(&caps, 0, sizeof(caps));
    mcu_device_caps_t dc;
    if (mcu_device_caps(0, &dc) != MCU_SUCCESS) return caps;  // no device: every query answers "unsupported"
    const double ghz = dc.sm_clock_mhz / 1000.0;
    caps.peak_flops_tflops_fp32 = (float)(dc.sm_count * 128 * 2 * ghz / 1000.0);
    // fifth-generation tensor cores: 8192 dense fp16/bf16 FMAs per SM and clock
    caps.peak_flops_tflops_fp16 = (float)(dc.sm_count * 8192.0 * 2 * ghz / 1000.0);
    caps.mem_bw_gbps = dc.mem_bw_gbps;
    caps.launch_overhead_us = 4.0f;
    caps.edge_penalty_alpha = 0.0f;
    caps.l1_cache_kb = (uint32_t)dc.shared_mem_kb;
    caps.l2_cache_kb = (uint32_t)dc.l2_cache_kb;
    caps.num_compute_units = (uint32_t)dc.sm_count;
    caps.simd_width = 32;
    caps.has_fma = true;
    caps.has_fp16_compute = true;
    caps.has_bf16_compute = true;
    caps.has_tensor_cores = true;
    caps.has_simdgroup_mm = false;
    caps.h2d_bw_gbps = 55.0f;  // PCIe 5 x16
    caps.d2h_bw_gbps = 55.0f;
    caps.d2d_bw_gbps = 900.0f;  // NVLink 5, per direction
    caps.d2d_lat_us = 2.0f;
    caps.copy_engines = (uint32_t)dc.copy_engines;
    caps.max_streams = 1;  // one stream per context
    caps.backend.cuda.sm_count = (uint32_t)dc.sm_count;
    caps.backend.cuda.shared_mem_kb = (uint32_t)dc.shared_mem_kb;
    caps.backend.cuda.compute_capability = (uint32_t)dc.compute_capability;
    return caps;
}

bool marmot_cuda_default_preferences(const marmot_device_caps_t *caps, marmot_backend_preferences_t *out) {
    if (out == nullptr) return false;
    (void)caps;
    *out = (marmot_backend_preferences_t){
        .policy =
            {
                .embedding_quant_output_dtype = MARMOT_DTYPE_FLOAT32,
                .quant_activation_mode = MARMOT_QUANT_ACTIVATION_AUTO,
                .variant_flags_mask = 0,  // no fused variants: the graph builder emits the plain operators
                .embedding_prefer_gpu_private = true,
                .embedding_allow_quant_decode_on_the_fly = true,
                .matmul_requires_temp_tensors = false,
                .matmul_prefer_packed_weights = false,  // raw GGUF blocks are what the kernels stream
            },
        .routing_policy = MARMOT_ROUTING_ALWAYS_GPU,
    };
    return true;
}
