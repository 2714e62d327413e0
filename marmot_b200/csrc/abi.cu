// extern "C" entry points of libmarmot_cuda.so (declared in include/marmot_cuda.h): context,
// device memory, regime selection and workspace handling around the kernels.  No CPU fallback:
// every operation either enqueues CUDA kernels or returns an error.
#include "../../include/marmot_cuda.h"

#include "common.cuh"
#include "kernels.h"
#include "moe.h"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <climits>
#include <mutex>
#include <vector>

namespace mcu {

std::atomic<uint64_t> g_kernel_launches{0};
void count_launches(int n) { g_kernel_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

static thread_local char g_err[512] = "";

static int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int set_error(int code, const char *message) { return fail(code, "%s", message); }

static int cuda_fail(cudaError_t e, const char *what) {
    const int code = e == cudaErrorMemoryAllocation ? MCU_ERROR_OUT_OF_MEMORY
        : (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver || e == cudaErrorInvalidDevice)
        ? MCU_ERROR_DEVICE_NOT_AVAILABLE
        : MCU_ERROR_INVALID_OPERATION;
    return fail(code, "%s: %s", what, cudaGetErrorString(e));
}

#define MCU_CUDA(expr)                                              \
    do {                                                            \
        cudaError_t e__ = (expr);                                   \
        if (e__ != cudaSuccess) return cuda_fail(e__, #expr);       \
    } while (0)

// SM count of the calling thread's current device (every launcher runs with its context's device current).
int device_sm_count() {
    static std::atomic<int> cache[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int v = cache[dev].load(std::memory_order_relaxed);
    if (v > 0) return v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 148;
    cache[dev].store(v, std::memory_order_relaxed);
    return v;
}

struct Buffer {
    void *ptr = nullptr;
    size_t cap = 0;
};

}  // namespace mcu

using namespace mcu;

constexpr int PIN_SLOTS = 16;
constexpr size_t PIN_SLOT_BYTES = 64 * 1024;

struct mcu_context {
    int device = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    int regime = MCU_REGIME_AUTO;
    std::mutex mu;  // guards the workspace; calls on one context are serialised
    // workspace (grows on demand, never shrinks)
    Buffer act_qs, act_d, act_bsums, act_half, act_rowscale, x_stage, out_stage, bias_stage;
    Buffer moe_meta, moe_hidden, moe_gate, moe_up, moe_down;
    Buffer gemm_partial;         // split-K partial tiles
    Buffer rope_table;              // {cos, sin} per token and pair when a decode attention call brings none
    Buffer attn_tickets;            // fused decode attention: one counter per (token, KV head)
    Buffer pro_h;                   // activations after a stand-alone prologue kernel (mcu_linear_multi's general form)
    Buffer i8_partial, i8_tickets;  // integer-MMA matmul: shares of row groups split between CTAs, and their tickets
    Buffer attn_partial;         // split-KV partial attention states
    int *gemm_counters = nullptr;  // split-K tile tickets (zero between launches)
    std::vector<int> host_counts;
    size_t moe_last_routes = 0, moe_last_experts = 0;  // shape of the last MoE call (mcu_moe_last_buffers)
    int moe_last_grouped = 0;
    int *dev_err = nullptr;  // set by kernels whose bounded device-side waits ran out
    int *err_host = nullptr; // page-locked word the flag is copied into on a synchronize
    // Small host <-> device copies go through page-locked slots owned by the context: an upload is a host memcpy into a
    // slot plus an asynchronous copy (the caller's buffer is free on return and nothing waits for the copy engine), a
    // download lands in a slot and is copied out after the one synchronize it needs anyway.
    uint8_t *pin_ring = nullptr;
    cudaEvent_t pin_event[PIN_SLOTS] = {};
    bool pin_used[PIN_SLOTS] = {};
    int pin_next = 0;
};

static bool stream_is_capturing(cudaStream_t s) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &st) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return st != cudaStreamCaptureStatusNone;
}

static int ensure(mcu_context *ctx, Buffer &b, size_t bytes) {
    if (bytes <= b.cap) return MCU_SUCCESS;
    // Growing means a synchronize, a free and an allocation: none of that can be recorded into a CUDA graph, and the
    // graph would keep the old address anyway.
    if (stream_is_capturing(ctx->stream))
        return fail(MCU_ERROR_INVALID_OPERATION,
                    "workspace would have to grow during stream capture: run the same call once before capturing");
    // Kernels already enqueued may still read the old allocation.
    MCU_CUDA(cudaStreamSynchronize(ctx->stream));
    if (b.ptr != nullptr) MCU_CUDA(cudaFree(b.ptr));
    b.ptr = nullptr;
    b.cap = 0;
    const size_t want = (bytes + 255) & ~(size_t)255;
    MCU_CUDA(cudaMalloc(&b.ptr, want));
    b.cap = want;
    return MCU_SUCCESS;
}

// After a synchronize: did a kernel give up on a bounded wait?
// Wait for the stream `s` of the context and report a device-side error flag, if one was set.  The flag travels with
// the wait (an asynchronous copy into a page-locked word enqueued ahead of the synchronize): a separate blocking copy
// of four bytes cost ten microseconds on every synchronising call.
static int sync_and_check(mcu_context *ctx, cudaStream_t s) {
    if (ctx->err_host == nullptr) {
        MCU_CUDA(cudaStreamSynchronize(s));
        int flag = 0;
        MCU_CUDA(cudaMemcpy(&flag, ctx->dev_err, sizeof(int), cudaMemcpyDeviceToHost));
        if (flag == 0) return MCU_SUCCESS;
        cudaMemset(ctx->dev_err, 0, sizeof(int));
        if (flag == 40) return fail(MCU_ERROR_INVALID_ARGUMENT, "MoE expert id is out of range (found by an earlier call)");
        return fail(MCU_ERROR_INVALID_OPERATION, "a device-side wait timed out (code %d)", flag);
    }
    MCU_CUDA(cudaMemcpyAsync(ctx->err_host, ctx->dev_err, sizeof(int), cudaMemcpyDeviceToHost, s));
    MCU_CUDA(cudaStreamSynchronize(s));
    const int flag = *(volatile int *)ctx->err_host;
    if (flag != 0) {
        cudaMemset(ctx->dev_err, 0, sizeof(int));
        if (flag == 40) return fail(MCU_ERROR_INVALID_ARGUMENT, "MoE expert id is out of range (found by an earlier call)");
        return fail(MCU_ERROR_INVALID_OPERATION, "a device-side wait timed out (code %d)", flag);
    }
    return MCU_SUCCESS;
}

namespace mcu {
int context_device(const mcu_context *ctx) { return ctx->device; }
int *context_err_flag(mcu_context *ctx) { return ctx->dev_err; }
int context_attention_scratch(mcu_context *ctx, size_t bytes, void **out) {
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (int rc = ensure(ctx, ctx->attn_partial, bytes)) return rc;
    *out = ctx->attn_partial.ptr;
    return MCU_SUCCESS;
}
int context_rope_table(mcu_context *ctx, size_t bytes, void **out) {
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (int rc = ensure(ctx, ctx->rope_table, bytes)) return rc;
    *out = ctx->rope_table.ptr;
    return MCU_SUCCESS;
}
// Zero-filled when it is (re)allocated; the attention kernel that uses the tickets leaves them at zero.
int context_attention_tickets(mcu_context *ctx, size_t bytes, void **out) {
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (bytes > ctx->attn_tickets.cap) {
        if (int rc = ensure(ctx, ctx->attn_tickets, bytes)) return rc;
        MCU_CUDA(cudaMemsetAsync(ctx->attn_tickets.ptr, 0, ctx->attn_tickets.cap, ctx->stream));
    }
    *out = ctx->attn_tickets.ptr;
    return MCU_SUCCESS;
}
}  // namespace mcu

static int check_ctx(mcu_context *ctx) {
    if (ctx == nullptr) return fail(MCU_ERROR_DEVICE_NOT_AVAILABLE, "CUDA context is not initialised");
    MCU_CUDA(cudaSetDevice(ctx->device));
    return MCU_SUCCESS;
}

extern "C" {

const char *mcu_last_error_message(void) { return g_err; }

uint64_t mcu_kernel_launch_count(const mcu_context_t *) { return g_kernel_launches.load(); }

int mcu_device_caps(int device, mcu_device_caps_t *out) {
    if (out == nullptr) return fail(MCU_ERROR_INVALID_ARGUMENT, "out is null");
    memset(out, 0, sizeof(*out));
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        return fail(MCU_ERROR_DEVICE_NOT_AVAILABLE, "no CUDA device: %s", cudaGetErrorString(e));
    }
    if (device < 0 || device >= n) return fail(MCU_ERROR_DEVICE_NOT_AVAILABLE, "device %d out of range (%d)", device, n);
    cudaDeviceProp prop;
    MCU_CUDA(cudaGetDeviceProperties(&prop, device));
    out->sm_count = prop.multiProcessorCount;
    out->compute_capability = prop.major * 10 + prop.minor;
    out->shared_mem_kb = (int)(prop.sharedMemPerMultiprocessor / 1024);
    out->l2_cache_kb = prop.l2CacheSize / 1024;
    out->sm_clock_mhz = prop.clockRate / 1000;
    out->mem_bw_gbps = 2.0f * (float)prop.memoryClockRate * 1e3f * (float)(prop.memoryBusWidth / 8) / 1e9f;
    out->total_mem_bytes = prop.totalGlobalMem;
    out->copy_engines = prop.asyncEngineCount;
    return MCU_SUCCESS;
}

int mcu_context_create(int device, mcu_context_t **out) {
    if (out == nullptr) return fail(MCU_ERROR_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0)
        return fail(MCU_ERROR_DEVICE_NOT_AVAILABLE, "no CUDA device: %s", cudaGetErrorString(e));
    if (device < 0 || device >= n) return fail(MCU_ERROR_DEVICE_NOT_AVAILABLE, "device %d out of range (%d)", device, n);
    MCU_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    MCU_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(MCU_ERROR_BACKEND_INIT_FAILED, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                    prop.major, prop.minor);
    mcu_context *ctx = new (std::nothrow) mcu_context();
    if (ctx == nullptr) return fail(MCU_ERROR_OUT_OF_MEMORY, "context allocation failed");
    ctx->device = device;
    e = cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        delete ctx;
        return cuda_fail(e, "cudaStreamCreate");
    }
    ctx->stream = ctx->own_stream;
    e = cudaMalloc(&ctx->dev_err, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(ctx->dev_err, 0, sizeof(int));
    if (e == cudaSuccess && cudaHostAlloc((void **)&ctx->err_host, sizeof(int), cudaHostAllocDefault) != cudaSuccess) {
        (void)cudaGetLastError();
        ctx->err_host = nullptr;  // the flag is then fetched with a blocking copy
    }
    if (ctx->err_host != nullptr) *ctx->err_host = 0;
    if (e == cudaSuccess) e = cudaMalloc(&ctx->gemm_counters, GEMM_TMA_MAX_TILE_COUNTERS * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(ctx->gemm_counters, 0, GEMM_TMA_MAX_TILE_COUNTERS * sizeof(int));
    if (e != cudaSuccess) {
        cudaStreamDestroy(ctx->own_stream);
        delete ctx;
        return cuda_fail(e, "cudaMalloc(error flag)");
    }
    const char *env = getenv("MARMOT_CUDA_FORCE_GEMV");
    if (env != nullptr && env[0] == '1') ctx->regime = MCU_REGIME_GEMV;
    env = getenv("MARMOT_CUDA_FORCE_GEMM");
    if (env != nullptr && env[0] == '1') ctx->regime = MCU_REGIME_GEMM;
    *out = ctx;
    return MCU_SUCCESS;
}

void mcu_context_destroy(mcu_context_t *ctx) {
    if (ctx == nullptr) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    Buffer *bufs[] = {&ctx->act_qs,   &ctx->act_d,      &ctx->act_bsums, &ctx->act_half, &ctx->act_rowscale, &ctx->x_stage, &ctx->out_stage,
                      &ctx->bias_stage, &ctx->moe_meta, &ctx->moe_hidden, &ctx->moe_gate, &ctx->moe_up, &ctx->moe_down, &ctx->gemm_partial, &ctx->attn_partial, &ctx->i8_partial, &ctx->i8_tickets, &ctx->pro_h, &ctx->attn_tickets, &ctx->rope_table};
    for (Buffer *b : bufs)
        if (b->ptr != nullptr) cudaFree(b->ptr);
    if (ctx->dev_err != nullptr) cudaFree(ctx->dev_err);
    if (ctx->err_host != nullptr) cudaFreeHost(ctx->err_host);
    if (ctx->pin_ring != nullptr) {
        for (int i = 0; i < PIN_SLOTS; ++i)
            if (ctx->pin_event[i] != nullptr) cudaEventDestroy(ctx->pin_event[i]);
        cudaFreeHost(ctx->pin_ring);
    }
    if (ctx->gemm_counters != nullptr) cudaFree(ctx->gemm_counters);
    if (ctx->own_stream != nullptr) cudaStreamDestroy(ctx->own_stream);
    delete ctx;
}

int mcu_context_set_stream(mcu_context_t *ctx, void *cuda_stream) {
    if (int rc = check_ctx(ctx)) return rc;
    std::lock_guard<std::mutex> lock(ctx->mu);
    MCU_CUDA(cudaStreamSynchronize(ctx->stream));
    ctx->stream = cuda_stream != nullptr ? (cudaStream_t)cuda_stream : ctx->own_stream;
    return MCU_SUCCESS;
}

void *mcu_context_get_stream(mcu_context_t *ctx) { return ctx != nullptr ? (void *)ctx->stream : nullptr; }

// ---- CUDA-graph capture of a sequence of calls on the context's stream ----
struct mcu_graph {
    cudaGraphExec_t exec = nullptr;
    mcu_context *ctx = nullptr;
};

int mcu_graph_capture_begin(mcu_context_t *ctx) {
    if (int rc = check_ctx(ctx)) return rc;
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (stream_is_capturing(ctx->stream)) return fail(MCU_ERROR_INVALID_OPERATION, "a capture is already in progress");
    if (ctx->stream == nullptr || ctx->stream == cudaStreamLegacy || ctx->stream == cudaStreamPerThread)
        return fail(MCU_ERROR_INVALID_OPERATION,
                    "the default stream cannot be captured: give the context a stream of its own (mcu_context_set_stream)");
    MCU_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    return MCU_SUCCESS;
}

int mcu_graph_capture_end(mcu_context_t *ctx, mcu_graph_t **out) {
    if (int rc = check_ctx(ctx)) return rc;
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (out != nullptr) *out = nullptr;
    if (!stream_is_capturing(ctx->stream)) return fail(MCU_ERROR_INVALID_OPERATION, "no capture in progress");
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    if (e != cudaSuccess || graph == nullptr) {
        (void)cudaGetLastError();
        return fail(MCU_ERROR_INVALID_OPERATION, "stream capture failed: %s", cudaGetErrorString(e));
    }
    if (out == nullptr) {  // the caller only wanted to end (discard) the capture
        cudaGraphDestroy(graph);
        return MCU_SUCCESS;
    }
    mcu_graph *g = new (std::nothrow) mcu_graph();
    if (g == nullptr) {
        cudaGraphDestroy(graph);
        return fail(MCU_ERROR_OUT_OF_MEMORY, "graph handle allocation failed");
    }
    e = cudaGraphInstantiate(&g->exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) {
        delete g;
        return cuda_fail(e, "cudaGraphInstantiate");
    }
    g->ctx = ctx;
    *out = g;
    return MCU_SUCCESS;
}

int mcu_graph_launch(mcu_graph_t *graph) {
    if (graph == nullptr || graph->exec == nullptr) return fail(MCU_ERROR_INVALID_ARGUMENT, "null graph");
    MCU_CUDA(cudaGraphLaunch(graph->exec, graph->ctx->stream));
    return MCU_SUCCESS;
}

void mcu_graph_destroy(mcu_graph_t *graph) {
    if (graph == nullptr) return;
    if (graph->exec != nullptr) cudaGraphExecDestroy(graph->exec);
    delete graph;
}

int mcu_context_set_regime(mcu_context_t *ctx, int regime) {
    if (ctx == nullptr) return fail(MCU_ERROR_DEVICE_NOT_AVAILABLE, "CUDA context is not initialised");
    if (regime < MCU_REGIME_AUTO || regime > MCU_REGIME_I8MMA) return fail(MCU_ERROR_INVALID_ARGUMENT, "bad regime");
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->regime = regime;
    return MCU_SUCCESS;
}

int mcu_synchronize(mcu_context_t *ctx) {
    if (int rc = check_ctx(ctx)) return rc;
    if (stream_is_capturing(ctx->stream)) return fail(MCU_ERROR_INVALID_OPERATION, "cannot synchronize during stream capture");
    return sync_and_check(ctx, ctx->stream);
}

int mcu_malloc(mcu_context_t *ctx, size_t bytes, void **out_dev) {
    if (int rc = check_ctx(ctx)) return rc;
    if (out_dev == nullptr) return fail(MCU_ERROR_INVALID_ARGUMENT, "out_dev is null");
    *out_dev = nullptr;
    MCU_CUDA(cudaMalloc(out_dev, bytes > 0 ? bytes : 1));
    return MCU_SUCCESS;
}

int mcu_free(mcu_context_t *ctx, void *dev) {
    if (int rc = check_ctx(ctx)) return rc;
    if (dev == nullptr) return MCU_SUCCESS;
    MCU_CUDA(cudaStreamSynchronize(ctx->stream));
    MCU_CUDA(cudaFree(dev));
    return MCU_SUCCESS;
}

// The next page-locked slot, free for reuse (its last copy has completed), or nullptr when the ring cannot be had.
static uint8_t *pin_slot(mcu_context *ctx, int *slot_out) {
    if (ctx->pin_ring == nullptr) {
        if (cudaHostAlloc((void **)&ctx->pin_ring, PIN_SLOTS * PIN_SLOT_BYTES, cudaHostAllocDefault) != cudaSuccess) {
            (void)cudaGetLastError();
            ctx->pin_ring = nullptr;
            return nullptr;
        }
        for (int i = 0; i < PIN_SLOTS; ++i)
            if (cudaEventCreateWithFlags(&ctx->pin_event[i], cudaEventDisableTiming) != cudaSuccess) {
                (void)cudaGetLastError();
                return nullptr;
            }
    }
    const int i = ctx->pin_next;
    if (ctx->pin_event[i] == nullptr) return nullptr;
    if (ctx->pin_used[i] && cudaEventSynchronize(ctx->pin_event[i]) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    ctx->pin_next = (i + 1) % PIN_SLOTS;
    *slot_out = i;
    return ctx->pin_ring + (size_t)i * PIN_SLOT_BYTES;
}

int mcu_memcpy_to_device(mcu_context_t *ctx, void *dst_dev, const void *src_host, size_t bytes) {
    if (int rc = check_ctx(ctx)) return rc;
    if (bytes == 0) return MCU_SUCCESS;
    if (dst_dev == nullptr || src_host == nullptr) return fail(MCU_ERROR_INVALID_ARGUMENT, "null pointer");
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (bytes <= PIN_SLOT_BYTES && !stream_is_capturing(ctx->stream)) {
        int slot = 0;
        if (uint8_t *pin = pin_slot(ctx, &slot)) {
            memcpy(pin, src_host, bytes);
            MCU_CUDA(cudaMemcpyAsync(dst_dev, pin, bytes, cudaMemcpyHostToDevice, ctx->stream));
            MCU_CUDA(cudaEventRecord(ctx->pin_event[slot], ctx->stream));
            ctx->pin_used[slot] = true;
            return MCU_SUCCESS;  // ordered before everything enqueued on the context's stream after it
        }
    }
    MCU_CUDA(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    MCU_CUDA(cudaStreamSynchronize(ctx->stream));
    return MCU_SUCCESS;
}

int mcu_memcpy_to_host(mcu_context_t *ctx, void *dst_host, const void *src_dev, size_t bytes) {
    if (int rc = check_ctx(ctx)) return rc;
    if (bytes == 0) return MCU_SUCCESS;
    if (dst_host == nullptr || src_dev == nullptr) return fail(MCU_ERROR_INVALID_ARGUMENT, "null pointer");
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (bytes <= PIN_SLOT_BYTES && !stream_is_capturing(ctx->stream)) {
        int slot = 0;
        if (uint8_t *pin = pin_slot(ctx, &slot)) {
            MCU_CUDA(cudaMemcpyAsync(pin, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
            MCU_CUDA(cudaStreamSynchronize(ctx->stream));
            ctx->pin_used[slot] = false;
            memcpy(dst_host, pin, bytes);
            return MCU_SUCCESS;
        }
    }
    MCU_CUDA(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    MCU_CUDA(cudaStreamSynchronize(ctx->stream));
    return MCU_SUCCESS;
}

size_t mcu_row_bytes(int kind, size_t K) {
    if (!kind_supported(kind)) return 0;
    const size_t bv = (size_t)block_values(kind);
    return (K + bv - 1) / bv * (size_t)block_bytes(kind);
}

int mcu_dequantize(mcu_context_t *ctx, int kind, const void *blocks_dev, size_t n_values, float *out_dev) {
    if (int rc = check_ctx(ctx)) return rc;
    if (!kind_supported(kind)) return fail(MCU_ERROR_NOT_IMPLEMENTED, "quant kind %d has no CUDA kernel", kind);
    if (n_values == 0) return MCU_SUCCESS;
    if (blocks_dev == nullptr || out_dev == nullptr) return fail(MCU_ERROR_INVALID_ARGUMENT, "null tensor data");
    if (kind == MCU_KIND_Q4_K && ((uintptr_t)blocks_dev & 3)) return fail(MCU_ERROR_INVALID_ARGUMENT, "Q4_K blocks must be 4-byte aligned");
    if ((uintptr_t)blocks_dev & 1) return fail(MCU_ERROR_INVALID_ARGUMENT, "blocks must be 2-byte aligned");
    MCU_CUDA(launch_dequantize(kind, blocks_dev, n_values, out_dev, ctx->stream));
    count_launches(1);
    return MCU_SUCCESS;
}

static int validate_linear(int kind, const void *x, const void *w, const void *out, size_t T, size_t K, size_t F,
                           size_t ldx, size_t ldo) {
    if (!kind_supported(kind)) return fail(MCU_ERROR_NOT_IMPLEMENTED, "quant kind %d has no CUDA kernel", kind);
    if (x == nullptr || w == nullptr || out == nullptr) return fail(MCU_ERROR_INVALID_ARGUMENT, "Tensor argument must not be null");
    if (K == 0) return fail(MCU_ERROR_DIMENSION_MISMATCH, "K must be positive");
    if (ldx < K || ldo < F) return fail(MCU_ERROR_DIMENSION_MISMATCH, "row stride smaller than the row");
    if (T > (size_t)1 << 30 || F > (size_t)1 << 30 || K > (size_t)1 << 30)
        return fail(MCU_ERROR_INVALID_ARGUMENT, "dimension too large");
    // the launchers carry row strides as int
    if (ldx > (size_t)INT_MAX || ldo > (size_t)INT_MAX) return fail(MCU_ERROR_INVALID_ARGUMENT, "row stride too large");
    const uintptr_t align = kind == MCU_KIND_Q4_K ? 15 : 1;
    if ((uintptr_t)w & align)
        return fail(MCU_ERROR_INVALID_ARGUMENT, "weight blocks must be %d-byte aligned", (int)align + 1);
    return MCU_SUCCESS;
}

// Quantize the activations into the context workspace.
static int pack_activations(mcu_context *ctx, int kind, const float *x, size_t ldx, size_t T, size_t K, bool want_half,
                            int k_order, ActBuffers &ab) {
    const size_t bv = (size_t)block_values(kind);
    const size_t nb = (K + bv - 1) / bv, kp = nb * bv;
    if (int rc = ensure(ctx, ctx->act_qs, T * kp)) return rc;
    if (int rc = ensure(ctx, ctx->act_d, T * nb * sizeof(float))) return rc;
    if (kind != MCU_KIND_Q8_0)
        if (int rc = ensure(ctx, ctx->act_bsums, T * nb * 16 * sizeof(int16_t))) return rc;
    if (want_half) {
        if (int rc = ensure(ctx, ctx->act_half, T * kp * sizeof(__half))) return rc;
        if (int rc = ensure(ctx, ctx->act_rowscale, T * sizeof(float))) return rc;
    }
    ab.qs = (int8_t *)ctx->act_qs.ptr;
    ab.d = (float *)ctx->act_d.ptr;
    ab.bsums = (int16_t *)ctx->act_bsums.ptr;
    MCU_CUDA(launch_quantize_act(kind, x, (int)ldx, (int)T, (int)K, ab, nullptr, ctx->stream));
    count_launches(1);
    if (want_half) {
        MCU_CUDA(launch_half_acts(kind, ab, (int)T, (int)K, k_order, (__half *)ctx->act_half.ptr,
                                  (float *)ctx->act_rowscale.ptr, ctx->stream));
        count_launches(1);
    }
    return MCU_SUCCESS;
}

// The device-side address of a page-locked, mapped host allocation (cudaHostAlloc / cudaHostRegister), or nullptr for
// pageable memory.
static void *mapped_host_pointer(const void *host) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, host) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    return attr.type == cudaMemoryTypeHost ? attr.devicePointer : nullptr;
}

// What the last staging launch of a multi-matmul call left in the context's fp16 activation buffer: a later matmul
// of the same call that wants the same block format class and K order reuses it.
struct Staged {
    bool valid = false, kq = false;
    int k_order = -1;
};

// The tensor-core matmuls (gemm_tc_supported shapes): stage the activations as fp16 (through `src` when the caller
// folds a gather, GLU or add + RMSNorm into the staging; needs the one-kernel staging), then the GEMM that suits the
// weights.  ctx->mu is held by the caller.
static int gemm_locked(mcu_context *ctx, int kind, const float *x, size_t ldx, const void *w, const void *w2, size_t T, size_t K,
                       size_t F, const float *bias, float *out, float *out2, size_t ldo, const ActSource *src, Staged *st) {
    const bool tma = gemm_tma_supported(kind, w, w2, (int)T, (int)K, (int)F);
    const bool warp_mma = gemm_warp_supported(kind, w, w2, (int)T, (int)K, (int)F);
    const int k_order = warp_mma ? ACT_ORDER_FRAG16 : tma ? ACT_ORDER_QUAD : ACT_ORDER_NATURAL;
    const bool kq = kind != MCU_KIND_Q8_0;
    const size_t bv = (size_t)block_values(kind);
    const size_t kp = (K + bv - 1) / bv * bv;
    if (st != nullptr && st->valid && st->kq == kq && st->k_order == k_order) {
        // staged by an earlier matmul of this call
    } else if (act_half_fused_smem(kind, (int)K) <= 48 * 1024) {
        if (int rc = ensure(ctx, ctx->act_half, T * kp * sizeof(__half))) return rc;
        if (int rc = ensure(ctx, ctx->act_rowscale, T * sizeof(float))) return rc;
        MCU_CUDA(launch_act_half_fused_from(kind, x, (int)ldx, src != nullptr ? *src : ActSource{}, (int)T, (int)K, k_order,
                                            (__half *)ctx->act_half.ptr, (float *)ctx->act_rowscale.ptr, ctx->stream));
        count_launches(1);
        if (st != nullptr) {
            st->valid = true;
            st->kq = kq;
            st->k_order = k_order;
        }
    } else {
        if (src != nullptr) return fail(MCU_ERROR_NOT_IMPLEMENTED, "rows too long for the one-kernel activation staging");
        ActBuffers ab;
        if (int rc = pack_activations(ctx, kind, x, ldx, T, K, true, k_order, ab)) return rc;
        if (st != nullptr) st->valid = false;
    }
    int launches = 0;
    if (warp_mma) {
        if (int rc = ensure(ctx, ctx->gemm_partial, gemm_warp_workspace_bytes(kind, (int)T, (int)K, (int)F, w2 != nullptr)))
            return rc;
        MCU_CUDA(launch_gemm_warp(kind, w, w2, (const __half *)ctx->act_half.ptr, (const float *)ctx->act_rowscale.ptr,
                                  (int)kp, (int)T, (int)K, (int)F, bias, out, out2, (int)ldo, (float *)ctx->gemm_partial.ptr,
                                  ctx->gemm_counters, ctx->dev_err, ctx->stream));
        launches = 1;
    } else if (tma) {
        if (int rc = ensure(ctx, ctx->gemm_partial, gemm_tma_workspace_bytes(kind, (int)T, (int)K, (int)F))) return rc;
        MCU_CUDA(launch_gemm_tma(kind, w, w2, (const __half *)ctx->act_half.ptr, (const float *)ctx->act_rowscale.ptr,
                                 (int)kp, (int)T, (int)K, (int)F, bias, out, out2, (int)ldo, (float *)ctx->gemm_partial.ptr,
                                 ctx->gemm_counters, ctx->dev_err, ctx->stream, &launches));
    } else {
        MCU_CUDA(launch_gemm_tc(kind, w, w2, (const __half *)ctx->act_half.ptr, (const float *)ctx->act_rowscale.ptr, (int)kp,
                                (int)T, (int)K, (int)F, bias, out, out2, (int)ldo, ctx->dev_err, ctx->stream, &launches));
    }
    count_launches(launches);
    return MCU_SUCCESS;
}

// Core of mcu_linear / mcu_linear_dual on device pointers; ctx->mu is held by the caller.
static int linear_locked(mcu_context *ctx, int kind, const float *x, size_t ldx, const void *w, const void *w2, size_t T,
                         size_t K, size_t F, const float *bias, float *out, float *out2, size_t ldo) {
    if (T == 0 || F == 0) return MCU_SUCCESS;
    const bool gemm = ctx->regime == MCU_REGIME_GEMM ||
        ((ctx->regime == MCU_REGIME_AUTO || ctx->regime == MCU_REGIME_I8MMA) && T > (size_t)GEMV_MAX_T);
    ActBuffers ab;
    // A handful of tokens: exact integer dots on mma.sync s8 (Q4_K, Q6_K).  Measured against the neighbours on
    // K = 4096 (F = 4096 / 14336, microseconds per call): 8 tokens 12.1 / 19.4 here, 15.3 / 33.6 on the dp4a kernel
    // (which re-reads the activations from shared memory per token); 16 tokens 13.4 / 22.5 here, 12.4 / 25.8 on the
    // tcgen05 kernel; below five tokens the dp4a kernel's single launch wins, beyond sixteen the integer MMA rate of
    // this part (about 30 cycles per m16n8k32 and SM sub-partition) does not keep up with the fp16 paths.
    static const bool no_i8 = getenv("MARMOT_CUDA_NO_I8MMA") != nullptr;  // diagnostic switch
    const size_t w_total = F * mcu_row_bytes(kind, K) * (w2 != nullptr ? 2 : 1);
    const bool i8_pays = ctx->regime == MCU_REGIME_I8MMA
        ? (T >= 2 && T <= 64)
        : (!no_i8 && ctx->regime == MCU_REGIME_AUTO && T >= 5 && T <= 16 && (T <= 12 || w_total >= ((size_t)24 << 20)));
    if (i8_pays &&
        gemm_i8_supported(kind, w, w2, (int)T, (int)K, (int)F) && (w2 == nullptr || bias == nullptr)) {
        size_t qs_b, dT_b, part_b, tick_b;
        gemm_i8_workspace_bytes((int)T, (int)K, (int)F, w2 != nullptr, &qs_b, &dT_b, &part_b, &tick_b);
        if (int rc = ensure(ctx, ctx->act_qs, qs_b)) return rc;
        if (int rc = ensure(ctx, ctx->act_d, dT_b)) return rc;
        if (int rc = ensure(ctx, ctx->i8_partial, part_b)) return rc;
        if (tick_b > ctx->i8_tickets.cap) {  // a fresh ticket area starts at zero; the kernel keeps it so
            if (int rc = ensure(ctx, ctx->i8_tickets, tick_b)) return rc;
            MCU_CUDA(cudaMemsetAsync(ctx->i8_tickets.ptr, 0, ctx->i8_tickets.cap, ctx->stream));
        }
        MCU_CUDA(launch_gemm_i8(kind, w, w2, x, (int)ldx, (int)T, (int)K, (int)F, bias, out, out2, (int)ldo,
                                (int8_t *)ctx->act_qs.ptr, (float *)ctx->act_d.ptr, (float *)ctx->i8_partial.ptr,
                                (int *)ctx->i8_tickets.ptr, ctx->dev_err, ctx->stream));
        count_launches(2);
        return MCU_SUCCESS;
    }
    if (gemm) {
        if (gemm_tc_supported(kind, (int)T, (int)K, (int)F))
            return gemm_locked(ctx, kind, x, ldx, w, w2, T, K, F, bias, out, out2, ldo, nullptr, nullptr);
        if (ctx->regime == MCU_REGIME_GEMM)
            return fail(MCU_ERROR_NOT_IMPLEMENTED, "tensor-core GEMM does not cover kind %d T=%zu K=%zu F=%zu", kind, T, K, F);
    }
    if (ctx->regime != MCU_REGIME_GEMV_PLAIN && T <= (size_t)GEMV_MAX_T &&
        gemv_stream_supported(kind, w, w2, (int)T, (int)K, (int)F)) {
        MCU_CUDA(launch_gemv_stream(kind, w, w2, x, (int)ldx, (int)T, (int)K, (int)F, bias, out, out2, (int)ldo,
                                    ctx->dev_err, ctx->stream));
        count_launches(1);
        return MCU_SUCCESS;
    }
    if (int rc = pack_activations(ctx, kind, x, ldx, T, K, false, ACT_ORDER_NATURAL, ab)) return rc;
    const size_t bv = (size_t)block_values(kind);
    const size_t nb = (K + bv - 1) / bv, kp = nb * bv;
    for (size_t t0 = 0; t0 < T; t0 += GEMV_MAX_T) {
        const size_t tc = T - t0 < (size_t)GEMV_MAX_T ? T - t0 : (size_t)GEMV_MAX_T;
        ActBuffers sub = ab;
        sub.qs += t0 * kp;
        sub.d += t0 * nb;
        if (sub.bsums != nullptr) sub.bsums += t0 * nb * 16;
        MCU_CUDA(launch_gemv(kind, w, w2, sub, (int)tc, (int)K, (int)F, bias, out + t0 * ldo,
                             out2 != nullptr ? out2 + t0 * ldo : nullptr, (int)ldo, ctx->stream));
        count_launches(1);
    }
    return MCU_SUCCESS;
}

extern "C++" {
namespace mcu {
int linear_fused_allreduce(mcu_context *ctx, int kind, const float *x, size_t ldx, const void *w, size_t T, size_t K,
                           size_t F, float *out, const PeerFuse &fuse) {
    if (int rc = check_ctx(ctx)) return rc;
    if (int rc = validate_linear(kind, x, w, out, T, K, F, ldx, F)) return rc;
    if (ctx->regime == MCU_REGIME_GEMV || ctx->regime == MCU_REGIME_GEMV_PLAIN || !gemm_tma_can_fuse(kind, (int)T, (int)F) ||
        !gemm_tma_supported(kind, w, nullptr, (int)T, (int)K, (int)F) || act_half_fused_smem(kind, (int)K) > 48 * 1024)
        return fail(MCU_ERROR_NOT_IMPLEMENTED, "shape or weights do not suit the fused matmul + all-reduce");
    std::lock_guard<std::mutex> lock(ctx->mu);
    const size_t bv = (size_t)block_values(kind);
    const size_t kp = (K + bv - 1) / bv * bv;
    if (int rc = ensure(ctx, ctx->act_half, T * kp * sizeof(__half))) return rc;
    if (int rc = ensure(ctx, ctx->act_rowscale, T * sizeof(float))) return rc;
    if (int rc = ensure(ctx, ctx->gemm_partial, gemm_tma_workspace_bytes(kind, (int)T, (int)K, (int)F))) return rc;
    MCU_CUDA(launch_act_half_fused(kind, x, (int)ldx, (int)T, (int)K, ACT_ORDER_QUAD, (__half *)ctx->act_half.ptr,
                                   (float *)ctx->act_rowscale.ptr, ctx->stream));
    int launches = 0;
    MCU_CUDA(launch_gemm_tma(kind, w, nullptr, (const __half *)ctx->act_half.ptr, (const float *)ctx->act_rowscale.ptr,
                             (int)kp, (int)T, (int)K, (int)F, nullptr, out, nullptr, (int)F, (float *)ctx->gemm_partial.ptr,
                             ctx->gemm_counters, ctx->dev_err, ctx->stream, &launches, &fuse));
    count_launches(1 + launches);
    return MCU_SUCCESS;
}
}  // namespace mcu
}  // extern "C++"

int mcu_quantize_activations(mcu_context_t *ctx, int weight_kind, const float *x_dev, size_t ldx, size_t T, size_t K,
                             int8_t *qs_dev, float *d_dev, int16_t *bsums_dev) {
    if (int rc = check_ctx(ctx)) return rc;
    if (!kind_supported(weight_kind)) return fail(MCU_ERROR_NOT_IMPLEMENTED, "quant kind %d has no CUDA kernel", weight_kind);
    if (T == 0) return MCU_SUCCESS;
    if (x_dev == nullptr || qs_dev == nullptr || d_dev == nullptr || (weight_kind != MCU_KIND_Q8_0 && bsums_dev == nullptr))
        return fail(MCU_ERROR_INVALID_ARGUMENT, "null tensor data");
    if (K == 0 || ldx < K) return fail(MCU_ERROR_DIMENSION_MISMATCH, "bad K / ldx");
    if (ldx > (size_t)INT_MAX || T > (size_t)1 << 30 || K > (size_t)1 << 30)
        return fail(MCU_ERROR_INVALID_ARGUMENT, "dimension or row stride too large");
    ActBuffers ab{qs_dev, d_dev, bsums_dev};
    MCU_CUDA(launch_quantize_act(weight_kind, x_dev, (int)ldx, (int)T, (int)K, ab, nullptr, ctx->stream));
    count_launches(1);
    return MCU_SUCCESS;
}

static float half_bits_to_float_host(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {  // subnormal: normalise
            int e = -1;
            uint32_t m = man;
            do {
                ++e;
                m <<= 1;
            } while ((m & 0x400u) == 0);
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, sizeof(f));
    return f;
}

int mcu_vec_dot_host(mcu_context_t *ctx, int weight_kind, const void *weights_host, const void *activations_host,
                     size_t num_blocks, float *result_host) {
    if (int rc = check_ctx(ctx)) return rc;
    if (result_host == nullptr) return fail(MCU_ERROR_INVALID_ARGUMENT, "vec_dot: null result");
    if (!kind_supported(weight_kind)) return fail(MCU_ERROR_NOT_IMPLEMENTED, "quant kind %d has no CUDA kernel", weight_kind);
    if (weights_host == nullptr || activations_host == nullptr || num_blocks == 0) {
        *result_host = 0.0f;  // as cpu_vec_dot
        return MCU_SUCCESS;
    }
    if (stream_is_capturing(ctx->stream))
        return fail(MCU_ERROR_INVALID_OPERATION, "mcu_vec_dot_host waits for its result: it cannot be captured");
    const bool kq = weight_kind != MCU_KIND_Q8_0;
    const size_t bv = (size_t)block_values(weight_kind), kp = num_blocks * bv;
    if (kp > ((size_t)1 << 24)) return fail(MCU_ERROR_INVALID_ARGUMENT, "vec_dot: row too long");
    // The activation blocks as the structure of arrays the decode kernels read (no arithmetic: bytes are moved).
    std::vector<int8_t> qs(kp);
    std::vector<float> d(num_blocks);
    std::vector<int16_t> bsums(kq ? num_blocks * 16 : 0);
    const uint8_t *a = (const uint8_t *)activations_host;
    for (size_t b = 0; b < num_blocks; ++b) {
        if (kq) {  // {f32 d, int8 qs[256], int16 bsums[16]}
            const uint8_t *blk = a + b * 292;
            memcpy(&d[b], blk, 4);
            for (int v = 0; v < 256; ++v) qs[b * 256 + ((v >> 5) & 1) * 128 + (v >> 6) * 32 + (v & 31)] = (int8_t)blk[4 + v];
            memcpy(&bsums[b * 16], blk + 260, 32);
        } else {  // {f16 d, int8 qs[32]}
            const uint8_t *blk = a + b * 34;
            uint16_t hb;
            memcpy(&hb, blk, 2);
            d[b] = half_bits_to_float_host(hb);
            memcpy(&qs[b * 32], blk + 2, 32);
        }
    }
    std::lock_guard<std::mutex> lock(ctx->mu);
    const size_t wbytes = num_blocks * (size_t)block_bytes(weight_kind);
    if (int rc = ensure(ctx, ctx->act_qs, kp)) return rc;
    if (int rc = ensure(ctx, ctx->act_d, num_blocks * sizeof(float))) return rc;
    if (int rc = ensure(ctx, ctx->act_bsums, (kq ? num_blocks * 16 : 1) * sizeof(int16_t))) return rc;
    if (int rc = ensure(ctx, ctx->x_stage, wbytes)) return rc;
    if (int rc = ensure(ctx, ctx->out_stage, sizeof(float))) return rc;
    cudaStream_t s = ctx->stream;
    MCU_CUDA(cudaMemcpyAsync(ctx->act_qs.ptr, qs.data(), kp, cudaMemcpyHostToDevice, s));
    MCU_CUDA(cudaMemcpyAsync(ctx->act_d.ptr, d.data(), num_blocks * sizeof(float), cudaMemcpyHostToDevice, s));
    if (kq) MCU_CUDA(cudaMemcpyAsync(ctx->act_bsums.ptr, bsums.data(), num_blocks * 32, cudaMemcpyHostToDevice, s));
    MCU_CUDA(cudaMemcpyAsync(ctx->x_stage.ptr, weights_host, wbytes, cudaMemcpyHostToDevice, s));
    ActBuffers ab{(int8_t *)ctx->act_qs.ptr, (float *)ctx->act_d.ptr, (int16_t *)ctx->act_bsums.ptr};
    MCU_CUDA(launch_gemv(weight_kind, ctx->x_stage.ptr, nullptr, ab, 1, (int)kp, 1, nullptr, (float *)ctx->out_stage.ptr,
                         nullptr, 1, s));
    count_launches(1);
    MCU_CUDA(cudaMemcpyAsync(result_host, ctx->out_stage.ptr, sizeof(float), cudaMemcpyDeviceToHost, s));
    return sync_and_check(ctx, s);  // the host vectors above must outlive the copies
}

int mcu_linear(mcu_context_t *ctx, int kind, const float *x_dev, size_t ldx, const void *w_dev, size_t T, size_t K,
               size_t F, const float *bias_dev, float *out_dev, size_t ldo) {
    if (int rc = check_ctx(ctx)) return rc;
    if (!kind_supported(kind)) return fail(MCU_ERROR_NOT_IMPLEMENTED, "quant kind %d has no CUDA kernel", kind);
    if (T == 0 || F == 0) return MCU_SUCCESS;
    if (int rc = validate_linear(kind, x_dev, w_dev, out_dev, T, K, F, ldx, ldo)) return rc;
    std::lock_guard<std::mutex> lock(ctx->mu);
    return linear_locked(ctx, kind, x_dev, ldx, w_dev, nullptr, T, K, F, bias_dev, out_dev, nullptr, ldo);
}

int mcu_linear_f16(mcu_context_t *ctx, int kind, const uint16_t *x_f16_dev, size_t ldx, const void *w_dev, size_t T, size_t K,
                   size_t F, const float *bias_dev, void *out_dev, size_t ldo, int out_dtype) {
    if (int rc = check_ctx(ctx)) return rc;
    if (!kind_supported(kind)) return fail(MCU_ERROR_NOT_IMPLEMENTED, "quant kind %d has no CUDA kernel", kind);
    if (T == 0 || F == 0) return MCU_SUCCESS;
    if (int rc = validate_linear(kind, x_f16_dev, w_dev, out_dev, T, K, F, ldx, ldo)) return rc;
    if (out_dtype != MCU_OUT_F32 && out_dtype != MCU_OUT_F16) return fail(MCU_ERROR_UNSUPPORTED_DTYPE, "output must be f32 or f16");
    if (out_dtype == MCU_OUT_F16 && bias_dev != nullptr)
        return fail(MCU_ERROR_NOT_IMPLEMENTED, "bias with an f16 output is not offered");
    if ((uintptr_t)x_f16_dev & 1) return fail(MCU_ERROR_INVALID_ARGUMENT, "f16 activations must be 2-byte aligned");
    std::lock_guard<std::mutex> lock(ctx->mu);
    MCU_CUDA(launch_linear_f16(kind, w_dev, (const __half *)x_f16_dev, ldx, (int)T, (int)K, (int)F, bias_dev,
                               out_dtype == MCU_OUT_F32 ? (float *)out_dev : nullptr,
                               out_dtype == MCU_OUT_F16 ? (__half *)out_dev : nullptr, ldo, ctx->stream));
    count_launches(1);
    return MCU_SUCCESS;
}

int mcu_linear_dual(mcu_context_t *ctx, int kind, const float *x_dev, size_t ldx, const void *w_a_dev,
                    const void *w_b_dev, size_t T, size_t K, size_t F, float *out_a_dev, float *out_b_dev, size_t ldo) {
    if (int rc = check_ctx(ctx)) return rc;
    if (w_b_dev == nullptr || out_b_dev == nullptr) return fail(MCU_ERROR_INVALID_ARGUMENT, "Tensor argument must not be null");
    if (int rc = validate_linear(kind, x_dev, w_a_dev, out_a_dev, T, K, F, ldx, ldo)) return rc;
    if (int rc = validate_linear(kind, x_dev, w_b_dev, out_b_dev, T, K, F, ldx, ldo)) return rc;
    std::lock_guard<std::mutex> lock(ctx->mu);
    return linear_locked(ctx, kind, x_dev, ldx, w_a_dev, w_b_dev, T, K, F, nullptr, out_a_dev, out_b_dev, ldo);
}

int mcu_linear_multi(mcu_context_t *ctx, const float *x_dev, size_t ldx, size_t T, size_t K, const mcu_prologue_t *prologue,
                     const mcu_linear_job_t *jobs, size_t n_jobs) {
    if (int rc = check_ctx(ctx)) return rc;
    if (jobs == nullptr || n_jobs == 0 || n_jobs > (size_t)MCU_LINEAR_MAX_JOBS)
        return fail(MCU_ERROR_INVALID_ARGUMENT, "between 1 and %d jobs", MCU_LINEAR_MAX_JOBS);
    static_assert(MCU_LINEAR_MAX_JOBS == GEMV_MAX_JOBS, "public and kernel job limits differ");
    if (T == 0) return MCU_SUCCESS;
    mcu_prologue_t none = {};
    const mcu_prologue_t &pr = prologue != nullptr ? *prologue : none;
    if (pr.op != MCU_PROLOGUE_NONE && pr.op != MCU_PROLOGUE_ADD_RMSNORM && pr.op != MCU_PROLOGUE_SWIGLU)
        return fail(MCU_ERROR_INVALID_ARGUMENT, "unknown prologue %d", pr.op);
    if (pr.op == MCU_PROLOGUE_SWIGLU && pr.aux_dev == nullptr) return fail(MCU_ERROR_INVALID_ARGUMENT, "SwiGLU needs the up projection");
    if (pr.op != MCU_PROLOGUE_NONE) {
        if ((pr.aux_dev != nullptr && pr.ld_aux < K) || (pr.x_out_dev != nullptr && pr.ld_x_out < K))
            return fail(MCU_ERROR_DIMENSION_MISMATCH, "row stride smaller than the row");
        if (pr.ld_aux > (size_t)INT_MAX || pr.ld_x_out > (size_t)INT_MAX) return fail(MCU_ERROR_INVALID_ARGUMENT, "row stride too large");
        if (pr.op == MCU_PROLOGUE_ADD_RMSNORM && pr.x_out_dev != nullptr &&
            (pr.x_out_dev == x_dev || pr.x_out_dev == pr.aux_dev))
            return fail(MCU_ERROR_INVALID_ARGUMENT, "x_out must not overlap the inputs");
    }
    GemvJobSpec specs[GEMV_MAX_JOBS];
    for (size_t j = 0; j < n_jobs; ++j) {
        const mcu_linear_job_t &jb = jobs[j];
        if (jb.F == 0) return fail(MCU_ERROR_DIMENSION_MISMATCH, "F must be positive");
        if (int rc = validate_linear(jb.kind, x_dev, jb.w_dev, jb.out_dev, T, K, jb.F, ldx, jb.ldo)) return rc;
        specs[j] = GemvJobSpec{jb.kind, jb.w_dev, (int)jb.F, jb.bias_dev, jb.out_dev, (int)jb.ldo};
    }
    GemvPrologue gp;
    gp.op = pr.op;
    if (pr.op != MCU_PROLOGUE_NONE) {
        gp.aux = pr.aux_dev;
        gp.ld_aux = (int)pr.ld_aux;
        gp.norm_w = pr.norm_weight_dev;
        gp.eps = pr.eps;
        gp.w_off = pr.weight_offset;
        gp.x_out = pr.op == MCU_PROLOGUE_ADD_RMSNORM ? pr.x_out_dev : nullptr;
        gp.ld_x_out = (int)pr.ld_x_out;
    }
    float *h = nullptr;
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        const bool contiguous = ldx == K && (pr.aux_dev == nullptr || pr.ld_aux == K) && (gp.x_out == nullptr || pr.ld_x_out == K);
        // Five to eight tokens over large K-quant matrices: the dp4a kernel is bound by its integer dots there (8 tokens,
        // 2 x 14336 x 4096 Q4_K: 73 us with the prologue folded in, 29 us on the integer-MMA kernel), so the prologue runs
        // as a kernel of its own and the matmuls take mcu_linear's regimes.  Small matrices keep the one-launch form.
        size_t w_total = 0;
        bool k_quants = true;
        for (size_t j = 0; j < n_jobs; ++j) {
            w_total += jobs[j].F * mcu_row_bytes(jobs[j].kind, K);
            k_quants = k_quants && (jobs[j].kind == KIND_Q4_K || jobs[j].kind == KIND_Q6_K);
        }
        static const bool no_i8 = getenv("MARMOT_CUDA_NO_I8MMA") != nullptr;  // diagnostic switch, as in linear_locked
        const bool integer_mma_pays = ctx->regime == MCU_REGIME_AUTO && !no_i8 && T >= 5 && k_quants &&
            w_total >= ((size_t)24 << 20) && (pr.op == MCU_PROLOGUE_NONE || contiguous);
        if (!integer_mma_pays && (ctx->regime == MCU_REGIME_AUTO || ctx->regime == MCU_REGIME_GEMV) && T <= (size_t)GEMV_MAX_T &&
            gemv_stream_jobs_supported(specs, (int)n_jobs, (int)T, (int)K, gp)) {
            MCU_CUDA(launch_gemv_stream_jobs(specs, (int)n_jobs, x_dev, (int)ldx, (int)T, (int)K, gp, ctx->dev_err, ctx->stream));
            count_launches(1);
            return MCU_SUCCESS;
        }
        // More than eight tokens on the tensor cores: one staging launch (the prologue folded into it) feeds every
        // matmul that wants the same staging; weights of the other block format class get a second one.
        bool tensor = (ctx->regime == MCU_REGIME_AUTO || ctx->regime == MCU_REGIME_GEMM) && T > 16 &&
            (pr.op == MCU_PROLOGUE_NONE || contiguous);
        for (size_t j = 0; j < n_jobs && tensor; ++j)
            tensor = gemm_tc_supported(jobs[j].kind, (int)T, (int)K, (int)jobs[j].F) &&
                act_half_fused_smem(jobs[j].kind, (int)K) <= 48 * 1024;
        if (tensor) {
            ActSource src;
            if (pr.op == MCU_PROLOGUE_ADD_RMSNORM) {
                src.norm = 1;
                src.add = pr.aux_dev;
                src.norm_w = pr.norm_weight_dev;
                src.eps = pr.eps;
                src.w_off = pr.weight_offset;
                src.x_out = gp.x_out;
            } else if (pr.op == MCU_PROLOGUE_SWIGLU) {
                src.x2 = pr.aux_dev;
                src.glu = 1;
            }
            Staged st;
            for (size_t j = 0; j < n_jobs;) {
                const mcu_linear_job_t &a = jobs[j];
                const bool pair = j + 1 < n_jobs && jobs[j + 1].kind == a.kind && jobs[j + 1].F == a.F && jobs[j + 1].ldo == a.ldo &&
                    a.bias_dev == nullptr && jobs[j + 1].bias_dev == nullptr;
                // x_out is written by the first staging launch only (a second one would add aux twice if x_out is x)
                ActSource use = src;
                if (st.valid || j > 0) {
                    if (use.norm && use.x_out != nullptr) {
                        use.add = nullptr;  // the sum is already in x_out
                        use.x_out = nullptr;
                    }
                }
                const float *from = (j > 0 && src.norm && src.x_out != nullptr) ? src.x_out : x_dev;
                if (int rc = gemm_locked(ctx, a.kind, from, ldx, a.w_dev, pair ? jobs[j + 1].w_dev : nullptr, T, K, a.F, a.bias_dev,
                                         a.out_dev, pair ? jobs[j + 1].out_dev : nullptr, a.ldo, &use, &st))
                    return rc;
                j += pair ? 2 : 1;
            }
            return MCU_SUCCESS;
        }
        if (pr.op != MCU_PROLOGUE_NONE) {
            if (!contiguous)
                return fail(MCU_ERROR_NOT_IMPLEMENTED, "the stand-alone prologue kernels need contiguous rows");
            if (int rc = ensure(ctx, ctx->pro_h, T * K * sizeof(float))) return rc;
            h = (float *)ctx->pro_h.ptr;
        }
    }
    // The general form: the prologue as its own kernel into the context's scratch, then the matmuls (pairs of equal
    // shape share their activation packing).
    const float *act = x_dev;
    size_t ld_act = ldx;
    if (pr.op == MCU_PROLOGUE_ADD_RMSNORM) {
        if (pr.aux_dev != nullptr && gp.x_out != nullptr) {
            if (int rc = mcu_add_rmsnorm(ctx, x_dev, pr.aux_dev, pr.norm_weight_dev, T, K, pr.eps, pr.weight_offset, gp.x_out, h))
                return rc;
        } else {
            if (int rc = mcu_rmsnorm(ctx, x_dev, pr.aux_dev, pr.norm_weight_dev, T, K, pr.eps, pr.weight_offset, h)) return rc;
            if (gp.x_out != nullptr)  // no aux: x' = x
                MCU_CUDA(cudaMemcpyAsync(gp.x_out, x_dev, T * K * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
        }
        act = h, ld_act = K;
    } else if (pr.op == MCU_PROLOGUE_SWIGLU) {
        if (int rc = mcu_swiglu(ctx, x_dev, pr.aux_dev, T * K, h)) return rc;
        act = h, ld_act = K;
    }
    std::lock_guard<std::mutex> lock(ctx->mu);
    for (size_t j = 0; j < n_jobs;) {
        const mcu_linear_job_t &a = jobs[j];
        const bool pair = j + 1 < n_jobs && jobs[j + 1].kind == a.kind && jobs[j + 1].F == a.F && jobs[j + 1].ldo == a.ldo &&
            a.bias_dev == nullptr && jobs[j + 1].bias_dev == nullptr;
        if (int rc = linear_locked(ctx, a.kind, act, ld_act, a.w_dev, pair ? jobs[j + 1].w_dev : nullptr, T, K, a.F, a.bias_dev,
                                   a.out_dev, pair ? jobs[j + 1].out_dev : nullptr, a.ldo))
            return rc;
        j += pair ? 2 : 1;
    }
    return MCU_SUCCESS;
}

int mcu_linear_host(mcu_context_t *ctx, int kind, const float *x_host, size_t ldx, const void *w_dev, size_t T,
                    size_t K, size_t F, const float *bias_host, float *out_host, size_t ldo) {
    if (int rc = check_ctx(ctx)) return rc;
    if (int rc = validate_linear(kind, x_host, w_dev, out_host, T, K, F, ldx, ldo)) return rc;
    if (T == 0 || F == 0) return MCU_SUCCESS;
    if (stream_is_capturing(ctx->stream))
        return fail(MCU_ERROR_INVALID_OPERATION, "mcu_linear_host waits for its result: it cannot be captured");
    std::lock_guard<std::mutex> lock(ctx->mu);
    // A page-locked result buffer that is mapped into the device's address space is written in place by the decode
    // kernels (a few KB of posted writes over PCIe), which saves the copy-back launch: 226 against 198 GB/s end to end
    // on the 4096 x 4096 GEMV.  The activations still go through a staging copy: every CTA reads all of them, and reads
    // of host memory are not cached (60 GB/s when tried).  Larger results are better moved by the copy engines.
    static const bool no_zero_copy = getenv("MARMOT_CUDA_HOST_NO_ZERO_COPY") != nullptr;  // diagnostic switch
    float *out_map =
        (T <= (size_t)GEMV_MAX_T && ldo == F && !no_zero_copy) ? (float *)mapped_host_pointer(out_host) : nullptr;
    float *xd = nullptr, *od = nullptr, *bd = nullptr;
    if (int rc = ensure(ctx, ctx->x_stage, T * K * sizeof(float))) return rc;
    xd = (float *)ctx->x_stage.ptr;
    if (ldx == K)
        MCU_CUDA(cudaMemcpyAsync(xd, x_host, T * K * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    else
        MCU_CUDA(cudaMemcpy2DAsync(xd, K * sizeof(float), x_host, ldx * sizeof(float), K * sizeof(float), T,
                                   cudaMemcpyHostToDevice, ctx->stream));
    if (out_map != nullptr) {
        od = out_map;
    } else {
        if (int rc = ensure(ctx, ctx->out_stage, T * F * sizeof(float))) return rc;
        od = (float *)ctx->out_stage.ptr;
    }
    if (bias_host != nullptr) {
        if (int rc = ensure(ctx, ctx->bias_stage, F * sizeof(float))) return rc;
        bd = (float *)ctx->bias_stage.ptr;
        MCU_CUDA(cudaMemcpyAsync(bd, bias_host, F * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    }
    if (int rc = linear_locked(ctx, kind, xd, K, w_dev, nullptr, T, K, F, bd, od, nullptr, F)) return rc;
    if (out_map == nullptr)
        MCU_CUDA(cudaMemcpy2DAsync(out_host, ldo * sizeof(float), od, F * sizeof(float), F * sizeof(float), T,
                                   cudaMemcpyDeviceToHost, ctx->stream));
    return sync_and_check(ctx, ctx->stream);
}

int mcu_topk(mcu_context_t *ctx, const float *x_dev, size_t rows, size_t cols, size_t ldx, size_t k, float *values_dev,
             int32_t *indices_dev) {
    if (int rc = check_ctx(ctx)) return rc;
    if (x_dev == nullptr || values_dev == nullptr || indices_dev == nullptr)
        return fail(MCU_ERROR_INVALID_ARGUMENT, "TopK descriptor is incomplete");
    if (k == 0 || k > cols || ldx < cols) return fail(MCU_ERROR_DIMENSION_MISMATCH, "TopK shapes do not match");
    MCU_CUDA(launch_topk(x_dev, (int)rows, (int)cols, ldx, (int)k, values_dev, indices_dev, ctx->stream));
    count_launches(1);
    return MCU_SUCCESS;
}

// Experts [e_begin, e_begin + e_count) are local: gate/up/down hold only those, and routes to other experts
// contribute nothing to out (their share is another rank's).
static int moe_experts_impl(mcu_context_t *ctx, int gate_kind, int up_kind, int down_kind, const float *hidden_dev,
                            size_t T, size_t H, size_t FF, size_t E, size_t e_begin, size_t e_count,
                            const void *gate_dev, const void *up_dev, const void *down_dev,
                            const int32_t *topk_ids_dev, const float *topk_weights_dev, size_t k, int ffn_type,
                            float weights_scale, int router_weight_policy, float *out_dev, float *routed_rows_ext = nullptr) {
    // routed_rows_ext: the rows of the down projection go there ([T * k][H], sorted-route order) and are NOT combined
    // into out_dev (expert parallelism: the token owners do that); only the grouped path offers it.
    if (int rc = check_ctx(ctx)) return rc;
    if (e_begin + e_count > E) return fail(MCU_ERROR_INVALID_ARGUMENT, "local expert range exceeds the expert count");
    if (hidden_dev == nullptr || gate_dev == nullptr || up_dev == nullptr || down_dev == nullptr ||
        topk_ids_dev == nullptr || topk_weights_dev == nullptr || out_dev == nullptr)
        return fail(MCU_ERROR_INVALID_ARGUMENT, "MoE experts descriptor is incomplete");
    if (!kind_supported(gate_kind) || !kind_supported(up_kind) || !kind_supported(down_kind))
        return fail(MCU_ERROR_NOT_IMPLEMENTED, "MoE expert quant kind has no CUDA kernel");
    if (ffn_type != MCU_FFN_SWIGLU && ffn_type != MCU_FFN_GEGLU)
        return fail(MCU_ERROR_NOT_IMPLEMENTED, "MoE experts supports SWIGLU and GEGLU only");
    if (k == 0 || k > (size_t)MOE_MAX_TOPK || E == 0 || H == 0 || FF == 0)
        return fail(MCU_ERROR_DIMENSION_MISMATCH, "MoE experts shapes do not match");
    if (T == 0) return MCU_SUCCESS;
    std::lock_guard<std::mutex> lock(ctx->mu);
    const size_t routes = T * k;
    // routing metadata: counts[E+1] | offsets[E+1] | sorted_tok | sorted_w | route_pos
    const size_t meta_bytes = (2 * (E + 1) + 3 * routes) * sizeof(int32_t);
    if (int rc = ensure(ctx, ctx->moe_meta, meta_bytes)) return rc;
    if (int rc = ensure(ctx, ctx->moe_hidden, routes * H * sizeof(float))) return rc;
    if (int rc = ensure(ctx, ctx->moe_gate, routes * FF * sizeof(float))) return rc;
    if (int rc = ensure(ctx, ctx->moe_up, routes * FF * sizeof(float))) return rc;
    if (int rc = ensure(ctx, ctx->moe_down, routes * H * sizeof(float))) return rc;
    MoeRouteBuffers rb;
    rb.counts = (int *)ctx->moe_meta.ptr;
    rb.offsets = rb.counts + (E + 1);
    rb.sorted_tok = (int32_t *)(rb.offsets + (E + 1));
    rb.sorted_w = (float *)(rb.sorted_tok + routes);
    rb.route_pos = (int32_t *)(rb.sorted_w + routes);
    cudaStream_t s = ctx->stream;
    ctx->moe_last_routes = routes;
    ctx->moe_last_experts = E;
    ctx->moe_last_grouped = 0;
    const int renorm = router_weight_policy == MCU_ROUTER_RENORMALIZE_SELECTED;
    MCU_CUDA(launch_moe_route(topk_ids_dev, topk_weights_dev, (int)T, (int)k, (int)E, weights_scale, renorm, rb, s));
    count_launches(3);
    float *route_hidden = (float *)ctx->moe_hidden.ptr, *gate_out = (float *)ctx->moe_gate.ptr;
    float *up_out = (float *)ctx->moe_up.ptr;
    float *route_down = routed_rows_ext != nullptr ? routed_rows_ext : (float *)ctx->moe_down.ptr;
    // Large batches: one grouped launch per projection over all local experts, sized from the device-resident counts.
    // Nothing is read back, so the call neither waits for the device nor breaks a stream capture.
    static const bool no_grouped = getenv("MARMOT_CUDA_MOE_NO_GROUPED") != nullptr;  // diagnostic switch
    // Fewer routes normally take per-expert launches sized from counts read back on the host (small groups then get the
    // GEMV kernels); a call that is being recorded into a CUDA graph cannot read anything back, so it takes the grouped
    // launches whatever its size.
    const bool grouped = !no_grouped && (routes >= 256 || stream_is_capturing(s) || routed_rows_ext != nullptr) &&
        gate_kind == up_kind &&
        gemm_tma_grouped_supported(gate_kind, gate_dev, (int)H, (int)FF) &&
        gemm_tma_grouped_supported(up_kind, up_dev, (int)H, (int)FF) &&
        gemm_tma_grouped_supported(down_kind, down_dev, (int)FF, (int)H) &&
        act_half_fused_smem(gate_kind, (int)H) <= 48 * 1024 && act_half_fused_smem(down_kind, (int)FF) <= 48 * 1024 &&
        routes < ((size_t)1 << 24);
    if (grouped) {
        const size_t kp_h = (H + block_values(gate_kind) - 1) / block_values(gate_kind) * block_values(gate_kind);
        const size_t kp_f = (FF + block_values(down_kind) - 1) / block_values(down_kind) * block_values(down_kind);
        const size_t kp_max = kp_h > kp_f ? kp_h : kp_f;
        if (int rc = ensure(ctx, ctx->act_half, routes * kp_max * sizeof(__half))) return rc;
        if (int rc = ensure(ctx, ctx->act_rowscale, routes * sizeof(float))) return rc;
        __half *xh = (__half *)ctx->act_half.ptr;
        float *rowscale = (float *)ctx->act_rowscale.ptr;
        const int *cnt = rb.counts + e_begin, *off = rb.offsets + e_begin;
        // The staging kernels fetch their rows themselves: the routed token's hidden row for gate/up, act(gate) * up
        // for down.  Routes of other ranks' experts (outside [offsets[e_begin], offsets[e_end])) are skipped there,
        // never multiplied and never combined.
        ActSource from_hidden, from_glu;
        from_hidden.row_index = rb.sorted_tok;
        from_hidden.row_lo = from_glu.row_lo = rb.offsets + e_begin;
        from_hidden.row_hi = from_glu.row_hi = rb.offsets + e_begin + e_count;
        from_glu.x2 = up_out;
        from_glu.glu = ffn_type == MCU_FFN_GEGLU ? 2 : 1;
        MCU_CUDA(launch_act_half_fused_from(gate_kind, hidden_dev, (int)H, from_hidden, (int)routes, (int)H, ACT_ORDER_QUAD,
                                            xh, rowscale, s));
        MCU_CUDA(launch_gemm_tma_grouped(gate_kind, gate_dev, (int)e_count, xh, rowscale, (int)kp_h, (int)routes, (int)H,
                                         (int)FF, cnt, off, gate_out, (int)FF, ctx->dev_err, s));
        MCU_CUDA(launch_gemm_tma_grouped(up_kind, up_dev, (int)e_count, xh, rowscale, (int)kp_h, (int)routes, (int)H, (int)FF,
                                         cnt, off, up_out, (int)FF, ctx->dev_err, s));
        MCU_CUDA(launch_act_half_fused_from(down_kind, gate_out, (int)FF, from_glu, (int)routes, (int)FF, ACT_ORDER_QUAD, xh,
                                            rowscale, s));
        MCU_CUDA(launch_gemm_tma_grouped(down_kind, down_dev, (int)e_count, xh, rowscale, (int)kp_f, (int)routes, (int)FF,
                                         (int)H, cnt, off, route_down, (int)H, ctx->dev_err, s));
        if (routed_rows_ext == nullptr) {
            MCU_CUDA(launch_moe_combine_dev(route_down, rb.sorted_w, rb.route_pos, (int)T, (int)k, (int)H, rb.offsets,
                                            (int)e_begin, (int)(e_begin + e_count), rb.counts + E, ctx->dev_err, out_dev, H, s));
            count_launches(1);
        }
        count_launches(5);
        ctx->moe_last_grouped = 1;
        return MCU_SUCCESS;
    }
    if (routed_rows_ext != nullptr)
        return fail(MCU_ERROR_NOT_IMPLEMENTED, "this MoE shape does not take the grouped path: no routed rows to exchange");
    if (stream_is_capturing(s))
        return fail(MCU_ERROR_INVALID_OPERATION,
                    "this MoE shape reads the group sizes back to size the per-expert launches: the call cannot be captured");
    // The per-expert launches need the group sizes on the host.
    ctx->host_counts.resize(2 * (E + 1));
    MCU_CUDA(cudaMemcpyAsync(ctx->host_counts.data(), rb.counts, 2 * (E + 1) * sizeof(int), cudaMemcpyDeviceToHost, s));
    MCU_CUDA(cudaStreamSynchronize(s));
    if (ctx->host_counts[E] != 0) return fail(MCU_ERROR_INVALID_ARGUMENT, "MoE expert id is out of range");
    const int *counts = ctx->host_counts.data();
    const int *offsets = counts + (E + 1);
    const int pos_lo = offsets[e_begin], pos_hi = offsets[e_begin + e_count];  // sorted positions of the local routes
    MCU_CUDA(launch_moe_gather(hidden_dev, H, rb.sorted_tok, pos_lo, pos_hi, (int)H, route_hidden, s));
    count_launches(1);
    const size_t gate_slice = FF * mcu_row_bytes(gate_kind, H), up_slice = FF * mcu_row_bytes(up_kind, H);
    const size_t down_slice = H * mcu_row_bytes(down_kind, FF);
    for (size_t e = e_begin; e < e_begin + e_count; ++e) {
        const size_t cnt = (size_t)counts[e], off = (size_t)offsets[e], le = e - e_begin;
        if (cnt == 0) continue;
        const float *hx = route_hidden + off * H;
        const uint8_t *ge = (const uint8_t *)gate_dev + le * gate_slice, *ue = (const uint8_t *)up_dev + le * up_slice;
        int rc;
        if (gate_kind == up_kind) {
            rc = linear_locked(ctx, gate_kind, hx, H, ge, ue, cnt, H, FF, nullptr, gate_out + off * FF, up_out + off * FF, FF);
        } else {
            rc = linear_locked(ctx, gate_kind, hx, H, ge, nullptr, cnt, H, FF, nullptr, gate_out + off * FF, nullptr, FF);
            if (rc == 0)
                rc = linear_locked(ctx, up_kind, hx, H, ue, nullptr, cnt, H, FF, nullptr, up_out + off * FF, nullptr, FF);
        }
        if (rc != 0) return rc;
        MCU_CUDA(launch_moe_glu(gate_out + off * FF, up_out + off * FF, cnt * FF, ffn_type == MCU_FFN_GEGLU, s));
        count_launches(1);
        rc = linear_locked(ctx, down_kind, gate_out + off * FF, FF, (const uint8_t *)down_dev + le * down_slice, nullptr,
                           cnt, FF, H, nullptr, route_down + off * H, nullptr, H);
        if (rc != 0) return rc;
    }
    MCU_CUDA(launch_moe_combine(route_down, rb.sorted_w, rb.route_pos, (int)T, (int)k, (int)H, pos_lo, pos_hi, out_dev, H,
                                s));
    count_launches(1);
    return MCU_SUCCESS;
}

int mcu_moe_last_buffers(mcu_context_t *ctx, mcu_moe_buffers_t *out) {
    if (int rc = check_ctx(ctx)) return rc;
    if (out == nullptr) return fail(MCU_ERROR_INVALID_ARGUMENT, "null output");
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (ctx->moe_last_routes == 0 || ctx->moe_meta.ptr == nullptr)
        return fail(MCU_ERROR_INVALID_OPERATION, "no MoE call has run on this context");
    const size_t E = ctx->moe_last_experts, routes = ctx->moe_last_routes;
    const int *counts = (const int *)ctx->moe_meta.ptr;
    out->offsets = counts + (E + 1);
    out->sorted_tok = (const int32_t *)(out->offsets + (E + 1));
    out->sorted_w = (const float *)(out->sorted_tok + routes);
    out->route_pos = (const int32_t *)(out->sorted_w + routes);
    out->gate_out = (const float *)ctx->moe_gate.ptr;
    out->up_out = (const float *)ctx->moe_up.ptr;
    out->route_down = (const float *)ctx->moe_down.ptr;
    out->routes = routes;
    out->experts = E;
    out->grouped = ctx->moe_last_grouped;
    return MCU_SUCCESS;
}

int mcu_moe_experts(mcu_context_t *ctx, int gate_kind, int up_kind, int down_kind, const float *hidden_dev, size_t T,
                    size_t H, size_t FF, size_t E, const void *gate_dev, const void *up_dev, const void *down_dev,
                    const int32_t *topk_ids_dev, const float *topk_weights_dev, size_t k, int ffn_type,
                    float weights_scale, int router_weight_policy, float *out_dev) {
    return moe_experts_impl(ctx, gate_kind, up_kind, down_kind, hidden_dev, T, H, FF, E, 0, E, gate_dev, up_dev, down_dev,
                            topk_ids_dev, topk_weights_dev, k, ffn_type, weights_scale, router_weight_policy, out_dev);
}

int mcu_moe_experts_local(mcu_context_t *ctx, int gate_kind, int up_kind, int down_kind, const float *hidden_dev,
                          size_t T, size_t H, size_t FF, size_t E, size_t expert_begin, size_t expert_count,
                          const void *gate_dev, const void *up_dev, const void *down_dev,
                          const int32_t *topk_ids_dev, const float *topk_weights_dev, size_t k, int ffn_type,
                          float weights_scale, int router_weight_policy, float *out_dev) {
    return moe_experts_impl(ctx, gate_kind, up_kind, down_kind, hidden_dev, T, H, FF, E, expert_begin, expert_count,
                            gate_dev, up_dev, down_dev, topk_ids_dev, topk_weights_dev, k, ffn_type, weights_scale,
                            router_weight_policy, out_dev);
}

int mcu_moe_experts_ep(mcu_context_t *ctx, mcu_peer_comm_t *comm, int gate_kind, int up_kind, int down_kind,
                       const float *hidden_dev, size_t T, size_t H, size_t FF, size_t E, const int32_t *expert_bounds,
                       const void *gate_dev, const void *up_dev, const void *down_dev, const int32_t *topk_ids_dev,
                       const float *topk_weights_dev, size_t k, int ffn_type, float weights_scale, int router_weight_policy,
                       float *out_dev) {
    if (comm == nullptr || expert_bounds == nullptr) return fail(MCU_ERROR_INVALID_ARGUMENT, "null argument");
    const int rank = mcu_peer_comm_rank(comm), world = mcu_peer_comm_world(comm);
    if (expert_bounds[0] != 0 || (size_t)expert_bounds[world] != E)
        return fail(MCU_ERROR_INVALID_ARGUMENT, "expert bounds must cover the experts 0..E");
    const size_t rows_bytes = (T * k * H * sizeof(float) + 255) & ~(size_t)255;
    if (rows_bytes + T * H * sizeof(float) > mcu_peer_comm_capacity(comm))
        return fail(MCU_ERROR_INVALID_ARGUMENT, "the communicator's staging slot must hold (T * k + T) * H floats");
    float *rows = (float *)mcu_peer_comm_staging(comm);
    const size_t e_begin = (size_t)expert_bounds[rank], e_count = (size_t)(expert_bounds[rank + 1] - expert_bounds[rank]);
    if (int rc = moe_experts_impl(ctx, gate_kind, up_kind, down_kind, hidden_dev, T, H, FF, E, e_begin, e_count, gate_dev, up_dev,
                                  down_dev, topk_ids_dev, topk_weights_dev, k, ffn_type, weights_scale, router_weight_policy,
                                  out_dev, rows))
        return rc;
    const size_t routes = T * k;
    const int32_t *counts = (const int32_t *)ctx->moe_meta.ptr;  // counts[E+1] | offsets[E+1] | sorted_tok | sorted_w | route_pos
    const int32_t *offsets = counts + (E + 1);
    const float *sorted_w = (const float *)(offsets + (E + 1) + routes);
    const int32_t *route_pos = (const int32_t *)(sorted_w + routes);
    return mcu_peer_moe_combine(comm, route_pos, sorted_w, offsets, counts + E, expert_bounds, T, k, H, out_dev);
}

}  // extern "C"
