// Streaming decode-regime matmul (T <= 8 tokens): planning and launch.  The kernel family lives in
// gemv_stream_kernel.cuh; this file instantiates the kernels without an activation prologue, gemv_stream_addnorm.cu
// and gemv_stream_swiglu.cu those with one.
#include "gemv_stream_kernel.cuh"

namespace mcu {

cudaError_t launch_gemv_stream_plain(int kind, int T, bool short_cfg, const GemvStreamParams &p, int gx, int smem, cudaStream_t s) {
    return launch_all_kinds<GEMV_PRO_NONE>(kind, T, short_cfg, p, gx, smem, s);
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
static int gcd_int(int a, int b) { return b == 0 ? a : gcd_int(b, a % b); }

struct StreamPlan {
    bool ok;
    bool short_cfg;
    int kind;  // template KIND of the launch
    int gx, stages, stage_stride, act_bytes, smem, nb;
    GemvJob job[GEMV_MAX_JOBS];
};

// Deals the CTAs of one wave to the jobs in proportion to their bytes (at least one each) and sizes the ring for the
// largest chunk.  The launch is "short" (half-SM CTAs, everything prefetched at once) when T = 1 and every CTA's share
// fits in three chunks.
static StreamPlan plan_stream(const GemvJobSpec *jobs, int n_jobs, int T, int K, const GemvPrologue &pro) {
    StreamPlan pl = {};
    if (T < 1 || T > GEMV_MAX_T || n_jobs < 1 || n_jobs > GEMV_MAX_JOBS || K < 1) return pl;
    const bool q8 = jobs[0].kind == KIND_Q8_0;
    pl.kind = jobs[0].kind;
    long row_bytes[GEMV_MAX_JOBS];
    int unit[GEMV_MAX_JOBS];
    double total = 0.0;
    for (int j = 0; j < n_jobs; ++j) {
        const GemvJobSpec &js = jobs[j];
        if (js.kind != KIND_Q4_K && js.kind != KIND_Q6_K && js.kind != KIND_Q8_0) return pl;
        if ((js.kind == KIND_Q8_0) != q8) return pl;  // one activation format per launch
        if (js.kind != pl.kind) pl.kind = KIND_MIXED;
        if (js.F < 1 || ((uintptr_t)js.W & 15)) return pl;  // bulk copies need 16-byte aligned sources
        const int bv = block_values(js.kind), nb = (K + bv - 1) / bv;
        row_bytes[j] = (long)nb * block_bytes(js.kind);
        if (row_bytes[j] > 64 * 1024) return pl;
        unit[j] = 16 / gcd_int((int)(row_bytes[j] % 16), 16);  // rows per 16-byte aligned group
        if (((long)js.F * row_bytes[j]) & 15) return pl;       // the last chunk of the last CTA must also be a 16-byte multiple
        total += (double)js.F * (double)row_bytes[j];
    }
    if (pro.op != GEMV_PRO_NONE && pro.op != GEMV_PRO_ADD_RMSNORM && pro.op != GEMV_PRO_SWIGLU) return pl;
    if (pro.op == GEMV_PRO_SWIGLU && pro.aux == nullptr) return pl;
    pl.nb = q8 ? (K + Q8_0_VALUES - 1) / Q8_0_VALUES : (K + QK_K - 1) / QK_K;
    pl.act_bytes = act_smem_bytes(!q8, T, pl.nb);
    const int sms = device_sm_count();
    if (sms < n_jobs) return pl;
    int ctas[GEMV_MAX_JOBS], given = 0;
    for (int j = 0; j < n_jobs; ++j) {
        ctas[j] = max(1, (int)((double)sms * ((double)jobs[j].F * (double)row_bytes[j]) / total));
        given += ctas[j];
    }
    // hand out what rounding left (or take back what the minimum of one added), largest share per CTA first
    while (given != sms) {
        int best = -1;
        double best_v = 0.0;
        for (int j = 0; j < n_jobs; ++j) {
            if (given > sms && ctas[j] <= 1) continue;
            const double per = (double)jobs[j].F * (double)row_bytes[j] / (double)ctas[j];
            const double v = given < sms ? per : -per;
            if (best < 0 || v > best_v) best = j, best_v = v;
        }
        if (best < 0) return pl;
        ctas[best] += given < sms ? 1 : -1;
        given += given < sms ? 1 : -1;
    }
    int rpc[GEMV_MAX_JOBS];
    for (int j = 0; j < n_jobs; ++j) {
        rpc[j] = (jobs[j].F + ctas[j] - 1) / ctas[j];
        rpc[j] = (rpc[j] + unit[j] - 1) / unit[j] * unit[j];
    }
    auto fill = [&](const int *rc, int stages, int stride, bool short_cfg) {
        pl.ok = true;
        pl.short_cfg = short_cfg;
        pl.stages = stages;
        pl.stage_stride = stride;
        pl.smem = GS_HEADER + pl.act_bytes + stages * stride;
        int begin = 0;
        for (int j = 0; j < n_jobs; ++j) {
            GemvJob &g = pl.job[j];
            g.W = (const uint8_t *)jobs[j].W;
            g.out = jobs[j].out;
            g.bias = jobs[j].bias;
            g.F = jobs[j].F;
            g.ldo = jobs[j].ldo;
            g.kind = jobs[j].kind;
            g.row_bytes = (int)row_bytes[j];
            g.rows_per_cta = rpc[j];
            g.rows_per_chunk = rc[j];
            g.cta_begin = begin;
            begin += (jobs[j].F + rpc[j] - 1) / rpc[j];
        }
        pl.gx = begin;
    };
    // Single-token launches whose per-CTA shares fit in the ring
    if (T == 1) {
        int rc[GEMV_MAX_JOBS], chunks = 0, stride = 0;
        bool ok = true;
        for (int j = 0; j < n_jobs && ok; ++j) {
            rc[j] = (int)min((long)NW_SHORT, (long)(40 * 1024) / row_bytes[j]) / unit[j] * unit[j];
            if (rc[j] < 1) {
                ok = false;
                break;
            }
            chunks = max(chunks, (rpc[j] + rc[j] - 1) / rc[j]);
            stride = max(stride, (int)((rc[j] * row_bytes[j] + 16 + 127) / 128 * 128));
        }
        static const int short_chunks = getenv("MARMOT_GS_SHORT_CHUNKS") ? atoi(getenv("MARMOT_GS_SHORT_CHUNKS")) : 3;  // diagnostic
        if (ok && chunks <= short_chunks && GS_HEADER + pl.act_bytes + chunks * stride <= 110 * 1024) {
            fill(rc, chunks, stride, true);
            return pl;
        }
    }
    // General case: one CTA per SM, sixteen consumer warps, as deep a ring as fits.
    {
        int rc[GEMV_MAX_JOBS], chunks = 0, stride = 0;
        for (int j = 0; j < n_jobs; ++j) {
            rc[j] = (int)min((long)NW_LONG, (long)(40 * 1024) / row_bytes[j]) / unit[j] * unit[j];
            if (rc[j] < 1) {
                if (row_bytes[j] * unit[j] > 64 * 1024 || unit[j] > NW_LONG) return pl;
                rc[j] = unit[j];
            }
            chunks = max(chunks, (rpc[j] + rc[j] - 1) / rc[j]);
            stride = max(stride, (int)((rc[j] * row_bytes[j] + 16 + 127) / 128 * 128));
        }
        const int budget = 200 * 1024 - GS_HEADER - pl.act_bytes;
        if (budget < 2 * stride) return pl;
        int stages = min(GS_MAX_STAGES, budget / stride);
        stages = min(stages, max(2, chunks));
        fill(rc, stages, stride, false);
        return pl;
    }
}

bool gemv_stream_jobs_supported(const GemvJobSpec *jobs, int n_jobs, int T, int K, const GemvPrologue &pro) {
    return plan_stream(jobs, n_jobs, T, K, pro).ok;
}

cudaError_t launch_gemv_stream_jobs(const GemvJobSpec *jobs, int n_jobs, const float *x, int ldx, int T, int K,
                                    const GemvPrologue &pro, int *err_flag, cudaStream_t s) {
    const StreamPlan pl = plan_stream(jobs, n_jobs, T, K, pro);
    if (!pl.ok) return cudaErrorInvalidValue;
    GemvStreamParams p = {};
    for (int j = 0; j < n_jobs; ++j) p.job[j] = pl.job[j];
    p.n_jobs = n_jobs;
    p.x = x;
    p.err = err_flag;
    p.ldx = ldx;
    p.K = K;
    p.nb = pl.nb;
    p.act_bytes = pl.act_bytes;
    p.stages = pl.stages;
    p.stage_stride = pl.stage_stride;
    p.pro = pro;
#ifdef MCU_TRACE
    static int trace_next = 0;
    p.trace_slot = trace_next++;
#endif
    if (pro.op == GEMV_PRO_ADD_RMSNORM) return launch_gemv_stream_addnorm(pl.kind, T, pl.short_cfg, p, pl.gx, pl.smem, s);
    if (pro.op == GEMV_PRO_SWIGLU) return launch_gemv_stream_swiglu(pl.kind, T, pl.short_cfg, p, pl.gx, pl.smem, s);
    return launch_gemv_stream_plain(pl.kind, T, pl.short_cfg, p, pl.gx, pl.smem, s);
}

static int specs_of(int kind, const void *W, const void *W2, int F, const float *bias, float *out, float *out2, int ldo,
                    GemvJobSpec (&js)[2]) {
    js[0] = GemvJobSpec{kind, W, F, bias, out, ldo};
    js[1] = GemvJobSpec{kind, W2, F, bias, out2, ldo};
    return W2 != nullptr ? 2 : 1;
}

bool gemv_stream_supported(int kind, const void *W, const void *W2, int T, int K, int F) {
    GemvJobSpec js[2];
    const int n = specs_of(kind, W, W2, F, nullptr, nullptr, nullptr, 0, js);
    return plan_stream(js, n, T, K, GemvPrologue{}).ok;
}

cudaError_t launch_gemv_stream(int kind, const void *W, const void *W2, const float *x, int ldx, int T, int K, int F,
                               const float *bias, float *out, float *out2, int ldo, int *err_flag, cudaStream_t s) {
    GemvJobSpec js[2];
    const int n = specs_of(kind, W, W2, F, bias, out, out2, ldo, js);
    return launch_gemv_stream_jobs(js, n, x, ldx, T, K, GemvPrologue{}, err_flag, s);
}

}  // namespace mcu
