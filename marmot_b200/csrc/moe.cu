// Device-side MoE routing and glue: top-k, per-expert histogram, exclusive prefix, stable scatter
// of (token, weight*norm), hidden-row gather, act(gate)*up, and the weighted combine.
// Order and arithmetic follow the reference's grouped path
// (src/backends/cpu/ops/moe/moe_ops.c:789-889 top-k, :891-1049 grouped execution).
#include "common.cuh"
#include "kernels.h"
#include "moe.h"

#include <float.h>

namespace mcu {

// One thread per row; insertion top-k, equal values keep the lower column first (moe_ops.c:851-875).
__global__ void topk_kernel(const float *__restrict__ x, int rows, int cols, size_t ldx, int k,
                            float *__restrict__ values, int32_t *__restrict__ indices) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    float *bv = values + (size_t)r * k;
    int32_t *bi = indices + (size_t)r * k;
    for (int i = 0; i < k; ++i) {
        bv[i] = -FLT_MAX;
        bi[i] = -1;
    }
    for (int c = 0; c < cols; ++c) {
        const float v = x[(size_t)r * ldx + c];
        int pos = k;
        for (int i = 0; i < k; ++i) {
            if (v > bv[i] || (v == bv[i] && c < bi[i])) {
                pos = i;
                break;
            }
        }
        if (pos == k) continue;
        for (int i = k - 1; i > pos; --i) {
            bv[i] = bv[i - 1];
            bi[i] = bi[i - 1];
        }
        bv[pos] = v;
        bi[pos] = c;
    }
}

// counts[e] = number of routes to expert e; bad_flag set when an id is out of range.  A route with such an id gets
// position -1, which the scatter kernel never overwrites and the combine kernels skip, so that no later kernel
// indexes with a stale or uninitialised position.
__global__ void moe_count_kernel(const int32_t *__restrict__ ids, int routes, int E, int *__restrict__ counts,
                                 int *__restrict__ bad_flag, int32_t *__restrict__ route_pos) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= routes) return;
    const int e = ids[i];
    if (e < 0 || e >= E) {
        atomicExch(bad_flag, 1);
        route_pos[i] = -1;
        return;
    }
    atomicAdd(&counts[e], 1);
}

// Single block: exclusive prefix over the experts (offsets[E] = routes).
__global__ void moe_prefix_kernel(const int *__restrict__ counts, int E, int *__restrict__ offsets) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int p = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = p;
            p += counts[e];
        }
        offsets[E] = p;
    }
}

// One CTA per expert assigns stable positions to its routes in route order (token-major, slot-minor): each of the 32
// warps takes a contiguous chunk of the routes, counts its matches with ballots, an exclusive prefix over the warps'
// counts gives every chunk its first position, and a second pass over the chunk places the routes.  Writes the sorted
// token ids, the normalised weights (renormalise policy: weight * (scale / sum of the token's weights), 0 when the
// sum <= FLT_MIN, moe_ops.c:960-967) and the inverse map route -> position.
__global__ void __launch_bounds__(1024)
moe_scatter_kernel(const int32_t *__restrict__ ids, const float *__restrict__ weights, int T, int k,
                   const int *__restrict__ offsets, float weights_scale, int renormalize,
                   int32_t *__restrict__ sorted_tok, float *__restrict__ sorted_w, int32_t *__restrict__ route_pos) {
    __shared__ int warp_first[32];
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int routes = T * k;
    const int chunk = ((routes + 31) / 32 + 31) & ~31;  // routes per warp, a multiple of the warp size
    const int lo = warp * chunk, hi = min(routes, lo + chunk);
    int n = 0;
    for (int base = lo; base < hi; base += 32) {
        const int i = base + lane;
        n += __popc(__ballot_sync(0xffffffffu, i < hi && ids[i] == e));
    }
    if (lane == 0) warp_first[warp] = n;
    __syncthreads();
    if (warp == 0) {
        const int mine = warp_first[lane];
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        warp_first[lane] = offsets[e] + incl - mine;
    }
    __syncthreads();
    int cursor = warp_first[warp];
    for (int base = lo; base < hi; base += 32) {
        const int i = base + lane;
        const bool mine = i < hi && ids[i] == e;
        const unsigned m = __ballot_sync(0xffffffffu, mine);
        if (mine) {
            const int pos = cursor + __popc(m & ((1u << lane) - 1u));
            const int t = i / k;
            float norm = weights_scale;
            if (renormalize) {
                float s = 0.0f;
                for (int j = 0; j < k; ++j) s = __fadd_rn(s, weights[(size_t)t * k + j]);
                norm = s > FLT_MIN ? __fdiv_rn(weights_scale, s) : 0.0f;
            }
            sorted_tok[pos] = t;
            sorted_w[pos] = __fmul_rn(weights[i], norm);
            route_pos[i] = pos;
        }
        cursor += __popc(m);
    }
}

// route_hidden[r][:] = hidden[sorted_tok[r]][:]
__global__ void moe_gather_kernel(const float *__restrict__ hidden, size_t ldh, const int32_t *__restrict__ sorted_tok,
                                  int r0, int H, float *__restrict__ route_hidden) {
    const int r = r0 + blockIdx.x;
    const float *src = hidden + (size_t)sorted_tok[r] * ldh;
    float *dst = route_hidden + (size_t)r * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) dst[c] = src[c];
}

// gate <- act(gate) * up; silu(x) = x / (1 + expf(-x)), gelu(x) = 0.5 x (1 + erff(x / sqrt 2))
// (moe_ops.c:318-324,552-556)
__global__ void moe_glu_kernel(float *__restrict__ gate, const float *__restrict__ up, size_t n, int geglu) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = gate[i];
    float a;
    if (geglu) a = __fmul_rn(__fmul_rn(0.5f, g), __fadd_rn(1.0f, erff(__fmul_rn(g, 0.7071067811865475f))));
    else a = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
    gate[i] = __fmul_rn(a, up[i]);
}

// out[t][c] = sum over the token's routes, in ascending sorted position (= the reference's route
// order, moe_ops.c:1034-1042), of w * down[pos][c]; products and sums rounded separately.
template <int MAXK>
__global__ void moe_combine_kernel(const float *__restrict__ route_down, const float *__restrict__ sorted_w,
                                   const int32_t *__restrict__ route_pos, int k, int H, int pos_lo, int pos_hi,
                                   float *__restrict__ out, size_t ldo) {
    const int t = blockIdx.x;
    int pos[MAXK];
    float w[MAXK];
    for (int j = 0; j < k; ++j) pos[j] = route_pos[(size_t)t * k + j];
    for (int i = 1; i < k; ++i) {  // insertion sort, k is tiny
        const int p = pos[i];
        int j = i;
        while (j > 0 && pos[j - 1] > p) {
            pos[j] = pos[j - 1];
            --j;
        }
        pos[j] = p;
    }
    for (int j = 0; j < k; ++j) w[j] = (pos[j] >= pos_lo && pos[j] < pos_hi) ? sorted_w[pos[j]] : 0.0f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < k; ++j) {
            if (pos[j] < pos_lo || pos[j] >= pos_hi) continue;  // another rank's expert, or a rejected id
            acc = __fadd_rn(acc, __fmul_rn(w[j], route_down[(size_t)pos[j] * H + c]));
        }
        out[(size_t)t * ldo + c] = acc;
    }
}

// The same with the local range of sorted positions taken from the device-resident offsets (experts
// [e_begin, e_end)): no host read-back.  Block 0 also reports an out-of-range expert id through the error flag.
template <int MAXK>
__global__ void moe_combine_dev_kernel(const float *__restrict__ route_down, const float *__restrict__ sorted_w,
                                       const int32_t *__restrict__ route_pos, int k, int H,
                                       const int *__restrict__ offsets, int e_begin, int e_end,
                                       const int *__restrict__ bad_id_count, int *err, float *__restrict__ out, size_t ldo) {
    const int t = blockIdx.x;
    const int pos_lo = offsets[e_begin], pos_hi = offsets[e_end];
    if (t == 0 && threadIdx.x == 0 && *bad_id_count != 0) atomicExch(err, 40);
    int pos[MAXK];
    float w[MAXK];
    for (int j = 0; j < k; ++j) pos[j] = route_pos[(size_t)t * k + j];
    for (int i = 1; i < k; ++i) {
        const int p = pos[i];
        int j = i;
        while (j > 0 && pos[j - 1] > p) {
            pos[j] = pos[j - 1];
            --j;
        }
        pos[j] = p;
    }
    const bool bad = *bad_id_count != 0;  // the call is rejected as a whole: zeros out, error at synchronize
    for (int j = 0; j < k; ++j) w[j] = (!bad && pos[j] >= pos_lo && pos[j] < pos_hi) ? sorted_w[pos[j]] : 0.0f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < k; ++j) {
            if (bad || pos[j] < pos_lo || pos[j] >= pos_hi) continue;
            acc = __fadd_rn(acc, __fmul_rn(w[j], route_down[(size_t)pos[j] * H + c]));
        }
        out[(size_t)t * ldo + c] = acc;
    }
}

cudaError_t launch_moe_combine_dev(const float *route_down, const float *sorted_w, const int32_t *route_pos, int T, int k,
                                   int H, const int *offsets, int e_begin, int e_end, const int *bad_id_count, int *err,
                                   float *out, size_t ldo, cudaStream_t s) {
    if (T <= 0) return cudaSuccess;
    if (k > MOE_MAX_TOPK) return cudaErrorInvalidValue;
    moe_combine_dev_kernel<MOE_MAX_TOPK><<<T, 256, 0, s>>>(route_down, sorted_w, route_pos, k, H, offsets, e_begin, e_end,
                                                            bad_id_count, err, out, ldo);
    return cudaGetLastError();
}

cudaError_t launch_topk(const float *x, int rows, int cols, size_t ldx, int k, float *values, int32_t *indices,
                        cudaStream_t s) {
    if (rows <= 0) return cudaSuccess;
    topk_kernel<<<(rows + 127) / 128, 128, 0, s>>>(x, rows, cols, ldx, k, values, indices);
    return cudaGetLastError();
}

cudaError_t launch_moe_route(const int32_t *ids, const float *weights, int T, int k, int E, float weights_scale,
                             int renormalize, const MoeRouteBuffers &b, cudaStream_t s) {
    const int routes = T * k;
    cudaError_t err = cudaMemsetAsync(b.counts, 0, (size_t)(E + 1) * sizeof(int), s);
    if (err != cudaSuccess) return err;
    moe_count_kernel<<<(routes + 255) / 256, 256, 0, s>>>(ids, routes, E, b.counts, b.counts + E, b.route_pos);
    moe_prefix_kernel<<<1, 32, 0, s>>>(b.counts, E, b.offsets);
    moe_scatter_kernel<<<E, 1024, 0, s>>>(ids, weights, T, k, b.offsets, weights_scale, renormalize, b.sorted_tok,
                                        b.sorted_w, b.route_pos);
    return cudaGetLastError();
}

cudaError_t launch_moe_gather(const float *hidden, size_t ldh, const int32_t *sorted_tok, int pos_lo, int pos_hi, int H,
                              float *route_hidden, cudaStream_t s) {
    if (pos_hi <= pos_lo) return cudaSuccess;
    moe_gather_kernel<<<pos_hi - pos_lo, 256, 0, s>>>(hidden, ldh, sorted_tok, pos_lo, H, route_hidden);
    return cudaGetLastError();
}

cudaError_t launch_moe_glu(float *gate, const float *up, size_t n, int geglu, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    moe_glu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(gate, up, n, geglu);
    return cudaGetLastError();
}

cudaError_t launch_moe_combine(const float *route_down, const float *sorted_w, const int32_t *route_pos, int T, int k,
                               int H, int pos_lo, int pos_hi, float *out, size_t ldo, cudaStream_t s) {
    if (T <= 0) return cudaSuccess;
    if (k > MOE_MAX_TOPK) return cudaErrorInvalidValue;
    moe_combine_kernel<MOE_MAX_TOPK><<<T, 256, 0, s>>>(route_down, sorted_w, route_pos, k, H, pos_lo, pos_hi, out, ldo);
    return cudaGetLastError();
}

}  // namespace mcu
