// MoE routing / glue launchers (internal).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace mcu {

constexpr int MOE_MAX_TOPK = 16;

struct MoeRouteBuffers {
    int *counts;           // [E] + one "bad id" flag at [E]
    int *offsets;          // [E + 1]
    int32_t *sorted_tok;   // [routes]
    float *sorted_w;       // [routes]
    int32_t *route_pos;    // [routes]: route (t*k + slot) -> sorted position
};

cudaError_t launch_topk(const float *x, int rows, int cols, size_t ldx, int k, float *values, int32_t *indices,
                        cudaStream_t s);
cudaError_t launch_moe_route(const int32_t *ids, const float *weights, int T, int k, int E, float weights_scale,
                             int renormalize, const MoeRouteBuffers &b, cudaStream_t s);
// rows [pos_lo, pos_hi) of the sorted route list only
cudaError_t launch_moe_gather(const float *hidden, size_t ldh, const int32_t *sorted_tok, int pos_lo, int pos_hi, int H,
                              float *route_hidden, cudaStream_t s);
cudaError_t launch_moe_glu(float *gate, const float *up, size_t n, int geglu, cudaStream_t s);
// routes whose sorted position lies outside [pos_lo, pos_hi) are skipped
cudaError_t launch_moe_combine(const float *route_down, const float *sorted_w, const int32_t *route_pos, int T, int k,
                               int H, int pos_lo, int pos_hi, float *out, size_t ldo, cudaStream_t s);

// combine with the local range given as experts [e_begin, e_end) and looked up in the device-resident offsets;
// *bad_id_count != 0 (an expert id out of range was seen while counting) sets *err to 40
cudaError_t launch_moe_combine_dev(const float *route_down, const float *sorted_w, const int32_t *route_pos, int T, int k,
                                   int H, const int *offsets, int e_begin, int e_end, const int *bad_id_count, int *err,
                                   float *out, size_t ldo, cudaStream_t s);

}  // namespace mcu
