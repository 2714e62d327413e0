// Few-token matmul on integer tensor-core instructions (2 <= T <= 64 tokens): the regime where the weights are read
// once from HBM and every weight value meets a handful of tokens.
//
// The arithmetic is the reference's, integer for integer: activations are packed to Q8_K exactly as the reference
// packs them (act_pack.cuh), and every 32-value (Q4_K) or 16-value (Q6_K) sub-block dot product is an exact int32 sum
// computed by `mma.sync.m16n8k32 / m16n8k16 .s8.s8.s32`: 16 weight rows x 8 tokens per instruction, the weight rows
// as the A operand built in registers straight from the packed block bytes, the tokens as the B operand fetched with
// `ldmatrix` from the quantized activation tile.  Sub-block sums are scaled by the integer sub-block scales, summed
// per 256-value block, converted once and scaled by d * d_act in f32 (the reference's vec_dot_q4_k_q8_k /
// vec_dot_q6_k_q8_k, vec_dot_impl.h:688-732,783-828).  The Q4_K min term sum_j m_j * bsum_j uses the activation
// packer's sub-block sums, two products per dp2a.
// Nothing is rounded to fp16 anywhere, so the results sit at the fp32-accumulate tolerance (about 1e-6 of the
// reference in practice), not the tensor-core one.
//
// Data movement: one launch quantizes the activations (qs [Tpad][K] int8 in the in-block order of act_pack.cuh,
// scales transposed to [column][Tpad]); the matmul kernel is persistent, one CTA per SM.  Work is cut into stage
// units (a group of 64 weight rows x WK block columns) laid out row-group major; CTA c takes the contiguous span
// [SU*c/C, SU*(c+1)/C) of them, so every SM streams the same number of bytes whatever F and K are.  A producer thread
// feeds a ring of stages with TMA: per stage the raw weight blocks (a [64 rows x one block column] box per column, no
// repacking: rows of a box are 144 / 240 bytes apart, which spreads the eight rows a warp touches over all banks) and
// the activation tile of the same columns ([Tpad x 128 B] boxes, 128-byte swizzle for conflict-free ldmatrix).  The
// consumer warps are 4 row tiles x WK columns.  When a CTA's span ends inside a row group its partial sums go to a
// workspace and the last CTA to finish that row group adds the partials in CTA order (deterministic) - nobody waits
// for anybody.  Weight boxes are requested before `griddepcontrol.wait` (they never depend on the previous kernel);
// every mbarrier wait is bounded and ends in an error flag, not a hang.  No TMA multicast.
#include "act_pack.cuh"
#include "common.cuh"
#include "kernels.h"
#include "tma_utils.cuh"

#include <cstdlib>
#include <cstring>

namespace mcu {

constexpr int I8_WM = 4;                     // 16-row tiles per row group
constexpr int I8_ROWS = 16 * I8_WM;          // weight rows per row group
constexpr int I8_MAX_STAGES = 8;
// Block columns per stage (WK, a template parameter): 4 for one or two token tiles (sixteen consumer warps: the
// integer MMA has a long latency and few of them are in flight per warp), 2 beyond (the activation tiles of a stage
// grow with the token count).
__host__ __device__ constexpr int i8_wk(int NT) { return NT <= 2 ? 4 : 2; }
constexpr int I8_HEADER = 1024;              // barriers; keeps the stages 1024-byte aligned for the swizzled tiles

template <int KIND>
struct I8Cfg;
template <>
struct I8Cfg<KIND_Q4_K> {
    static constexpr int COL_BYTES = 144, BOX_W = 144;
};
template <>
struct I8Cfg<KIND_Q6_K> {
    static constexpr int COL_BYTES = 210, BOX_W = 240;  // the box starts on the 16-byte boundary below the column
};

struct GemmI8Params {
    float *out[2];
    const float *bias;
    const float *dT;   // activation scales [columns][Tpad]
    const int16_t *bsT; // sums of the 32-value sub-blocks of the activations [columns][Tpad][8] (Q4_K mins)
    float *partial;    // [CTAs][2][I8_WM][Tpad * 16] partial sums of row groups shared between CTAs
    int *tickets;      // [row groups * I8_WM], zero between launches
    int *err;
    int ldo, T, Tpad, F, ncols, NJ, RG, n_mats, SU, stages;
    int w_bytes, x_bytes, d_bytes, bs_bytes, stage_bytes;  // per stage: offsets / sizes of the three parts, stride of a stage
    int tx_bytes;                                // bytes the copies of one stage deliver
};

// first stage unit of CTA c of C
__host__ __device__ inline int i8_span_begin(int SU, int c, int C) { return (int)(((long long)SU * c) / C); }
// the CTA whose span holds stage unit x
__host__ __device__ inline int i8_owner(int SU, int x, int C) {
    return (int)((((long long)(x + 1) * C + SU - 1) / SU) - 1);
}

__device__ __forceinline__ void mma_s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
// 32-bit word at a 2-byte aligned shared-memory address
__device__ __forceinline__ uint32_t lds_u32_a2(const uint8_t *p) {
    const uint32_t a = tm_smem_u32(p);
    const uint32_t *w = (const uint32_t *)(p - (a & 3u));
    return (a & 2u) ? __funnelshift_r(w[0], w[1], 16) : w[0];
}

// Address of 16-byte chunk `chunk` of row `row` in a [rows][128 B] tile stored with the 128-byte swizzle.
__device__ __forceinline__ uint32_t swz128(uint32_t tile, int row, int chunk) {
    return tile + (uint32_t)row * 128u + (uint32_t)((chunk ^ (row & 7)) << 4);
}

// One Q4_K block column of one 16-row tile against NT token tiles.  wbox: the tile's rows in the weight box (row stride
// 144); xa / xb: the activation half tiles (sub-blocks 0,2,4,6 and 1,3,5,7 of the column, in-block order of
// act_pack.cuh); dcol: the column's activation scales.  acc[nt][i]: rows (g, g, g+8, g+8) x tokens (2t, 2t+1, ...).
template <int NT>
__device__ __forceinline__ void unit_q4_k(const uint8_t *wbox, uint32_t xa, uint32_t xb, const float *dcol,
                                          const int16_t *bscol, int lane, float (&acc)[NT][4]) {
    const int g = lane >> 2, t = lane & 3;
    const uint8_t *r0 = wbox + g * 144, *r1 = r0 + 8 * 144;
    const uint32_t h0 = *(const uint32_t *)r0, h1 = *(const uint32_t *)r1;
    uint32_t sc[2][2], mn[2][2];  // [row][low / high four sub-blocks], one byte per sub-block
    {
        const uint32_t a0 = *(const uint32_t *)(r0 + 4), a1 = *(const uint32_t *)(r0 + 8), a2 = *(const uint32_t *)(r0 + 12);
        sc[0][0] = a0 & 0x3F3F3F3Fu;
        mn[0][0] = a1 & 0x3F3F3F3Fu;
        sc[0][1] = (a2 & 0x0F0F0F0Fu) | (((a0 >> 6) & 0x03030303u) << 4);
        mn[0][1] = ((a2 >> 4) & 0x0F0F0F0Fu) | (((a1 >> 6) & 0x03030303u) << 4);
        const uint32_t b0 = *(const uint32_t *)(r1 + 4), b1 = *(const uint32_t *)(r1 + 8), b2 = *(const uint32_t *)(r1 + 12);
        sc[1][0] = b0 & 0x3F3F3F3Fu;
        mn[1][0] = b1 & 0x3F3F3F3Fu;
        sc[1][1] = (b2 & 0x0F0F0F0Fu) | (((b0 >> 6) & 0x03030303u) << 4);
        mn[1][1] = ((b2 >> 4) & 0x0F0F0F0Fu) | (((b1 >> 6) & 0x03030303u) << 4);
    }
    int p[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) p[nt][i] = 0;
    const int mat = lane >> 3, lrow = lane & 7;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {  // 64-value group: sub-blocks 2jj (low nibbles) and 2jj+1 (high nibbles)
        const uint32_t q00 = *(const uint32_t *)(r0 + 16 + 32 * jj + 4 * t), q01 = *(const uint32_t *)(r0 + 32 + 32 * jj + 4 * t);
        const uint32_t q10 = *(const uint32_t *)(r1 + 16 + 32 * jj + 4 * t), q11 = *(const uint32_t *)(r1 + 32 + 32 * jj + 4 * t);
        const int s0 = 2 * jj, s1 = 2 * jj + 1;
        const int sc00 = (int)((sc[0][s0 >> 2] >> (8 * (s0 & 3))) & 0xFFu), sc01 = (int)((sc[0][s1 >> 2] >> (8 * (s1 & 3))) & 0xFFu);
        const int sc10 = (int)((sc[1][s0 >> 2] >> (8 * (s0 & 3))) & 0xFFu), sc11 = (int)((sc[1][s1 >> 2] >> (8 * (s1 & 3))) & 0xFFu);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            // matrices: (xa, chunk 2jj), (xa, chunk 2jj+1), (xb, chunk 2jj), (xb, chunk 2jj+1)
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(swz128((mat & 2) ? xb : xa, nt * 8 + lrow, 2 * jj + (mat & 1)), b0, b1, b2, b3);
            int c[4] = {0, 0, 0, 0};
            mma_s8_k32(c, q00 & 0x0F0F0F0Fu, q10 & 0x0F0F0F0Fu, q01 & 0x0F0F0F0Fu, q11 & 0x0F0F0F0Fu, b0, b1);
            p[nt][0] += sc00 * c[0], p[nt][1] += sc00 * c[1], p[nt][2] += sc10 * c[2], p[nt][3] += sc10 * c[3];
            int e[4] = {0, 0, 0, 0};
            mma_s8_k32(e, (q00 >> 4) & 0x0F0F0F0Fu, (q10 >> 4) & 0x0F0F0F0Fu, (q01 >> 4) & 0x0F0F0F0Fu,
                       (q11 >> 4) & 0x0F0F0F0Fu, b2, b3);
            p[nt][0] += sc01 * e[0], p[nt][1] += sc01 * e[1], p[nt][2] += sc11 * e[2], p[nt][3] += sc11 * e[3];
        }
    }
    const float d0 = half_bits_to_float((uint16_t)(h0 & 0xFFFFu)), dm0 = half_bits_to_float((uint16_t)(h0 >> 16));
    const float d1 = half_bits_to_float((uint16_t)(h1 & 0xFFFFu)), dm1 = half_bits_to_float((uint16_t)(h1 >> 16));
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const float2 ad = *(const float2 *)(dcol + nt * 8 + 2 * t);
        // sum_j m_j * bsum_j (the reference's sumi): eight 16-bit sub-block sums per token against the eight 6-bit mins
        // of a row, two products per dp2a
        const int4 bs0 = *(const int4 *)(bscol + (nt * 8 + 2 * t) * 8), bs1 = *(const int4 *)(bscol + (nt * 8 + 2 * t + 1) * 8);
        int sm[4];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            sm[2 * r] = __dp2a_hi(bs0.w, (int)mn[r][1], __dp2a_lo(bs0.z, (int)mn[r][1], __dp2a_hi(bs0.y, (int)mn[r][0], __dp2a_lo(bs0.x, (int)mn[r][0], 0))));
            sm[2 * r + 1] = __dp2a_hi(bs1.w, (int)mn[r][1], __dp2a_lo(bs1.z, (int)mn[r][1], __dp2a_hi(bs1.y, (int)mn[r][0], __dp2a_lo(bs1.x, (int)mn[r][0], 0))));
        }
        acc[nt][0] = fmaf(ad.x, __fsub_rn(__fmul_rn(d0, (float)p[nt][0]), __fmul_rn(dm0, (float)sm[0])), acc[nt][0]);
        acc[nt][1] = fmaf(ad.y, __fsub_rn(__fmul_rn(d0, (float)p[nt][1]), __fmul_rn(dm0, (float)sm[1])), acc[nt][1]);
        acc[nt][2] = fmaf(ad.x, __fsub_rn(__fmul_rn(d1, (float)p[nt][2]), __fmul_rn(dm1, (float)sm[2])), acc[nt][2]);
        acc[nt][3] = fmaf(ad.y, __fsub_rn(__fmul_rn(d1, (float)p[nt][3]), __fmul_rn(dm1, (float)sm[3])), acc[nt][3]);
    }
}

// The same for a Q6_K block column: sixteen 16-value sub-blocks, int8 scales, values q - 32.  wbox rows are 240 bytes
// apart and the block starts `roff` bytes into the row (the box begins on a 16-byte boundary).
template <int NT>
__device__ __forceinline__ void unit_q6_k(const uint8_t *wbox, int roff, uint32_t xa, uint32_t xb, const float *dcol,
                                          int lane, float (&acc)[NT][4]) {
    const int g = lane >> 2, t = lane & 3;
    const uint8_t *r0 = wbox + g * 240 + roff, *r1 = r0 + 8 * 240;
    int p[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) p[nt][i] = 0;
    const int mat = lane >> 3, lrow = lane & 7;
#pragma unroll
    for (int n = 0; n < 2; ++n) {  // 128-value halves of the block
        const uint32_t s0w[2] = {lds_u32_a2(r0 + 192 + 8 * n), lds_u32_a2(r0 + 196 + 8 * n)};
        const uint32_t s1w[2] = {lds_u32_a2(r1 + 192 + 8 * n), lds_u32_a2(r1 + 196 + 8 * n)};
#pragma unroll
        for (int lh = 0; lh < 2; ++lh) {  // values l = 16 lh + 4t .. of the 32-value runs
            const uint32_t qh0 = lds_u32_a2(r0 + 128 + 32 * n + 16 * lh + 4 * t), qh1 = lds_u32_a2(r1 + 128 + 32 * n + 16 * lh + 4 * t);
            uint32_t a0[4], a1[4];  // A operands of sub-blocks 8n + 2c + lh, c = 0..3
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const uint32_t ql0 = lds_u32_a2(r0 + 64 * n + 32 * cc + 16 * lh + 4 * t), ql1 = lds_u32_a2(r1 + 64 * n + 32 * cc + 16 * lh + 4 * t);
#pragma unroll
                for (int chi = 0; chi < 2; ++chi) {
                    const int c = cc + 2 * chi;
                    a0[c] = __vsub4(((ql0 >> (4 * chi)) & 0x0F0F0F0Fu) | (((qh0 >> (2 * c)) & 0x03030303u) << 4), 0x20202020u);
                    a1[c] = __vsub4(((ql1 >> (4 * chi)) & 0x0F0F0F0Fu) | (((qh1 >> (2 * c)) & 0x03030303u) << 4), 0x20202020u);
                }
            }
            int sc0[4], sc1[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {  // scale index 8n + 2c + lh -> byte 2c + lh of this half's eight
                const int b = 2 * c + lh;
                sc0[c] = (int)(int8_t)((s0w[b >> 2] >> (8 * (b & 3))) & 0xFFu);
                sc1[c] = (int)(int8_t)((s1w[b >> 2] >> (8 * (b & 3))) & 0xFFu);
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                // sub-block 8n + 2c + lh lives in half (c & 1), 16-byte chunk 4n + 2(c >> 1) + lh: matrices c = 0..3
                uint32_t b[4];
                ldmatrix_x4(swz128((mat & 1) ? xb : xa, nt * 8 + lrow, 4 * n + 2 * (mat >> 1) + lh), b[0], b[1], b[2], b[3]);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    int e[4] = {0, 0, 0, 0};
                    mma_s8_k16(e, a0[c], a1[c], b[c]);
                    p[nt][0] += sc0[c] * e[0], p[nt][1] += sc0[c] * e[1], p[nt][2] += sc1[c] * e[2], p[nt][3] += sc1[c] * e[3];
                }
            }
        }
    }
    const float d0 = half_bits_to_float(*(const uint16_t *)(r0 + 208)), d1 = half_bits_to_float(*(const uint16_t *)(r1 + 208));
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const float2 ad = *(const float2 *)(dcol + nt * 8 + 2 * t);
        acc[nt][0] = fmaf(ad.x, __fmul_rn(d0, (float)p[nt][0]), acc[nt][0]);
        acc[nt][1] = fmaf(ad.y, __fmul_rn(d0, (float)p[nt][1]), acc[nt][1]);
        acc[nt][2] = fmaf(ad.x, __fmul_rn(d1, (float)p[nt][2]), acc[nt][2]);
        acc[nt][3] = fmaf(ad.y, __fmul_rn(d1, (float)p[nt][3]), acc[nt][3]);
    }
}

template <int KIND, int NT>
__global__ void __launch_bounds__((I8_WM * i8_wk(NT) + 1) * 32, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap map_w0, const __grid_constant__ CUtensorMap map_w1,
               const __grid_constant__ CUtensorMap map_x, const GemmI8Params p) {
    using Cfg = I8Cfg<KIND>;
    constexpr int I8_WK = i8_wk(NT), I8_WARPS = I8_WM * I8_WK;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t *full = (uint64_t *)smem;
    uint64_t *empty = full + I8_MAX_STAGES;
    uint8_t *stage0 = smem + I8_HEADER;
    uint8_t *red_buf = stage0 + (size_t)p.stages * p.stage_bytes;  // [I8_WM][NT * 4 * 32] floats
    const int S = p.stages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int C = gridDim.x, c = blockIdx.x;
    const int su0 = i8_span_begin(p.SU, c, C), su1 = i8_span_begin(p.SU, c + 1, C);

    if (threadIdx.x == 0) {
        for (int i = 0; i < S; ++i) {
            tm_mbar_init(tm_smem_u32(&full[i]), 1);
            tm_mbar_init(tm_smem_u32(&empty[i]), I8_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == I8_WARPS) {
        // ---------------- producer ----------------
        if (lane == 0) {
            const int n = su1 - su0;
            auto issue_w = [&](int i) {
                const int su = su0 + i, st = i % S;
                const int rgg = su / p.NJ, jj = su - rgg * p.NJ;  // row group over both matrices, column pair
                const int mat = rgg >= p.RG ? 1 : 0, rg = rgg - mat * p.RG;
                const uint32_t bar = tm_smem_u32(&full[st]);
                tm_mbar_expect_tx(bar, (uint32_t)p.tx_bytes);
                uint8_t *dst = stage0 + (size_t)st * p.stage_bytes;
                for (int k = 0; k < I8_WK; ++k) {
                    const int j = min(jj * I8_WK + k, p.ncols - 1);  // a column past the end repeats the last one (unused)
                    const int x = (j * Cfg::COL_BYTES) & ~15;
                    tm_tma_load_2d(tm_smem_u32(dst + k * (I8_ROWS * Cfg::BOX_W)), mat ? &map_w1 : &map_w0, x, rg * I8_ROWS, bar);
                }
            };
            auto issue_x = [&](int i) {
                const int su = su0 + i, st = i % S;
                const int jj = su % p.NJ;
                const uint32_t bar = tm_smem_u32(&full[st]);
                uint8_t *dst = stage0 + (size_t)st * p.stage_bytes + p.w_bytes;
                for (int k = 0; k < I8_WK; ++k) {
                    const int j = min(jj * I8_WK + k, p.ncols - 1);
                    for (int h = 0; h < 2; ++h)
                        tm_tma_load_2d(tm_smem_u32(dst + (k * 2 + h) * (p.Tpad * 128)), &map_x, j * 256 + h * 128, 0, bar);
                    const uint32_t dd = tm_smem_u32(dst + p.x_bytes + k * (p.Tpad * 4));
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dd),
                                 "l"(p.dT + (size_t)j * p.Tpad), "r"((uint32_t)(p.Tpad * 4)), "r"(bar)
                                 : "memory");
                    if (KIND == KIND_Q4_K) {
                        const uint32_t bb = tm_smem_u32(dst + p.x_bytes + p.d_bytes + k * (p.Tpad * 16));
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(bb),
                                     "l"(p.bsT + (size_t)j * p.Tpad * 8), "r"((uint32_t)(p.Tpad * 16)), "r"(bar)
                                     : "memory");
                    }
                }
            };
            // the weights never depend on the previous kernel in the stream: ask for the first ring's worth before
            // waiting for it; the activations are that kernel's output
            const int first = min(n, S);
            for (int i = 0; i < first; ++i) issue_w(i);
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int i = 0; i < first; ++i) issue_x(i);
            bool ok = true;
            for (int i = S; i < n && ok; ++i) {
                const int st = i % S, round = i / S;
                ok = tm_mbar_wait(tm_smem_u32(&empty[st]), (uint32_t)((round - 1) & 1));
                if (!ok) {
                    atomicExch(p.err, 11);
                    break;
                }
                issue_w(i);
                issue_x(i);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the output buffer may still be read by the previous kernel
    const int wm = warp / I8_WK, wk = warp - wm * I8_WK;
    const int g = lane >> 2, t = lane & 3;
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;

    for (int su = su0; su < su1; ++su) {
        const int i = su - su0, st = i % S;
        const int rgg = su / p.NJ, jj = su - rgg * p.NJ;
        if (!tm_mbar_wait(tm_smem_u32(&full[st]), (uint32_t)((i / S) & 1))) {
            if (lane == 0) atomicExch(p.err, 12);
            return;
        }
        const int j = jj * I8_WK + wk;
        if (j < p.ncols) {
            const uint8_t *sb = stage0 + (size_t)st * p.stage_bytes;
            const uint8_t *wbox = sb + wk * (I8_ROWS * Cfg::BOX_W) + (wm * 16) * Cfg::BOX_W;
            const uint32_t xa = tm_smem_u32(sb + p.w_bytes + (wk * 2) * (p.Tpad * 128)), xb = xa + p.Tpad * 128;
            const float *dcol = (const float *)(sb + p.w_bytes + p.x_bytes + wk * (p.Tpad * 4));
            const int16_t *bscol = (const int16_t *)(sb + p.w_bytes + p.x_bytes + p.d_bytes + wk * (p.Tpad * 16));
            if (KIND == KIND_Q4_K) unit_q4_k<NT>(wbox, xa, xb, dcol, bscol, lane, acc);
            else unit_q6_k<NT>(wbox, (j * Cfg::COL_BYTES) & 15, xa, xb, dcol, lane, acc);
        }
        __syncwarp();
        if (lane == 0) tm_mbar_arrive(tm_smem_u32(&empty[st]));

        // last stage unit of this row group within the span: reduce over the column warps and write
        const bool flush = su + 1 == su1 || (su + 1) / p.NJ != rgg;
        if (!flush) continue;
        float *redw = (float *)red_buf + (size_t)wm * (I8_WK - 1) * (NT * 4 * 32);
        if (wk != 0) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int k = 0; k < 4; ++k) redw[(size_t)(wk - 1) * (NT * 4 * 32) + (nt * 4 + k) * 32 + lane] = acc[nt][k];
        }
        asm volatile("bar.sync 1, %0;" ::"n"(I8_WARPS * 32) : "memory");
        if (wk == 0) {
#pragma unroll
            for (int w = 0; w < I8_WK - 1; ++w)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        acc[nt][k] = __fadd_rn(acc[nt][k], redw[(size_t)w * (NT * 4 * 32) + (nt * 4 + k) * 32 + lane]);
            const int mat = rgg >= p.RG ? 1 : 0, rg = rgg - mat * p.RG;
            const int row_lo = rg * I8_ROWS + wm * 16 + g;
            float *out = p.out[mat];
            const int first_su = rgg * p.NJ, last_su = first_su + p.NJ - 1;
            const int cf = i8_owner(p.SU, first_su, C), cl = i8_owner(p.SU, last_su, C);
            bool write_out = cf == cl;
            if (!write_out) {
                // this CTA holds a share of the row group: park it and take a ticket; the last one adds the shares up
                const int which = (rgg == su0 / p.NJ) ? 0 : 1;
                float *mine = p.partial + ((size_t)(c * 2 + which) * I8_WM + wm) * (NT * 4 * 32);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int k = 0; k < 4; ++k) __stcg(mine + (nt * 4 + k) * 32 + lane, acc[nt][k]);
                __threadfence();
                __syncwarp();
                int ticket = 0;
                if (lane == 0) ticket = atomicAdd(&p.tickets[rgg * I8_WM + wm], 1);
                ticket = __shfl_sync(0xffffffffu, ticket, 0);
                if (ticket == cl - cf) {
                    __threadfence();
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int k = 0; k < 4; ++k) acc[nt][k] = 0.0f;
                    for (int cc = cf; cc <= cl; ++cc) {
                        const int w2 = (rgg == i8_span_begin(p.SU, cc, C) / p.NJ) ? 0 : 1;
                        const float *src = p.partial + ((size_t)(cc * 2 + w2) * I8_WM + wm) * (NT * 4 * 32);
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                            for (int k = 0; k < 4; ++k) acc[nt][k] = __fadd_rn(acc[nt][k], __ldcg(src + (nt * 4 + k) * 32 + lane));
                    }
                    if (lane == 0) p.tickets[rgg * I8_WM + wm] = 0;  // ready for the next launch
                    write_out = true;
                }
            }
            if (write_out) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int row = row_lo + (k >> 1) * 8, tok = nt * 8 + 2 * t + (k & 1);
                        if (row < p.F && tok < p.T) {
                            const float v = acc[nt][k];
                            out[(size_t)tok * p.ldo + row] = p.bias != nullptr ? __fadd_rn(v, p.bias[row]) : v;
                        }
                    }
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int k = 0; k < 4; ++k) acc[nt][k] = 0.0f;
        asm volatile("bar.sync 1, %0;" ::"n"(I8_WARPS * 32) : "memory");  // the reduction buffer is free again
    }
}

// ---- activation packing for this kernel: qs [Tpad][kp] (rows T..Tpad-1 are never read: the tensor map ends at T),
//      scales transposed to dT [columns][Tpad] with zeros for the padding tokens ----
__global__ void __launch_bounds__(256) quantize_i8_kernel(const float *__restrict__ x, int ldx, int T, int Tpad, int K, int nb,
                                                         int8_t *__restrict__ qs, float *__restrict__ dT,
                                                         int16_t *__restrict__ bsT) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const int task = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // (block column, token): tokens fastest
    if (task >= nb * Tpad) return;
    const int j = task / Tpad, t = task - j * Tpad;
    if (t >= T) {
        if (lane == 0) dT[(size_t)j * Tpad + t] = 0.0f;
        return;
    }
    const float *row = x + (size_t)t * ldx + (size_t)j * QK_K;
    const int len = min(QK_K, K - j * QK_K);
    const bool vec_ok = (((uintptr_t)x & 15) == 0) && ((ldx & 3) == 0);
    float v[8];
    load_values_q8_k<32>(row, len, vec_ok, lane, v);
    pack_values_q8_k<32>(v, true, lane, qs + (size_t)t * nb * QK_K + (size_t)j * QK_K, dT + (size_t)j * Tpad + t,
                         bsT != nullptr ? bsT + ((size_t)j * Tpad + t) * 8 : nullptr);
}

// ---- host side ----
static int i8_stage_bytes(int kind, int Tpad, int *w, int *x, int *d, int *bs) {
    const int box_w = kind == KIND_Q4_K ? I8Cfg<KIND_Q4_K>::BOX_W : I8Cfg<KIND_Q6_K>::BOX_W;
    const int wk = i8_wk(Tpad / 8);
    *w = wk * I8_ROWS * box_w;
    *w = (*w + 1023) & ~1023;  // the swizzled activation tiles that follow need 1024-byte alignment
    *x = wk * 2 * Tpad * 128;
    *d = wk * Tpad * 4;
    *bs = kind == KIND_Q4_K ? wk * Tpad * 16 : 0;
    return (*w + *x + *d + *bs + 1023) & ~1023;
}

bool gemm_i8_supported(int kind, const void *W, const void *W2, int T, int K, int F) {
    if (kind != KIND_Q4_K && kind != KIND_Q6_K) return false;
    if (T < 2 || T > 64 || K < 1 || F < 1) return false;
    if (((uintptr_t)W & 15) || ((uintptr_t)W2 & 15)) return false;
    const int nb = (K + QK_K - 1) / QK_K;
    const long row_bytes = (long)nb * block_bytes(kind);
    if (row_bytes % 16) return false;  // tensor-map row stride
    return encode_tiled_fn() != nullptr;
}

// Workspace the caller provides: the packed activations (qs, dT), the parking area for row groups shared between
// CTAs, and the tickets (which must be zero before the first launch; the kernel leaves them zero).
void gemm_i8_workspace_bytes(int T, int K, int F, bool dual, size_t *qs_bytes, size_t *dT_bytes, size_t *partial_bytes,
                             size_t *ticket_bytes) {
    const int Tpad = (T + 7) & ~7, nb = (K + QK_K - 1) / QK_K;
    const int RG = (F + I8_ROWS - 1) / I8_ROWS;
    *qs_bytes = (size_t)Tpad * nb * QK_K;
    *dT_bytes = (size_t)nb * Tpad * (sizeof(float) + 8 * sizeof(int16_t));  // scales, then the sub-block sums
    *partial_bytes = (size_t)device_sm_count() * 2 * I8_WM * (Tpad / 8) * 4 * 32 * sizeof(float);
    *ticket_bytes = (size_t)RG * (dual ? 2 : 1) * I8_WM * sizeof(int);
}

template <int KIND, int NT>
static cudaError_t launch_i8(const CUtensorMap &mw0, const CUtensorMap &mw1, const CUtensorMap &mx, const GemmI8Params &p, int grid,
                             int smem, cudaStream_t s) {
    static int configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_i8_kernel<KIND, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        configured = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((I8_WM * i8_wk(NT) + 1) * 32, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemm_i8_kernel<KIND, NT>, mw0, mw1, mx, p);
}

template <int KIND>
static cudaError_t launch_i8_nt(int NT, const CUtensorMap &mw0, const CUtensorMap &mw1, const CUtensorMap &mx, const GemmI8Params &p,
                                int grid, int smem, cudaStream_t s) {
    switch (NT) {
    case 1: return launch_i8<KIND, 1>(mw0, mw1, mx, p, grid, smem, s);
    case 2: return launch_i8<KIND, 2>(mw0, mw1, mx, p, grid, smem, s);
    case 3: return launch_i8<KIND, 3>(mw0, mw1, mx, p, grid, smem, s);
    case 4: return launch_i8<KIND, 4>(mw0, mw1, mx, p, grid, smem, s);
    case 5: return launch_i8<KIND, 5>(mw0, mw1, mx, p, grid, smem, s);
    case 6: return launch_i8<KIND, 6>(mw0, mw1, mx, p, grid, smem, s);
    case 7: return launch_i8<KIND, 7>(mw0, mw1, mx, p, grid, smem, s);
    default: return launch_i8<KIND, 8>(mw0, mw1, mx, p, grid, smem, s);
    }
}

// Two launches: the activation packer and the matmul.
cudaError_t launch_gemm_i8(int kind, const void *W, const void *W2, const float *x, int ldx, int T, int K, int F, const float *bias,
                           float *out, float *out2, int ldo, int8_t *qs, float *dT, float *partial, int *tickets, int *err_flag,
                           cudaStream_t s) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr) return cudaErrorNotSupported;
    const int Tpad = (T + 7) & ~7, NT = Tpad / 8, nb = (K + QK_K - 1) / QK_K;
    const long row_bytes = (long)nb * block_bytes(kind);
    const int WK = i8_wk(NT);
    int16_t *bsT = kind == KIND_Q4_K ? (int16_t *)(dT + (size_t)nb * Tpad) : nullptr;
    {
        cudaLaunchConfig_t cfg = {};
        const int tasks = nb * Tpad;
        cfg.gridDim = dim3((unsigned)((tasks + 7) / 8), 1, 1);
        cfg.blockDim = dim3(256, 1, 1);
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, quantize_i8_kernel, x, ldx, T, Tpad, K, nb, qs, dT, bsT);
        if (e != cudaSuccess) return e;
    }

    const int box_w = kind == KIND_Q4_K ? I8Cfg<KIND_Q4_K>::BOX_W : I8Cfg<KIND_Q6_K>::BOX_W;
    alignas(64) CUtensorMap mw0, mw1, mx;
    auto encode_w = [&](CUtensorMap *m, const void *w) {
        const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)F};
        const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
        const cuuint32_t box[2] = {(cuuint32_t)box_w, (cuuint32_t)I8_ROWS};
        const cuuint32_t es[2] = {1, 1};
        return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(w), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    };
    if (encode_w(&mw0, W) != CUDA_SUCCESS) return cudaErrorInvalidValue;
    if (encode_w(&mw1, W2 != nullptr ? W2 : W) != CUDA_SUCCESS) return cudaErrorInvalidValue;
    {
        const cuuint64_t dims[2] = {(cuuint64_t)nb * QK_K, (cuuint64_t)T};
        const cuuint64_t strides[1] = {(cuuint64_t)nb * QK_K};
        const cuuint32_t box[2] = {128, (cuuint32_t)Tpad};
        const cuuint32_t es[2] = {1, 1};
        if (enc(&mx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, qs, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }

    GemmI8Params p;
    memset(&p, 0, sizeof(p));
    p.out[0] = out;
    p.out[1] = out2;
    p.bias = bias;
    p.dT = dT;
    p.bsT = bsT;
    p.partial = partial;
    p.tickets = tickets;
    p.err = err_flag;
    p.ldo = ldo;
    p.T = T;
    p.Tpad = Tpad;
    p.F = F;
    p.ncols = nb;
    p.NJ = (nb + WK - 1) / WK;
    p.RG = (F + I8_ROWS - 1) / I8_ROWS;
    p.n_mats = W2 != nullptr ? 2 : 1;
    p.SU = p.RG * p.n_mats * p.NJ;
    p.stage_bytes = i8_stage_bytes(kind, Tpad, &p.w_bytes, &p.x_bytes, &p.d_bytes, &p.bs_bytes);
    p.tx_bytes = WK * I8_ROWS * box_w + p.x_bytes + p.d_bytes + p.bs_bytes;
    if (W2 != nullptr && bias != nullptr) return cudaErrorInvalidValue;  // the dual form has no epilogue
    const int red_bytes = I8_WM * (WK - 1) * NT * 4 * 32 * (int)sizeof(float);
    const int budget = 220 * 1024 - I8_HEADER - red_bytes;
    p.stages = budget / p.stage_bytes;
    if (p.stages > I8_MAX_STAGES) p.stages = I8_MAX_STAGES;
    if (p.stages < 2) return cudaErrorInvalidValue;
    const int grid = device_sm_count() < p.SU ? device_sm_count() : p.SU;
    const int smem = I8_HEADER + p.stages * p.stage_bytes + red_bytes;
    if (kind == KIND_Q4_K) return launch_i8_nt<KIND_Q4_K>(NT, mw0, mw1, mx, p, grid, smem, s);
    return launch_i8_nt<KIND_Q6_K>(NT, mw0, mw1, mx, p, grid, smem, s);
}

}  // namespace mcu
