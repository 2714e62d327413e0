// Quantized matmul for 8 < T <= 64 tokens on Q6_K (and, behind a switch, Q4_K) weights, bound by the weight stream.
//
// With this few tokens the tcgen05 path spends its time writing dequantised fp16 weight tiles to shared memory
// and handing them to the MMA issuer; the weights are used once, so staging them buys nothing.  Here the
// dequantised weights never leave the registers:
//
//   producer warp   one thread streams slabs of RAW packed blocks (128 or 256 weight rows x one 256-value block
//                   column, no swizzle) and the matching fp16 activation boxes (MT*16 tokens x 64 values,
//                   SWIZZLE_128B) into a ring of shared-memory stages with cp.async.bulk.tensor (TMA); the weight
//                   slabs of the first stages are requested before griddepcontrol.wait, i.e. while the kernel ahead
//                   in the stream is still running.
//   consumer warps  each owns 32 weight rows (four n-tiles of mma.sync m16n8k16; the tokens are the M dimension).
//                   A lane (g, t) of the quad layout reads one 32-bit word of packed weights per row and 16-value
//                   group, turns it into the two fp16 pairs of the B fragment with packed-half arithmetic (nibble ->
//                   1024+q by mask-and-or, -1024, one HFMA2 with the block's d*sc and -dmin*m), loads the A
//                   fragments of the activations with ldmatrix and accumulates in f32 registers.
//
// A word holds values 4t..4t+3 of its 16-value group and mask-and-or yields the pairs (4t, 4t+2) and (4t+1, 4t+3),
// so the activation rows are staged with every 16 values in the order that puts 4t and 4t+2 at positions 2t, 2t+1 and
// 4t+1, 4t+3 at positions 8+2t, 9+2t (act_half_fused_kernel, order 2): the k index of the MMA is only a label, as
// long as both operands agree on it.
//
// Few row tiles: K is split over blockIdx.z; partial tiles go to workspace and the last CTA of a tile (ticket) adds
// them in split order.  blockIdx.y selects the second weight matrix of a dual (gate/up) call.
// No TMA multicast; every mbarrier wait is bounded.
#include "common.cuh"
#include "kernels.h"
#include "tma_utils.cuh"

#include <cstdlib>

namespace mcu {

constexpr int GW_ROWS_PER_WARP = 32;
constexpr int GW_MAX_STAGES = 4;
constexpr int GW_MAX_SPLITS = 16;

template <int KIND>
struct GwCfg;
template <>
struct GwCfg<KIND_Q4_K> {
    static constexpr int UNIT = 144;   // bytes of one block
    static constexpr int BOX_W = 144;  // bytes fetched per row and slab
};
template <>
struct GwCfg<KIND_Q6_K> {
    static constexpr int UNIT = 210;
    static constexpr int BOX_W = 240;  // covers 210 bytes from a 16-byte boundary; 240 = 112 mod 128 keeps the eight
                                       // rows of a fragment on distinct shared-memory banks
};

struct GemmWarpParams {
    const float *bias;
    const float *rowscale;
    float *out0, *out1;  // second matrix of a dual call (blockIdx.y == 1)
    int *err;
    int ldo, T, F;
    int n_slabs, splits, slabs_per_split;
    int stages, stage_bytes;
    float *partial;  // [2][splits][T][F]
    int *counters;   // [2][tiles]
};

__device__ __forceinline__ void gw_ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void gw_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// A 32-bit word from a shared-memory address that is 2-byte aligned (Q6_K blocks are 210 bytes).
__device__ __forceinline__ uint32_t gw_lds32(const uint8_t *p, bool aligned4) {
    if (aligned4) return *(const uint32_t *)p;
    return (uint32_t) * (const uint16_t *)p | ((uint32_t) * (const uint16_t *)(p + 2) << 16);
}

template <int KIND, int MT, int NW>
__global__ void __launch_bounds__((NW + 1) * 32, NW == 4 ? (MT == 1 ? 3 : 2) : 1)
gemm_warp_kernel(const __grid_constant__ CUtensorMap map_w0, const __grid_constant__ CUtensorMap map_w1,
                 const __grid_constant__ CUtensorMap map_x, const GemmWarpParams p) {
    extern __shared__ uint8_t smem_raw[];
    using C = GwCfg<KIND>;
    constexpr int BM = NW * GW_ROWS_PER_WARP;
    constexpr int X_BOX = MT * 16 * 128;  // one activation box: MT*16 tokens x 64 fp16
    constexpr int X_BYTES = 4 * X_BOX;    // the 256 values of a slab
    constexpr uint32_t W_BYTES = (uint32_t)BM * C::BOX_W;

    const uint32_t raw_addr = tm_smem_u32(smem_raw);
    const uint32_t bar_base = (raw_addr + 7u) & ~7u;
    const uint32_t full = bar_base, empty = bar_base + 8u * GW_MAX_STAGES;
    volatile int *abort_flag = (volatile int *)(smem_raw + (bar_base - raw_addr) + 16 * GW_MAX_STAGES);
    const uint32_t ring = (bar_base + 16u * GW_MAX_STAGES + 16u + 1023u) & ~1023u;
    const uint8_t *ring_ptr = smem_raw + (ring - raw_addr);
    const int S = p.stages;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, which = blockIdx.y, z = blockIdx.z;
    const int f0 = tile * BM;
    const int rows_here = min(BM, p.F - f0);
    const int j0 = z * p.slabs_per_split;
    const int j1 = min(p.n_slabs, j0 + p.slabs_per_split);
    const int n = j1 - j0;

    __shared__ int last_s;
    if (threadIdx.x == 0) {
        last_s = 1;
        for (int i = 0; i < S; ++i) {
            tm_mbar_init(full + 8u * i, 1);
            tm_mbar_init(empty + 8u * i, NW);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // The next kernel of the stream may start its own prologue (and weight prefetch) from here on.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == NW) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            const CUtensorMap *mw = which ? &map_w1 : &map_w0;
            const int pre = min(S, n);
            // Weights are model constants: their first slabs are requested at once.  The activations belong to the
            // kernel ahead in the stream until griddepcontrol.wait returns.
            for (int i = 0; i < pre; ++i) {
                tm_mbar_expect_tx(full + 8u * i, W_BYTES + (uint32_t)X_BYTES);
                tm_tma_load_2d(ring + (uint32_t)(i * p.stage_bytes + X_BYTES), mw, ((j0 + i) * C::UNIT) & ~15, f0, full + 8u * i);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int i = 0; i < pre; ++i)
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    tm_tma_load_2d(ring + (uint32_t)(i * p.stage_bytes + b * X_BOX), &map_x, (j0 + i) * QK_K + 64 * b, 0,
                                   full + 8u * i);
            bool ok = true;
            int st = 0;
            uint32_t phase = 0;  // parity of the first release of a stage
            for (int i = pre; i < n && ok; ++i) {
                ok = tm_mbar_wait(empty + 8u * st, phase);
                if (!ok) break;
                tm_mbar_expect_tx(full + 8u * st, W_BYTES + (uint32_t)X_BYTES);
                tm_tma_load_2d(ring + (uint32_t)(st * p.stage_bytes + X_BYTES), mw, ((j0 + i) * C::UNIT) & ~15, f0, full + 8u * st);
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    tm_tma_load_2d(ring + (uint32_t)(st * p.stage_bytes + b * X_BOX), &map_x, (j0 + i) * QK_K + 64 * b, 0,
                                   full + 8u * st);
                if (++st == S) {
                    st = 0;
                    phase ^= 1u;
                }
            }
            if (!ok) {
                atomicExch(p.err, 30);
                *abort_flag = 1;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------ consumers ------------------------------
        const int g = lane >> 2, tq = lane & 3;
        const int mi = lane >> 3;
        // ldmatrix: lanes 8i..8i+7 give the row addresses of matrix i = (tokens 0-7 | 8-15) x (first | second
        // 16-byte piece of the 16-value group); the box is swizzled in 16-byte pieces by (row & 7)
        uint32_t a_row[MT];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) a_row[mt] = (uint32_t)((16 * mt + 8 * (mi & 1) + (lane & 7)) * 128);
        const uint32_t a_sw = (uint32_t)(lane & 7), a_piece = (uint32_t)(mi >> 1);
        float acc[MT][4][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.0f;

        bool ok = true;
        int st = 0;
        uint32_t phase = 0;
        const __half2 k1024 = as_half2(0x64006400u), k64 = as_half2(0x54005400u);
        for (int i = 0; i < n; ++i) {
            ok = tm_mbar_wait(full + 8u * st, phase);
            ok = __all_sync(0xffffffffu, ok) && !*abort_flag;
            if (!ok) break;
            const int j = j0 + i;
            const uint32_t xst = ring + (uint32_t)(st * p.stage_bytes);
            const uint8_t *wst = ring_ptr + (size_t)st * p.stage_bytes + X_BYTES + ((j * C::UNIT) & 15);
            const uint8_t *rowp[4];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) rowp[nt] = wst + (size_t)(warp * GW_ROWS_PER_WARP + 8 * nt + g) * C::BOX_W;

            if constexpr (KIND == KIND_Q4_K) {
                // lane (g, t) prepares d*sc and -dmin*m of the sub-block pair t of its four rows; the quad shares them
                uint32_t s2[4], m2[4];
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const uint4 hdr = *(const uint4 *)rowp[nt];  // d, dmin | scales[12]
                    uint32_t sc2, mn2;
                    q4k_scale_bytes(hdr, tq, sc2, mn2);
                    const __half2 sc_h = __hsub2(as_half2(__byte_perm(sc2, 0x64646464u, 0x4140)), k1024);
                    const __half2 mn_h = __hsub2(as_half2(__byte_perm(mn2, 0x64646464u, 0x4140)), k1024);
                    const __half2 dd = as_half2(__byte_perm(hdr.x, 0u, 0x1010));
                    const __half2 nd = as_half2(__byte_perm(hdr.x, 0u, 0x3232) ^ 0x80008000u);
                    s2[nt] = as_u32(__hmul2(sc_h, dd));
                    m2[nt] = as_u32(__hmul2(mn_h, nd));
                }
#pragma unroll
                for (int kq = 0; kq < 4; ++kq) {
                    const int src = (lane & ~3) | kq;
                    uint32_t w0[4], w1[4];
                    __half2 sa[4], sb[4], ma[4], mb[4];
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) {
                        const __half2 s = as_half2(__shfl_sync(0xffffffffu, s2[nt], src));
                        const __half2 m = as_half2(__shfl_sync(0xffffffffu, m2[nt], src));
                        sa[nt] = bcast_lo(s);
                        sb[nt] = bcast_hi(s);
                        ma[nt] = bcast_lo(m);
                        mb[nt] = bcast_hi(m);
                        w0[nt] = *(const uint32_t *)(rowp[nt] + 16 + 32 * kq + 4 * tq);
                        w1[nt] = *(const uint32_t *)(rowp[nt] + 32 + 32 * kq + 4 * tq);
                    }
                    const uint32_t xbox = xst + (uint32_t)(kq * X_BOX);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {  // 16-value groups: low nibbles of bytes 0-15, 16-31, then the high ones
                        uint32_t a[MT][4];
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) gw_ldsm_x4(xbox + a_row[mt] + (((2u * u + a_piece) ^ a_sw) << 4), a[mt]);
#pragma unroll
                        for (int nt = 0; nt < 4; ++nt) {
                            const uint32_t w = (u & 1) ? w1[nt] : w0[nt];
                            uint32_t b0, b1;
                            if (u < 2) {
                                const __half2 v02 = as_half2((w & 0x000F000Fu) | 0x64006400u);
                                const __half2 v13 = as_half2(((w >> 8) & 0x000F000Fu) | 0x64006400u);
                                b0 = as_u32(__hfma2(__hsub2(v02, k1024), sa[nt], ma[nt]));
                                b1 = as_u32(__hfma2(__hsub2(v13, k1024), sa[nt], ma[nt]));
                            } else {
                                const __half2 v02 = as_half2((w & 0x00F000F0u) | 0x54005400u);
                                const __half2 v13 = as_half2(((w >> 8) & 0x00F000F0u) | 0x54005400u);
                                b0 = as_u32(__hfma2(__hsub2(v02, k64), sb[nt], mb[nt]));
                                b1 = as_u32(__hfma2(__hsub2(v13, k64), sb[nt], mb[nt]));
                            }
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt) gw_mma(acc[mt][nt], a[mt], b0, b1);
                        }
                    }
                }
            } else {
                // Q6_K: ql[128] | qh[64] | scales[16] (int8) | d.  Group u (16 values) = half n = u / 8, quadrant
                // qd = (u % 8) / 2, 16-byte half lh = u % 2: low or high nibbles of ql[64n + 32(qd & 1) + 16lh ..],
                // bits 2qd.. of qh[32n + 16lh ..], scale u.
                const bool al4 = (tm_smem_u32(wst) & 3u) == 0;  // the same for every row of the slab
                const __half2 k1152 = as_half2(0x64806480u);     // 1024 + 128
                const __half2 k1056 = as_half2(0x64206420u);     // 1024 + 32
                uint32_t sp[4][8];  // per row: d*scale pairs (4i, 4i+2) and (4i+1, 4i+3), i = 0..3
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const uint32_t dbits = *(const uint16_t *)(rowp[nt] + 208);
                    const __half2 dd = as_half2(dbits | (dbits << 16));
#pragma unroll
                    for (int i2 = 0; i2 < 4; ++i2) {
                        const uint32_t sw = gw_lds32(rowp[nt] + 192 + 4 * i2, al4) ^ 0x80808080u;  // int8 + 128
                        __half2 e, o;
                        bytes_to_half2(sw, k1152, e, o);
                        sp[nt][2 * i2] = as_u32(__hmul2(e, dd));
                        sp[nt][2 * i2 + 1] = as_u32(__hmul2(o, dd));
                    }
                }
#pragma unroll
                for (int nh = 0; nh < 2; ++nh)
#pragma unroll
                    for (int lh = 0; lh < 2; ++lh) {
                        uint32_t qh[4], ql0[4], ql1[4];
#pragma unroll
                        for (int nt = 0; nt < 4; ++nt) {
                            qh[nt] = gw_lds32(rowp[nt] + 128 + 32 * nh + 16 * lh + 4 * tq, al4);
                            ql0[nt] = gw_lds32(rowp[nt] + 64 * nh + 16 * lh + 4 * tq, al4);
                            ql1[nt] = gw_lds32(rowp[nt] + 64 * nh + 32 + 16 * lh + 4 * tq, al4);
                        }
#pragma unroll
                        for (int qd = 0; qd < 4; ++qd) {
                            const int u = 8 * nh + 2 * qd + lh;  // group index inside the slab
                            const uint32_t xbox = xst + (uint32_t)((u >> 2) * X_BOX);
                            uint32_t a[MT][4];
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt)
                                gw_ldsm_x4(xbox + a_row[mt] + (((2u * (u & 3) + a_piece) ^ a_sw) << 4), a[mt]);
#pragma unroll
                            for (int nt = 0; nt < 4; ++nt) {
                                const uint32_t lo = ((qd & 1) ? ql1[nt] : ql0[nt]) >> (4 * (qd >> 1));
                                const uint32_t q = (lo & 0x0F0F0F0Fu) | (((qh[nt] >> (2 * qd)) & 0x03030303u) << 4);
                                __half2 e, o;
                                bytes_to_half2(q, k1056, e, o);  // (q - 32) of values (4t, 4t+2) and (4t+1, 4t+3)
                                const uint32_t pair = sp[nt][2 * (u >> 2) + (u & 1)];  // scales (4i + j&1) and (.. + 2)
                                const __half2 sc = (u & 2) ? bcast_hi(as_half2(pair)) : bcast_lo(as_half2(pair));
                                const uint32_t b0 = as_u32(__hmul2(e, sc)), b1 = as_u32(__hmul2(o, sc));
#pragma unroll
                                for (int mt = 0; mt < MT; ++mt) gw_mma(acc[mt][nt], a[mt], b0, b1);
                            }
                        }
                    }
            }
            __syncwarp();
            if (lane == 0) tm_mbar_arrive(empty + 8u * st);  // this warp no longer reads the stage
            if (++st == S) {
                st = 0;
                phase ^= 1u;
            }
        }
        if (!ok && lane == 0) {
            atomicExch(p.err, 31);
            *abort_flag = 1;
        }

        // ------------------------------ epilogue ------------------------------
        // acc[mt][nt] = {(token 16mt+g, feature 8nt+2t), (.., +1), (token +8, ..), (token +8, +1)}
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (ok) {
            float *dst = p.splits == 1 ? (which ? p.out1 : p.out0) : p.partial + ((size_t)which * p.splits + z) * (size_t)p.T * p.F;
            const size_t ld = p.splits == 1 ? (size_t)p.ldo : (size_t)p.F;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int tok = 16 * mt + 8 * hh + g;
                    if (tok >= p.T) continue;
                    const float rs = p.splits == 1 ? p.rowscale[tok] : 1.0f;
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) {
                        const int fr = warp * GW_ROWS_PER_WARP + 8 * nt + 2 * tq;
                        const int f = f0 + fr;
                        float v0 = acc[mt][nt][2 * hh] * rs, v1 = acc[mt][nt][2 * hh + 1] * rs;
                        if (p.splits == 1 && p.bias != nullptr) {
                            if (fr < rows_here) v0 += p.bias[f];
                            if (fr + 1 < rows_here) v1 += p.bias[f + 1];
                        }
                        float *o = dst + (size_t)tok * ld + f;
                        if (fr + 1 < rows_here && (((uintptr_t)o) & 7) == 0) {
                            *(float2 *)o = make_float2(v0, v1);
                        } else {
                            if (fr < rows_here) o[0] = v0;
                            if (fr + 1 < rows_here) o[1] = v1;
                        }
                    }
                }
        }
    }

    if (p.splits > 1) {
        // The last CTA of this tile to finish adds the partial tiles, in split order.
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            int *ctr = p.counters + which * gridDim.x + tile;
            const int ticket = atomicAdd(ctr, 1);
            last_s = ticket == p.splits - 1;
            if (last_s) *ctr = 0;  // ready for the next launch
        }
        __syncthreads();
        if (last_s && !*abort_flag) {
            __threadfence();
            const float *part = p.partial + (size_t)which * p.splits * (size_t)p.T * p.F;
            float *out = which ? p.out1 : p.out0;
            if ((p.F & 3) == 0 && (rows_here & 3) == 0 && (p.ldo & 3) == 0 && (((uintptr_t)out) & 15) == 0) {
                const int r4 = rows_here >> 2;
                for (int i = threadIdx.x; i < p.T * r4; i += blockDim.x) {
                    const int t = i / r4, f = f0 + ((i - t * r4) << 2);
                    float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                    for (int z0 = 0; z0 < GW_MAX_SPLITS; z0 += 8) {
                        if (z0 >= p.splits) break;
                        float4 v[8];
#pragma unroll
                        for (int zz = 0; zz < 8; ++zz)
                            if (z0 + zz < p.splits)
                                v[zz] = __ldcg((const float4 *)(part + ((size_t)(z0 + zz) * p.T + t) * p.F + f));
#pragma unroll
                        for (int zz = 0; zz < 8; ++zz)
                            if (z0 + zz < p.splits) {
                                sum.x += v[zz].x;
                                sum.y += v[zz].y;
                                sum.z += v[zz].z;
                                sum.w += v[zz].w;
                            }
                    }
                    const float rs = p.rowscale[t];
                    float4 b = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (p.bias != nullptr) b = *(const float4 *)(p.bias + f);
                    *(float4 *)(out + (size_t)t * p.ldo + f) =
                        make_float4(sum.x * rs + b.x, sum.y * rs + b.y, sum.z * rs + b.z, sum.w * rs + b.w);
                }
            } else {
                for (int i = threadIdx.x; i < p.T * rows_here; i += blockDim.x) {
                    const int t = i / rows_here, f = f0 + (i - t * rows_here);
                    float sum = 0.0f;
                    for (int zz = 0; zz < p.splits; ++zz) sum += __ldcg(part + ((size_t)zz * p.T + t) * p.F + f);
                    out[(size_t)t * p.ldo + f] = sum * p.rowscale[t] + (p.bias != nullptr ? p.bias[f] : 0.0f);
                }
            }
        }
    }
    __syncthreads();
    if (*abort_flag) {
        // A wait ran out and the agents stopped early: bulk tensor copies may still be landing in this CTA's shared
        // memory.  Give them time to finish before the CTA (and its shared memory) goes away.
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
struct WarpPlan {
    int nw;  // consumer warps per CTA: 4 (two or three CTAs per SM) or 8
    int ctas_per_sm;
    int stages, stage_bytes, splits, slabs_per_split, tiles;
};

static int box_w(int kind) { return kind == KIND_Q4_K ? GwCfg<KIND_Q4_K>::BOX_W : GwCfg<KIND_Q6_K>::BOX_W; }

static WarpPlan plan_warp(int kind, int T, int K, int F, bool dual) {
    const int mt = (T + 15) / 16;
    const int x_bytes = 4 * mt * 16 * 128;
    WarpPlan pl;
    // The consumers are bound by instruction latency, so resident warps count for more than a deep ring: three CTAs per
    // SM when the registers allow it (one token tile), else two, each with at least two stages.
    pl.nw = 4;
    pl.ctas_per_sm = mt == 1 ? 3 : 2;
    pl.stage_bytes = x_bytes + (4 * GW_ROWS_PER_WARP * box_w(kind) + 1023) / 1024 * 1024;
    pl.stages = (227 * 1024 / pl.ctas_per_sm - 3 * 1024) / pl.stage_bytes;
    if (pl.stages < 2 && pl.ctas_per_sm == 3) {
        pl.ctas_per_sm = 2;
        pl.stages = (227 * 1024 / 2 - 3 * 1024) / pl.stage_bytes;
    }
    if (pl.stages < 2) {  // one CTA of eight warps per SM, sharing the activation boxes
        pl.nw = 8;
        pl.ctas_per_sm = 1;
        pl.stage_bytes = x_bytes + (8 * GW_ROWS_PER_WARP * box_w(kind) + 1023) / 1024 * 1024;
        pl.stages = (222 * 1024) / pl.stage_bytes;
    }
    if (pl.stages > GW_MAX_STAGES) pl.stages = GW_MAX_STAGES;
    const int bm = pl.nw * GW_ROWS_PER_WARP;
    pl.tiles = (F + bm - 1) / bm;
    const int n_slabs = (K + QK_K - 1) / QK_K;
    if (pl.stages > n_slabs) pl.stages = n_slabs;
    const int slots = device_sm_count() * pl.ctas_per_sm;
    int splits = slots / (pl.tiles * (dual ? 2 : 1));
    if (splits > GW_MAX_SPLITS) splits = GW_MAX_SPLITS;
    if (splits > n_slabs / 2) splits = n_slabs / 2;  // at least two slabs per CTA: a partial tile costs as much traffic
    if (splits < 1) splits = 1;
    static const bool no_split = getenv("MARMOT_CUDA_GEMM_NO_SPLITK") != nullptr;  // diagnostic switch
    if (no_split) splits = 1;
    pl.slabs_per_split = (n_slabs + splits - 1) / splits;
    pl.splits = (n_slabs + pl.slabs_per_split - 1) / pl.slabs_per_split;
    return pl;
}

bool gemm_warp_supported(int kind, const void *W, const void *W2, int T, int K, int F) {
    static const bool off = getenv("MARMOT_CUDA_GEMM_NO_WARP") != nullptr;      // diagnostic switches
    static const bool q4k_too = getenv("MARMOT_CUDA_GEMM_WARP_Q4K") != nullptr;
    // Measured on B200 (K = 4096, F = 14336): Q6_K 25 / 30 / 37 / 45 us at T = 16 / 32 / 48 / 64 against 45 - 49 us on the
    // tcgen05 path; Q4_K 25 / 28 / 35 / 44 us against 26 / 28 / 30 / 31 us, so Q4_K stays on the tcgen05 path (mma.sync
    // runs at about a sixth of the tcgen05 rate and bounds this kernel from T = 48 on).
    if (off || !(kind == KIND_Q6_K || (kind == KIND_Q4_K && q4k_too))) return false;
    if (T <= GEMV_MAX_T || T > 64 || K % QK_K != 0 || F < 1) return false;
    if (!gemm_tma_supported(kind, W, W2, T, K, F)) return false;  // 16-byte aligned weights and rows
    const WarpPlan pl = plan_warp(kind, T, K, F, W2 != nullptr);
    return pl.stages >= 1 && pl.tiles * (W2 != nullptr ? 2 : 1) <= GEMM_TMA_MAX_TILE_COUNTERS;
}

size_t gemm_warp_workspace_bytes(int kind, int T, int K, int F, bool dual) {
    const WarpPlan pl = plan_warp(kind, T, K, F, dual);
    return pl.splits > 1 ? (size_t)(dual ? 2 : 1) * pl.splits * T * F * sizeof(float) : 0;
}

template <int KIND, int MT, int NW>
static cudaError_t launch_warp(const CUtensorMap &mw0, const CUtensorMap &mw1, const CUtensorMap &mx,
                               const GemmWarpParams &p, const WarpPlan &pl, bool dual, cudaStream_t s) {
    const int smem = 2048 + pl.stages * pl.stage_bytes;
    cudaError_t e = cudaFuncSetAttribute(gemm_warp_kernel<KIND, MT, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)pl.tiles, dual ? 2u : 1u, (unsigned)pl.splits);
    cfg.blockDim = dim3((NW + 1) * 32, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const bool no_pdl = getenv("MARMOT_CUDA_NO_PDL") != nullptr;  // diagnostic switch
    cfg.numAttrs = no_pdl ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, gemm_warp_kernel<KIND, MT, NW>, mw0, mw1, mx, p);
}

template <int KIND>
static cudaError_t launch_warp_kind(const CUtensorMap &mw0, const CUtensorMap &mw1, const CUtensorMap &mx,
                                    const GemmWarpParams &p, const WarpPlan &pl, bool dual, cudaStream_t s) {
    const int mt = (p.T + 15) / 16;
#define GW_CASE(M, N) \
    if (mt == M && pl.nw == N) return launch_warp<KIND, M, N>(mw0, mw1, mx, p, pl, dual, s)
    GW_CASE(1, 4);
    GW_CASE(2, 4);
    GW_CASE(3, 4);
    GW_CASE(4, 4);
    GW_CASE(1, 8);
    GW_CASE(2, 8);
    GW_CASE(3, 8);
    GW_CASE(4, 8);
#undef GW_CASE
    return cudaErrorInvalidConfiguration;
}

cudaError_t launch_gemm_warp(int kind, const void *W, const void *W2, const __half *xh, const float *rowscale, int ldxh,
                             int T, int K, int F, const float *bias, float *out, float *out2, int ldo, float *partial,
                             int *counters, int *err_flag, cudaStream_t s) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr) return cudaErrorNotSupported;
    const bool dual = W2 != nullptr;
    const WarpPlan pl = plan_warp(kind, T, K, F, dual);
    if (pl.splits > 1 && (partial == nullptr || counters == nullptr)) return cudaErrorInvalidValue;
    const int mt = (T + 15) / 16;
    const long row_bytes = (long)(K / QK_K) * block_bytes(kind);
    alignas(64) CUtensorMap mw[2], mx;
    for (int i = 0; i < (dual ? 2 : 1); ++i) {
        const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)F};
        const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
        const cuuint32_t box[2] = {(cuuint32_t)box_w(kind), (cuuint32_t)(pl.nw * GW_ROWS_PER_WARP)};
        const cuuint32_t es[2] = {1, 1};
        if (enc(&mw[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(i == 0 ? W : W2), dims, strides, box, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    if (!dual) mw[1] = mw[0];
    {
        const cuuint64_t dims[2] = {(cuuint64_t)ldxh, (cuuint64_t)T};
        const cuuint64_t strides[1] = {(cuuint64_t)ldxh * 2};
        const cuuint32_t box[2] = {64u, (cuuint32_t)(mt * 16)};
        const cuuint32_t es[2] = {1, 1};
        if (enc(&mx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(xh), dims, strides, box, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    GemmWarpParams p;
    p.bias = bias;
    p.rowscale = rowscale;
    p.out0 = out;
    p.out1 = dual ? out2 : out;
    p.err = err_flag;
    p.ldo = ldo;
    p.T = T;
    p.F = F;
    p.n_slabs = K / QK_K;
    p.splits = pl.splits;
    p.slabs_per_split = pl.slabs_per_split;
    p.stages = pl.stages;
    p.stage_bytes = pl.stage_bytes;
    p.partial = partial;
    p.counters = counters;
    return kind == KIND_Q4_K ? launch_warp_kind<KIND_Q4_K>(mw[0], mw[1], mx, p, pl, dual, s)
                             : launch_warp_kind<KIND_Q6_K>(mw[0], mw[1], mx, p, pl, dual, s);
}

}  // namespace mcu
