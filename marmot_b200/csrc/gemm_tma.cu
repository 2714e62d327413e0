// TMA-fed variant of the tensor-core quantized matmul (tcgen05 + TMEM), used when the weight rows are
// 16-byte multiples (K % 2048 == 0 for Q6_K, K % 256 == 0 for Q8_0, always for Q4_K).
//
//   warp 21     one thread streams slabs of RAW packed weight blocks (rows_box rows x one super-block
//               column, no swizzle) from HBM into a ring with cp.async.bulk.tensor.
//   warp 20     one thread loads the BN x 64 fp16 activation tile of every K step (SWIZZLE_128B) straight
//               into the MMA stage, also with cp.async.bulk.tensor.
//   warps 0..15 converters, four groups of four warps, group g taking the K steps with ks % 4 == g: every
//               thread dequantises the 64 values of one weight row from the packed blocks in shared memory
//               with packed-half arithmetic (nibble -> 1024+q by mask-and-or, -1024, one HFMA2 per two
//               values) and stores them into the fp16 A tile in the canonical K-major SWIZZLE_128B layout;
//               warps 0..7 later run the epilogue (tcgen05.ld, + bias, coalesced stores).
//   warps 16..19 one thread each issues tcgen05.mma (M = 128, N = BN, K = 16) and tcgen05.commit for the K
//               steps ks % issuers == i into its own TMEM accumulator (narrow tiles are issue bound).
//
// For few tokens (T <= 64) the matmul is bound by the weight stream, so the CTAs take fewer than 128
// weight rows each (F split evenly over the SMs, rounded up to 8) instead of full 128-row tiles that
// would leave SMs idle; the unused accumulator lanes are simply not read back.
// No TMA multicast anywhere; every mbarrier wait is bounded.
#include "common.cuh"
#include "kernels.h"
#include "tma_utils.cuh"

#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>

namespace mcu {

constexpr int TM_BK = 64;
constexpr int TM_ALL_CONV = 16;  // converter warps, split into G groups (template parameter of the kernel):
                                 // G = 4: one weight row (64 values) per thread, group g takes the K steps ks % 4 == g;
                                 // G = 2: half a row (32 values) per thread, the groups alternate K steps.
                                 // A group must never be two uses of a stage ahead of the MMA (a parity wait cannot
                                 // tell them apart), which holds when the stage ring is at least G deep.
constexpr int TM_MAX_ISSUERS = 4;  // MMA-issuing warps, each with its own TMEM accumulator (see NACC in the kernel)
constexpr int TM_B_PRODUCER = TM_ALL_CONV + TM_MAX_ISSUERS;
constexpr int TM_W_PRODUCER = TM_B_PRODUCER + 1;
constexpr int TM_THREADS = (TM_W_PRODUCER + 1) * 32;
constexpr int TM_A_BYTES = TM_BM * TM_BK * 2;
constexpr int TM_MAX_RING = 8;

template <int KIND>
struct RawCfg;
template <>
struct RawCfg<KIND_Q4_K> {
    static constexpr int KR = 4;         // K steps per raw slab (one 256-value super-block)
    static constexpr int UNIT = 144;     // bytes of packed data per slab and row
    static constexpr int BOX_W = 144;    // bytes fetched per row (16-byte aligned window covering UNIT)
};
template <>
struct RawCfg<KIND_Q6_K> {
    static constexpr int KR = 4;
    static constexpr int UNIT = 210;
    static constexpr int BOX_W = 224;
};
template <>
struct RawCfg<KIND_Q8_0> {
    static constexpr int KR = 2;         // four 32-value blocks
    static constexpr int UNIT = 136;
    static constexpr int BOX_W = 144;
};

struct GemmTmaParams {
    const float *bias;
    const float *rowscale;  // per-token power-of-two factor undone in the epilogue
    float *out;
    int *err;
    int ldo, T, F, nb;
    int ksteps;
    int rows_per_cta;  // weight rows per CTA (= tensor-map box rows): <= 128, or 256 for two row tiles
    int stages;        // MMA stage ring depth
    int raw_stages;    // raw slab ring depth
    int raw_stage_bytes;  // bytes of one slab slot (a multiple of 128)
    int issuers;       // MMA-issuing warps in use (1..4), a divisor of `stages`
    // Split K (few tokens, few row tiles): blockIdx.z takes `slabs_per_split` slabs of K; every CTA writes its
    // partial tile to `partial` [split][T][F] and the last CTA of a tile to arrive (ticket in `counters`) adds the
    // partials in split order, so the result does not depend on the arrival order.
    int splits, slabs_per_split;
    float *partial;
    int *counters;
    PeerFuse fuse;  // world > 0: finished tiles go to all ranks' slots and are summed there (see kernels.h)
    // Grouped launch (MoE experts): blockIdx.z is the group; it owns group_counts[z] activation rows starting at row
    // group_offsets[z] of xh / rowscale / out, and the weight rows [z * F, (z + 1) * F) of the stacked matrix.  The
    // counts live in device memory (no host read-back); token tiles beyond a group's count exit at once.
    const int *group_counts, *group_offsets;
#ifdef MCU_TRACE
    long long *trace;  // development aid: clock64 samples of CTA 0, [agent][step][point]
#endif
};

#ifdef MCU_TRACE
#define MCU_TRACE_POINT(agent, step, point)                                                          \
    do {                                                                                             \
        if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (step) < 64)                 \
            p.trace[((agent) * 64 + (step)) * 4 + (point)] = clock64();                               \
    } while (0)
#else
#define MCU_TRACE_POINT(agent, step, point) do { } while (0)
#endif

// ---- converters: the 64 values of one weight row for K step KQ of the slab, as eight 16-byte chunks ----

// Q4_K: bytes 32*kq .. 32*kq+31 of qs hold sub-block 2*kq in their low nibbles and 2*kq+1 in their high nibbles.
// Everything stays in packed-half and integer lanes: 6-bit scales become fp16 through the 0x6400 pattern, the
// products d*sc and dmin*m are single fp16 roundings of exact values (11-bit x 6-bit), exactly what rounding the
// f32 products would give.
__device__ __forceinline__ void conv_q4k(const uint8_t *rowp, int kq, uint4 (&outv)[8]) {
    const uint4 hdr = *(const uint4 *)rowp;  // d, dmin | scales[0..3] | scales[4..7] | scales[8..11]
    const uint4 q0 = *(const uint4 *)(rowp + 16 + 32 * kq), q1 = *(const uint4 *)(rowp + 32 + 32 * kq);
    uint32_t sc2, mn2;
    q4k_scale_bytes(hdr, kq, sc2, mn2);
    const __half2 k1024 = as_half2(0x64006400u), k64 = as_half2(0x54005400u);
    const __half2 sc_h = __hsub2(as_half2(__byte_perm(sc2, 0x64646464u, 0x4140)), k1024);  // (sc_a, sc_b)
    const __half2 mn_h = __hsub2(as_half2(__byte_perm(mn2, 0x64646464u, 0x4140)), k1024);
    const __half2 dd = as_half2(__byte_perm(hdr.x, 0u, 0x1010));                     // (d, d)
    const __half2 nd = as_half2(__byte_perm(hdr.x, 0u, 0x3232) ^ 0x80008000u);       // (-dmin, -dmin)
    const __half2 s2 = __hmul2(sc_h, dd), m2 = __hmul2(mn_h, nd);
    const __half2 sa = bcast_lo(s2), sb = bcast_hi(s2), ma = bcast_lo(m2), mb = bcast_hi(m2);
    const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    uint32_t oa[16], ob[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t ws = w[i] >> 8;
        // 0x6400 | n = 1024 + n;  0x5400 | (n << 4) = 64 + n
        const __half2 a0 = as_half2((w[i] & 0x000F000Fu) | 0x64006400u), a1 = as_half2((ws & 0x000F000Fu) | 0x64006400u);
        const __half2 b0 = as_half2((w[i] & 0x00F000F0u) | 0x54005400u), b1 = as_half2((ws & 0x00F000F0u) | 0x54005400u);
        oa[2 * i] = as_u32(__hfma2(__hsub2(a0, k1024), sa, ma));
        oa[2 * i + 1] = as_u32(__hfma2(__hsub2(a1, k1024), sa, ma));
        ob[2 * i] = as_u32(__hfma2(__hsub2(b0, k64), sb, mb));
        ob[2 * i + 1] = as_u32(__hfma2(__hsub2(b1, k64), sb, mb));
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        outv[c] = make_uint4(oa[4 * c], oa[4 * c + 1], oa[4 * c + 2], oa[4 * c + 3]);
        outv[4 + c] = make_uint4(ob[4 * c], ob[4 * c + 1], ob[4 * c + 2], ob[4 * c + 3]);
    }
}

// The same for half a row: h = 0 takes the low nibbles (sub-block 2*kq), h = 1 the high nibbles (2*kq+1) of the
// step's 32 bytes; out[0..3] are the 16-byte chunks 4h .. 4h+3 of the tile row.
__device__ __forceinline__ void conv_q4k_half(const uint8_t *rowp, int kq, int h, uint4 (&outv)[4]) {
    const uint4 hdr = *(const uint4 *)rowp;
    const uint4 q0 = *(const uint4 *)(rowp + 16 + 32 * kq), q1 = *(const uint4 *)(rowp + 32 + 32 * kq);
    uint32_t sc2, mn2;
    q4k_scale_bytes(hdr, kq, sc2, mn2);
    const __half2 k1024 = as_half2(0x64006400u);
    const __half2 sc_h = __hsub2(as_half2(__byte_perm(sc2, 0x64646464u, 0x4140)), k1024);
    const __half2 mn_h = __hsub2(as_half2(__byte_perm(mn2, 0x64646464u, 0x4140)), k1024);
    const __half2 dd = as_half2(__byte_perm(hdr.x, 0u, 0x1010));
    const __half2 nd = as_half2(__byte_perm(hdr.x, 0u, 0x3232) ^ 0x80008000u);
    const __half2 s2 = __hmul2(sc_h, dd), m2 = __hmul2(mn_h, nd);
    const __half2 sv = h ? bcast_hi(s2) : bcast_lo(s2), mv = h ? bcast_hi(m2) : bcast_lo(m2);
    const uint32_t mask = h ? 0x00F000F0u : 0x000F000Fu, magic = h ? 0x54005400u : 0x64006400u;
    const __half2 off = as_half2(magic);
    const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    uint32_t o[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const __half2 v0 = as_half2((w[i] & mask) | magic), v1 = as_half2(((w[i] >> 8) & mask) | magic);
        o[2 * i] = as_u32(__hfma2(__hsub2(v0, off), sv, mv));
        o[2 * i + 1] = as_u32(__hfma2(__hsub2(v1, off), sv, mv));
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) outv[c] = make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
}

// Q6_K: 32 values (half h of K step kq) of one block.
__device__ __forceinline__ void conv_q6k(const uint8_t *blk, int kq, int h, uint4 *outv) {
    const int n = kq >> 1, c = 2 * (kq & 1) + h;  // values 128n + 32c + l
    uint32_t ql[8], qh[8];
    tm_lds_words<8>(blk + n * 64 + (c & 1) * 32, ql);
    tm_lds_words<8>(blk + 128 + n * 32, qh);
    const uint32_t sc2 = *(const uint16_t *)(blk + 192 + n * 8 + 2 * c);
    const float d = half_bits_to_float(*(const uint16_t *)(blk + 208));
    const __half2 ds0 = __float2half2_rn(__fmul_rn(d, (float)(int8_t)(sc2 & 0xFFu)));
    const __half2 ds1 = __float2half2_rn(__fmul_rn(d, (float)(int8_t)(sc2 >> 8)));
    const __half2 off = __float2half2_rn(1056.0f);  // 1024 + 32
    uint32_t o[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t lo4 = (c & 2) ? ((ql[j] >> 4) & 0x0F0F0F0Fu) : (ql[j] & 0x0F0F0F0Fu);
        const uint32_t u = lo4 | (((qh[j] >> (2 * c)) & 0x03030303u) << 4);
        __half2 a, b;
        bytes_to_half2(u, off, a, b);
        const __half2 ds = j < 4 ? ds0 : ds1;
        o[2 * j] = as_u32(__hmul2(a, ds));
        o[2 * j + 1] = as_u32(__hmul2(b, ds));
    }
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) outv[cc] = make_uint4(o[4 * cc], o[4 * cc + 1], o[4 * cc + 2], o[4 * cc + 3]);
}

// Q8_0: one 32-value block.
__device__ __forceinline__ void conv_q8_0(const uint8_t *blk, uint4 *outv) {
    const __half2 dh = __half2half2(__ushort_as_half(*(const uint16_t *)blk));
    uint32_t q[8];
    tm_lds_words<8>(blk + 2, q);
    const __half2 off = __float2half2_rn(1152.0f);  // 1024 + 128
    uint32_t o[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        __half2 a, b;
        bytes_to_half2(q[j] ^ 0x80808080u, off, a, b);
        o[2 * j] = as_u32(__hmul2(a, dh));
        o[2 * j + 1] = as_u32(__hmul2(b, dh));
    }
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) outv[cc] = make_uint4(o[4 * cc], o[4 * cc + 1], o[4 * cc + 2], o[4 * cc + 3]);
}

// RT = 2 (with BN = 256, G = 1): the CTA owns two 128-row weight tiles and multiplies both with the same activation
// tile of a K step into two accumulators (all 512 TMEM columns).  With one row tile the 256-token activation tile
// (32 KB from L2 per K step) bounds the step at about half the tensor rate; two row tiles halve the activation bytes
// per MMA.  All sixteen converter warps then work on the same K step (half a row per thread, 256 rows).
template <int KIND, int BN, int G, int RT = 1>
__global__ void __launch_bounds__(TM_THREADS, 1)
gemm_tma_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                const GemmTmaParams p) {
    extern __shared__ uint8_t smem_raw[];
    using RC = RawCfg<KIND>;
    constexpr int B_BYTES = BN * TM_BK * 2;
    static_assert(RT == 1 || (RT == 2 && BN == 256 && G == 1), "two row tiles need the 256-token tile");
    constexpr int A_BYTES = RT * TM_A_BYTES;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    const int RAW_STAGE_BYTES = p.raw_stage_bytes;  // rows_per_cta * BOX_W rounded to 128, + slack for the one-word over-read
    // One thread can issue tcgen05.mma only so fast (a few hundred cycles per K step including its barrier
    // wait and commit), which is far slower than the tensor core for narrow tiles.  NACC threads therefore issue
    // interleaved K steps (step ks -> issuer ks % NACC), each into its own accumulator; the epilogue adds them.
    constexpr int NACC = BN == 64 ? 4 : (BN == 128 ? 2 : 1);
    constexpr uint32_t TMEM_COLS = RT * NACC * BN;  // 256 for every BN with one row tile, 512 with two
    constexpr int GW = TM_ALL_CONV / G;        // warps per converter group

    const uint32_t raw_addr = tm_smem_u32(smem_raw);
    const uint32_t bar_base = (raw_addr + 7u) & ~7u;
    const uint32_t tile_base = (bar_base + 512u + 1023u) & ~1023u;
    uint8_t *tiles = smem_raw + (tile_base - raw_addr);
    const int S = p.stages, R = p.raw_stages;
    uint8_t *raw_ring = tiles + (size_t)S * STAGE_BYTES;
    const uint32_t raw_ring_addr = tile_base + (uint32_t)S * STAGE_BYTES;
    // barrier slots (8 bytes each): full[8] stage_empty_odd[8] stage_empty[8] raw_full[8] raw_empty[8] accum
    // Stage-release barriers come in two sets used by alternate uses of a stage (use = ks / S): the converter
    // groups wait for a stage only at every G-th step, and with one barrier per stage a group could be two
    // phases ahead of it, which a parity wait cannot tell from "done".  With two sets the phases of one barrier
    // are 2*S steps apart, and everything up to step ks - 3*S is complete before any group reaches step ks
    // (the activation producer walks the steps in order), as long as S >= G.
    const uint32_t a_full = bar_base, st_empty = bar_base + 128u, st_empty_odd = bar_base + 64u, raw_full = bar_base + 192u,
                   raw_empty = bar_base + 256u, accum_bar = bar_base + 320u;
    uint32_t *tmem_slot = (uint32_t *)(smem_raw + (bar_base - raw_addr) + 336);
    volatile int *abort_flag = (volatile int *)(smem_raw + (bar_base - raw_addr) + 344);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) MCU_TRACE_POINT(3, 32, 0);
    const int f0 = blockIdx.x * p.rows_per_cta, t0 = blockIdx.y * BN;
    const int rows_here = min(p.rows_per_cta, p.F - f0);
    const bool grouped = p.group_counts != nullptr;
    // The group tables were written by kernels that finished before the kernel ahead of this one started (they do
    // not trigger their dependents early), so they may be read before griddepcontrol.wait.
    const int T_here = grouped ? p.group_counts[blockIdx.z] : p.T;
    const int row_off = grouped ? p.group_offsets[blockIdx.z] : 0;  // first activation / output row of the group
    const int w_row0 = (grouped ? (int)blockIdx.z * p.F : 0) + f0;  // first weight row in the (stacked) matrix
    if (t0 >= T_here) return;  // uniform over the CTA, before any barrier or tensor memory exists
    // this CTA's share of K: slabs [j0, j1), K steps [ks0, ks0 + nsteps)
    const int j0 = grouped ? 0 : (int)blockIdx.z * p.slabs_per_split;
    const int j1 = min((p.ksteps + RC::KR - 1) / RC::KR, j0 + p.slabs_per_split);
    const int ks0 = j0 * RC::KR;
    const int nsteps = min(p.ksteps, j1 * RC::KR) - ks0;

    __shared__ uint32_t epoch_s;
    __shared__ int last_s, peer_ok_s;
    if (threadIdx.x == 0) {
        last_s = 1;
        peer_ok_s = 1;
        for (int i = 0; i < S; ++i) {
            tm_mbar_init(a_full + 8u * i, GW + 1);  // a group's converter warps + the activation tile's expect_tx
            tm_mbar_init(st_empty + 8u * i, 1);
            tm_mbar_init(st_empty_odd + 8u * i, 1);
        }
        for (int i = 0; i < R; ++i) {
            tm_mbar_init(raw_full + 8u * i, 1);
            tm_mbar_init(raw_empty + 8u * i, TM_ALL_CONV);
        }
        tm_mbar_init(accum_bar, (uint32_t)p.issuers);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TM_ALL_CONV) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tm_smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) MCU_TRACE_POINT(3, 33, 0);
    // Programmatic dependent launch: the next kernel of the stream may start its own prologue now.  Here the packed
    // weights are taken to be final when the call is enqueued, so their stream starts at once; the activations,
    // the per-token scales and the output belong to earlier kernels until griddepcontrol.wait returns.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == TM_B_PRODUCER) {
        // ------------------------------ TMA producer: activation tiles ------------------------------
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            bool ok = true;
            int st = 0;
            uint32_t use = 0;  // ks / S
            for (int ks = 0; ks < nsteps && ok; ++ks) {  // ks: step index inside this CTA's share
                MCU_TRACE_POINT(2, ks, 0);
                if (use >= 1)  // release of the previous use of this stage
                    ok = tm_mbar_wait_relaxed((((use - 1) & 1u) ? st_empty_odd : st_empty) + 8u * st, ((use - 1) >> 1) & 1u);
                if (!ok) break;
                tm_mbar_expect_tx(a_full + 8u * st, (uint32_t)B_BYTES);
                tm_tma_load_2d(tile_base + (uint32_t)st * STAGE_BYTES + A_BYTES, &map_x, (ks0 + ks) * TM_BK, row_off + t0, a_full + 8u * st);
                MCU_TRACE_POINT(2, ks, 1);
                if (++st == S) {
                    st = 0;
                    ++use;
                }
            }
            if (!ok) {
                atomicExch(p.err, 6);
                *abort_flag = 1;
            }
        }
        __syncwarp();
    } else if (warp == TM_W_PRODUCER) {
        // ------------------------------ TMA producer: packed weight slabs ------------------------------
        // Runs ahead by the depth of the slab ring, independently of the MMA stages: this is the HBM stream.
        if (lane == 0) {
            bool ok = true;
            const uint32_t raw_bytes = (uint32_t)p.rows_per_cta * RC::BOX_W;
            int rs = 0;
            uint32_t phase = 1;  // parity of the previous use of the slab slot
            for (int j = j0; j < j1 && ok; ++j) {
                MCU_TRACE_POINT(3, j - j0, 0);
                if (j - j0 >= R) ok = tm_mbar_wait_relaxed(raw_empty + 8u * rs, phase);
                if (!ok) break;
                tm_mbar_expect_tx(raw_full + 8u * rs, raw_bytes);
                tm_tma_load_2d(raw_ring_addr + (uint32_t)rs * RAW_STAGE_BYTES, &map_w, (j * RC::UNIT) & ~15, w_row0,
                               raw_full + 8u * rs);
                MCU_TRACE_POINT(3, j - j0, 1);
                if (++rs == R) {
                    rs = 0;
                    phase ^= 1u;
                }
            }
            if (!ok) {
                atomicExch(p.err, 10);
                *abort_flag = 1;
            }
        }
        __syncwarp();
    } else if (warp >= TM_ALL_CONV) {
        // ------------------------------ MMA issuers ------------------------------
        // The whole warp runs the loop; one elected lane issues the MMAs and commits (always the same lane, so
        // tcgen05.commit covers every MMA of this issuer).
        const int issuer = warp - TM_ALL_CONV;
        if (issuer < p.issuers) {
            constexpr uint32_t idesc = tm_idesc(BN);
            bool ok = true;
            const uint64_t a_desc0 = tm_smem_desc(tile_base), b_desc0 = tm_smem_desc(tile_base + A_BYTES);
            constexpr uint64_t desc_step = (uint64_t)(STAGE_BYTES >> 4);
            const uint32_t tmem_acc = tmem_base + (uint32_t)(issuer * BN);
            int st = issuer % S;
            uint32_t use = (uint32_t)(issuer / S), acc = 0;
            const int nacc = p.issuers;
            for (int ks = issuer; ks < nsteps; ks += nacc) {
                if (lane == 0) MCU_TRACE_POINT(0, ks, 0);
                ok = tm_mbar_wait(a_full + 8u * st, use & 1u);  // weight tile converted and activation tile landed
                ok = __all_sync(0xffffffffu, ok);
                if (lane == 0) MCU_TRACE_POINT(0, ks, 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (tm_elect_one()) {
                    const uint64_t a_desc = a_desc0 + desc_step * (uint64_t)st, b_desc = b_desc0 + desc_step * (uint64_t)st;
                    tm_mma(tmem_acc, a_desc, b_desc, idesc, acc);
                    tm_mma(tmem_acc, a_desc + 2, b_desc + 2, idesc, 1u);  // +32 bytes along K inside the swizzle row
                    tm_mma(tmem_acc, a_desc + 4, b_desc + 4, idesc, 1u);
                    tm_mma(tmem_acc, a_desc + 6, b_desc + 6, idesc, 1u);
                    if constexpr (RT == 2) {  // the second row tile: next 16 KB of the stage, next BN columns of TMEM
                        constexpr uint64_t a2 = (uint64_t)(TM_A_BYTES >> 4);
                        tm_mma(tmem_acc + BN, a_desc + a2, b_desc, idesc, acc);
                        tm_mma(tmem_acc + BN, a_desc + a2 + 2, b_desc + 2, idesc, 1u);
                        tm_mma(tmem_acc + BN, a_desc + a2 + 4, b_desc + 4, idesc, 1u);
                        tm_mma(tmem_acc + BN, a_desc + a2 + 6, b_desc + 6, idesc, 1u);
                    }
                    MCU_TRACE_POINT(0, ks, 2);
                    tm_commit(((use & 1u) ? st_empty_odd : st_empty) + 8u * st);
                    MCU_TRACE_POINT(0, ks, 3);
                }
                __syncwarp();
                acc = 1u;
                st += nacc;
                while (st >= S) {
                    st -= S;
                    ++use;
                }
            }
            if (!ok && lane == 0) {
                atomicExch(p.err, 7);
                *abort_flag = 1;
            }
            __syncwarp();
            if (tm_elect_one()) tm_commit(accum_bar);  // arrives when every MMA this issuer issued has completed
        }
        __syncwarp();
    } else {
        // ------------------------------ converters ------------------------------
        // G groups of GW warps; group g converts the K steps with ks % G == g.
        const int group = warp / GW;
        const int gtid = threadIdx.x - group * (GW * 32);
        const int r = G == 4 ? gtid : gtid >> 1;  // weight row of this thread
        const int hc = gtid & 1;                  // G == 2: which half of the row's step
        const bool row_live = r < rows_here;
        bool ok = true;
        // Every warp visits every slab in order (wait for it, release it), and converts the K steps of its group
        // that fall into it: one code path, no per-step template copies (the instruction cache matters here).
        int rs = 0, st = group, ks = ks0 + group;  // ring positions of the slab and of this group's next K step
        uint32_t raw_phase = 0, use = 0;           // use = (ks - ks0) / S
        bool raw_ready = false;                    // answer of the early test for the slab about to be visited
        for (int j = j0; j < j1 && ok; ++j) {
            if (threadIdx.x == 0) MCU_TRACE_POINT(3, j - j0, 2);
            if (!raw_ready) ok = tm_mbar_wait_relaxed(raw_full + 8u * rs, raw_phase);
            if (threadIdx.x == 0) MCU_TRACE_POINT(3, j - j0, 3);
            if (!ok || *abort_flag) {
                if (!ok && lane == 0) atomicExch(p.err, 8);
                ok = false;
                break;
            }
            const uint8_t *rowp = raw_ring + (size_t)rs * RAW_STAGE_BYTES + (size_t)r * RC::BOX_W + ((j * RC::UNIT) & 15);
            for (; ks < (j + 1) * RC::KR && ks < ks0 + nsteps; ks += G) {
                const int kq = ks - j * RC::KR;
                if (gtid == 0) MCU_TRACE_POINT(1, ks - ks0, 0);
                // Has the MMA that read the previous contents of this stage completed?  Asked now, needed only
                // before the stores: the conversion in between hides the answer's latency.
                const uint32_t rel_bar = (((use - 1) & 1u) ? st_empty_odd : st_empty) + 8u * st;
                const uint32_t rel_parity = ((use - 1) >> 1) & 1u;
                const bool stage_free = use >= 1 ? tm_mbar_test(rel_bar, rel_parity) : true;
                uint8_t *a_row = tiles + (size_t)st * STAGE_BYTES + r * 128;
                if constexpr (G == 4) {
                    uint4 wv[8];
                    if (row_live) {
                        if constexpr (KIND == KIND_Q4_K) {
                            conv_q4k(rowp, kq, wv);
                        } else if constexpr (KIND == KIND_Q6_K) {
                            conv_q6k(rowp, kq, 0, wv);
                            conv_q6k(rowp, kq, 1, wv + 4);
                        } else {
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const int blk = 4 * j + 2 * kq + h;
                                if (blk < p.nb) conv_q8_0(rowp + (2 * kq + h) * Q8_0_BYTES, wv + 4 * h);
                                else wv[4 * h] = wv[4 * h + 1] = wv[4 * h + 2] = wv[4 * h + 3] = make_uint4(0, 0, 0, 0);
                            }
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < 8; ++c) wv[c] = make_uint4(0, 0, 0, 0);
                    }
                    if (!stage_free) ok = tm_mbar_wait_relaxed(rel_bar, rel_parity);
                    if (gtid == 0) MCU_TRACE_POINT(1, ks - ks0, 1);
                    if (ok) {
#pragma unroll
                        for (int c = 0; c < 8; ++c) *(uint4 *)(a_row + ((c ^ (r & 7)) << 4)) = wv[c];
                    }
                } else {
                    uint4 wv[4];
                    if (row_live) {
                        if constexpr (KIND == KIND_Q4_K) {
                            conv_q4k_half(rowp, kq, hc, wv);
                        } else if constexpr (KIND == KIND_Q6_K) {
                            conv_q6k(rowp, kq, hc, wv);
                        } else {
                            const int blk = 4 * j + 2 * kq + hc;
                            if (blk < p.nb) conv_q8_0(rowp + (2 * kq + hc) * Q8_0_BYTES, wv);
                            else wv[0] = wv[1] = wv[2] = wv[3] = make_uint4(0, 0, 0, 0);
                        }
                    } else {
                        wv[0] = wv[1] = wv[2] = wv[3] = make_uint4(0, 0, 0, 0);
                    }
                    if (!stage_free) ok = tm_mbar_wait_relaxed(rel_bar, rel_parity);
                    if (gtid == 0) MCU_TRACE_POINT(1, ks - ks0, 1);
                    if (ok) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) *(uint4 *)(a_row + (((4 * hc + c) ^ (r & 7)) << 4)) = wv[c];
                    }
                }
                if (!__all_sync(0xffffffffu, ok)) {  // a wait ran out: the stage was not written, nothing is signalled
                    ok = false;
                    if (lane == 0) atomicExch(p.err, 8);
                    break;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) tm_mbar_arrive(a_full + 8u * st);
                if (gtid == 0) MCU_TRACE_POINT(1, ks - ks0, 2);
                st += G;
                while (st >= S) {
                    st -= S;
                    ++use;
                }
            }
            if (!ok) break;
            const int released = rs;
            if (++rs == R) {
                rs = 0;
                raw_phase ^= 1u;
            }
            raw_ready = j + 1 < j1 ? tm_mbar_test(raw_full + 8u * rs, raw_phase) : false;  // asked early
            __syncwarp();
            if (lane == 0) tm_mbar_arrive(raw_empty + 8u * released);  // this warp no longer reads the slab
        }

        // ------------------------------ epilogue ------------------------------
        if (warp < 8) asm volatile("griddepcontrol.wait;" ::: "memory");
        // the epoch of this collective: only now is the previous kernel of the stream (which may have been the
        // previous collective) certain to have published its own
        if (threadIdx.x == 0 && p.fuse.world > 0) epoch_s = *(volatile uint32_t *)p.fuse.ctr + 1u;
        if (threadIdx.x == 0) MCU_TRACE_POINT(3, 34, 0);
        if (ok && warp < 8) ok = tm_mbar_wait_relaxed(accum_bar, 0);
        if (threadIdx.x == 0) MCU_TRACE_POINT(3, 35, 0);
        if (!ok && lane == 0) atomicExch(p.err, 9);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok && warp < 8 && !*abort_flag) {
            const int q = warp & 3;
            const int col0 = (warp >> 2) * (BN / 2);
#pragma unroll 1
            for (int rt = 0; rt < RT; ++rt) {
            const int fr = TM_BM * rt + 32 * q + lane;
            const int f = f0 + fr;
            const bool f_ok = fr < rows_here;
            const float bias = (p.bias != nullptr && f_ok) ? p.bias[f] : 0.0f;
            for (int cb = 0; cb < BN / 2; cb += 32) {
                if (t0 + col0 + cb >= T_here) break;  // warp-uniform: no tokens left in this column block
                float sum[32];
#pragma unroll
                for (int jj = 0; jj < 32; ++jj) sum[jj] = 0.0f;
                const int n_used = nsteps < p.issuers ? nsteps : p.issuers;  // accumulators that received a K step
#pragma unroll
                for (int a = 0; a < NACC; ++a) {
                    if (a >= n_used) break;  // warp-uniform
                    uint32_t v[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)((rt * NACC + a) * BN + col0 + cb);
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
                          "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
                          "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
                          "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                        : "r"(taddr)
                        : "memory");
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) sum[jj] += __uint_as_float(v[jj]);
                }
                if (f_ok) {
                    if (p.splits == 1 && p.fuse.world > 0) {
                        // partial result of this rank: into its own peer-visible staging buffer; bias comes later
                        float *mine = p.fuse.slots[p.fuse.rank];
#pragma unroll
                        for (int jj = 0; jj < 32; ++jj) {
                            const int t = t0 + col0 + cb + jj;
                            if (t < p.T) __stcg(mine + (size_t)t * p.F + f, sum[jj] * p.rowscale[t]);
                        }
                    } else if (p.splits == 1) {
#pragma unroll
                        for (int jj = 0; jj < 32; ++jj) {
                            const int t = t0 + col0 + cb + jj;
                            if (t < T_here)
                                p.out[(size_t)(row_off + t) * p.ldo + f] = sum[jj] * p.rowscale[row_off + t] + bias;
                        }
                    } else {
                        float *part = p.partial + (size_t)blockIdx.z * p.T * p.F;
#pragma unroll
                        for (int jj = 0; jj < 32; ++jj) {
                            const int t = t0 + col0 + cb + jj;
                            if (t < p.T) __stcg(part + (size_t)t * p.F + f, sum[jj]);
                        }
                    }
                }
            }
            }  // row tiles
        }
    }
    if (threadIdx.x == 0) MCU_TRACE_POINT(3, 36, 0);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    if (p.splits > 1) {
        // Last CTA of this tile to finish adds the partial tiles, in split order.
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            int *ctr = p.counters + blockIdx.y * gridDim.x + blockIdx.x;
            const int ticket = atomicAdd(ctr, 1);
            last_s = ticket == p.splits - 1;
            if (last_s) *ctr = 0;  // ready for the next launch
        }
        __syncthreads();
        if (threadIdx.x == 0) MCU_TRACE_POINT(3, 37, 0);
        if (last_s && !*abort_flag) {
            __threadfence();
            const int t_here = min(BN, p.T - t0);
            constexpr int MAXS = 16;  // plan_tma never asks for more splits
            if ((p.F & 3) == 0 && (rows_here & 3) == 0 && (p.ldo & 3) == 0 && p.splits <= MAXS) {
                // four features per thread and all splits' loads in flight at once: the tile is small, the reads are
                // L2 latency bound
                const int r4 = rows_here >> 2;
                for (int i = threadIdx.x; i < t_here * r4; i += blockDim.x) {
                    const int tt = i / r4, fr = (i - tt * r4) << 2;
                    const int t = t0 + tt, f = f0 + fr;
                    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                    for (int z0 = 0; z0 < MAXS; z0 += 8) {
                        if (z0 >= p.splits) break;
                        float4 v[8];
#pragma unroll
                        for (int z = 0; z < 8; ++z)
                            if (z0 + z < p.splits)
                                v[z] = __ldcg((const float4 *)(p.partial + ((size_t)(z0 + z) * p.T + t) * p.F + f));
#pragma unroll
                        for (int z = 0; z < 8; ++z)
                            if (z0 + z < p.splits) {
                                acc.x += v[z].x;
                                acc.y += v[z].y;
                                acc.z += v[z].z;
                                acc.w += v[z].w;
                            }
                    }
                    const float rsc = p.rowscale[t];
                    if (p.fuse.world > 0) {
                        __stcg((float4 *)(p.fuse.slots[p.fuse.rank] + (size_t)t * p.F + f),
                               make_float4(acc.x * rsc, acc.y * rsc, acc.z * rsc, acc.w * rsc));
                        continue;
                    }
                    float4 b = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (p.bias != nullptr) b = *(const float4 *)(p.bias + f);
                    *(float4 *)(p.out + (size_t)t * p.ldo + f) =
                        make_float4(acc.x * rsc + b.x, acc.y * rsc + b.y, acc.z * rsc + b.z, acc.w * rsc + b.w);
                }
            } else {
                for (int i = threadIdx.x; i < t_here * rows_here; i += blockDim.x) {
                    const int tt = i / rows_here, fr = i - tt * rows_here;
                    const int t = t0 + tt, f = f0 + fr;
                    float acc = 0.0f;
                    for (int z = 0; z < p.splits; ++z) acc += __ldcg(p.partial + ((size_t)z * p.T + t) * p.F + f);
                    p.out[(size_t)t * p.ldo + f] = acc * p.rowscale[t] + (p.bias != nullptr ? p.bias[f] : 0.0f);
                }
            }
        }
    }
    if (p.fuse.world > 0 && last_s) {
        // This CTA has written a finished tile of this rank's partial result to the rank's staging buffer.  Publish it
        // (one flag per rank and tile), wait for the same tile of the other ranks, pull their tiles over NVLink with
        // plain loads and add in rank order.  (last_s is CTA-uniform; with split K only the CTA that summed the
        // splits gets here.)
        const uint32_t epoch = epoch_s;
        const int tile = blockIdx.x;
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x < p.fuse.world) {
            if ((epoch & 1u) != p.fuse.parity_of_next) {
                atomicExch(p.err, 22);  // host and device disagree about the epoch: skip the exchange
                peer_ok_s = 0;
            } else {
                uint32_t *f = p.fuse.flags[threadIdx.x] + p.fuse.rank * PEER_FUSE_MAX_TILES + tile;
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
                const uint32_t *mine = p.fuse.flags[p.fuse.rank] + threadIdx.x * PEER_FUSE_MAX_TILES + tile;
                unsigned long long t_start, t_now;
                asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_start));
                for (;;) {
                    uint32_t v;
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
                    if ((int32_t)(v - epoch) >= 0) break;
                    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_now));
                    if (t_now - t_start > 2000000000ull) {  // a peer that never arrives: report, do not hang
                        atomicExch(p.err, 21);
                        peer_ok_s = 0;
                        break;
                    }
                    __nanosleep(100);
                }
            }
        }
        __syncthreads();
        if (peer_ok_s) {
            const int t_here = min(BN, p.T - t0);
            const int r4 = rows_here >> 2;  // fused launches use F % 4 == 0 and full-width tiles
            for (int i = threadIdx.x; i < t_here * r4; i += blockDim.x) {
                const int tt = i / r4, fr = (i - tt * r4) << 2;
                const int t = t0 + tt, f = f0 + fr;
                const size_t at = (size_t)t * p.F + f;
                float4 v[PEER_FUSE_MAX_WORLD];
#pragma unroll
                for (int r = 0; r < PEER_FUSE_MAX_WORLD; ++r)
                    if (r < p.fuse.world) v[r] = __ldcg((const float4 *)(p.fuse.slots[r] + at));  // all loads in flight
                float4 acc = v[0];
#pragma unroll
                for (int r = 1; r < PEER_FUSE_MAX_WORLD; ++r)
                    if (r < p.fuse.world) {
                        acc.x += v[r].x;
                        acc.y += v[r].y;
                        acc.z += v[r].z;
                        acc.w += v[r].w;
                    }
                float4 b = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (p.bias != nullptr) b = *(const float4 *)(p.bias + f);
                *(float4 *)(p.out + (size_t)t * p.ldo + f) = make_float4(acc.x + b.x, acc.y + b.y, acc.z + b.z, acc.w + b.w);
            }
        }
        // the last tile owner of the grid publishes the epoch for the next collective of this communicator
        if (threadIdx.x == 0) {
            __threadfence();
            if (atomicAdd(p.fuse.ctr + 1, 1u) == gridDim.x * gridDim.y - 1) {
                p.fuse.ctr[1] = 0;
                __threadfence();
                *(volatile uint32_t *)p.fuse.ctr = epoch;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) MCU_TRACE_POINT(3, 38, 0);
    if (*abort_flag) {
        // A wait ran out and the agents stopped early: bulk tensor copies may still be landing in this CTA's
        // shared memory.  Give them time to finish before the CTA (and its shared memory) goes away.
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == TM_ALL_CONV) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
static bool force_v1() {
    static const bool v = getenv("MARMOT_CUDA_GEMM_NO_TMA") != nullptr;
    return v;
}

// Tiling for few tokens (T <= 64), where the matmul is bound by the weight stream and by the latency of the K loop:
// full 128-row tiles when K can be split so that tiles x splits still fills the SMs (the serial K loop gets
// shorter), otherwise the rows spread evenly over the SMs.
struct TmaPlan {
    int rows_per_cta, splits, slabs_per_split;
};
static TmaPlan plan_tma(int kind, int T, int K, int F) {
    const int bv = block_values(kind), nb = (K + bv - 1) / bv;
    const int ksteps = (nb * bv + TM_BK - 1) / TM_BK;
    const int kr = kind == KIND_Q8_0 ? 2 : 4;
    const int n_slabs = (ksteps + kr - 1) / kr;
    TmaPlan pl{TM_BM, 1, n_slabs};
    const int sms = device_sm_count();
    // T > 64: full tiles (shorter tiles that would fill the last wave better finish no sooner: the MMA computes
    // M = 128 rows whatever the tile holds, and a converter warp takes as long for a half-empty tile).  With 256-token
    // tiles and enough work to fill most SMs a CTA takes two row tiles (see the kernel's RT parameter); Q6_K slabs are
    // too large for that.
    if (T > 64) {
        static const bool one_tile = getenv("MARMOT_CUDA_GEMM_ONE_ROW_TILE") != nullptr;  // diagnostic switch
        // Measured K-step times: about 1290 cycles with one row tile, 2250 with two (F = 14336, T = 512: 99 -> 90 us for
        // Q8_0, 83 -> 76 us for Q4_K); two tiles win when they save a wave (224 units on 148 SMs -> 112).
        const long t_tiles = (T + 255) / 256;
        const long waves2 = ((long)((F + 2 * TM_BM - 1) / (2 * TM_BM)) * t_tiles + sms - 1) / sms;
        const long waves1 = ((long)((F + TM_BM - 1) / TM_BM) * t_tiles + sms - 1) / sms;
        if (T > 128 && kind != KIND_Q6_K && !one_tile && waves2 * 175 < waves1 * 97) pl.rows_per_cta = 2 * TM_BM;
        return pl;
    }
    static const bool no_split = getenv("MARMOT_CUDA_GEMM_NO_SPLITK") != nullptr;  // diagnostic switch
    const int tiles = (F + TM_BM - 1) / TM_BM;
    int splits = no_split ? 1 : sms / tiles;
    if (splits > 16) splits = 16;
    if (splits >= 2 && n_slabs >= 2) {
        if (splits > n_slabs) splits = n_slabs;
        pl.slabs_per_split = (n_slabs + splits - 1) / splits;
        pl.splits = (n_slabs + pl.slabs_per_split - 1) / pl.slabs_per_split;
        if (pl.splits >= 2) return pl;
        pl.splits = 1;
        pl.slabs_per_split = n_slabs;
    }
    const int waves = (F + TM_BM * sms - 1) / (TM_BM * sms);  // passes over the SMs with full tiles
    int rows = (F + sms * waves - 1) / (sms * waves);
    rows = (rows + 7) / 8 * 8;
    if (rows > TM_BM) rows = TM_BM;
    if (rows < 8) rows = 8;
    pl.rows_per_cta = rows;
    return pl;
}

bool gemm_tma_can_fuse(int kind, int T, int F) {
    return kind_supported(kind) && T > GEMV_MAX_T && T <= 64 && F % 4 == 0 && (F + TM_BM - 1) / TM_BM <= PEER_FUSE_MAX_TILES;
}

size_t gemm_tma_workspace_bytes(int kind, int T, int K, int F) {
    const TmaPlan pl = plan_tma(kind, T, K, F);
    return pl.splits > 1 ? (size_t)pl.splits * T * F * sizeof(float) : 0;
}

bool gemm_tma_supported(int kind, const void *W, const void *W2, int T, int K, int F) {
    if (force_v1() || !kind_supported(kind) || T < 1 || F < 1 || K < 1) return false;
    if (((uintptr_t)W & 15) || ((uintptr_t)W2 & 15)) return false;
    const int bv = block_values(kind), nb = (K + bv - 1) / bv;
    const long row_bytes = (long)nb * block_bytes(kind);
    if (row_bytes % 16) return false;  // tensor-map row stride
    return encode_tiled_fn() != nullptr;
}

template <int KIND, int BN, int G, int RT = 1>
static cudaError_t launch_tma_bn(const void *W, const __half *xh, int ldxh, GemmTmaParams p, long row_bytes,
                                 cudaStream_t s, int groups = 0, int total_rows = 0) {
    using RC = RawCfg<KIND>;
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr) return cudaErrorNotSupported;
    alignas(64) CUtensorMap map_w, map_x;
    {
        const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)p.F * (cuuint64_t)(groups > 0 ? groups : 1)};
        const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
        const cuuint32_t box[2] = {(cuuint32_t)RC::BOX_W, (cuuint32_t)p.rows_per_cta};
        const cuuint32_t es[2] = {1, 1};
        if (enc(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(W), dims, strides, box, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    {
        const cuuint64_t dims[2] = {(cuuint64_t)ldxh, (cuuint64_t)(groups > 0 ? total_rows : p.T)};
        const cuuint64_t strides[1] = {(cuuint64_t)ldxh * 2};
        const cuuint32_t box[2] = {(cuuint32_t)TM_BK, (cuuint32_t)BN};
        const cuuint32_t es[2] = {1, 1};
        if (enc(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(xh), dims, strides, box, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    constexpr int stage_bytes = RT * TM_A_BYTES + BN * TM_BK * 2;
    const int raw_stage_bytes = (p.rows_per_cta * RC::BOX_W + 127) / 128 * 128 + 128;
    const int budget = 210 * 1024 - 2048;
    const int raw_slabs = p.slabs_per_split;
    // The slab ring carries the HBM stream (about 50 KB in flight per SM); the MMA stages get the rest.  The
    // stage ring is at least G deep (see TM_ALL_CONV) and is cut to a multiple of the issuer count: issuer i takes
    // the K steps ks = i (mod issuers) and with that always the same stages, so successive uses of one
    // full-barrier are waited on by one thread in order.  (A parity wait cannot tell "this phase" from "two
    // phases ago"; an issuer that got ahead of the thread owning the previous use of the stage would fall
    // through its wait.)
    int R = RT == 2 ? 2 : (BN <= 128 ? 4 : 3);  // two row tiles: two 64 KB stages and two 256-row slabs fill the SM
    if (R > raw_slabs) R = raw_slabs;
    int S = (budget - R * raw_stage_bytes) / stage_bytes;
    if (S < G + 2 && R > 3) {  // a ring deeper than G lets a group convert while its previous step is still in the MMA
        --R;
        S = (budget - R * raw_stage_bytes) / stage_bytes;
    }
    while (S < G && R > 1) {
        --R;
        S = (budget - R * raw_stage_bytes) / stage_bytes;
    }
    if (S < G) return cudaErrorInvalidConfiguration;
    if (S > TM_MAX_RING) S = TM_MAX_RING;
    constexpr int NACC = BN == 64 ? 4 : (BN == 128 ? 2 : 1);
    static const int issuer_cap = getenv("MARMOT_CUDA_GEMM_ISSUERS") ? atoi(getenv("MARMOT_CUDA_GEMM_ISSUERS")) : NACC;
    int max_issuers = NACC;
    if (issuer_cap >= 1 && max_issuers > issuer_cap) max_issuers = issuer_cap;
    int issuers = 1;  // the count that keeps most stages after rounding down (at least G); ties go to more issuers
    for (int i = 2; i <= max_issuers; ++i)
        if (S / i * i >= G && S / i * i >= S / issuers * issuers) issuers = i;
    S = S / issuers * issuers;
    p.raw_stage_bytes = raw_stage_bytes;
    p.issuers = issuers;
    p.stages = S;
    p.raw_stages = R;
    const int smem = 2048 + S * stage_bytes + R * raw_stage_bytes;
    static int configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tma_kernel<KIND, BN, G, RT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        configured = smem;
    }
    dim3 grid((unsigned)((p.F + p.rows_per_cta - 1) / p.rows_per_cta), (unsigned)((p.T + BN - 1) / BN), (unsigned)p.splits);
    if (groups > 0) grid = dim3(grid.x, (unsigned)((total_rows + BN - 1) / BN), (unsigned)groups);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(TM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const bool no_pdl = getenv("MARMOT_CUDA_NO_PDL") != nullptr;  // diagnostic switch
    cfg.numAttrs = no_pdl ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, gemm_tma_kernel<KIND, BN, G, RT>, map_w, map_x, p);
}

template <int KIND>
static cudaError_t launch_tma_kind(const void *W, const __half *xh, int ldxh, const GemmTmaParams &p, long row_bytes,
                                   cudaStream_t s) {
    if (p.T <= 64) return launch_tma_bn<KIND, 64, 4>(W, xh, ldxh, p, row_bytes, s);
    if (p.T <= 128) return launch_tma_bn<KIND, 128, 4>(W, xh, ldxh, p, row_bytes, s);
    if constexpr (KIND != KIND_Q6_K)
        if (p.rows_per_cta == 2 * TM_BM) return launch_tma_bn<KIND, 256, 1, 2>(W, xh, ldxh, p, row_bytes, s);
    return launch_tma_bn<KIND, 256, 2>(W, xh, ldxh, p, row_bytes, s);
}

#ifdef MCU_TRACE
long long *g_trace_buf = nullptr;
extern "C" long long *mcu_debug_trace_buffer() { return g_trace_buf; }
#endif

cudaError_t launch_gemm_tma(int kind, const void *W, const void *W2, const __half *xh, const float *rowscale, int ldxh,
                            int T, int K, int F, const float *bias, float *out, float *out2, int ldo, float *partial,
                            int *counters, int *err_flag, cudaStream_t s, int *launches, const PeerFuse *fuse) {
    GemmTmaParams p;
    p.bias = bias;
    p.rowscale = rowscale;
    p.err = err_flag;
    p.ldo = ldo;
    p.T = T;
    p.F = F;
    const int bv = block_values(kind);
    p.nb = (K + bv - 1) / bv;
    p.ksteps = (p.nb * bv + TM_BK - 1) / TM_BK;
    const long row_bytes = (long)p.nb * block_bytes(kind);
    TmaPlan pl = plan_tma(kind, T, K, F);
    memset(&p.fuse, 0, sizeof(p.fuse));
    p.group_counts = p.group_offsets = nullptr;
    if (fuse != nullptr && fuse->world > 0) {
        if (!gemm_tma_can_fuse(kind, T, F) || W2 != nullptr || ldo != F || (size_t)T * F > fuse->slot_floats)
            return cudaErrorInvalidValue;
        pl.rows_per_cta = TM_BM;  // tiles must be the same on every rank, whatever its share of K
        p.fuse = *fuse;
    }
    p.rows_per_cta = pl.rows_per_cta;
    p.splits = pl.splits;
    p.slabs_per_split = pl.slabs_per_split;
    p.partial = partial;
    p.counters = counters;
    if (p.splits > 1 && (partial == nullptr || counters == nullptr || (F + TM_BM - 1) / TM_BM > GEMM_TMA_MAX_TILE_COUNTERS))
        return cudaErrorInvalidValue;
    p.stages = p.raw_stages = p.issuers = p.raw_stage_bytes = 0;
#ifdef MCU_TRACE
    {
        static long long *trace_buf = nullptr;
        if (trace_buf == nullptr) cudaMalloc(&trace_buf, 4 * 64 * 4 * sizeof(long long));
        cudaMemsetAsync(trace_buf, 0, 4 * 64 * 4 * sizeof(long long), s);
        p.trace = trace_buf;
        g_trace_buf = trace_buf;
    }
#endif
    int n = 0;
    for (int pass = 0; pass < (W2 != nullptr ? 2 : 1); ++pass) {
        const void *w = pass == 0 ? W : W2;
        p.out = pass == 0 ? out : out2;
        cudaError_t e = kind == KIND_Q4_K ? launch_tma_kind<KIND_Q4_K>(w, xh, ldxh, p, row_bytes, s)
            : kind == KIND_Q6_K           ? launch_tma_kind<KIND_Q6_K>(w, xh, ldxh, p, row_bytes, s)
                                          : launch_tma_kind<KIND_Q8_0>(w, xh, ldxh, p, row_bytes, s);
        if (e != cudaSuccess) return e;
        ++n;
    }
    if (launches != nullptr) *launches = n;
    return cudaSuccess;
}

bool gemm_tma_grouped_supported(int kind, const void *W, int K, int F) {
    return gemm_tma_supported(kind, W, nullptr, 256, K, F);
}

// n_groups matmuls in one launch: group g multiplies its group_counts[g] rows of xh (from row group_offsets[g]) with the
// weight rows [g * F, (g + 1) * F) of the stacked matrix W.  The 256-token tile configuration is used whatever the
// counts turn out to be (they are device data): meant for batches with many rows per group.
cudaError_t launch_gemm_tma_grouped(int kind, const void *W, int n_groups, const __half *xh, const float *rowscale,
                                    int ldxh, int total_rows, int K, int F, const int *group_counts,
                                    const int *group_offsets, float *out, int ldo, int *err_flag, cudaStream_t s) {
    if (n_groups <= 0 || total_rows <= 0) return cudaSuccess;
    if (n_groups > 65535 || (total_rows + 255) / 256 > 65535) return cudaErrorInvalidValue;
    GemmTmaParams p;
    memset(&p, 0, sizeof(p));
    p.rowscale = rowscale;
    p.out = out;
    p.err = err_flag;
    p.ldo = ldo;
    p.T = total_rows;
    p.F = F;
    const int bv = block_values(kind);
    p.nb = (K + bv - 1) / bv;
    p.ksteps = (p.nb * bv + TM_BK - 1) / TM_BK;
    const long row_bytes = (long)p.nb * block_bytes(kind);
    p.splits = 1;
    p.slabs_per_split = (p.ksteps + (kind == KIND_Q8_0 ? 2 : 4) - 1) / (kind == KIND_Q8_0 ? 2 : 4);
    p.group_counts = group_counts;
    p.group_offsets = group_offsets;
    static const bool one_tile = getenv("MARMOT_CUDA_GEMM_ONE_ROW_TILE") != nullptr;  // diagnostic switch
    const bool two = kind != KIND_Q6_K && !one_tile && F % (2 * TM_BM) == 0;
    p.rows_per_cta = two ? 2 * TM_BM : TM_BM;
    if (kind == KIND_Q4_K)
        return two ? launch_tma_bn<KIND_Q4_K, 256, 1, 2>(W, xh, ldxh, p, row_bytes, s, n_groups, total_rows)
                   : launch_tma_bn<KIND_Q4_K, 256, 2>(W, xh, ldxh, p, row_bytes, s, n_groups, total_rows);
    if (kind == KIND_Q8_0)
        return two ? launch_tma_bn<KIND_Q8_0, 256, 1, 2>(W, xh, ldxh, p, row_bytes, s, n_groups, total_rows)
                   : launch_tma_bn<KIND_Q8_0, 256, 2>(W, xh, ldxh, p, row_bytes, s, n_groups, total_rows);
    return launch_tma_bn<KIND_Q6_K, 256, 2>(W, xh, ldxh, p, row_bytes, s, n_groups, total_rows);
}

}  // namespace mcu
