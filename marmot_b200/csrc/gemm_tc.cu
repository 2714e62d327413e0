// Prefill / batched-decode quantized matmul on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   out[t][f] = sum_k xh[t][k] * fp16(dequant(W)[f][k])          (f32 accumulation in tensor memory)
//
// xh is the fp16 value d*q of the exactly emulated activation quantizer (act_quant.cu), so the only
// deviation from the reference's integer path is the fp16 rounding of the two operands (~2^-12
// relative each); fp16 rather than bf16 keeps the result within ~1e-3 of the reference.
//
// One CTA computes a 128-feature x BN-token tile.  Warp roles:
//   warps 0..7  producers: dequantise a 128 x 64 weight tile to fp16 and copy a BN x 64 activation
//               tile into shared memory in the canonical K-major SWIZZLE_128B layout (16-byte chunk
//               c of row r at r*128 + ((c ^ (r & 7)) * 16)), fence to the async proxy, arrive on
//               full[stage].  Global loads of step s+1 are issued before step s is converted.
//               After the K loop the same warps run the epilogue: tcgen05.ld of the accumulator
//               (lane = feature, column = token) and coalesced f32 stores (+ bias).
//   warp 8      one elected lane issues tcgen05.mma (M=128, N=BN, K=16, kind::f16) four times per
//               stage and tcgen05.commit to release the stage / publish the accumulator; the warp
//               also owns the TMEM allocation.
// Every mbarrier wait is bounded; a timeout sets *err and the CTA drains and returns (TMEM is still
// released).
#include "common.cuh"
#include "kernels.h"

namespace mcu {

constexpr int TC_BM = 128;      // features per CTA (MMA M)
constexpr int TC_BK = 64;       // K values per stage: one 128-byte swizzle row of fp16
constexpr int TC_PRODUCERS = 8; // producer / epilogue warps
constexpr int TC_THREADS = (TC_PRODUCERS + 1) * 32;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;  // 16 KiB
constexpr uint32_t TC_SPIN_LIMIT = 1u << 22;

struct GemmTcParams {
    const uint8_t *W;
    const __half *xh;
    const float *bias;
    const float *rowscale;  // per-token power-of-two factor undone in the epilogue
    float *out;
    int *err;
    int ldxh, ldo, T, K, F, nb;
    int ksteps;  // ceil(K / 64)
    int stages;
};

__device__ __forceinline__ uint32_t tc_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tc_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void tc_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool tc_mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool tc_mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i)
        if (tc_mbar_try_wait(bar, parity)) return true;
    return false;
}

// Shared-memory matrix descriptor: K-major, SWIZZLE_128B, rows of 128 bytes, 8-row groups 1024 bytes
// apart (stride byte offset), leading byte offset 16 (unused for swizzled K-major), version 1.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor for kind::f16: f16 A and B (K-major), f32 accumulator, M = 128, N = BN.
__host__ __device__ constexpr uint32_t tc_idesc(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}

__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *(const uint32_t *)&h;
}
// byte `idx` (0..3) of w as an exact float: 2^23 + byte, then minus 2^23
__device__ __forceinline__ float byte_to_float(uint32_t w, int idx) {
    return __int_as_float((int)__byte_perm(w, 0x4B000000u, 0x7650 | idx << 0 | 0x0000)) - 8388608.0f;
}

// store eight fp16 (16 bytes) as chunk c of row r of a swizzled tile
__device__ __forceinline__ void st_chunk(uint8_t *tile, int r, int c, uint4 v) {
    *(uint4 *)(tile + r * 128 + ((c ^ (r & 7)) << 4)) = v;
}

// ---------------------------------------------------------------------------------------------
// Weight tile producers: thread (r = row 0..127, h = half 0/1) produces 32 consecutive K values
// [64*kstep + 32*h, +32) of row r.  `Raw` holds the global loads of one step.
// ---------------------------------------------------------------------------------------------
struct RawQ4K {
    uint4 hdr, q0, q1;
};
__device__ __forceinline__ void load_q4k(const uint8_t *W, int nb, int row, bool valid, int kstep, RawQ4K &raw) {
    raw.hdr = raw.q0 = raw.q1 = make_uint4(0, 0, 0, 0);
    if (!valid) return;
    const uint4 *bp = (const uint4 *)(W + ((size_t)row * nb + (kstep >> 2)) * Q4_K_BYTES);
    raw.hdr = __ldg(bp);
    raw.q0 = __ldg(bp + 1 + 2 * (kstep & 3));
    raw.q1 = __ldg(bp + 2 + 2 * (kstep & 3));
}
__device__ __forceinline__ void convert_q4k(const RawQ4K &raw, int kstep, int h, uint4 (&outv)[4]) {
    const int sb = 2 * (kstep & 3) + h;  // sub-block: low nibbles -> 2g, high nibbles -> 2g+1
    int sc, mn;
    k4_scale_min_w(sb, raw.hdr.y, raw.hdr.z, raw.hdr.w, sc, mn);
    const float d = half_bits_to_float((uint16_t)(raw.hdr.x & 0xFFFFu));
    const float dmin = half_bits_to_float((uint16_t)(raw.hdr.x >> 16));
    const float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(dmin, (float)mn);
    const uint32_t w[8] = {raw.q0.x, raw.q0.y, raw.q0.z, raw.q0.w, raw.q1.x, raw.q1.y, raw.q1.z, raw.q1.w};
    uint32_t o[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t nib = (w[j] >> (4 * h)) & 0x0F0F0F0Fu;
        const float v0 = __fsub_rn(__fmul_rn(d1, byte_to_float(nib, 0)), m1);
        const float v1 = __fsub_rn(__fmul_rn(d1, byte_to_float(nib, 1)), m1);
        const float v2 = __fsub_rn(__fmul_rn(d1, byte_to_float(nib, 2)), m1);
        const float v3 = __fsub_rn(__fmul_rn(d1, byte_to_float(nib, 3)), m1);
        o[2 * j] = pack_half2(v0, v1);
        o[2 * j + 1] = pack_half2(v2, v3);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) outv[c] = make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
}

// nine aligned words covering 36 bytes that start at a 2-byte aligned address
__device__ __forceinline__ void ldg_words9(const uint8_t *p, uint32_t (&w)[9], uint32_t &sh) {
    const uintptr_t a = (uintptr_t)p;
    const uint32_t *al = (const uint32_t *)(a & ~(uintptr_t)3);
    sh = (uint32_t)(a & 3) * 8;
#pragma unroll
    for (int i = 0; i < 9; ++i) w[i] = __ldg(al + i);
}

struct RawQ8_0 {
    uint32_t w[9];
    uint32_t sh;
    bool valid;
};
__device__ __forceinline__ void load_q8_0(const uint8_t *W, int nb, int row, bool valid, int kstep, int h, RawQ8_0 &raw) {
    const int blk = 2 * kstep + h;
    raw.valid = valid && blk < nb;
    raw.sh = 0;
#pragma unroll
    for (int i = 0; i < 9; ++i) raw.w[i] = 0;
    if (!raw.valid) return;
    const uint8_t *bp = W + ((size_t)row * nb + blk) * Q8_0_BYTES;
    // block = [bp, bp+34).  Aligned start (sh = 0): words 0..7 + the two bytes 32,33; otherwise the block
    // starts in the upper half of word 0 and ends exactly at the end of word 8.
    const uintptr_t a = (uintptr_t)bp;
    const uint32_t *al = (const uint32_t *)(a & ~(uintptr_t)3);
    raw.sh = (uint32_t)(a & 3) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) raw.w[i] = __ldg(al + i);
    raw.w[8] = raw.sh == 0 ? (uint32_t)__ldg((const uint16_t *)(bp + 32)) : __ldg(al + 8);
}
__device__ __forceinline__ void convert_q8_0(const RawQ8_0 &raw, uint4 (&outv)[4]) {
    uint32_t q[8];
    float d;
    if (raw.sh == 0) {
        d = half_bits_to_float((uint16_t)(raw.w[0] & 0xFFFFu));
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = __funnelshift_r(raw.w[i], raw.w[i + 1], 16);
    } else {
        d = half_bits_to_float((uint16_t)(raw.w[0] >> 16));
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = raw.w[i + 1];
    }
    if (!raw.valid) d = 0.0f;
    uint32_t o[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t u = q[j] ^ 0x80808080u;  // int8 + 128 as unsigned bytes
        const float v0 = __fmul_rn(byte_to_float(u, 0) - 128.0f, d);
        const float v1 = __fmul_rn(byte_to_float(u, 1) - 128.0f, d);
        const float v2 = __fmul_rn(byte_to_float(u, 2) - 128.0f, d);
        const float v3 = __fmul_rn(byte_to_float(u, 3) - 128.0f, d);
        o[2 * j] = pack_half2(v0, v1);
        o[2 * j + 1] = pack_half2(v2, v3);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) outv[c] = make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
}

struct RawQ6K {
    uint32_t ql[9], qh[9];
    uint32_t sh_l, sh_h;
    uint32_t sc2;  // the two int8 scales of this thread's 32 values
    uint32_t dbits;
};
__device__ __forceinline__ void load_q6k(const uint8_t *W, int nb, int row, bool valid, int kstep, int h, RawQ6K &raw) {
#pragma unroll
    for (int i = 0; i < 9; ++i) raw.ql[i] = raw.qh[i] = 0;
    raw.sh_l = raw.sh_h = raw.sc2 = raw.dbits = 0;
    if (!valid) return;
    const uint8_t *bp = W + ((size_t)row * nb + (kstep >> 2)) * Q6_K_BYTES;
    const int qk = kstep & 3, n = qk >> 1, c = 2 * (qk & 1) + h;  // values 128n + 32c + l, l = 0..31
    ldg_words9(bp + n * 64 + (c & 1) * 32, raw.ql, raw.sh_l);
    ldg_words9(bp + 128 + n * 32, raw.qh, raw.sh_h);
    raw.sc2 = (uint32_t)__ldg((const uint16_t *)(bp + 192 + n * 8 + 2 * c));
    raw.dbits = (uint32_t)__ldg((const uint16_t *)(bp + 208));
}
__device__ __forceinline__ void convert_q6k(const RawQ6K &raw, int kstep, int h, uint4 (&outv)[4]) {
    const int c = 2 * (kstep & 1) + h;
    const float d = half_bits_to_float((uint16_t)raw.dbits);
    const float ds0 = __fmul_rn(d, (float)(int8_t)(raw.sc2 & 0xFFu));
    const float ds1 = __fmul_rn(d, (float)(int8_t)((raw.sc2 >> 8) & 0xFFu));
    uint32_t o[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t ql = raw.sh_l ? __funnelshift_r(raw.ql[j], raw.ql[j + 1], 16) : raw.ql[j];
        const uint32_t qh = raw.sh_h ? __funnelshift_r(raw.qh[j], raw.qh[j + 1], 16) : raw.qh[j];
        const uint32_t lo4 = (c & 2) ? ((ql >> 4) & 0x0F0F0F0Fu) : (ql & 0x0F0F0F0Fu);
        const uint32_t u = lo4 | (((qh >> (2 * c)) & 0x03030303u) << 4);  // 0..63 per byte, value = u - 32
        const float ds = j < 4 ? ds0 : ds1;
        const float v0 = __fmul_rn(ds, byte_to_float(u, 0) - 32.0f);
        const float v1 = __fmul_rn(ds, byte_to_float(u, 1) - 32.0f);
        const float v2 = __fmul_rn(ds, byte_to_float(u, 2) - 32.0f);
        const float v3 = __fmul_rn(ds, byte_to_float(u, 3) - 32.0f);
        o[2 * j] = pack_half2(v0, v1);
        o[2 * j + 1] = pack_half2(v2, v3);
    }
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) outv[cc] = make_uint4(o[4 * cc], o[4 * cc + 1], o[4 * cc + 2], o[4 * cc + 3]);
}

template <int KIND>
struct RawOf;
template <>
struct RawOf<KIND_Q4_K> { using type = RawQ4K; };
template <>
struct RawOf<KIND_Q6_K> { using type = RawQ6K; };
template <>
struct RawOf<KIND_Q8_0> { using type = RawQ8_0; };

template <int KIND>
__device__ __forceinline__ void load_w(const uint8_t *W, int nb, int row, bool valid, int kstep, int h,
                                       typename RawOf<KIND>::type &raw) {
    if constexpr (KIND == KIND_Q4_K) load_q4k(W, nb, row, valid, kstep, raw);
    else if constexpr (KIND == KIND_Q6_K) load_q6k(W, nb, row, valid, kstep, h, raw);
    else load_q8_0(W, nb, row, valid, kstep, h, raw);
}
template <int KIND>
__device__ __forceinline__ void convert_w(const typename RawOf<KIND>::type &raw, int kstep, int h, uint4 (&outv)[4]) {
    if constexpr (KIND == KIND_Q4_K) convert_q4k(raw, kstep, h, outv);
    else if constexpr (KIND == KIND_Q6_K) convert_q6k(raw, kstep, h, outv);
    else convert_q8_0(raw, outv);
}

// ---------------------------------------------------------------------------------------------
// Kernel
// ---------------------------------------------------------------------------------------------
template <int KIND, int BN>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const GemmTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    constexpr int B_BYTES = BN * TC_BK * 2;
    constexpr int STAGE_BYTES = TC_A_BYTES + B_BYTES;
    constexpr int ACT_CHUNKS = BN * 8 / (TC_PRODUCERS * 32);  // 16-byte chunks of the activation tile per thread
    static_assert(ACT_CHUNKS >= 1, "BN too small for the producer count");

    // barriers first, tiles at the next 1024-byte boundary (SWIZZLE_128B atoms are 1024-byte aligned)
    const uint32_t raw_addr = tc_smem_u32(smem_raw);
    const uint32_t bar_base = (raw_addr + 7u) & ~7u;
    const uint32_t tile_base = (bar_base + 256u + 1023u) & ~1023u;
    uint8_t *tiles = smem_raw + (tile_base - raw_addr);
    const int S = p.stages;
    const uint32_t full0 = bar_base, empty0 = bar_base + 8u * 8u, accum_bar = bar_base + 8u * 16u;
    uint32_t *tmem_slot = (uint32_t *)(smem_raw + (bar_base - raw_addr) + 8 * 17);
    volatile int *abort_flag = (volatile int *)(smem_raw + (bar_base - raw_addr) + 8 * 17 + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f0 = blockIdx.x * TC_BM, t0 = blockIdx.y * BN;

    if (threadIdx.x == 0) {
        for (int i = 0; i < S; ++i) {
            tc_mbar_init(full0 + 8u * i, TC_PRODUCERS);
            tc_mbar_init(empty0 + 8u * i, 1);
        }
        tc_mbar_init(accum_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TC_PRODUCERS) {
        // TMEM: BN columns of 128 lanes x 32 bit
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(tmem_slot)),
                     "r"((uint32_t)BN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == TC_PRODUCERS) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = tc_idesc(BN);
            bool ok = true;
            for (int ks = 0; ks < p.ksteps && ok; ++ks) {
                const int st = ks % S, round = ks / S;
                ok = tc_mbar_wait(full0 + 8u * st, (uint32_t)(round & 1));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = tile_base + (uint32_t)st * STAGE_BYTES;
                const uint32_t b_addr = a_addr + TC_A_BYTES;
                const uint64_t a_desc = tc_smem_desc(a_addr), b_desc = tc_smem_desc(b_addr);
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k) {
                    // 16 fp16 = 32 bytes further along K inside the 128-byte swizzle row: +2 in the address field
                    tc_mma(tmem_base, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc,
                           (ks > 0 || k > 0) ? 1u : 0u);
                }
                tc_commit(empty0 + 8u * st);  // the stage may be overwritten once these MMAs have read it
            }
            if (!ok) {
                atomicExch(p.err, 3);
                *abort_flag = 1;
            }
            tc_commit(accum_bar);  // arrives when every MMA issued so far has completed
        }
        __syncwarp();
    } else {
        // ------------------------------ producers ------------------------------
        const int tid = threadIdx.x;            // 0..255
        const int r = tid >> 1, h = tid & 1;    // weight row inside the tile, 32-value half of the K step
        const int row = f0 + r;
        const bool row_ok = row < p.F;
        typename RawOf<KIND>::type raw;
        uint4 act[ACT_CHUNKS];
        auto load_act = [&](int ks) {
#pragma unroll
            for (int i = 0; i < ACT_CHUNKS; ++i) {
                const int ch = tid + i * (TC_PRODUCERS * 32);  // chunk index: row = ch / 8, chunk = ch % 8
                const int t = t0 + (ch >> 3);
                // rows past T and chunks past the padded row length (odd Q8_0 block counts) are zero
                const bool in_range = t < p.T && ks * TC_BK + (ch & 7) * 8 < p.ldxh;
                act[i] = in_range ? __ldg((const uint4 *)(p.xh + (size_t)t * p.ldxh + (size_t)ks * TC_BK) + (ch & 7))
                                  : make_uint4(0, 0, 0, 0);
            }
        };
        load_w<KIND>(p.W, p.nb, row, row_ok, 0, h, raw);
        load_act(0);
        bool ok = true;
        for (int ks = 0; ks < p.ksteps; ++ks) {
            const int st = ks % S, round = ks / S;
            // convert the step in registers, then prefetch the next one before waiting for the stage
            uint4 wv[4];
            convert_w<KIND>(raw, ks, h, wv);
            uint4 av[ACT_CHUNKS];
#pragma unroll
            for (int i = 0; i < ACT_CHUNKS; ++i) av[i] = act[i];
            if (ks + 1 < p.ksteps) {
                load_w<KIND>(p.W, p.nb, row, row_ok, ks + 1, h, raw);
                load_act(ks + 1);
            }
            if (round > 0) {
                ok = tc_mbar_wait(empty0 + 8u * st, (uint32_t)((round - 1) & 1));
                if (!ok || *abort_flag) {
                    if (!ok && lane == 0) atomicExch(p.err, 4);
                    ok = false;
                    break;
                }
            }
            uint8_t *a_tile = tiles + (size_t)st * STAGE_BYTES;
            uint8_t *b_tile = a_tile + TC_A_BYTES;
#pragma unroll
            for (int c = 0; c < 4; ++c) st_chunk(a_tile, r, 4 * h + c, wv[c]);
#pragma unroll
            for (int i = 0; i < ACT_CHUNKS; ++i) {
                const int ch = tid + i * (TC_PRODUCERS * 32);
                st_chunk(b_tile, ch >> 3, ch & 7, av[i]);
            }
            // make the generic-proxy stores visible to the tensor core's async-proxy reads
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(full0 + 8u * st);
        }

        // ------------------------------ epilogue ------------------------------
        if (ok) ok = tc_mbar_wait(accum_bar, 0);
        if (!ok && lane == 0) atomicExch(p.err, 5);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok && !*abort_flag) {
            const int q = warp & 3;                      // TMEM lane quarter this warp may read
            const int col0 = (warp >> 2) * (BN / 2);     // warps w and w+4 split the columns
            const int f = f0 + 32 * q + lane;
            const float bias = (p.bias != nullptr && f < p.F) ? p.bias[f] : 0.0f;
            for (int cb = 0; cb < BN / 2; cb += 32) {
                uint32_t v[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(col0 + cb);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                      "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]),
                      "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]),
                      "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (f < p.F) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int t = t0 + col0 + cb + j;
                        if (t < p.T) p.out[(size_t)t * p.ldo + f] = __uint_as_float(v[j]) * p.rowscale[t] + bias;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == TC_PRODUCERS) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
bool gemm_tc_supported(int kind, int T, int K, int F) {
    if (!kind_supported(kind) || T < 1 || F < 1 || K < 1) return false;
    return true;
}

template <int KIND, int BN>
static cudaError_t launch_bn(const GemmTcParams &p0, cudaStream_t s) {
    GemmTcParams p = p0;
    constexpr int stage_bytes = TC_A_BYTES + BN * TC_BK * 2;
    int stages = (200 * 1024) / stage_bytes;
    if (stages > 8) stages = 8;
    if (stages > p.ksteps) stages = p.ksteps < 2 ? 2 : p.ksteps;
    p.stages = stages;
    const int smem = 256 + 8 + 1024 + stages * stage_bytes;
    static int configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<KIND, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        configured = smem;
    }
    dim3 grid((unsigned)((p.F + TC_BM - 1) / TC_BM), (unsigned)((p.T + BN - 1) / BN), 1);
    gemm_tc_kernel<KIND, BN><<<grid, TC_THREADS, smem, s>>>(p);
    return cudaGetLastError();
}

template <int KIND>
static cudaError_t launch_kind(const GemmTcParams &p, cudaStream_t s) {
    if (p.T <= 64) return launch_bn<KIND, 64>(p, s);
    if (p.T <= 128) return launch_bn<KIND, 128>(p, s);
    return launch_bn<KIND, 256>(p, s);
}

cudaError_t launch_gemm_tc(int kind, const void *W, const void *W2, const __half *xh, const float *rowscale, int ldxh,
                           int T, int K, int F, const float *bias, float *out, float *out2, int ldo, int *err_flag,
                           cudaStream_t s, int *launches) {
    GemmTcParams p;
    p.xh = xh;
    p.bias = bias;
    p.rowscale = rowscale;
    p.err = err_flag;
    p.ldxh = ldxh;
    p.ldo = ldo;
    p.T = T;
    p.K = K;
    p.F = F;
    const int bv = block_values(kind);
    p.nb = (K + bv - 1) / bv;
    p.ksteps = (p.nb * bv + TC_BK - 1) / TC_BK;
    p.stages = 0;
    int n = 0;
    for (int pass = 0; pass < (W2 != nullptr ? 2 : 1); ++pass) {
        p.W = (const uint8_t *)(pass == 0 ? W : W2);
        p.out = pass == 0 ? out : out2;
        cudaError_t e = kind == KIND_Q4_K ? launch_kind<KIND_Q4_K>(p, s)
            : kind == KIND_Q6_K           ? launch_kind<KIND_Q6_K>(p, s)
                                          : launch_kind<KIND_Q8_0>(p, s);
        if (e != cudaSuccess) return e;
        ++n;
    }
    if (launches != nullptr) *launches = n;
    return cudaSuccess;
}

}  // namespace mcu
