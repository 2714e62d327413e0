// Device-side helpers shared by the TMA-fed matmul kernels: mbarrier and bulk-tensor-copy wrappers (every wait
// bounded), tcgen05 wrappers, packed-half conversion helpers, and the host-side tensor-map encoder lookup.
#pragma once

#include "common.cuh"

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <mutex>

namespace mcu {

constexpr int TM_BM = 128;  // rows of a tcgen05 weight tile (used by the instruction descriptor below)
constexpr uint32_t TM_SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t tm_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tm_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void tm_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tm_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait on an mbarrier phase.  try_wait suspends the thread in hardware for a short, system-chosen time and
// returns early when the phase completes, so a waiting warp executes few instructions; TM_SPIN_LIMIT tries
// bound the whole wait, after which the caller records an error and winds down.
__device__ __forceinline__ bool tm_mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < TM_SPIN_LIMIT; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
        __nanosleep(32);  // a failed try costs issue slots the dequantising warps need
    }
    return false;
}
__device__ __forceinline__ bool tm_mbar_wait_relaxed(uint32_t bar, uint32_t parity) { return tm_mbar_wait(bar, parity); }
// Non-blocking test, issued ahead of the work that hides its latency; a negative answer is followed by a real wait.
__device__ __forceinline__ bool tm_mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// 2-D tiled tensor load, completion counted in bytes on an mbarrier of this CTA (no multicast).
__device__ __forceinline__ void tm_tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}
__device__ __forceinline__ uint64_t tm_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__host__ __device__ constexpr uint32_t tm_idesc(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TM_BM >> 4) << 24);
}
__device__ __forceinline__ void tm_mma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void tm_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// N words from a 2-byte aligned shared-memory address (reads one aligned word beyond the last).
template <int N>
__device__ __forceinline__ void tm_lds_words(const uint8_t *p, uint32_t (&out)[N]) {
    const uint32_t a = tm_smem_u32(p);
    const uint32_t *w = (const uint32_t *)(p - (a & 3u));
    const uint32_t sh = (a & 3u) * 8u;
    uint32_t prev = w[0];
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const uint32_t next = w[i + 1];
        out[i] = __funnelshift_r(prev, next, sh);
        prev = next;
    }
}

__device__ __forceinline__ __half2 as_half2(uint32_t v) { return *(const __half2 *)&v; }
__device__ __forceinline__ uint32_t as_u32(__half2 v) { return *(const uint32_t *)&v; }

// The fp16 tiles hold every group of four consecutive K values in the order (0, 2, 1, 3): the two 16-bit lanes of
// a 32-bit word then come from bytes (0, 2) and (1, 3) of a packed word, which is what mask-and-or extraction
// yields without shuffling bytes.  The activation rows are written in the same order (half_acts_kernel).

// Four unsigned bytes (each < 256) -> two half2 holding byte - offset: bytes (0, 2) and bytes (1, 3).
__device__ __forceinline__ void bytes_to_half2(uint32_t w, __half2 offset, __half2 &v02, __half2 &v13) {
    // 0x64xx is the fp16 bit pattern of 1024 + xx
    v02 = __hsub2(as_half2(__byte_perm(w, 0x64646464u, 0x4240)), offset);
    v13 = __hsub2(as_half2(__byte_perm(w, 0x64646464u, 0x4341)), offset);
}
__device__ __forceinline__ __half2 bcast_lo(__half2 v) { return as_half2(__byte_perm(as_u32(v), 0u, 0x1010)); }
__device__ __forceinline__ __half2 bcast_hi(__half2 v) { return as_half2(__byte_perm(as_u32(v), 0u, 0x3232)); }

// 6-bit scales and mins of the sub-blocks 2*kq (byte 0) and 2*kq+1 (byte 1): the bit selection of
// get_scale_min_k4 on two bytes at once.  kq is uniform over the warp.
__device__ __forceinline__ void q4k_scale_bytes(const uint4 &hdr, int kq, uint32_t &sc2, uint32_t &mn2) {
    const int sh = 16 * (kq & 1);
    if (kq < 2) {
        sc2 = (hdr.y >> sh) & 0x3F3Fu;
        mn2 = (hdr.z >> sh) & 0x3F3Fu;
    } else {
        sc2 = ((hdr.w >> sh) & 0x0F0Fu) | (((hdr.y >> (sh + 6)) & 0x0303u) << 4);
        mn2 = ((hdr.w >> (sh + 4)) & 0x0F0Fu) | (((hdr.z >> (sh + 6)) & 0x0303u) << 4);
    }
}

__device__ __forceinline__ bool tm_elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ---- host side ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult st;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &st) == cudaSuccess &&
            st == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

}  // namespace mcu
