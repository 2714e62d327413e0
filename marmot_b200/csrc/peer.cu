// Peer communicator for tensor-parallel row-parallel outputs: one staging buffer per rank, mapped into every
// other rank of the box (CUDA IPC over NVLink), and a one-shot all-reduce kernel that sums the ranks' partial
// results with plain peer loads in a fixed rank order, so every rank gets bit-identical sums.
//
// Protocol (per rank, everything on the context's stream):
//   1. the producer (a matmul) writes its partial result into this rank's staging slot of parity p = epoch & 1;
//   2. allreduce kernel: one thread per peer stores `epoch` into flag[p][rank] of that peer (release, system
//      scope); every CTA then waits (acquire, bounded) until all world flags of its own rank have reached
//      `epoch`, and sums the world staging slots element-wise, rank 0 first.
// Two parities are enough: a rank can only pass the wait of call n+1 after every peer has started call n+1,
// i.e. finished reading call n, and it overwrites parity n & 1 again in call n+2 at the earliest.
// The epoch lives in device memory (read by every CTA at its start, advanced by the last CTA to finish), so a
// captured CUDA graph can be replayed; the staging pointer a producer writes to is fixed at capture, so with the two
// alternating slots a graph must hold an even number of collectives per communicator.  mcu_peer_comm_set_one_slot
// lifts that: one slot, and every kernel ends with a second flag exchange ("finished reading"), after which nothing
// can still be reading what the next producer overwrites.
// A wait that runs out (a peer that never arrives) sets the context's error flag and skips the sum; the
// kernel always terminates.
#include "../../include/marmot_cuda.h"

#include "common.cuh"
#include "kernels.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

namespace mcu {

constexpr int PEER_MAX_WORLD = 8;
constexpr size_t PEER_CTR_OFFSET = 2 * PEER_MAX_WORLD * 128;  // epoch counter and CTA ticket of the owning rank
// flags of the fused matmul + all-reduce: [parity][source rank][tile] u32
constexpr size_t PEER_FUSE_FLAG_OFFSET = 4096;
constexpr size_t PEER_FUSE_FLAG_BYTES = 2 * (size_t)PEER_FUSE_MAX_WORLD * PEER_FUSE_MAX_TILES * sizeof(uint32_t);
// all flags and counters; the staging buffers follow: [parity][capacity]
constexpr size_t PEER_FLAG_BYTES = PEER_FUSE_FLAG_OFFSET + PEER_FUSE_FLAG_BYTES;
static_assert(PEER_CTR_OFFSET + 128 <= PEER_FUSE_FLAG_OFFSET && PEER_FLAG_BYTES % 256 == 0, "layout");
constexpr unsigned long long PEER_WAIT_NS = 2000000000ull;    // 2 s
constexpr size_t PEER_TWO_PHASE_BYTES = (size_t)2 << 20;      // all-reduces from this size on go reduce-scatter + all-gather

struct PeerParams {
    const uint8_t *base[PEER_MAX_WORLD];  // every rank's buffer as mapped in this process
    uint8_t *flag_base[PEER_MAX_WORLD];
    int rank, world;
    uint32_t *ctr;    // this rank's {epoch of the last finished all-reduce, ticket}
    size_t capacity;  // bytes of one staging slot
    size_t n;         // floats
    float *out;
    int *err;
    // One-slot mode (mcu_peer_comm_set_one_slot): always parity 0, and the kernel ends only when every peer has finished
    // reading this rank's slot, so that whatever writes the slot next -- however many all-reduces a replayed CUDA graph
    // holds -- cannot overtake a reader.  done[r]: rank r's array of "finished reading" epochs, one entry per rank.
    int one_slot;
    uint32_t *done[PEER_MAX_WORLD];
};

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// The end of every collective kernel of this file: the last CTA of the grid to get here (ticket) publishes the epoch
// for the next launch.  In one-slot mode it first tells every peer that this rank has finished reading, and waits,
// bounded, until every peer has said the same.
__device__ __forceinline__ void peer_finish(const PeerParams &p, uint32_t epoch) {
    __syncthreads();
    if (threadIdx.x != 0) return;
    __threadfence();
    if (atomicAdd(p.ctr + 1, 1u) != gridDim.x - 1) return;
    p.ctr[1] = 0;
    if (p.one_slot) {
        __threadfence_system();
        for (int r = 0; r < p.world; ++r) st_release_sys(p.done[r] + (size_t)p.rank * 16, epoch);
        for (int r = 0; r < p.world; ++r) {
            const unsigned long long t0 = global_ns();
            while ((int32_t)(ld_acquire_sys(p.done[p.rank] + (size_t)r * 16) - epoch) < 0) {
                if (global_ns() - t0 > PEER_WAIT_NS) {
                    atomicExch(p.err, 25);
                    break;
                }
                __nanosleep(200);
            }
        }
    }
    __threadfence();
    *(volatile uint32_t *)p.ctr = epoch;
}

__global__ void __launch_bounds__(512) allreduce_oneshot_kernel(const PeerParams p) {
    __shared__ int ok_s;
    __shared__ uint32_t epoch_s;
    if (threadIdx.x == 0) {
        ok_s = 1;
        epoch_s = *(volatile uint32_t *)p.ctr + 1u;
    }
    __syncthreads();
    const uint32_t epoch = epoch_s;
    const int parity = p.one_slot ? 0 : (int)(epoch & 1u);
    const size_t slot_offset = PEER_FLAG_BYTES + (size_t)parity * p.capacity;
    if (blockIdx.x == 0 && threadIdx.x < p.world) {
        // this rank's partial result was written by earlier work on this stream
        __threadfence_system();
        uint32_t *f = (uint32_t *)(p.flag_base[threadIdx.x] + ((size_t)parity * PEER_MAX_WORLD + p.rank) * 128);
        st_release_sys(f, epoch);
    }
    __syncthreads();
    if (threadIdx.x < p.world) {
        const uint32_t *f =
            (const uint32_t *)(p.flag_base[p.rank] + ((size_t)parity * PEER_MAX_WORLD + threadIdx.x) * 128);
        const unsigned long long t0 = global_ns();
        // epochs only grow; the signed difference tolerates wrap-around
        while ((int32_t)(ld_acquire_sys(f) - epoch) < 0) {
            if (global_ns() - t0 > PEER_WAIT_NS) {
                atomicExch(p.err, 21);
                ok_s = 0;
                break;
            }
            __nanosleep(200);
        }
    }
    __syncthreads();
    const size_t n4 = ok_s ? p.n / 4 : 0;
    const size_t n_all = ok_s ? p.n : 0;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 acc = __ldcg((const float4 *)(p.base[0] + slot_offset) + i);
        for (int r = 1; r < p.world; ++r) {
            const float4 v = __ldcg((const float4 *)(p.base[r] + slot_offset) + i);
            acc.x = __fadd_rn(acc.x, v.x);
            acc.y = __fadd_rn(acc.y, v.y);
            acc.z = __fadd_rn(acc.z, v.z);
            acc.w = __fadd_rn(acc.w, v.w);
        }
        ((float4 *)p.out)[i] = acc;
    }
    for (size_t i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_all; i += stride) {
        float acc = __ldcg((const float *)(p.base[0] + slot_offset) + i);
        for (int r = 1; r < p.world; ++r) acc = __fadd_rn(acc, __ldcg((const float *)(p.base[r] + slot_offset) + i));
        p.out[i] = acc;
    }
    peer_finish(p, epoch);
}


// The same sum for large messages as reduce-scatter + all-gather in one kernel.  The message is cut into `world`
// slices (whole float4s).  Phase 1: this rank sums slice `rank` over all ranks' staging slots, rank 0 first, and
// writes the result over slice `rank` of ITS OWN slot (nobody else reads that slice of any slot in phase 1); the last
// CTA to finish raises this rank's phase-2 flag on every peer.  Phase 2: every rank copies slice q out of rank q's
// slot, for all q, once rank q's phase-2 flag is up.  A rank pulls 2 (world - 1) / world of the message instead of
// (world - 1) times the message; the sums are formed once, by one rank each, so all ranks hold the same bits.
// The grid must be co-resident (CTAs of phase 2 wait for flags that CTAs of phase 1 raise): the host sizes it from
// the occupancy of this kernel.  The flags of the two phases live side by side: [parity][phase][rank].
constexpr size_t PEER_CTR2_OFFSET = PEER_CTR_OFFSET + 128;    // phase-1 ticket of the owning rank
constexpr size_t PEER_PHASE2_OFFSET = PEER_CTR_OFFSET + 256;  // [parity][rank] u32, 64 bytes apart
constexpr size_t PEER_DONE_OFFSET = PEER_PHASE2_OFFSET + 2 * PEER_MAX_WORLD * 64;  // [rank] u32, 64 bytes apart (one-slot mode)
static_assert(PEER_DONE_OFFSET + PEER_MAX_WORLD * 64 <= PEER_FUSE_FLAG_OFFSET, "layout");

__device__ __forceinline__ bool peer_wait_flag(const uint32_t *f, uint32_t epoch, int *err, int code) {
    const unsigned long long t0 = global_ns();
    while ((int32_t)(ld_acquire_sys(f) - epoch) < 0) {
        if (global_ns() - t0 > PEER_WAIT_NS) {
            atomicExch(err, code);
            return false;
        }
        __nanosleep(200);
    }
    return true;
}

struct PeerParams2 {
    PeerParams base;
    uint32_t *phase2[PEER_MAX_WORLD];  // every rank's phase-2 flag array [parity][rank]
    uint32_t *ctr2;                    // this rank's phase-1 ticket
};

__global__ void __launch_bounds__(512) allreduce_rs_ag_kernel(const PeerParams2 q) {
    const PeerParams &p = q.base;
    __shared__ int ok_s;
    __shared__ uint32_t epoch_s;
    if (threadIdx.x == 0) {
        ok_s = 1;
        epoch_s = *(volatile uint32_t *)p.ctr + 1u;
    }
    __syncthreads();
    const uint32_t epoch = epoch_s;
    const int parity = p.one_slot ? 0 : (int)(epoch & 1u);
    const size_t slot_offset = PEER_FLAG_BYTES + (size_t)parity * p.capacity;
    if (blockIdx.x == 0 && threadIdx.x < p.world) {
        __threadfence_system();  // this rank's partial result was written by earlier work on this stream
        st_release_sys((uint32_t *)(p.flag_base[threadIdx.x] + ((size_t)parity * PEER_MAX_WORLD + p.rank) * 128), epoch);
    }
    __syncthreads();
    if (threadIdx.x < p.world) {
        const uint32_t *f = (const uint32_t *)(p.flag_base[p.rank] + ((size_t)parity * PEER_MAX_WORLD + threadIdx.x) * 128);
        if (!peer_wait_flag(f, epoch, p.err, 21)) ok_s = 0;
    }
    __syncthreads();
    const size_t n4 = (p.n + 3) / 4;                            // the staging slot is padded to whole float4s
    const size_t per = (n4 + p.world - 1) / p.world;            // float4s per slice
    const size_t stride = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (ok_s) {
        const size_t lo = per * p.rank, hi = min(n4, lo + per);
        float4 *mine = (float4 *)(p.base[p.rank] + slot_offset);
        for (size_t i = lo + tid; i < hi; i += stride) {
            float4 acc = __ldcg((const float4 *)(p.base[0] + slot_offset) + i);
            for (int r = 1; r < p.world; ++r) {
                const float4 v = __ldcg((const float4 *)(p.base[r] + slot_offset) + i);
                acc.x = __fadd_rn(acc.x, v.x);
                acc.y = __fadd_rn(acc.y, v.y);
                acc.z = __fadd_rn(acc.z, v.z);
                acc.w = __fadd_rn(acc.w, v.w);
            }
            mine[i] = acc;
        }
    }
    // the last CTA through phase 1 tells every rank that this rank's slice is summed
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        if (atomicAdd(q.ctr2, 1u) == gridDim.x - 1) {
            *q.ctr2 = 0;
            __threadfence_system();
            for (int r = 0; r < p.world; ++r) st_release_sys(q.phase2[r] + ((size_t)parity * PEER_MAX_WORLD + p.rank) * 16, epoch);
        }
    }
    // phase 2: the summed slices, each from the rank that formed it
    for (int step = 0; step < p.world; ++step) {
        const int src = (p.rank + step) % p.world;  // own slice first, then round the ring: the ranks pull from different peers
        __syncthreads();
        if (threadIdx.x == 0 && ok_s)
            if (!peer_wait_flag(q.phase2[p.rank] + ((size_t)parity * PEER_MAX_WORLD + src) * 16, epoch, p.err, 22)) ok_s = 0;
        __syncthreads();
        if (!ok_s) break;
        const size_t lo = per * src, hi = min(n4, lo + per);
        const float4 *from = (const float4 *)(p.base[src] + slot_offset);
        for (size_t i = lo + tid; i < hi; i += stride) {
            const float4 v = __ldcg(from + i);
            if (4 * i + 3 < p.n) {
                ((float4 *)p.out)[i] = v;
            } else {  // the ragged end of the message
                const float e[4] = {v.x, v.y, v.z, v.w};
                for (int j = 0; j < 4; ++j)
                    if (4 * i + j < p.n) p.out[4 * i + j] = e[j];
            }
        }
    }
    peer_finish(p, epoch);
}


// Expert-parallel MoE: the routed rows go back to the owners of their tokens and the token slices are gathered, in
// one kernel of the same two-phase shape.  Every rank ran the (replicated) router, so all agree on the sorted order of
// the routes; rank q's grouped down projection left its experts' rows [offsets[bound[q]], offsets[bound[q + 1]]) of the
// [routes][H] matrix in ITS staging slot.  Phase 1: this rank owns the tokens of slice `rank` and adds up each one's k
// routed rows, pulled from the slot of whichever rank owns the route's expert, weighted, in the order of the sorted
// positions -- the order and the operations of the one-GPU combine kernel, so the result has the same bits.  The
// combined rows go to `out` and to the result region behind the route rows of this rank's slot.  Phase 2: every rank
// copies the other ranks' token slices out of their result regions.  A rank pulls (world - 1) / world of
// (T / world) * k rows, then (world - 1) / world of the [T][H] output, instead of adding up `world` whole outputs.
struct PeerMoeParams {
    PeerParams2 pp;  // pp.base.out: [T][H]; pp.base.n is not used
    const int32_t *route_pos;
    const float *sorted_w;
    const int *offsets;
    const int *bad_id_count;
    int bound[PEER_MAX_WORLD + 1];  // rank q owns experts [bound[q], bound[q + 1])
    int T, k, H;
    size_t result_offset;           // bytes from the start of a slot to its [T][H] result region
};

template <int MAXK>
__global__ void __launch_bounds__(512) moe_ep_combine_kernel(const PeerMoeParams m) {
    const PeerParams &p = m.pp.base;
    __shared__ int ok_s;
    __shared__ uint32_t epoch_s;
    if (threadIdx.x == 0) {
        ok_s = 1;
        epoch_s = *(volatile uint32_t *)p.ctr + 1u;
    }
    __syncthreads();
    const uint32_t epoch = epoch_s;
    const int parity = p.one_slot ? 0 : (int)(epoch & 1u);
    const size_t slot_offset = PEER_FLAG_BYTES + (size_t)parity * p.capacity;
    if (blockIdx.x == 0 && threadIdx.x < p.world) {
        __threadfence_system();  // this rank's routed rows were written by the down projection earlier on this stream
        st_release_sys((uint32_t *)(p.flag_base[threadIdx.x] + ((size_t)parity * PEER_MAX_WORLD + p.rank) * 128), epoch);
    }
    __syncthreads();
    if (threadIdx.x < p.world) {
        const uint32_t *f = (const uint32_t *)(p.flag_base[p.rank] + ((size_t)parity * PEER_MAX_WORLD + threadIdx.x) * 128);
        if (!peer_wait_flag(f, epoch, p.err, 23)) ok_s = 0;
    }
    __syncthreads();
    const bool bad = *m.bad_id_count != 0;  // an expert id out of range rejects the call as a whole: zeros, error at synchronize
    if (bad && blockIdx.x == 0 && threadIdx.x == 0) atomicExch(p.err, 40);
    const int per_tok = (m.T + p.world - 1) / p.world, H4 = m.H / 4;
    float4 *out4 = (float4 *)p.out;
    if (ok_s) {
        const int lo = per_tok * p.rank, hi = min(m.T, lo + per_tok);
        float4 *mine = (float4 *)(p.base[p.rank] + slot_offset + m.result_offset);
        for (int t = lo + (int)blockIdx.x; t < hi; t += (int)gridDim.x) {
            int pos[MAXK];
            float w[MAXK];
            const float4 *rows[MAXK];
            for (int j = 0; j < m.k; ++j) pos[j] = m.route_pos[(size_t)t * m.k + j];
            for (int i = 1; i < m.k; ++i) {  // by sorted position, as the one-GPU combine
                const int v = pos[i];
                int j = i;
                while (j > 0 && pos[j - 1] > v) {
                    pos[j] = pos[j - 1];
                    --j;
                }
                pos[j] = v;
            }
            for (int j = 0; j < m.k; ++j) {
                rows[j] = nullptr;
                w[j] = 0.0f;
                if (bad || pos[j] < 0) continue;  // a rejected id has no row
                int q = 0;
                while (q + 1 < p.world && pos[j] >= m.offsets[m.bound[q + 1]]) ++q;
                rows[j] = (const float4 *)(p.base[q] + slot_offset) + (size_t)pos[j] * H4;
                w[j] = m.sorted_w[pos[j]];
            }
            for (int c = threadIdx.x; c < H4; c += blockDim.x) {
                float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                for (int j = 0; j < m.k; ++j) {
                    if (rows[j] == nullptr) continue;
                    const float4 v = __ldcg(rows[j] + c);
                    acc.x = __fadd_rn(acc.x, __fmul_rn(w[j], v.x));
                    acc.y = __fadd_rn(acc.y, __fmul_rn(w[j], v.y));
                    acc.z = __fadd_rn(acc.z, __fmul_rn(w[j], v.z));
                    acc.w = __fadd_rn(acc.w, __fmul_rn(w[j], v.w));
                }
                mine[(size_t)t * H4 + c] = acc;
                out4[(size_t)t * H4 + c] = acc;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        if (atomicAdd(m.pp.ctr2, 1u) == gridDim.x - 1) {
            *m.pp.ctr2 = 0;
            __threadfence_system();
            for (int r = 0; r < p.world; ++r) st_release_sys(m.pp.phase2[r] + ((size_t)parity * PEER_MAX_WORLD + p.rank) * 16, epoch);
        }
    }
    const size_t stride = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (int step = 1; step < p.world; ++step) {
        const int src = (p.rank + step) % p.world;
        __syncthreads();
        if (threadIdx.x == 0 && ok_s)
            if (!peer_wait_flag(m.pp.phase2[p.rank] + ((size_t)parity * PEER_MAX_WORLD + src) * 16, epoch, p.err, 24)) ok_s = 0;
        __syncthreads();
        if (!ok_s) break;
        const int lo = per_tok * src, hi = min(m.T, lo + per_tok);
        const float4 *from = (const float4 *)(p.base[src] + slot_offset + m.result_offset);
        for (size_t i = (size_t)lo * H4 + tid; i < (size_t)max(hi, lo) * H4; i += stride) out4[i] = __ldcg(from + i);
    }
    peer_finish(p, epoch);
}

}  // namespace mcu

using namespace mcu;

struct mcu_peer_comm {
    mcu_context_t *ctx = nullptr;
    int rank = 0, world = 1;
    size_t capacity = 0;  // bytes of one staging slot
    uint8_t *local = nullptr;
    uint8_t *mapped[PEER_MAX_WORLD] = {};
    bool connected = false;
    bool fused = false;  // mcu_linear_allreduce as one kernel (see mcu_peer_comm_set_fused)
    bool one_slot = false;  // see PeerParams::one_slot
    uint32_t epoch = 0;
};

#define PEER_CUDA(expr)                                                                   \
    do {                                                                                  \
        cudaError_t e__ = (expr);                                                         \
        if (e__ != cudaSuccess) {                                                         \
            char msg__[256];                                                              \
            snprintf(msg__, sizeof(msg__), "%s: %s", #expr, cudaGetErrorString(e__));     \
            return set_error(MCU_ERROR_INVALID_OPERATION, msg__);                         \
        }                                                                                 \
    } while (0)

extern "C" {

int mcu_peer_comm_create(mcu_context_t *ctx, int rank, int world, size_t max_bytes, mcu_peer_comm_t **out) {
    if (out == nullptr) return set_error(MCU_ERROR_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    if (ctx == nullptr) return set_error(MCU_ERROR_DEVICE_NOT_AVAILABLE, "CUDA context is not initialised");
    if (world < 1 || world > PEER_MAX_WORLD || rank < 0 || rank >= world)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "peer communicator: bad rank / world (at most 8 ranks)");
    if (max_bytes == 0) return set_error(MCU_ERROR_INVALID_ARGUMENT, "peer communicator: empty staging buffer");
    PEER_CUDA(cudaSetDevice(context_device(ctx)));
    mcu_peer_comm *c = new (std::nothrow) mcu_peer_comm;
    if (c == nullptr) return set_error(MCU_ERROR_OUT_OF_MEMORY, "peer communicator allocation failed");
    c->ctx = ctx;
    c->rank = rank;
    c->world = world;
    c->capacity = (max_bytes + 255) & ~(size_t)255;
    const size_t total = PEER_FLAG_BYTES + 2 * c->capacity;
    cudaError_t e = cudaMalloc((void **)&c->local, total);
    if (e != cudaSuccess) {
        delete c;
        return set_error(MCU_ERROR_OUT_OF_MEMORY, "peer communicator: cudaMalloc failed");
    }
    e = cudaMemset(c->local, 0, total);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(c->local);
        delete c;
        return set_error(MCU_ERROR_INVALID_OPERATION, cudaGetErrorString(e));
    }
    c->mapped[rank] = c->local;
    c->connected = world == 1;
    *out = c;
    return MCU_SUCCESS;
}

int mcu_peer_comm_export(mcu_peer_comm_t *c, void *handle_out) {
    if (c == nullptr || handle_out == nullptr) return set_error(MCU_ERROR_INVALID_ARGUMENT, "null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == MCU_PEER_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    PEER_CUDA(cudaSetDevice(context_device(c->ctx)));
    PEER_CUDA(cudaIpcGetMemHandle(&h, c->local));
    memcpy(handle_out, &h, sizeof(h));
    return MCU_SUCCESS;
}

int mcu_peer_comm_connect(mcu_peer_comm_t *c, const void *all_handles) {
    if (c == nullptr || all_handles == nullptr) return set_error(MCU_ERROR_INVALID_ARGUMENT, "null argument");
    if (c->connected) return MCU_SUCCESS;
    PEER_CUDA(cudaSetDevice(context_device(c->ctx)));
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const uint8_t *)all_handles + (size_t)r * MCU_PEER_HANDLE_BYTES, sizeof(h));
        void *p = nullptr;
        PEER_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        c->mapped[r] = (uint8_t *)p;
    }
    c->connected = true;
    return MCU_SUCCESS;
}

int mcu_peer_comm_set_fused(mcu_peer_comm_t *c, int enabled) {
    if (c == nullptr) return set_error(MCU_ERROR_INVALID_ARGUMENT, "null argument");
    c->fused = enabled != 0;
    return MCU_SUCCESS;
}

void *mcu_peer_comm_staging(mcu_peer_comm_t *c) {
    if (c == nullptr) return nullptr;
    // slot of the NEXT collective: the two slots take turns, unless the communicator keeps to one
    return c->local + PEER_FLAG_BYTES + (c->one_slot ? 0 : (size_t)((c->epoch + 1) & 1u) * c->capacity);
}

int mcu_peer_comm_set_one_slot(mcu_peer_comm_t *c, int enabled) {
    if (c == nullptr) return set_error(MCU_ERROR_INVALID_ARGUMENT, "null argument");
    PEER_CUDA(cudaSetDevice(context_device(c->ctx)));
    PEER_CUDA(cudaStreamSynchronize((cudaStream_t)mcu_context_get_stream(c->ctx)));  // nothing of the other mode in flight here
    c->one_slot = enabled != 0;
    return MCU_SUCCESS;
}

int mcu_peer_allreduce(mcu_peer_comm_t *c, size_t n_floats, float *out_dev) {
    if (c == nullptr || out_dev == nullptr) return set_error(MCU_ERROR_INVALID_ARGUMENT, "null argument");
    if (!c->connected) return set_error(MCU_ERROR_INVALID_OPERATION, "peer communicator is not connected");
    if (n_floats * sizeof(float) > c->capacity)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "all-reduce larger than the communicator's staging buffer");
    if (n_floats == 0) return MCU_SUCCESS;
    if ((uintptr_t)out_dev & 15) return set_error(MCU_ERROR_INVALID_ARGUMENT, "all-reduce output must be 16-byte aligned");
    PEER_CUDA(cudaSetDevice(context_device(c->ctx)));
    c->epoch += 1;  // host mirror: only its parity is used (mcu_peer_comm_staging)
    PeerParams p;
    memset(&p, 0, sizeof(p));
    for (int r = 0; r < c->world; ++r) {
        p.base[r] = c->mapped[r];
        p.flag_base[r] = c->mapped[r];
    }
    for (int r = 0; r < c->world; ++r) p.done[r] = (uint32_t *)(c->mapped[r] + PEER_DONE_OFFSET);
    p.one_slot = c->one_slot ? 1 : 0;
    p.rank = c->rank;
    p.world = c->world;
    p.ctr = (uint32_t *)(c->local + PEER_CTR_OFFSET);
    p.capacity = c->capacity;
    p.n = n_floats;
    p.out = out_dev;
    p.err = context_err_flag(c->ctx);
    const size_t n4 = (n_floats + 3) / 4;
    static const bool no_two_phase = getenv("MARMOT_CUDA_ALLREDUCE_ONESHOT") != nullptr;  // diagnostic switch
    if (c->world > 1 && n_floats * sizeof(float) >= PEER_TWO_PHASE_BYTES && !no_two_phase) {
        // large message: reduce-scatter + all-gather; the grid must be resident at once (its CTAs wait on one another)
        static int per_sm = 0;
        if (per_sm == 0) {
            PEER_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, allreduce_rs_ag_kernel, 512, 0));
            if (per_sm < 1) return set_error(MCU_ERROR_INVALID_OPERATION, "all-reduce kernel does not fit an SM");
        }
        PeerParams2 q;
        memset(&q, 0, sizeof(q));
        q.base = p;
        for (int r = 0; r < c->world; ++r) q.phase2[r] = (uint32_t *)(c->mapped[r] + PEER_PHASE2_OFFSET);
        q.ctr2 = (uint32_t *)(c->local + PEER_CTR2_OFFSET);
        const size_t per = (n4 + c->world - 1) / c->world;
        int blocks = (int)((per + 511) / 512);
        const int max_blocks = (per_sm > 2 ? 2 : per_sm) * device_sm_count();
        if (blocks > max_blocks) blocks = max_blocks;
        if (blocks < 1) blocks = 1;
        allreduce_rs_ag_kernel<<<blocks, 512, 0, (cudaStream_t)mcu_context_get_stream(c->ctx)>>>(q);
        PEER_CUDA(cudaGetLastError());
        count_launches(1);
        return MCU_SUCCESS;
    }
    int blocks = (int)((n4 + 511) / 512);
    const int max_blocks = 2 * device_sm_count();
    if (blocks > max_blocks) blocks = max_blocks;
    if (blocks < 1) blocks = 1;
    allreduce_oneshot_kernel<<<blocks, 512, 0, (cudaStream_t)mcu_context_get_stream(c->ctx)>>>(p);
    PEER_CUDA(cudaGetLastError());
    count_launches(1);
    return MCU_SUCCESS;
}

int mcu_linear_allreduce(mcu_context_t *ctx, mcu_peer_comm_t *c, int kind, const float *x_dev, size_t ldx,
                         const void *w_dev, size_t T, size_t K, size_t F, float *out_dev) {
    if (c == nullptr || c->ctx != ctx) return set_error(MCU_ERROR_INVALID_ARGUMENT, "communicator of another context");
    if (T * F * sizeof(float) > c->capacity)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "result larger than the communicator's staging buffer");
    if (!c->connected) return set_error(MCU_ERROR_INVALID_OPERATION, "peer communicator is not connected");
    if (c->fused && !c->one_slot && c->world > 1 && gemm_tma_can_fuse(kind, (int)T, (int)F) && ((uintptr_t)out_dev & 15) == 0) {
        // one kernel: the matmul's epilogue publishes its tiles and pulls the peers' tiles
        const uint32_t parity = (c->epoch + 1) & 1u;
        PeerFuse f;
        memset(&f, 0, sizeof(f));
        const size_t slots_off = PEER_FLAG_BYTES + (size_t)parity * c->capacity;
        const size_t flags_off = PEER_FUSE_FLAG_OFFSET + (size_t)parity * PEER_FUSE_MAX_WORLD * PEER_FUSE_MAX_TILES * sizeof(uint32_t);
        for (int r = 0; r < c->world; ++r) {
            f.slots[r] = (float *)(c->mapped[r] + slots_off);
            f.flags[r] = (uint32_t *)(c->mapped[r] + flags_off);
        }
        f.ctr = (uint32_t *)(c->local + PEER_CTR_OFFSET);
        f.slot_floats = c->capacity / sizeof(float);
        f.rank = c->rank;
        f.world = c->world;
        f.parity_of_next = parity;
        const int rc = linear_fused_allreduce(ctx, kind, x_dev, ldx, w_dev, T, K, F, out_dev, f);
        if (rc == MCU_SUCCESS) {
            c->epoch += 1;
            return rc;
        }
        if (rc != MCU_ERROR_NOT_IMPLEMENTED) return rc;
        // the weights do not suit the TMA matmul: two kernels below (all ranks take the same decision when their
        // shards are cut in k_granule units)
    }
    float *staging = (float *)mcu_peer_comm_staging(c);
    if (int rc = mcu_linear(ctx, kind, x_dev, ldx, w_dev, T, K, F, nullptr, staging, F)) return rc;
    return mcu_peer_allreduce(c, T * F, out_dev);
}

size_t mcu_peer_comm_capacity(mcu_peer_comm_t *c) { return c == nullptr ? 0 : c->capacity; }
int mcu_peer_comm_rank(mcu_peer_comm_t *c) { return c == nullptr ? 0 : c->rank; }
int mcu_peer_comm_world(mcu_peer_comm_t *c) { return c == nullptr ? 1 : c->world; }

int mcu_peer_moe_combine(mcu_peer_comm_t *c, const int32_t *route_pos_dev, const float *sorted_w_dev, const int32_t *offsets_dev,
                         const int32_t *bad_id_count_dev, const int32_t *expert_bounds, size_t T, size_t k, size_t H,
                         float *out_dev) {
    if (c == nullptr || route_pos_dev == nullptr || sorted_w_dev == nullptr || offsets_dev == nullptr ||
        bad_id_count_dev == nullptr || expert_bounds == nullptr || out_dev == nullptr)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "null argument");
    if (!c->connected) return set_error(MCU_ERROR_INVALID_OPERATION, "peer communicator is not connected");
    if (T == 0) return MCU_SUCCESS;
    if (k == 0 || k > 8 || H == 0 || H % 4 != 0 || ((uintptr_t)out_dev & 15) || T > (size_t)1 << 24)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "expert-parallel combine: k <= 8, H a multiple of 4, 16-byte aligned output");
    const size_t rows_bytes = (T * k * H * sizeof(float) + 255) & ~(size_t)255;
    if (rows_bytes + T * H * sizeof(float) > c->capacity)
        return set_error(MCU_ERROR_INVALID_ARGUMENT, "expert-parallel combine: the staging slot must hold (T * k + T) * H floats");
    for (int r = 0; r < c->world; ++r)
        if (expert_bounds[r] > expert_bounds[r + 1] || expert_bounds[0] != 0)
            return set_error(MCU_ERROR_INVALID_ARGUMENT, "expert-parallel combine: expert bounds must start at 0 and not decrease");
    PEER_CUDA(cudaSetDevice(context_device(c->ctx)));
    static int per_sm = 0;
    if (per_sm == 0) {
        PEER_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moe_ep_combine_kernel<8>, 512, 0));
        if (per_sm < 1) return set_error(MCU_ERROR_INVALID_OPERATION, "combine kernel does not fit an SM");
    }
    c->epoch += 1;
    PeerMoeParams m;
    memset(&m, 0, sizeof(m));
    for (int r = 0; r < c->world; ++r) {
        m.pp.base.base[r] = c->mapped[r];
        m.pp.base.flag_base[r] = c->mapped[r];
        m.pp.phase2[r] = (uint32_t *)(c->mapped[r] + PEER_PHASE2_OFFSET);
        m.pp.base.done[r] = (uint32_t *)(c->mapped[r] + PEER_DONE_OFFSET);
    }
    m.pp.base.one_slot = c->one_slot ? 1 : 0;
    m.pp.base.rank = c->rank;
    m.pp.base.world = c->world;
    m.pp.base.ctr = (uint32_t *)(c->local + PEER_CTR_OFFSET);
    m.pp.base.capacity = c->capacity;
    m.pp.base.out = out_dev;
    m.pp.base.err = context_err_flag(c->ctx);
    m.pp.ctr2 = (uint32_t *)(c->local + PEER_CTR2_OFFSET);
    m.route_pos = route_pos_dev;
    m.sorted_w = sorted_w_dev;
    m.offsets = offsets_dev;
    m.bad_id_count = bad_id_count_dev;
    for (int r = 0; r <= c->world; ++r) m.bound[r] = expert_bounds[r];
    m.T = (int)T;
    m.k = (int)k;
    m.H = (int)H;
    m.result_offset = rows_bytes;
    int blocks = (per_sm > 2 ? 2 : per_sm) * device_sm_count();  // resident at once: its CTAs wait on one another
    const size_t per_tok = (T + c->world - 1) / c->world;
    if ((size_t)blocks > per_tok * 2 && per_tok > 0) blocks = (int)(per_tok * 2);
    if (blocks < 1) blocks = 1;
    moe_ep_combine_kernel<8><<<blocks, 512, 0, (cudaStream_t)mcu_context_get_stream(c->ctx)>>>(m);
    PEER_CUDA(cudaGetLastError());
    count_launches(1);
    return MCU_SUCCESS;
}

void mcu_peer_comm_destroy(mcu_peer_comm_t *c) {
    if (c == nullptr) return;
    cudaSetDevice(context_device(c->ctx));
    cudaStreamSynchronize((cudaStream_t)mcu_context_get_stream(c->ctx));
    for (int r = 0; r < c->world; ++r)
        if (r != c->rank && c->mapped[r] != nullptr) cudaIpcCloseMemHandle(c->mapped[r]);
    if (c->local != nullptr) cudaFree(c->local);
    delete c;
}

}  // extern "C"
