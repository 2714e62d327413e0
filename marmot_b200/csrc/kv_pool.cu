// Paged KV-cache pool with HBM-resident blocks: the block allocator of the reference's serving path
// (src/inference/kv_pool/kv_pool.cpp, C API include/marmot/inference/kv_pool.h:65-101) for a CUDA device.
//
// The bookkeeping is the reference's, decision for decision, so that a scheduler sees the same slots, block ids
// and error codes: sequence slots and free blocks are handed out last-freed-first (or lowest-id-first with the
// deterministic flag), blocks are reference counted so that sequences can share a prefix, a shared partially
// filled block is cloned before it is appended to (copy on write), blocks marked "retained" are reused only when
// nothing else is free, and a sequence can be swapped out to host memory and back (by exchange with another
// resident sequence of the same size when the device pool is full).
//
// What differs is where things live and how they move:
//   * K and V pools [blocks][layers][kv_heads][block_size][head_dim] are device allocations; the block table
//     [max_seqs][max_blocks_per_seq] u32 exists twice, a host shadow that the bookkeeping edits and a device copy
//     the attention kernel reads.  Every call that edits rows uploads exactly those rows with an asynchronous copy
//     on the context's stream before it returns, so kernels enqueued afterwards see the new table and nothing ever
//     waits for the device.
//   * Copy-on-write clones are device-to-device copies on the same stream.
//   * Swap blocks are page-locked host memory; swapping out and in are asynchronous copies on the same stream.  The
//     stream order alone makes them safe: a swapped-out block may be handed to another sequence at once, because
//     whatever overwrites it is enqueued after the copy that saved it.  The exchange path goes through one spare
//     device block instead of host staging buffers.
//   * A pool created without a context keeps books only (no storage): what a scheduler needs to plan admission.
#include "../../include/marmot_cuda.h"

#include "kernels.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <functional>
#include <mutex>
#include <new>
#include <vector>

using namespace mcu;

namespace {

constexpr uint32_t kInvalid = MCU_BLOCK_ID_INVALID;

// Free blocks: a stack (last freed, first reused) or, deterministic, a min-heap with lazy deletion.
struct FreeSet {
    bool deterministic = false;
    std::vector<uint32_t> blocks;
    std::vector<int32_t> index;  // stack mode: position of a block in `blocks`, -1 if absent
    std::vector<uint8_t> mask;   // heap mode: membership
    size_t count = 0;

    void init(size_t capacity, bool det) {
        deterministic = det;
        blocks.clear();
        blocks.reserve(capacity);
        index.clear();
        mask.clear();
        count = 0;
        if (det) mask.assign(capacity, 0);
        else index.assign(capacity, -1);
    }
    void push(uint32_t b) {
        if (deterministic) {
            if (b >= mask.size() || mask[b]) return;
            mask[b] = 1;
            blocks.push_back(b);
            std::push_heap(blocks.begin(), blocks.end(), std::greater<uint32_t>());
            ++count;
            return;
        }
        if (b >= index.size() || index[b] >= 0) return;
        index[b] = (int32_t)blocks.size();
        blocks.push_back(b);
        ++count;
    }
    bool remove(uint32_t b) {
        if (deterministic) {
            if (b >= mask.size() || !mask[b]) return false;
            mask[b] = 0;  // the heap entry stays and is skipped when it surfaces
            if (count > 0) --count;
            return true;
        }
        if (blocks.empty() || b >= index.size() || index[b] < 0) return false;
        const size_t at = (size_t)index[b];
        const uint32_t last = blocks.back();
        blocks[at] = last;
        index[last] = (int32_t)at;
        blocks.pop_back();
        index[b] = -1;
        if (count > 0) --count;
        return true;
    }
    bool pop(uint32_t &out) {
        if (deterministic) {
            while (!blocks.empty()) {
                std::pop_heap(blocks.begin(), blocks.end(), std::greater<uint32_t>());
                out = blocks.back();
                blocks.pop_back();
                if (out < mask.size() && mask[out]) {
                    mask[out] = 0;
                    if (count > 0) --count;
                    return true;
                }
            }
            return false;
        }
        if (blocks.empty()) return false;
        out = blocks.back();
        blocks.pop_back();
        if (out < index.size()) index[out] = -1;
        if (count > 0) --count;
        return true;
    }
};

struct BlockAlloc {
    uint32_t block, logical;
};
struct BlockClone {
    uint32_t old_block, new_block, logical;
};
struct PendingPlan {  // at most one per sequence (the reference refuses a second plan while one is pending)
    uint64_t cookie = 0;
    bool is_prefix = false;
    size_t start_pos = 0, token_count = 0, prefix_len = 0;
    std::vector<BlockAlloc> new_blocks;
    std::vector<BlockClone> cloned;
    std::vector<uint32_t> prefix_blocks;
};

}  // namespace

struct mcu_kv_pool {
    mcu_kv_pool_options_t o{};
    mcu_context_t *ctx = nullptr;
    cudaStream_t stream() const { return (cudaStream_t)mcu_context_get_stream(ctx); }
    size_t max_blocks_per_seq = 0, block_bytes = 0;
    uint32_t shift = 0, mask = 0;
    bool deterministic = false;

    uint8_t *k_dev = nullptr, *v_dev = nullptr;  // num_blocks + 1 blocks: the last one is the exchange spare
    uint32_t *table_dev = nullptr;
    uint8_t *swap_k = nullptr, *swap_v = nullptr;  // page-locked host memory
    std::vector<uint32_t> table, swap_table;       // host shadows [max_seqs][max_blocks_per_seq]

    std::vector<size_t> seq_len;
    std::vector<uint8_t> active, pending, swapped;
    std::vector<uint32_t> free_seqs;
    FreeSet free_blocks, retained_free, swap_free;
    std::vector<uint32_t> refcount, generation;
    std::vector<uint8_t> retained;
    uint32_t next_generation = 1;
    std::vector<PendingPlan> plans;
    uint64_t next_cookie = 1;
    std::mutex mu;

    uint32_t *row(uint32_t seq) { return table.data() + (size_t)seq * max_blocks_per_seq; }
    uint32_t *swap_row(uint32_t seq) { return swap_table.data() + (size_t)seq * max_blocks_per_seq; }
    bool seq_ok(uint32_t seq) const { return (size_t)seq < o.max_seqs; }
    void bump_generation(uint32_t b) {
        if (b >= generation.size()) return;
        generation[b] = next_generation++;
        if (next_generation == 0) next_generation = 1;
    }
    void release_block(uint32_t b) {
        if (b >= retained.size()) return;
        (retained[b] ? retained_free : free_blocks).push(b);
    }
    void unref(uint32_t b) {
        if (b < refcount.size() && refcount[b] > 0 && --refcount[b] == 0) release_block(b);
    }
    void restore_block(uint32_t b) {  // take a block back that an aborted plan had let go of
        if (b >= refcount.size()) return;
        if (refcount[b] == 0) {
            (void)free_blocks.remove(b);
            (void)retained_free.remove(b);
        }
        ++refcount[b];
    }
    bool pop_free(uint32_t &b) {
        if (!free_blocks.pop(b) && !retained_free.pop(b)) return false;
        if (b < retained.size()) retained[b] = 0;
        return true;
    }

    // ---- data movement (all asynchronous, all on the context's stream) ----
    int upload_row(uint32_t seq, size_t first, size_t count) {
        if (table_dev == nullptr || count == 0) return MCU_SUCCESS;
        const size_t at = (size_t)seq * max_blocks_per_seq + first;
        const cudaError_t e = cudaMemcpyAsync(table_dev + at, table.data() + at, count * sizeof(uint32_t),
                                              cudaMemcpyHostToDevice, stream());
        return e == cudaSuccess ? MCU_SUCCESS : set_error(MCU_ERROR_INVALID_OPERATION, cudaGetErrorString(e));
    }
    int copy_blocks(uint8_t *dst_k, uint8_t *dst_v, const uint8_t *src_k, const uint8_t *src_v, cudaMemcpyKind kind) {
        if (k_dev == nullptr) return MCU_SUCCESS;  // a pool that only keeps books
        cudaError_t e = cudaMemcpyAsync(dst_k, src_k, block_bytes, kind, stream());
        if (e == cudaSuccess) e = cudaMemcpyAsync(dst_v, src_v, block_bytes, kind, stream());
        return e == cudaSuccess ? MCU_SUCCESS : set_error(MCU_ERROR_INVALID_OPERATION, cudaGetErrorString(e));
    }
    int clone_block(uint32_t dst, uint32_t src) {
        return copy_blocks(k_dev + (size_t)dst * block_bytes, v_dev + (size_t)dst * block_bytes, k_dev + (size_t)src * block_bytes,
                           v_dev + (size_t)src * block_bytes, cudaMemcpyDeviceToDevice);
    }
    int save_block(uint32_t swap_b, uint32_t dev_b) {
        return copy_blocks(swap_k + (size_t)swap_b * block_bytes, swap_v + (size_t)swap_b * block_bytes,
                           k_dev + (size_t)dev_b * block_bytes, v_dev + (size_t)dev_b * block_bytes, cudaMemcpyDeviceToHost);
    }
    int load_block(uint32_t dev_b, uint32_t swap_b) {
        return copy_blocks(k_dev + (size_t)dev_b * block_bytes, v_dev + (size_t)dev_b * block_bytes,
                           swap_k + (size_t)swap_b * block_bytes, swap_v + (size_t)swap_b * block_bytes, cudaMemcpyHostToDevice);
    }
};

static int pool_fail(int code, const char *msg) { return set_error(code, msg); }

extern "C" {

int mcu_kv_pool_options_init(mcu_kv_pool_options_t *opts) {
    if (opts == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    memset(opts, 0, sizeof(*opts));
    opts->max_seqs = 1;
    opts->max_seq_len = 2048;
    opts->block_size = 16;
    opts->num_blocks = 256;
    opts->num_layers = 1;
    opts->num_kv_heads = 1;
    opts->head_dim = 64;
    opts->kv_dtype = MCU_KV_F16;
    return MCU_SUCCESS;
}

int mcu_kv_pool_create(mcu_context_t *ctx, const mcu_kv_pool_options_t *opts, mcu_kv_pool_t **out_pool) {
    if (out_pool == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    *out_pool = nullptr;
    if (opts == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    if (opts->max_seqs == 0 || opts->max_seq_len == 0 || opts->block_size == 0 || opts->num_blocks == 0 ||
        opts->num_layers == 0 || opts->num_kv_heads == 0 || opts->head_dim == 0)
        return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool options must be non-zero");
    if (opts->block_size <= 1 || (opts->block_size & (opts->block_size - 1)) != 0)
        return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool block_size must be power-of-two > 1");
    if (opts->kv_dtype != MCU_KV_F32 && opts->kv_dtype != MCU_KV_F16)
        return pool_fail(MCU_ERROR_UNSUPPORTED_DTYPE, "KV pool dtype must be FLOAT32 or FLOAT16");
    if (opts->num_blocks >= (size_t)kInvalid || opts->num_swap_blocks >= (size_t)kInvalid)
        return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool block count exceeds the block id range");
    mcu_kv_pool *p = new (std::nothrow) mcu_kv_pool();
    if (p == nullptr) return pool_fail(MCU_ERROR_OUT_OF_MEMORY, "Failed to allocate KV pool");
    p->o = *opts;
    p->ctx = ctx;
    p->deterministic = (opts->flags & MCU_KV_POOL_FLAG_DETERMINISTIC_ALLOC) != 0;
    p->max_blocks_per_seq = (opts->max_seq_len + opts->block_size - 1) / opts->block_size;
    while (((size_t)1 << p->shift) < opts->block_size) ++p->shift;
    p->mask = (1u << p->shift) - 1u;
    const size_t elem = opts->kv_dtype == MCU_KV_F16 ? 2 : 4;
    p->block_bytes = opts->num_layers * opts->num_kv_heads * opts->block_size * opts->head_dim * elem;
    if (opts->num_blocks > (((size_t)kInvalid) >> p->shift)) {
        delete p;
        return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool slots exceed 32 bits");
    }
    const size_t cells = opts->max_seqs * p->max_blocks_per_seq;
    p->table.assign(cells, kInvalid);
    p->swap_table.assign(cells, kInvalid);
    p->seq_len.assign(opts->max_seqs, 0);
    p->active.assign(opts->max_seqs, 0);
    p->pending.assign(opts->max_seqs, 0);
    p->swapped.assign(opts->max_seqs, 0);
    p->plans.resize(opts->max_seqs);
    p->free_seqs.reserve(opts->max_seqs);
    for (size_t i = 0; i < opts->max_seqs; ++i) p->free_seqs.push_back((uint32_t)(opts->max_seqs - 1 - i));
    p->free_blocks.init(opts->num_blocks, p->deterministic);
    p->retained_free.init(opts->num_blocks, p->deterministic);
    for (size_t i = 0; i < opts->num_blocks; ++i) p->free_blocks.push((uint32_t)(opts->num_blocks - 1 - i));
    p->refcount.assign(opts->num_blocks, 0);
    p->retained.assign(opts->num_blocks, 0);
    p->generation.assign(opts->num_blocks, 0);
    if (opts->num_swap_blocks > 0) {
        p->swap_free.init(opts->num_swap_blocks, p->deterministic);
        for (size_t i = 0; i < opts->num_swap_blocks; ++i) p->swap_free.push((uint32_t)(opts->num_swap_blocks - 1 - i));
    }
    if (ctx != nullptr) {
        cudaError_t e = cudaSetDevice(context_device(ctx));
        const size_t pool_bytes = (opts->num_blocks + 1) * p->block_bytes;  // + the exchange spare
        if (e == cudaSuccess) e = cudaMalloc(&p->k_dev, pool_bytes);
        if (e == cudaSuccess) e = cudaMalloc(&p->v_dev, pool_bytes);
        if (e == cudaSuccess) e = cudaMalloc(&p->table_dev, cells * sizeof(uint32_t));
        if (e == cudaSuccess) e = cudaMemsetAsync(p->k_dev, 0, pool_bytes, p->stream());
        if (e == cudaSuccess) e = cudaMemsetAsync(p->v_dev, 0, pool_bytes, p->stream());
        if (e == cudaSuccess) e = cudaMemsetAsync(p->table_dev, 0xFF, cells * sizeof(uint32_t), p->stream());
        if (e == cudaSuccess && opts->num_swap_blocks > 0) {
            e = cudaHostAlloc(&p->swap_k, opts->num_swap_blocks * p->block_bytes, cudaHostAllocDefault);
            if (e == cudaSuccess) e = cudaHostAlloc(&p->swap_v, opts->num_swap_blocks * p->block_bytes, cudaHostAllocDefault);
        }
        if (e != cudaSuccess) {
            const int rc = pool_fail(e == cudaErrorMemoryAllocation ? MCU_ERROR_OUT_OF_MEMORY : MCU_ERROR_INVALID_OPERATION,
                                     cudaGetErrorString(e));
            (void)cudaGetLastError();
            mcu_kv_pool_destroy(p);
            return rc;
        }
    }
    *out_pool = p;
    return MCU_SUCCESS;
}

void mcu_kv_pool_destroy(mcu_kv_pool_t *p) {
    if (p == nullptr) return;
    if (p->ctx != nullptr) {
        // copies of this pool may still be in flight on the stream
        (void)cudaStreamSynchronize(p->stream());
        if (p->k_dev != nullptr) cudaFree(p->k_dev);
        if (p->v_dev != nullptr) cudaFree(p->v_dev);
        if (p->table_dev != nullptr) cudaFree(p->table_dev);
        if (p->swap_k != nullptr) cudaFreeHost(p->swap_k);
        if (p->swap_v != nullptr) cudaFreeHost(p->swap_v);
    }
    delete p;
}

int mcu_kv_pool_acquire_seq(mcu_kv_pool_t *p, uint32_t *out_seq) {
    if (p == nullptr || out_seq == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    if (p->free_seqs.empty()) return pool_fail(MCU_ERROR_OUT_OF_MEMORY, "KV pool has no free sequence slots");
    const uint32_t seq = p->free_seqs.back();
    p->free_seqs.pop_back();
    p->active[seq] = 1;
    p->pending[seq] = 0;
    p->swapped[seq] = 0;
    p->seq_len[seq] = 0;
    std::fill(p->row(seq), p->row(seq) + p->max_blocks_per_seq, kInvalid);
    std::fill(p->swap_row(seq), p->swap_row(seq) + p->max_blocks_per_seq, kInvalid);
    *out_seq = seq;
    return p->upload_row(seq, 0, p->max_blocks_per_seq);
}

int mcu_kv_pool_release_seq(mcu_kv_pool_t *p, uint32_t seq) {
    if (p == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    if (!p->seq_ok(seq) || !p->active[seq])
        return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool release requires active sequence slot");
    if (p->pending[seq]) return pool_fail(MCU_ERROR_INVALID_OPERATION, "KV pool release requires no pending plan");
    uint32_t *row = p->row(seq);
    if (p->swapped[seq]) {
        uint32_t *srow = p->swap_row(seq);
        for (size_t i = 0; i < p->max_blocks_per_seq; ++i)
            if (srow[i] != kInvalid) {
                p->swap_free.push(srow[i]);
                srow[i] = kInvalid;
            }
        p->swapped[seq] = 0;
    }
    for (size_t i = 0; i < p->max_blocks_per_seq; ++i) {
        if (row[i] == kInvalid) continue;
        p->unref(row[i]);
        row[i] = kInvalid;
    }
    p->seq_len[seq] = 0;
    p->active[seq] = 0;
    p->pending[seq] = 0;
    p->free_seqs.push_back(seq);
    return p->upload_row(seq, 0, p->max_blocks_per_seq);
}

// Undo what prepare_append did to the books (shared by the failure path of prepare and by abort).
static void rollback_append(mcu_kv_pool *p, uint32_t seq, const PendingPlan &plan) {
    uint32_t *row = p->row(seq);
    for (const BlockClone &c : plan.cloned) {
        row[c.logical] = c.old_block;
        p->unref(c.new_block);
        p->restore_block(c.old_block);
    }
    for (const BlockAlloc &a : plan.new_blocks) {
        row[a.logical] = kInvalid;
        p->unref(a.block);
    }
}

int mcu_kv_pool_prepare_append(mcu_kv_pool_t *p, uint32_t seq, size_t token_count, mcu_kv_append_plan_t *out_plan,
                               uint32_t *out_slots, size_t *out_start_pos) {
    if (p == nullptr || out_plan == nullptr || out_start_pos == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    out_plan->seq = seq;
    out_plan->token_count = token_count;
    out_plan->cookie = 0;
    *out_start_pos = 0;
    if (!p->seq_ok(seq) || !p->active[seq])
        return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool append requires active sequence slot");
    if (p->pending[seq]) return pool_fail(MCU_ERROR_INVALID_OPERATION, "KV pool append requires no pending plan");
    if (p->swapped[seq]) return pool_fail(MCU_ERROR_INVALID_OPERATION, "KV pool append requires resident sequence");
    if (token_count == 0) {
        *out_start_pos = p->seq_len[seq];
        return MCU_SUCCESS;
    }
    if (out_slots == nullptr) return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool append requires output slots");
    const size_t start = p->seq_len[seq];
    if (start > p->o.max_seq_len) return pool_fail(MCU_ERROR_INVALID_OPERATION, "KV pool sequence length exceeds max_seq_len");
    if (token_count > p->o.max_seq_len - start) return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool append exceeds max_seq_len");
    const size_t end = start + token_count;
    const size_t first_block = start >> p->shift, last_block = (end - 1) >> p->shift;
    if (last_block >= p->max_blocks_per_seq) return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool append exceeds block table");
    uint32_t *row = p->row(seq);
    PendingPlan plan;
    plan.start_pos = start;
    plan.token_count = token_count;
    // copy on write: the block the append continues in is shared with another sequence
    if ((start & p->mask) != 0) {
        const uint32_t existing = row[first_block];
        if (existing != kInvalid && existing < p->refcount.size() && p->refcount[existing] > 1) {
            uint32_t fresh = kInvalid;
            if (!p->pop_free(fresh)) return pool_fail(MCU_ERROR_OUT_OF_MEMORY, "KV pool out of blocks");
            if (int rc = p->clone_block(fresh, existing)) {
                p->release_block(fresh);
                return rc;
            }
            row[first_block] = fresh;
            ++p->refcount[fresh];
            p->unref(existing);
            p->bump_generation(fresh);
            plan.cloned.push_back(BlockClone{existing, fresh, (uint32_t)first_block});
        }
    }
    for (size_t b = first_block; b <= last_block; ++b) {
        if (row[b] != kInvalid) continue;
        uint32_t fresh = kInvalid;
        if (!p->pop_free(fresh)) {
            rollback_append(p, seq, plan);
            (void)p->upload_row(seq, first_block, last_block - first_block + 1);
            return pool_fail(MCU_ERROR_OUT_OF_MEMORY, "KV pool out of blocks");
        }
        row[b] = fresh;
        ++p->refcount[fresh];
        p->bump_generation(fresh);
        plan.new_blocks.push_back(BlockAlloc{fresh, (uint32_t)b});
    }
    for (size_t i = 0; i < token_count; ++i) {
        const size_t pos = start + i;
        out_slots[i] = (row[pos >> p->shift] << p->shift) | (uint32_t)(pos & p->mask);
    }
    *out_start_pos = start;
    plan.cookie = p->next_cookie++;
    out_plan->cookie = plan.cookie;
    p->plans[seq] = std::move(plan);
    p->pending[seq] = 1;
    return p->upload_row(seq, first_block, last_block - first_block + 1);
}

int mcu_kv_pool_commit_append(mcu_kv_pool_t *p, const mcu_kv_append_plan_t *plan) {
    if (p == nullptr || plan == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    if (plan->token_count == 0) return MCU_SUCCESS;
    const uint32_t seq = plan->seq;
    if (!p->seq_ok(seq) || !p->active[seq])
        return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool commit requires active sequence slot");
    if (!p->pending[seq] || p->plans[seq].cookie != plan->cookie || p->plans[seq].is_prefix)
        return pool_fail(MCU_ERROR_INVALID_OPERATION, "KV pool commit requires pending plan");
    if (p->seq_len[seq] != p->plans[seq].start_pos)
        return pool_fail(MCU_ERROR_INVALID_OPERATION, "KV pool commit start_pos mismatch");
    p->seq_len[seq] += p->plans[seq].token_count;
    p->pending[seq] = 0;
    p->plans[seq] = PendingPlan();
    return MCU_SUCCESS;
}

void mcu_kv_pool_abort_append(mcu_kv_pool_t *p, const mcu_kv_append_plan_t *plan) {
    if (p == nullptr || plan == nullptr || plan->token_count == 0) return;
    std::lock_guard<std::mutex> lock(p->mu);
    const uint32_t seq = plan->seq;
    if (!p->seq_ok(seq) || !p->active[seq] || !p->pending[seq]) return;
    if (p->plans[seq].cookie != plan->cookie || p->plans[seq].is_prefix) return;
    rollback_append(p, seq, p->plans[seq]);
    p->pending[seq] = 0;
    p->plans[seq] = PendingPlan();
    (void)p->upload_row(seq, 0, p->max_blocks_per_seq);
}

int mcu_kv_pool_prepare_prefix_attach(mcu_kv_pool_t *p, uint32_t seq, const uint32_t *block_ids, size_t num_blocks,
                                      size_t prefix_len, mcu_kv_prefix_plan_t *out_plan) {
    if (p == nullptr || out_plan == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    out_plan->seq = seq;
    out_plan->num_blocks = num_blocks;
    out_plan->prefix_len = prefix_len;
    out_plan->cookie = 0;
    if (!p->seq_ok(seq) || !p->active[seq])
        return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool prefix attach requires active sequence slot");
    if (p->pending[seq]) return pool_fail(MCU_ERROR_INVALID_OPERATION, "KV pool prefix attach requires no pending plan");
    if (p->swapped[seq]) return pool_fail(MCU_ERROR_INVALID_OPERATION, "KV pool prefix attach requires resident sequence");
    if (p->seq_len[seq] != 0) return pool_fail(MCU_ERROR_INVALID_OPERATION, "KV pool prefix attach requires empty sequence");
    if (num_blocks == 0) {
        if (prefix_len != 0) return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool prefix attach requires blocks for prefix_len");
        return MCU_SUCCESS;
    }
    if (block_ids == nullptr) return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool prefix attach requires block IDs");
    if (prefix_len == 0) return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool prefix attach requires prefix_len > 0");
    if (prefix_len > p->o.max_seq_len) return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool prefix attach exceeds max_seq_len");
    if ((prefix_len + p->o.block_size - 1) / p->o.block_size != num_blocks)
        return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool prefix attach block count mismatch");
    if (num_blocks > p->max_blocks_per_seq) return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool prefix attach exceeds block table");
    std::vector<uint8_t> seen(p->o.num_blocks, 0);
    for (size_t i = 0; i < num_blocks; ++i) {
        const uint32_t b = block_ids[i];
        if (b == kInvalid || b >= p->o.num_blocks) return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool prefix attach block ID invalid");
        if (seen[b]) return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool prefix attach has duplicate block ID");
        seen[b] = 1;
    }
    uint32_t *row = p->row(seq);
    std::fill(row, row + p->max_blocks_per_seq, kInvalid);
    PendingPlan plan;
    plan.is_prefix = true;
    plan.prefix_len = prefix_len;
    for (size_t i = 0; i < num_blocks; ++i) {
        const uint32_t b = block_ids[i];
        if (p->refcount[b] == 0) {
            (void)p->free_blocks.remove(b);
            (void)p->retained_free.remove(b);
        }
        row[i] = b;
        ++p->refcount[b];
        plan.prefix_blocks.push_back(b);
    }
    plan.cookie = p->next_cookie++;
    out_plan->cookie = plan.cookie;
    p->plans[seq] = std::move(plan);
    p->pending[seq] = 1;
    return p->upload_row(seq, 0, p->max_blocks_per_seq);
}

int mcu_kv_pool_commit_prefix_attach(mcu_kv_pool_t *p, const mcu_kv_prefix_plan_t *plan) {
    if (p == nullptr || plan == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    if (plan->num_blocks == 0) return MCU_SUCCESS;
    const uint32_t seq = plan->seq;
    if (!p->seq_ok(seq) || !p->active[seq])
        return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool commit requires active sequence slot");
    if (!p->pending[seq] || p->plans[seq].cookie != plan->cookie || !p->plans[seq].is_prefix)
        return pool_fail(MCU_ERROR_INVALID_OPERATION, "KV pool commit requires pending plan");
    p->seq_len[seq] = p->plans[seq].prefix_len;
    p->pending[seq] = 0;
    p->plans[seq] = PendingPlan();
    return MCU_SUCCESS;
}

void mcu_kv_pool_abort_prefix_attach(mcu_kv_pool_t *p, const mcu_kv_prefix_plan_t *plan) {
    if (p == nullptr || plan == nullptr || plan->num_blocks == 0) return;
    std::lock_guard<std::mutex> lock(p->mu);
    const uint32_t seq = plan->seq;
    if (!p->seq_ok(seq) || !p->active[seq] || !p->pending[seq]) return;
    if (p->plans[seq].cookie != plan->cookie || !p->plans[seq].is_prefix) return;
    uint32_t *row = p->row(seq);
    const std::vector<uint32_t> &blocks = p->plans[seq].prefix_blocks;
    for (size_t i = 0; i < blocks.size(); ++i) {
        row[i] = kInvalid;
        p->unref(blocks[i]);
    }
    p->pending[seq] = 0;
    p->plans[seq] = PendingPlan();
    (void)p->upload_row(seq, 0, p->max_blocks_per_seq);
}

int mcu_kv_pool_get_pointers(mcu_kv_pool_t *p, void **out_k_dev, void **out_v_dev, uint32_t **out_block_table_dev,
                             size_t *out_max_blocks_per_seq) {
    if (p == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    if (out_k_dev != nullptr) *out_k_dev = p->k_dev;
    if (out_v_dev != nullptr) *out_v_dev = p->v_dev;
    if (out_block_table_dev != nullptr) *out_block_table_dev = p->table_dev;
    if (out_max_blocks_per_seq != nullptr) *out_max_blocks_per_seq = p->max_blocks_per_seq;
    return MCU_SUCCESS;
}

size_t mcu_kv_pool_free_block_count(mcu_kv_pool_t *p) {
    if (p == nullptr) return 0;
    std::lock_guard<std::mutex> lock(p->mu);
    return p->free_blocks.count + p->retained_free.count;
}

size_t mcu_kv_pool_total_block_count(mcu_kv_pool_t *p) { return p == nullptr ? 0 : p->o.num_blocks; }

size_t mcu_kv_pool_seq_len(mcu_kv_pool_t *p, uint32_t seq) {
    if (p == nullptr) return 0;
    std::lock_guard<std::mutex> lock(p->mu);
    return p->seq_ok(seq) ? p->seq_len[seq] : 0;
}

uint32_t mcu_kv_pool_block_id(mcu_kv_pool_t *p, uint32_t seq, size_t logical_block) {
    if (p == nullptr) return kInvalid;
    std::lock_guard<std::mutex> lock(p->mu);
    if (!p->seq_ok(seq) || logical_block >= p->max_blocks_per_seq) return kInvalid;
    return p->row(seq)[logical_block];
}

uint32_t mcu_kv_pool_block_generation(mcu_kv_pool_t *p, uint32_t block_id) {
    if (p == nullptr) return 0;
    std::lock_guard<std::mutex> lock(p->mu);
    return block_id < p->generation.size() ? p->generation[block_id] : 0;
}

void mcu_kv_pool_set_block_retained(mcu_kv_pool_t *p, uint32_t b, int keep) {
    if (p == nullptr) return;
    std::lock_guard<std::mutex> lock(p->mu);
    if (b >= p->retained.size()) return;
    const uint8_t value = keep ? 1 : 0;
    if (p->retained[b] == value) return;
    p->retained[b] = value;
    if (p->refcount[b] != 0) return;
    if (keep) {
        (void)p->free_blocks.remove(b);
        p->retained_free.push(b);
    } else {
        (void)p->retained_free.remove(b);
        p->free_blocks.push(b);
    }
}

int mcu_kv_pool_is_seq_swapped(mcu_kv_pool_t *p, uint32_t seq, int *out_swapped) {
    if (p == nullptr || out_swapped == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    *out_swapped = p->seq_ok(seq) && p->swapped[seq] ? 1 : 0;
    return MCU_SUCCESS;
}

static int swap_precheck(mcu_kv_pool *p, uint32_t seq) {
    if (p->o.num_swap_blocks == 0) return pool_fail(MCU_ERROR_INVALID_OPERATION, "KV pool swap not configured");
    if (!p->seq_ok(seq) || !p->active[seq]) return pool_fail(MCU_ERROR_INVALID_ARGUMENT, "KV pool swap requires active sequence slot");
    if (p->pending[seq]) return pool_fail(MCU_ERROR_INVALID_OPERATION, "KV pool swap requires no pending plan");
    return MCU_SUCCESS;
}

int mcu_kv_pool_swap_out_seq(mcu_kv_pool_t *p, uint32_t seq) {
    if (p == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    if (int rc = swap_precheck(p, seq)) return rc;
    if (p->swapped[seq]) return MCU_SUCCESS;
    uint32_t *row = p->row(seq), *srow = p->swap_row(seq);
    std::fill(srow, srow + p->max_blocks_per_seq, kInvalid);
    struct Move {
        size_t logical;
        uint32_t dev, swap;
    };
    std::vector<Move> moves;
    auto undo = [&]() {
        for (const Move &m : moves) {
            p->swap_free.push(m.swap);
            srow[m.logical] = kInvalid;
        }
    };
    for (size_t b = 0; b < p->max_blocks_per_seq; ++b) {
        if (row[b] == kInvalid) continue;
        uint32_t sb = kInvalid;
        if (!p->swap_free.pop(sb)) {
            undo();
            return pool_fail(MCU_ERROR_OUT_OF_MEMORY, "KV pool swap out of host blocks");
        }
        if (int rc = p->save_block(sb, row[b])) {
            p->swap_free.push(sb);
            undo();
            return rc;
        }
        srow[b] = sb;
        moves.push_back(Move{b, row[b], sb});
    }
    if (moves.empty()) return MCU_SUCCESS;
    for (const Move &m : moves) {
        row[m.logical] = kInvalid;
        p->unref(m.dev);
    }
    p->swapped[seq] = 1;
    return p->upload_row(seq, 0, p->max_blocks_per_seq);
}

// No free device block: trade places with a resident sequence that owns (unshared, not retained) exactly as many
// blocks.  Each pair goes device -> spare, host -> device, spare -> host, in stream order.
static int swap_exchange(mcu_kv_pool *p, uint32_t seq) {
    uint32_t *row = p->row(seq), *srow = p->swap_row(seq);
    std::vector<size_t> target;
    for (size_t b = 0; b < p->max_blocks_per_seq; ++b)
        if (srow[b] != kInvalid) target.push_back(b);
    if (target.empty()) {
        p->swapped[seq] = 0;
        return MCU_SUCCESS;
    }
    uint32_t victim = (uint32_t)p->o.max_seqs;
    std::vector<size_t> victim_blocks;
    for (uint32_t cand = 0; cand < p->o.max_seqs; ++cand) {
        if (cand == seq || !p->active[cand] || p->pending[cand] || p->swapped[cand]) continue;
        const uint32_t *crow = p->row(cand);
        victim_blocks.clear();
        bool usable = true;
        for (size_t b = 0; b < p->max_blocks_per_seq && usable; ++b) {
            if (crow[b] == kInvalid) continue;
            if (crow[b] >= p->refcount.size() || p->refcount[crow[b]] != 1 || p->retained[crow[b]]) usable = false;
            else victim_blocks.push_back(b);
        }
        if (usable && victim_blocks.size() == target.size()) {
            victim = cand;
            break;
        }
    }
    if (victim == p->o.max_seqs) return pool_fail(MCU_ERROR_OUT_OF_MEMORY, "KV pool out of blocks");
    uint32_t *vrow = p->row(victim), *vsrow = p->swap_row(victim);
    const uint32_t spare = (uint32_t)p->o.num_blocks;
    std::fill(vsrow, vsrow + p->max_blocks_per_seq, kInvalid);
    for (size_t i = 0; i < target.size(); ++i) {
        const uint32_t dev_b = vrow[victim_blocks[i]], swap_b = srow[target[i]];
        int rc = p->clone_block(spare, dev_b);
        if (rc == MCU_SUCCESS) rc = p->load_block(dev_b, swap_b);
        if (rc == MCU_SUCCESS && p->k_dev != nullptr)
            rc = p->copy_blocks(p->swap_k + (size_t)swap_b * p->block_bytes, p->swap_v + (size_t)swap_b * p->block_bytes,
                                p->k_dev + (size_t)spare * p->block_bytes, p->v_dev + (size_t)spare * p->block_bytes,
                                cudaMemcpyDeviceToHost);
        if (rc != MCU_SUCCESS) return rc;  // a failed enqueue: the context is unusable, nothing to roll back to
        row[target[i]] = dev_b;
        srow[target[i]] = kInvalid;
        vrow[victim_blocks[i]] = kInvalid;
        vsrow[victim_blocks[i]] = swap_b;
        p->retained[dev_b] = 0;
        p->bump_generation(dev_b);
    }
    p->swapped[seq] = 0;
    p->swapped[victim] = 1;
    if (int rc = p->upload_row(victim, 0, p->max_blocks_per_seq)) return rc;
    return p->upload_row(seq, 0, p->max_blocks_per_seq);
}

int mcu_kv_pool_swap_in_seq(mcu_kv_pool_t *p, uint32_t seq) {
    if (p == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    if (int rc = swap_precheck(p, seq)) return rc;
    if (!p->swapped[seq]) return MCU_SUCCESS;
    uint32_t *row = p->row(seq), *srow = p->swap_row(seq);
    struct Move {
        size_t logical;
        uint32_t dev, swap;
    };
    std::vector<Move> moves;
    for (size_t b = 0; b < p->max_blocks_per_seq; ++b) {
        if (srow[b] == kInvalid) continue;
        if (row[b] != kInvalid) return pool_fail(MCU_ERROR_INVALID_OPERATION, "KV pool swap-in encountered resident block");
        uint32_t db = kInvalid;
        if (!p->pop_free(db)) {
            if (moves.empty() && swap_exchange(p, seq) == MCU_SUCCESS) return MCU_SUCCESS;
            for (const Move &m : moves) p->release_block(m.dev);
            return pool_fail(MCU_ERROR_OUT_OF_MEMORY, "KV pool out of blocks");
        }
        if (int rc = p->load_block(db, srow[b])) {
            p->release_block(db);
            for (const Move &m : moves) p->release_block(m.dev);
            return rc;
        }
        moves.push_back(Move{b, db, srow[b]});
    }
    for (const Move &m : moves) {
        row[m.logical] = m.dev;
        if (m.dev < p->refcount.size()) ++p->refcount[m.dev];
        p->bump_generation(m.dev);
        srow[m.logical] = kInvalid;
        p->swap_free.push(m.swap);
    }
    p->swapped[seq] = 0;
    return p->upload_row(seq, 0, p->max_blocks_per_seq);
}

}  // extern "C"
