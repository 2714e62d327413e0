// Paged KV-cache pool with HBM-resident blocks: what marmot_kv_pool_* (include/marmot/inference/kv_pool.h:65-101,
// src/inference/kv_pool/kv_pool.cpp) does for the reference's serving path, for a CUDA device.
//
// A scheduler that drives this pool sees the slots, block ids and error codes it would see from the reference's (the
// tests replay seeded schedules against traces of the reference pool): sequence slots and free blocks come back
// last-freed-first (lowest-id-first with the deterministic flag), blocks are reference counted so that sequences can
// share a prefix, a shared partially filled block is cloned before it is appended to, blocks marked "retained" are
// reused only when nothing else is free, and a sequence can be moved to host memory and back (trading places with a
// resident sequence of the same size when the device pool is full).
//
// How it is organised here:
//   * IdBag hands out ids (blocks, host swap blocks, sequence slots).  Two policies behind one interface: "latest"
//     (an array of the free ids and each id's position in it; taking a specific id out moves the top entry into
//     its place) and "lowest" (a two-level bitmap searched with count-trailing-zeros).
//   * A sequence's pending plan is a journal of block-table edits {logical block, id before, id after}.  Abort replays
//     the journal; commit forgets it.  Appends and prefix attaches differ only in what they write to the journal.
//   * Every table row that a call edits is noted in a RowSync, which uploads the touched span of each row to the
//     device copy of the table with one asynchronous copy on the context's stream when the call returns.  K and V
//     pools [blocks][layers][kv_heads][block_size][head_dim] are device allocations; copy-on-write clones are
//     device-to-device copies, swap blocks are page-locked host memory, and all of them ride the same stream: a block
//     that was just saved may be handed out at once, because whatever overwrites it is enqueued after the copy.  The
//     exchange path goes through one spare device block.  Nothing here waits for the device.
//   * A pool created without a context keeps books only (no storage): what a scheduler needs to plan admission.
#include "../../include/marmot_cuda.h"

#include "kernels.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

using namespace mcu;

namespace {

constexpr uint32_t NO_BLOCK = MCU_BLOCK_ID_INVALID;

class IdBag {
  public:
    void reset(size_t capacity, bool lowest_first) {
        lowest_ = lowest_first;
        n_ = 0;
        order_.clear();
        where_.clear();
        bits_.clear();
        summary_.clear();
        if (lowest_) {
            bits_.assign((capacity + 63) / 64, 0);
            summary_.assign((bits_.size() + 63) / 64, 0);
        } else {
            order_.reserve(capacity);
            where_.assign(capacity, -1);
        }
        cap_ = capacity;
    }
    // all ids, arranged so that they come out 0, 1, 2, ...
    void fill() {
        for (size_t i = cap_; i-- > 0;) put((uint32_t)i);
    }
    size_t size() const { return n_; }
    bool has(uint32_t id) const {
        if (id >= cap_) return false;
        return lowest_ ? ((bits_[id >> 6] >> (id & 63)) & 1u) != 0 : where_[id] >= 0;
    }
    void put(uint32_t id) {
        if (id >= cap_ || has(id)) return;
        if (lowest_) {
            bits_[id >> 6] |= 1ull << (id & 63);
            summary_[id >> 12] |= 1ull << ((id >> 6) & 63);
        } else {
            where_[id] = (int32_t)order_.size();
            order_.push_back(id);
        }
        ++n_;
    }
    bool take(uint32_t &id) {
        if (n_ == 0) return false;
        if (lowest_) {
            size_t s = 0;
            while (summary_[s] == 0) ++s;
            const size_t w = s * 64 + (size_t)__builtin_ctzll(summary_[s]);
            id = (uint32_t)(w * 64 + (size_t)__builtin_ctzll(bits_[w]));
        } else {
            id = order_.back();
        }
        return pull(id);
    }
    // a specific id leaves the bag
    bool pull(uint32_t id) {
        if (!has(id)) return false;
        if (lowest_) {
            bits_[id >> 6] &= ~(1ull << (id & 63));
            if (bits_[id >> 6] == 0) summary_[id >> 12] &= ~(1ull << ((id >> 6) & 63));
        } else {
            const uint32_t top = order_.back();
            order_[(size_t)where_[id]] = top;
            where_[top] = where_[id];
            order_.pop_back();
            where_[id] = -1;
        }
        --n_;
        return true;
    }

  private:
    bool lowest_ = false;
    size_t cap_ = 0, n_ = 0;
    std::vector<uint32_t> order_;   // "latest": the free ids, top at the back
    std::vector<int32_t> where_;    //           position of an id in order_, -1 when it is out
    std::vector<uint64_t> bits_, summary_;  // "lowest": one bit per id, one bit per non-empty word
};

struct Edit {
    uint32_t logical, before, after;
};
enum class PlanKind : uint8_t { None, Append, Prefix };
struct Plan {
    PlanKind kind = PlanKind::None;
    uint64_t cookie = 0;
    size_t first_pos = 0, tokens = 0;  // Append: where the tokens go; Prefix: tokens = the prefix length
    std::vector<Edit> journal;
};
struct Sequence {
    bool live = false, on_host = false;
    size_t length = 0;
    Plan plan;
};

}  // namespace

struct mcu_kv_pool {
    mcu_kv_pool_options_t o{};
    mcu_context_t *ctx = nullptr;
    size_t row_len = 0, block_bytes = 0;  // row_len: table entries per sequence
    uint32_t shift = 0, in_block = 0;

    uint8_t *k_dev = nullptr, *v_dev = nullptr;    // num_blocks + 1 blocks: the last one is the exchange spare
    uint32_t *table_dev = nullptr;
    uint8_t *host_k = nullptr, *host_v = nullptr;  // page-locked swap space
    std::vector<uint32_t> table, host_table;       // [max_seqs][row_len]: device block / swap block per logical block

    std::vector<Sequence> seqs;
    IdBag idle_seqs, idle_blocks, idle_kept, idle_host;  // idle_kept: free blocks marked "retained"
    struct BlockState {
        uint32_t users = 0, generation = 0;
        bool kept = false;
    };
    std::vector<BlockState> blocks;
    uint32_t generation_clock = 1;
    uint64_t cookie_clock = 1;
    std::mutex mu;

    cudaStream_t stream() const { return (cudaStream_t)mcu_context_get_stream(ctx); }
    uint32_t *row(uint32_t s) { return table.data() + (size_t)s * row_len; }
    uint32_t *host_row(uint32_t s) { return host_table.data() + (size_t)s * row_len; }
    Sequence *live_seq(uint32_t s) { return (size_t)s < seqs.size() && seqs[s].live ? &seqs[s] : nullptr; }

    // ---- block ledger ----
    void stamp(uint32_t b) {
        blocks[b].generation = generation_clock++;
        if (generation_clock == 0) generation_clock = 1;
    }
    void to_idle(uint32_t b) { (blocks[b].kept ? idle_kept : idle_blocks).put(b); }
    void drop_user(uint32_t b) {
        if (b < blocks.size() && blocks[b].users > 0 && --blocks[b].users == 0) to_idle(b);
    }
    void add_user(uint32_t b) {  // also for a block that had gone idle: it comes back out of the bags
        if (blocks[b].users == 0) {
            idle_blocks.pull(b);
            idle_kept.pull(b);
        }
        ++blocks[b].users;
    }
    bool fresh_block(uint32_t &b) {
        if (!idle_blocks.take(b) && !idle_kept.take(b)) return false;
        blocks[b].kept = false;
        return true;
    }
    // Take back a plan's table edits, in the order they were made.
    void undo_plan(uint32_t s, const Plan &plan) {
        uint32_t *r = row(s);
        for (const Edit &e : plan.journal) {
            r[e.logical] = e.before;
            drop_user(e.after);
            if (e.before != NO_BLOCK) add_user(e.before);
        }
    }

    // ---- data movement (asynchronous, on the context's stream) ----
    int move_block(uint8_t *dst_k, uint8_t *dst_v, const uint8_t *src_k, const uint8_t *src_v, cudaMemcpyKind kind) {
        if (k_dev == nullptr) return MCU_SUCCESS;  // books only
        cudaError_t e = cudaMemcpyAsync(dst_k, src_k, block_bytes, kind, stream());
        if (e == cudaSuccess) e = cudaMemcpyAsync(dst_v, src_v, block_bytes, kind, stream());
        return e == cudaSuccess ? MCU_SUCCESS : set_error(MCU_ERROR_INVALID_OPERATION, cudaGetErrorString(e));
    }
    size_t at(uint32_t b) const { return (size_t)b * block_bytes; }
    int device_to_device(uint32_t dst, uint32_t src) {
        return move_block(k_dev + at(dst), v_dev + at(dst), k_dev + at(src), v_dev + at(src), cudaMemcpyDeviceToDevice);
    }
    int device_to_host(uint32_t host_b, uint32_t dev_b) {
        return move_block(host_k + at(host_b), host_v + at(host_b), k_dev + at(dev_b), v_dev + at(dev_b), cudaMemcpyDeviceToHost);
    }
    int host_to_device(uint32_t dev_b, uint32_t host_b) {
        return move_block(k_dev + at(dev_b), v_dev + at(dev_b), host_k + at(host_b), host_v + at(host_b), cudaMemcpyHostToDevice);
    }
};

namespace {

// Notes which span of which table rows a call edited and uploads those spans when the call is over.
class RowSync {
  public:
    explicit RowSync(mcu_kv_pool *p) : p_(p) {}
    void touched(uint32_t seq, size_t first, size_t last) {  // inclusive
        for (Span &s : spans_)
            if (s.seq == seq) {
                s.first = std::min(s.first, first);
                s.last = std::max(s.last, last);
                return;
            }
        spans_.push_back(Span{seq, first, last});
    }
    void whole(uint32_t seq) { touched(seq, 0, p_->row_len - 1); }
    // status in, status out: an upload failure only shows when the call itself succeeded
    int finish(int rc) {
        if (p_->table_dev != nullptr)
            for (const Span &s : spans_) {
                const size_t off = (size_t)s.seq * p_->row_len + s.first;
                const cudaError_t e = cudaMemcpyAsync(p_->table_dev + off, p_->table.data() + off,
                                                      (s.last - s.first + 1) * sizeof(uint32_t), cudaMemcpyHostToDevice, p_->stream());
                if (e != cudaSuccess && rc == MCU_SUCCESS) rc = set_error(MCU_ERROR_INVALID_OPERATION, cudaGetErrorString(e));
            }
        spans_.clear();
        return rc;
    }

  private:
    struct Span {
        uint32_t seq;
        size_t first, last;
    };
    mcu_kv_pool *p_;
    std::vector<Span> spans_;
};

int refuse(int code, const char *why) { return set_error(code, why); }

}  // namespace

extern "C" {

int mcu_kv_pool_options_init(mcu_kv_pool_options_t *opts) {
    if (opts == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    *opts = mcu_kv_pool_options_t{};
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
    const size_t dims[] = {opts->max_seqs, opts->max_seq_len, opts->block_size, opts->num_blocks,
                           opts->num_layers, opts->num_kv_heads, opts->head_dim};
    for (size_t d : dims)
        if (d == 0) return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: every size in the options must be at least 1");
    if (opts->block_size < 2 || (opts->block_size & (opts->block_size - 1)) != 0)
        return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: block_size must be 2, 4, 8, ...");
    if (opts->kv_dtype != MCU_KV_F32 && opts->kv_dtype != MCU_KV_F16)
        return refuse(MCU_ERROR_UNSUPPORTED_DTYPE, "kv pool: K/V are stored as f32 or f16");
    if (opts->num_blocks >= (size_t)NO_BLOCK || opts->num_swap_blocks >= (size_t)NO_BLOCK)
        return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: more blocks than 32-bit block ids");
    uint32_t shift = 0;
    while (((size_t)1 << shift) < opts->block_size) ++shift;
    if (opts->num_blocks > (((size_t)NO_BLOCK) >> shift))
        return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: more token slots than 32-bit slot numbers");
    mcu_kv_pool *p = new (std::nothrow) mcu_kv_pool();
    if (p == nullptr) return refuse(MCU_ERROR_OUT_OF_MEMORY, "kv pool: no host memory for the books");
    p->o = *opts;
    p->ctx = ctx;
    p->shift = shift;
    p->in_block = (1u << shift) - 1u;
    p->row_len = (opts->max_seq_len + opts->block_size - 1) / opts->block_size;
    p->block_bytes = opts->num_layers * opts->num_kv_heads * opts->block_size * opts->head_dim * (opts->kv_dtype == MCU_KV_F16 ? 2 : 4);
    const bool lowest = (opts->flags & MCU_KV_POOL_FLAG_DETERMINISTIC_ALLOC) != 0;
    p->table.assign(opts->max_seqs * p->row_len, NO_BLOCK);
    p->host_table = p->table;
    p->seqs.resize(opts->max_seqs);
    p->blocks.resize(opts->num_blocks);
    p->idle_seqs.reset(opts->max_seqs, false);  // sequence slots are always reused latest-first
    p->idle_seqs.fill();
    p->idle_blocks.reset(opts->num_blocks, lowest);
    p->idle_blocks.fill();
    p->idle_kept.reset(opts->num_blocks, lowest);
    p->idle_host.reset(opts->num_swap_blocks, lowest);
    p->idle_host.fill();
    if (ctx != nullptr) {
        const size_t pool_bytes = (opts->num_blocks + 1) * p->block_bytes;  // + the exchange spare
        const size_t table_bytes = p->table.size() * sizeof(uint32_t);
        cudaError_t e = cudaSetDevice(context_device(ctx));
        if (e == cudaSuccess) e = cudaMalloc(&p->k_dev, pool_bytes);
        if (e == cudaSuccess) e = cudaMalloc(&p->v_dev, pool_bytes);
        if (e == cudaSuccess) e = cudaMalloc(&p->table_dev, table_bytes);
        if (e == cudaSuccess) e = cudaMemsetAsync(p->k_dev, 0, pool_bytes, p->stream());
        if (e == cudaSuccess) e = cudaMemsetAsync(p->v_dev, 0, pool_bytes, p->stream());
        if (e == cudaSuccess) e = cudaMemsetAsync(p->table_dev, 0xFF, table_bytes, p->stream());
        if (e == cudaSuccess && opts->num_swap_blocks > 0) {
            e = cudaHostAlloc(&p->host_k, opts->num_swap_blocks * p->block_bytes, cudaHostAllocDefault);
            if (e == cudaSuccess) e = cudaHostAlloc(&p->host_v, opts->num_swap_blocks * p->block_bytes, cudaHostAllocDefault);
        }
        if (e != cudaSuccess) {
            const int rc = refuse(e == cudaErrorMemoryAllocation ? MCU_ERROR_OUT_OF_MEMORY : MCU_ERROR_INVALID_OPERATION,
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
        (void)cudaStreamSynchronize(p->stream());  // copies of this pool may still be in flight
        if (p->k_dev != nullptr) cudaFree(p->k_dev);
        if (p->v_dev != nullptr) cudaFree(p->v_dev);
        if (p->table_dev != nullptr) cudaFree(p->table_dev);
        if (p->host_k != nullptr) cudaFreeHost(p->host_k);
        if (p->host_v != nullptr) cudaFreeHost(p->host_v);
    }
    delete p;
}

int mcu_kv_pool_acquire_seq(mcu_kv_pool_t *p, uint32_t *out_seq) {
    if (p == nullptr || out_seq == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    uint32_t s;
    if (!p->idle_seqs.take(s)) return refuse(MCU_ERROR_OUT_OF_MEMORY, "kv pool: every sequence slot is taken");
    p->seqs[s] = Sequence{};
    p->seqs[s].live = true;
    std::fill_n(p->row(s), p->row_len, NO_BLOCK);
    std::fill_n(p->host_row(s), p->row_len, NO_BLOCK);
    *out_seq = s;
    RowSync sync(p);
    sync.whole(s);
    return sync.finish(MCU_SUCCESS);
}

int mcu_kv_pool_release_seq(mcu_kv_pool_t *p, uint32_t s) {
    if (p == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    Sequence *q = p->live_seq(s);
    if (q == nullptr) return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: release of a slot that is not in use");
    if (q->plan.kind != PlanKind::None) return refuse(MCU_ERROR_INVALID_OPERATION, "kv pool: release while a plan is open");
    if (q->on_host) {
        uint32_t *hr = p->host_row(s);
        for (size_t i = 0; i < p->row_len; ++i)
            if (hr[i] != NO_BLOCK) {
                p->idle_host.put(hr[i]);
                hr[i] = NO_BLOCK;
            }
    }
    uint32_t *r = p->row(s);
    for (size_t i = 0; i < p->row_len; ++i)
        if (r[i] != NO_BLOCK) {
            p->drop_user(r[i]);
            r[i] = NO_BLOCK;
        }
    *q = Sequence{};
    p->idle_seqs.put(s);
    RowSync sync(p);
    sync.whole(s);
    return sync.finish(MCU_SUCCESS);
}

int mcu_kv_pool_prepare_append(mcu_kv_pool_t *p, uint32_t s, size_t token_count, mcu_kv_append_plan_t *out_plan,
                               uint32_t *out_slots, size_t *out_start_pos) {
    if (p == nullptr || out_plan == nullptr || out_start_pos == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    *out_plan = mcu_kv_append_plan_t{};
    out_plan->seq = s;
    out_plan->token_count = token_count;
    *out_start_pos = 0;
    Sequence *q = p->live_seq(s);
    if (q == nullptr) return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: append to a slot that is not in use");
    if (q->plan.kind != PlanKind::None) return refuse(MCU_ERROR_INVALID_OPERATION, "kv pool: the sequence already has an open plan");
    if (q->on_host) return refuse(MCU_ERROR_INVALID_OPERATION, "kv pool: the sequence is swapped out");
    if (token_count == 0) {
        *out_start_pos = q->length;
        return MCU_SUCCESS;
    }
    if (out_slots == nullptr) return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: nowhere to write the token slots");
    const size_t from = q->length;
    if (from > p->o.max_seq_len) return refuse(MCU_ERROR_INVALID_OPERATION, "kv pool: the sequence is longer than max_seq_len");
    if (token_count > p->o.max_seq_len - from) return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: the append would pass max_seq_len");
    const size_t lb0 = from >> p->shift, lb1 = (from + token_count - 1) >> p->shift;
    if (lb1 >= p->row_len) return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: the append would pass the block table");
    uint32_t *r = p->row(s);
    Plan plan;
    plan.kind = PlanKind::Append;
    plan.first_pos = from;
    plan.tokens = token_count;
    RowSync sync(p);
    sync.touched(s, lb0, lb1);
    // the append continues inside a block that another sequence also reads: give this one a private copy first
    const uint32_t tail = r[lb0];
    if ((from & p->in_block) != 0 && tail != NO_BLOCK && tail < p->blocks.size() && p->blocks[tail].users > 1) {
        uint32_t copy;
        if (!p->fresh_block(copy)) return refuse(MCU_ERROR_OUT_OF_MEMORY, "kv pool: no free block");
        if (int rc = p->device_to_device(copy, tail)) {
            p->to_idle(copy);
            return rc;
        }
        r[lb0] = copy;
        ++p->blocks[copy].users;
        p->drop_user(tail);
        p->stamp(copy);
        plan.journal.push_back(Edit{(uint32_t)lb0, tail, copy});
    }
    for (size_t lb = lb0; lb <= lb1; ++lb) {
        if (r[lb] != NO_BLOCK) continue;
        uint32_t b;
        if (!p->fresh_block(b)) {
            p->undo_plan(s, plan);
            return sync.finish(refuse(MCU_ERROR_OUT_OF_MEMORY, "kv pool: no free block"));
        }
        r[lb] = b;
        ++p->blocks[b].users;
        p->stamp(b);
        plan.journal.push_back(Edit{(uint32_t)lb, NO_BLOCK, b});
    }
    for (size_t i = 0; i < token_count; ++i) {
        const size_t pos = from + i;
        out_slots[i] = (r[pos >> p->shift] << p->shift) | (uint32_t)(pos & p->in_block);
    }
    *out_start_pos = from;
    plan.cookie = p->cookie_clock++;
    out_plan->cookie = plan.cookie;
    q->plan = std::move(plan);
    return sync.finish(MCU_SUCCESS);
}

// The open plan of `s` if it is of `kind` and carries `cookie`; sets *code to why not otherwise.
static Plan *open_plan(mcu_kv_pool *p, uint32_t s, uint64_t cookie, PlanKind kind, int *code) {
    Sequence *q = p->live_seq(s);
    if (q == nullptr) {
        *code = MCU_ERROR_INVALID_ARGUMENT;
        return nullptr;
    }
    if (q->plan.kind != kind || q->plan.cookie != cookie) {
        *code = MCU_ERROR_INVALID_OPERATION;
        return nullptr;
    }
    return &q->plan;
}

int mcu_kv_pool_commit_append(mcu_kv_pool_t *p, const mcu_kv_append_plan_t *plan) {
    if (p == nullptr || plan == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    if (plan->token_count == 0) return MCU_SUCCESS;
    int code = MCU_SUCCESS;
    Plan *open = open_plan(p, plan->seq, plan->cookie, PlanKind::Append, &code);
    if (open == nullptr) return refuse(code, "kv pool: commit without a matching open append plan");
    Sequence &q = p->seqs[plan->seq];
    if (q.length != open->first_pos) return refuse(MCU_ERROR_INVALID_OPERATION, "kv pool: the sequence moved since the plan was made");
    q.length += open->tokens;
    q.plan = Plan{};
    return MCU_SUCCESS;
}

void mcu_kv_pool_abort_append(mcu_kv_pool_t *p, const mcu_kv_append_plan_t *plan) {
    if (p == nullptr || plan == nullptr || plan->token_count == 0) return;
    std::lock_guard<std::mutex> lock(p->mu);
    int code;
    Plan *open = open_plan(p, plan->seq, plan->cookie, PlanKind::Append, &code);
    if (open == nullptr) return;
    p->undo_plan(plan->seq, *open);
    *open = Plan{};
    RowSync sync(p);
    sync.whole(plan->seq);
    (void)sync.finish(MCU_SUCCESS);
}

int mcu_kv_pool_prepare_prefix_attach(mcu_kv_pool_t *p, uint32_t s, const uint32_t *block_ids, size_t num_blocks,
                                      size_t prefix_len, mcu_kv_prefix_plan_t *out_plan) {
    if (p == nullptr || out_plan == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    *out_plan = mcu_kv_prefix_plan_t{};
    out_plan->seq = s;
    out_plan->num_blocks = num_blocks;
    out_plan->prefix_len = prefix_len;
    Sequence *q = p->live_seq(s);
    if (q == nullptr) return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: prefix for a slot that is not in use");
    if (q->plan.kind != PlanKind::None) return refuse(MCU_ERROR_INVALID_OPERATION, "kv pool: the sequence already has an open plan");
    if (q->on_host) return refuse(MCU_ERROR_INVALID_OPERATION, "kv pool: the sequence is swapped out");
    if (q->length != 0) return refuse(MCU_ERROR_INVALID_OPERATION, "kv pool: a prefix can only start an empty sequence");
    if (num_blocks == 0)
        return prefix_len == 0 ? MCU_SUCCESS : refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: a prefix length without blocks");
    if (block_ids == nullptr) return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: no block ids given");
    if (prefix_len == 0) return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: blocks without a prefix length");
    if (prefix_len > p->o.max_seq_len) return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: the prefix is longer than max_seq_len");
    if (((prefix_len + p->in_block) >> p->shift) != num_blocks)
        return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: the prefix length does not fill that many blocks");
    if (num_blocks > p->row_len) return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: more prefix blocks than table entries");
    for (size_t i = 0; i < num_blocks; ++i) {
        if (block_ids[i] == NO_BLOCK || block_ids[i] >= p->blocks.size())
            return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: a prefix block id is out of range");
        for (size_t j = 0; j < i; ++j)
            if (block_ids[j] == block_ids[i]) return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: a prefix block is listed twice");
    }
    uint32_t *r = p->row(s);
    std::fill_n(r, p->row_len, NO_BLOCK);
    Plan plan;
    plan.kind = PlanKind::Prefix;
    plan.tokens = prefix_len;
    for (size_t i = 0; i < num_blocks; ++i) {
        p->add_user(block_ids[i]);
        r[i] = block_ids[i];
        plan.journal.push_back(Edit{(uint32_t)i, NO_BLOCK, block_ids[i]});
    }
    plan.cookie = p->cookie_clock++;
    out_plan->cookie = plan.cookie;
    q->plan = std::move(plan);
    RowSync sync(p);
    sync.whole(s);
    return sync.finish(MCU_SUCCESS);
}

int mcu_kv_pool_commit_prefix_attach(mcu_kv_pool_t *p, const mcu_kv_prefix_plan_t *plan) {
    if (p == nullptr || plan == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    if (plan->num_blocks == 0) return MCU_SUCCESS;
    int code = MCU_SUCCESS;
    Plan *open = open_plan(p, plan->seq, plan->cookie, PlanKind::Prefix, &code);
    if (open == nullptr) return refuse(code, "kv pool: commit without a matching open prefix plan");
    p->seqs[plan->seq].length = open->tokens;
    *open = Plan{};
    return MCU_SUCCESS;
}

void mcu_kv_pool_abort_prefix_attach(mcu_kv_pool_t *p, const mcu_kv_prefix_plan_t *plan) {
    if (p == nullptr || plan == nullptr || plan->num_blocks == 0) return;
    std::lock_guard<std::mutex> lock(p->mu);
    int code;
    Plan *open = open_plan(p, plan->seq, plan->cookie, PlanKind::Prefix, &code);
    if (open == nullptr) return;
    p->undo_plan(plan->seq, *open);
    *open = Plan{};
    RowSync sync(p);
    sync.whole(plan->seq);
    (void)sync.finish(MCU_SUCCESS);
}

int mcu_kv_pool_get_pointers(mcu_kv_pool_t *p, void **out_k_dev, void **out_v_dev, uint32_t **out_block_table_dev,
                             size_t *out_max_blocks_per_seq) {
    if (p == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    if (out_k_dev != nullptr) *out_k_dev = p->k_dev;
    if (out_v_dev != nullptr) *out_v_dev = p->v_dev;
    if (out_block_table_dev != nullptr) *out_block_table_dev = p->table_dev;
    if (out_max_blocks_per_seq != nullptr) *out_max_blocks_per_seq = p->row_len;
    return MCU_SUCCESS;
}

size_t mcu_kv_pool_free_block_count(mcu_kv_pool_t *p) {
    if (p == nullptr) return 0;
    std::lock_guard<std::mutex> lock(p->mu);
    return p->idle_blocks.size() + p->idle_kept.size();
}

size_t mcu_kv_pool_total_block_count(mcu_kv_pool_t *p) { return p == nullptr ? 0 : p->o.num_blocks; }

size_t mcu_kv_pool_seq_len(mcu_kv_pool_t *p, uint32_t s) {
    if (p == nullptr) return 0;
    std::lock_guard<std::mutex> lock(p->mu);
    return (size_t)s < p->seqs.size() ? p->seqs[s].length : 0;
}

uint32_t mcu_kv_pool_block_id(mcu_kv_pool_t *p, uint32_t s, size_t logical_block) {
    if (p == nullptr) return NO_BLOCK;
    std::lock_guard<std::mutex> lock(p->mu);
    if ((size_t)s >= p->seqs.size() || logical_block >= p->row_len) return NO_BLOCK;
    return p->row(s)[logical_block];
}

uint32_t mcu_kv_pool_block_generation(mcu_kv_pool_t *p, uint32_t b) {
    if (p == nullptr) return 0;
    std::lock_guard<std::mutex> lock(p->mu);
    return b < p->blocks.size() ? p->blocks[b].generation : 0;
}

void mcu_kv_pool_set_block_retained(mcu_kv_pool_t *p, uint32_t b, int keep) {
    if (p == nullptr) return;
    std::lock_guard<std::mutex> lock(p->mu);
    if (b >= p->blocks.size() || p->blocks[b].kept == (keep != 0)) return;
    const bool idle = p->blocks[b].users == 0;
    if (idle) (p->blocks[b].kept ? p->idle_kept : p->idle_blocks).pull(b);
    p->blocks[b].kept = keep != 0;
    if (idle) p->to_idle(b);
}

int mcu_kv_pool_is_seq_swapped(mcu_kv_pool_t *p, uint32_t s, int *out_swapped) {
    if (p == nullptr || out_swapped == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    *out_swapped = (size_t)s < p->seqs.size() && p->seqs[s].on_host ? 1 : 0;
    return MCU_SUCCESS;
}

// Common refusals of the two swap directions; *q is the sequence when the answer is MCU_SUCCESS.
static int swappable(mcu_kv_pool *p, uint32_t s, Sequence **q) {
    if (p->o.num_swap_blocks == 0) return refuse(MCU_ERROR_INVALID_OPERATION, "kv pool: created without swap blocks");
    *q = p->live_seq(s);
    if (*q == nullptr) return refuse(MCU_ERROR_INVALID_ARGUMENT, "kv pool: swap of a slot that is not in use");
    if ((*q)->plan.kind != PlanKind::None) return refuse(MCU_ERROR_INVALID_OPERATION, "kv pool: swap while a plan is open");
    return MCU_SUCCESS;
}

int mcu_kv_pool_swap_out_seq(mcu_kv_pool_t *p, uint32_t s) {
    if (p == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    Sequence *q;
    if (int rc = swappable(p, s, &q)) return rc;
    if (q->on_host) return MCU_SUCCESS;
    uint32_t *r = p->row(s), *hr = p->host_row(s);
    std::fill_n(hr, p->row_len, NO_BLOCK);
    // first find a host block for, and enqueue the copy of, every block; only then let the device blocks go
    int rc = MCU_SUCCESS;
    size_t moved = 0;
    for (size_t lb = 0; lb < p->row_len && rc == MCU_SUCCESS; ++lb) {
        if (r[lb] == NO_BLOCK) continue;
        uint32_t hb;
        if (!p->idle_host.take(hb)) {
            rc = refuse(MCU_ERROR_OUT_OF_MEMORY, "kv pool: no free swap block");
        } else if ((rc = p->device_to_host(hb, r[lb])) != MCU_SUCCESS) {
            p->idle_host.put(hb);
        } else {
            hr[lb] = hb;
            ++moved;
        }
    }
    if (rc != MCU_SUCCESS) {  // hand the host blocks back in the order they were taken
        for (size_t lb = 0; lb < p->row_len; ++lb)
            if (hr[lb] != NO_BLOCK) {
                p->idle_host.put(hr[lb]);
                hr[lb] = NO_BLOCK;
            }
        return rc;
    }
    if (moved == 0) return MCU_SUCCESS;
    for (size_t lb = 0; lb < p->row_len; ++lb)
        if (r[lb] != NO_BLOCK) {
            p->drop_user(r[lb]);
            r[lb] = NO_BLOCK;
        }
    q->on_host = true;
    RowSync sync(p);
    sync.whole(s);
    return sync.finish(MCU_SUCCESS);
}

// No free device block: trade places with a resident sequence that owns (alone, not retained) exactly as many blocks.
// Each pair goes device -> spare, host -> device, spare -> host, in stream order.
static int trade_places(mcu_kv_pool *p, uint32_t s) {
    uint32_t *r = p->row(s), *hr = p->host_row(s);
    std::vector<uint32_t> mine;  // logical blocks of s that are on the host
    for (size_t lb = 0; lb < p->row_len; ++lb)
        if (hr[lb] != NO_BLOCK) mine.push_back((uint32_t)lb);
    if (mine.empty()) {
        p->seqs[s].on_host = false;
        return MCU_SUCCESS;
    }
    std::vector<uint32_t> theirs;
    uint32_t other = 0;
    bool found = false;
    for (; other < p->seqs.size() && !found; ++other) {
        const Sequence &c = p->seqs[other];
        if (other == s || !c.live || c.on_host || c.plan.kind != PlanKind::None) continue;
        const uint32_t *cr = p->row(other);
        theirs.clear();
        bool sole_owner = true;
        for (size_t lb = 0; lb < p->row_len && sole_owner; ++lb) {
            if (cr[lb] == NO_BLOCK) continue;
            sole_owner = cr[lb] < p->blocks.size() && p->blocks[cr[lb]].users == 1 && !p->blocks[cr[lb]].kept;
            theirs.push_back((uint32_t)lb);
        }
        found = sole_owner && theirs.size() == mine.size();
    }
    if (!found) return refuse(MCU_ERROR_OUT_OF_MEMORY, "kv pool: no free block");
    --other;  // the loop stepped past it
    uint32_t *orow = p->row(other), *ohr = p->host_row(other);
    const uint32_t spare = (uint32_t)p->o.num_blocks;
    std::fill_n(ohr, p->row_len, NO_BLOCK);
    for (size_t i = 0; i < mine.size(); ++i) {
        const uint32_t dev_b = orow[theirs[i]], host_b = hr[mine[i]];
        int rc = p->device_to_device(spare, dev_b);
        if (rc == MCU_SUCCESS) rc = p->host_to_device(dev_b, host_b);
        if (rc == MCU_SUCCESS) rc = p->device_to_host(host_b, spare);
        if (rc != MCU_SUCCESS) return rc;  // a failed enqueue: the context is unusable, nothing to go back to
        r[mine[i]] = dev_b;
        hr[mine[i]] = NO_BLOCK;
        orow[theirs[i]] = NO_BLOCK;
        ohr[theirs[i]] = host_b;
        p->blocks[dev_b].kept = false;
        p->stamp(dev_b);
    }
    p->seqs[s].on_host = false;
    p->seqs[other].on_host = true;
    RowSync sync(p);
    sync.whole(other);
    sync.whole(s);
    return sync.finish(MCU_SUCCESS);
}

int mcu_kv_pool_swap_in_seq(mcu_kv_pool_t *p, uint32_t s) {
    if (p == nullptr) return MCU_ERROR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(p->mu);
    Sequence *q;
    if (int rc = swappable(p, s, &q)) return rc;
    if (!q->on_host) return MCU_SUCCESS;
    uint32_t *r = p->row(s), *hr = p->host_row(s);
    std::vector<Edit> landed;  // {logical, host block, device block}
    auto give_back = [&]() {
        for (const Edit &e : landed) p->to_idle(e.after);
    };
    for (size_t lb = 0; lb < p->row_len; ++lb) {
        if (hr[lb] == NO_BLOCK) continue;
        if (r[lb] != NO_BLOCK) return refuse(MCU_ERROR_INVALID_OPERATION, "kv pool: a swapped-out sequence still holds a device block");
        uint32_t b;
        if (!p->fresh_block(b)) {
            if (landed.empty() && trade_places(p, s) == MCU_SUCCESS) return MCU_SUCCESS;
            give_back();
            return refuse(MCU_ERROR_OUT_OF_MEMORY, "kv pool: no free block");
        }
        if (int rc = p->host_to_device(b, hr[lb])) {
            p->to_idle(b);
            give_back();
            return rc;
        }
        landed.push_back(Edit{(uint32_t)lb, hr[lb], b});
    }
    for (const Edit &e : landed) {
        r[e.logical] = e.after;
        ++p->blocks[e.after].users;
        p->stamp(e.after);
        hr[e.logical] = NO_BLOCK;
        p->idle_host.put(e.before);
    }
    q->on_host = false;
    RowSync sync(p);
    sync.whole(s);
    return sync.finish(MCU_SUCCESS);
}

}  // extern "C"
