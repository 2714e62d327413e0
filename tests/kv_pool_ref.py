"""ctypes binding of the reference's own KV-cache pool (marmot_kv_pool_*, built by oracle/build_ref.py) and a
recorder that drives any pool with a seeded random operation sequence (tests only)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from oracle import build_ref


class _RefOptions(C.Structure):
    """marmot_kv_pool_options_t, include/marmot/inference/kv_pool.h:29-50."""
    _fields_ = [("struct_size", C.c_uint32), ("struct_version", C.c_uint32), ("flags", C.c_uint64),
                ("backend", C.c_int), ("max_seqs", C.c_size_t), ("max_seq_len", C.c_size_t), ("block_size", C.c_size_t),
                ("num_blocks", C.c_size_t), ("num_swap_blocks", C.c_size_t), ("num_layers", C.c_size_t),
                ("num_kv_heads", C.c_size_t), ("head_dim", C.c_size_t), ("kv_dtype", C.c_int), ("pnext", C.c_void_p),
                ("reserved", C.c_uint64 * 4)]


class _RefAppendPlan(C.Structure):
    _fields_ = [("seq", C.c_uint32), ("token_count", C.c_size_t), ("cookie", C.c_uint64)]


class _RefPrefixPlan(C.Structure):
    _fields_ = [("seq", C.c_uint32), ("num_blocks", C.c_size_t), ("prefix_len", C.c_size_t), ("cookie", C.c_uint64)]


class RefKvPool:
    """Same method surface as marmot_b200.runtime.KvPool, on the reference's CPU pool."""

    def __init__(self, reference, *, max_seqs, max_seq_len, block_size, num_blocks, num_swap_blocks=0, num_layers=1,
                 num_kv_heads=1, head_dim=64, kv_f16=True, deterministic=False):
        C.CDLL(str(build_ref.OUT_LIB), mode=C.RTLD_GLOBAL)
        self.lib = L = C.CDLL(str(build_ref.KV_POOL_LIB))
        vp, sz, u32 = C.c_void_p, C.c_size_t, C.c_uint32
        L.marmot_kv_pool_create.argtypes = [vp, C.POINTER(_RefOptions), C.POINTER(vp)]
        L.marmot_kv_pool_destroy.argtypes = [vp]
        L.marmot_kv_pool_destroy.restype = None
        L.marmot_kv_pool_acquire_seq.argtypes = [vp, C.POINTER(u32)]
        L.marmot_kv_pool_release_seq.argtypes = [vp, u32]
        L.marmot_kv_pool_prepare_append.argtypes = [vp, u32, sz, C.POINTER(_RefAppendPlan), C.POINTER(u32), C.POINTER(sz)]
        L.marmot_kv_pool_commit_append.argtypes = [vp, C.POINTER(_RefAppendPlan)]
        L.marmot_kv_pool_abort_append.argtypes = [vp, C.POINTER(_RefAppendPlan)]
        L.marmot_kv_pool_abort_append.restype = None
        L.marmot_kv_pool_prepare_prefix_attach.argtypes = [vp, u32, C.POINTER(u32), sz, sz, C.POINTER(_RefPrefixPlan)]
        L.marmot_kv_pool_commit_prefix_attach.argtypes = [vp, C.POINTER(_RefPrefixPlan)]
        L.marmot_kv_pool_abort_prefix_attach.argtypes = [vp, C.POINTER(_RefPrefixPlan)]
        L.marmot_kv_pool_abort_prefix_attach.restype = None
        L.marmot_kv_pool_get_tensors.argtypes = [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp)]
        L.marmot_kv_pool_free_block_count.argtypes = [vp]
        L.marmot_kv_pool_free_block_count.restype = sz
        L.marmot_kv_pool_total_block_count.argtypes = [vp]
        L.marmot_kv_pool_total_block_count.restype = sz
        L.marmot_kv_pool_swap_out_seq.argtypes = [vp, u32]
        L.marmot_kv_pool_swap_in_seq.argtypes = [vp, u32]
        L.marmot_kv_pool_is_seq_swapped.argtypes = [vp, u32, C.POINTER(C.c_bool)]
        opts = _RefOptions()
        L.marmot_kv_pool_options_init(C.byref(opts))
        opts.flags = 1 if deterministic else 0
        opts.backend = 0  # MARMOT_BACKEND_CPU
        opts.max_seqs, opts.max_seq_len, opts.block_size = max_seqs, max_seq_len, block_size
        opts.num_blocks, opts.num_swap_blocks = num_blocks, num_swap_blocks
        opts.num_layers, opts.num_kv_heads, opts.head_dim = num_layers, num_kv_heads, head_dim
        opts.kv_dtype = 1 if kv_f16 else 0  # MARMOT_DTYPE_FLOAT16 / FLOAT32
        self.max_blocks_per_seq = (max_seq_len + block_size - 1) // block_size
        self.max_seqs = max_seqs
        h = vp()
        rc = L.marmot_kv_pool_create(reference.ctx, C.byref(opts), C.byref(h))
        if rc != 0:
            raise RuntimeError(f"marmot_kv_pool_create: {rc}")
        self.handle = h
        self._tensor_type = None

    def close(self):
        if self.handle:
            self.lib.marmot_kv_pool_destroy(self.handle)
            self.handle = None

    def acquire_seq(self):
        seq = C.c_uint32(0xFFFFFFFF)
        rc = self.lib.marmot_kv_pool_acquire_seq(self.handle, C.byref(seq))
        return rc, seq.value

    def release_seq(self, seq):
        return self.lib.marmot_kv_pool_release_seq(self.handle, seq)

    def prepare_append(self, seq, n):
        plan, slots, start = _RefAppendPlan(), (C.c_uint32 * max(n, 1))(), C.c_size_t(0)
        rc = self.lib.marmot_kv_pool_prepare_append(self.handle, seq, n, C.byref(plan), slots, C.byref(start))
        return rc, plan, list(slots[:n]) if rc == 0 else [], start.value

    def commit_append(self, plan):
        return self.lib.marmot_kv_pool_commit_append(self.handle, C.byref(plan))

    def abort_append(self, plan):
        self.lib.marmot_kv_pool_abort_append(self.handle, C.byref(plan))

    def prepare_prefix_attach(self, seq, block_ids, prefix_len):
        plan = _RefPrefixPlan()
        ids = (C.c_uint32 * max(len(block_ids), 1))(*block_ids)
        rc = self.lib.marmot_kv_pool_prepare_prefix_attach(self.handle, seq, ids, len(block_ids), prefix_len, C.byref(plan))
        return rc, plan

    def commit_prefix_attach(self, plan):
        return self.lib.marmot_kv_pool_commit_prefix_attach(self.handle, C.byref(plan))

    def abort_prefix_attach(self, plan):
        self.lib.marmot_kv_pool_abort_prefix_attach(self.handle, C.byref(plan))

    def free_block_count(self):
        return self.lib.marmot_kv_pool_free_block_count(self.handle)

    def total_block_count(self):
        return self.lib.marmot_kv_pool_total_block_count(self.handle)

    def swap_out(self, seq):
        return self.lib.marmot_kv_pool_swap_out_seq(self.handle, seq)

    def swap_in(self, seq):
        return self.lib.marmot_kv_pool_swap_in_seq(self.handle, seq)

    def is_swapped(self, seq):
        out = C.c_bool(False)
        self.lib.marmot_kv_pool_is_seq_swapped(self.handle, seq, C.byref(out))
        return bool(out.value)

    def block_id(self, seq, logical):
        """Read the block table tensor the pool hands to the attention operator."""
        from oracle.bindings import _Tensor

        k, v, t = C.c_void_p(), C.c_void_p(), C.c_void_p()
        self.lib.marmot_kv_pool_get_tensors(self.handle, C.byref(k), C.byref(v), C.byref(t))
        data = C.cast(t, C.POINTER(_Tensor)).contents.data
        table = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint32)), shape=(self.max_seqs * self.max_blocks_per_seq,))
        return int(table[seq * self.max_blocks_per_seq + logical])


def drive(pool, seed: int, steps: int, *, max_seqs: int, max_seq_len: int, block_size: int, swap: bool):
    """A seeded random schedule of pool operations; returns the trace of everything observable (status codes, sequence
    slots, kv slots, start positions, free counts, block ids).  Two pools with the same books give the same trace."""
    rng = np.random.default_rng(seed)
    max_blocks = (max_seq_len + block_size - 1) // block_size
    live: list[int] = []
    lengths: dict[int, int] = {}
    trace = []
    for _ in range(steps):
        op = rng.choice(["acquire", "append", "append", "append", "abort", "release", "prefix", "swap_out", "swap_in"])
        if op == "acquire":
            rc, seq = pool.acquire_seq()
            trace.append(("acquire", rc, seq if rc == 0 else None))
            if rc == 0:
                live.append(seq)
                lengths[seq] = 0
        elif op in ("append", "abort") and live:
            seq = int(rng.choice(live))
            n = int(rng.integers(0, 2 * block_size + 3))
            rc, plan, slots, start = pool.prepare_append(seq, n)
            trace.append(("prepare", seq, n, rc, tuple(slots), start if rc == 0 else None))
            if rc == 0:
                if op == "abort":
                    pool.abort_append(plan)
                    trace.append(("abort", seq))
                else:
                    trace.append(("commit", seq, pool.commit_append(plan)))
                    lengths[seq] += n
        elif op == "release" and live:
            seq = live.pop(int(rng.integers(0, len(live))))
            trace.append(("release", seq, pool.release_seq(seq)))
            lengths.pop(seq, None)
        elif op == "prefix" and len(live) >= 2:
            donors = [s for s in live if lengths[s] >= block_size and not pool.is_swapped(s)]
            takers = [s for s in live if lengths[s] == 0 and not pool.is_swapped(s)]
            if donors and takers:
                donor, taker = int(rng.choice(donors)), int(rng.choice(takers))
                if donor != taker:
                    plen = int(rng.integers(1, lengths[donor] + 1))
                    nb = (plen + block_size - 1) // block_size
                    ids = [pool.block_id(donor, b) for b in range(nb)]
                    rc, plan = pool.prepare_prefix_attach(taker, ids, plen)
                    trace.append(("prefix", donor, taker, plen, tuple(ids), rc))
                    if rc == 0:
                        if rng.random() < 0.2:
                            pool.abort_prefix_attach(plan)
                            trace.append(("prefix_abort", taker))
                        else:
                            trace.append(("prefix_commit", taker, pool.commit_prefix_attach(plan)))
                            lengths[taker] = plen
        elif op == "swap_out" and swap and live:
            seq = int(rng.choice(live))
            trace.append(("swap_out", seq, pool.swap_out(seq), pool.is_swapped(seq)))
        elif op == "swap_in" and swap and live:
            seq = int(rng.choice(live))
            trace.append(("swap_in", seq, pool.swap_in(seq), pool.is_swapped(seq)))
        trace.append(("free", pool.free_block_count()))
        if live:
            seq = int(rng.choice(live))
            trace.append(("table", seq, tuple(pool.block_id(seq, b) for b in range(max_blocks))))
    return trace
