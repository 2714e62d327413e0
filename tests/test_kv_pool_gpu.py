"""The KV-cache pool with storage on the GPU: the device block table follows the books, copy-on-write clones and swaps
move the right bytes, and the attention operator runs on pool-managed blocks."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from marmot_b200 import Context
from marmot_b200.runtime import KvPool

pytestmark = pytest.mark.gpu
INVALID = 0xFFFFFFFF


@pytest.fixture(scope="module")
def ctx():
    c = Context(0)
    yield c
    c.close()


def table_on_device(pool):
    return pool.tensors()[2].cpu().numpy().view(np.uint32)


def books(pool, max_seqs, max_blocks):
    return np.array([[pool.block_id(s, b) for b in range(max_blocks)] for s in range(max_seqs)], dtype=np.uint32)


def fill(pool, slots, seed):
    """Write recognisable K/V rows at the given kv slots (all layers and heads); returns what was written."""
    k, v, _ = pool.tensors()
    nb, L, H, bs, hd = k.shape
    g = torch.Generator(device="cuda").manual_seed(seed)
    data_k = torch.randn((len(slots), L, H, hd), device="cuda", generator=g).to(k.dtype)
    data_v = torch.randn((len(slots), L, H, hd), device="cuda", generator=g).to(k.dtype)
    for i, s in enumerate(slots):
        k[s // bs, :, :, s % bs, :] = data_k[i]
        v[s // bs, :, :, s % bs, :] = data_v[i]
    return data_k, data_v


def read(pool, slots):
    k, v, _ = pool.tensors()
    bs = k.shape[3]
    return (torch.stack([k[s // bs, :, :, s % bs, :] for s in slots]), torch.stack([v[s // bs, :, :, s % bs, :] for s in slots]))


def slots_of(pool, seq, n, bs):
    return [pool.block_id(seq, p // bs) * bs + p % bs for p in range(n)]


def test_device_table_follows_the_books(ctx):
    cfg = dict(max_seqs=3, max_seq_len=64, block_size=16, num_blocks=8, num_layers=2, num_kv_heads=2, head_dim=64)
    pool = KvPool(ctx, **cfg)
    try:
        k, v, t = pool.tensors()
        assert tuple(k.shape) == (8, 2, 2, 16, 64) and k.dtype == torch.float16 and tuple(t.shape) == (3, 4)
        assert np.all(table_on_device(pool) == INVALID)
        seqs = [pool.acquire_seq()[1] for _ in range(3)]
        for seq, n in zip(seqs, (20, 5, 33)):
            rc, plan, slots, start = pool.prepare_append(seq, n)
            assert rc == 0 and start == 0
            assert pool.commit_append(plan) == 0
        ctx.synchronize()
        assert np.array_equal(table_on_device(pool), books(pool, 3, 4))
        rc, plan, _, _ = pool.prepare_append(seqs[1], 30)
        pool.abort_append(plan)
        assert pool.release_seq(seqs[0]) == 0
        ctx.synchronize()
        assert np.array_equal(table_on_device(pool), books(pool, 3, 4))
        assert np.all(table_on_device(pool)[seqs[0]] == INVALID)
    finally:
        pool.close()


def test_copy_on_write_clones_the_shared_block(ctx):
    bs = 16
    pool = KvPool(ctx, max_seqs=2, max_seq_len=64, block_size=bs, num_blocks=6, num_layers=2, num_kv_heads=2, head_dim=64)
    try:
        a, b = pool.acquire_seq()[1], pool.acquire_seq()[1]
        rc, plan, slots_a, _ = pool.prepare_append(a, 20)
        assert pool.commit_append(plan) == 0
        want_k, want_v = fill(pool, slots_a, seed=1)
        ids = [pool.block_id(a, 0), pool.block_id(a, 1)]
        rc, pplan = pool.prepare_prefix_attach(b, ids, 20)
        assert rc == 0 and pool.commit_prefix_attach(pplan) == 0 and pool.seq_len(b) == 20
        assert pool.free_block_count() == 4  # shared, not copied
        rc, plan, slots_b, start = pool.prepare_append(b, 3)  # continues inside the shared, partially filled block
        assert rc == 0 and start == 20 and pool.commit_append(plan) == 0
        assert pool.block_id(b, 0) == ids[0] and pool.block_id(b, 1) not in ids  # block 0 still shared, block 1 cloned
        assert pool.free_block_count() == 3
        fill(pool, slots_b, seed=2)  # b writes its own tokens: a must not see them
        got_k, got_v = read(pool, slots_a)
        assert torch.equal(got_k, want_k) and torch.equal(got_v, want_v)
        clone_k, clone_v = read(pool, slots_of(pool, b, 20, bs))  # b sees a's first twenty positions
        assert torch.equal(clone_k, want_k) and torch.equal(clone_v, want_v)
        ctx.synchronize()
        assert np.array_equal(table_on_device(pool), books(pool, 2, 4))
    finally:
        pool.close()


@pytest.mark.parametrize("kv_f16", [True, False])
def test_swap_round_trip_keeps_the_data(ctx, kv_f16):
    bs = 16
    pool = KvPool(ctx, max_seqs=3, max_seq_len=64, block_size=bs, num_blocks=4, num_swap_blocks=4, num_layers=2,
                  num_kv_heads=2, head_dim=64, kv_f16=kv_f16)
    try:
        a, b = pool.acquire_seq()[1], pool.acquire_seq()[1]
        rc, plan, slots_a, _ = pool.prepare_append(a, 40)
        assert rc == 0 and pool.commit_append(plan) == 0
        want_k, want_v = fill(pool, slots_a, seed=3)
        assert pool.swap_out(a) == 0 and pool.is_swapped(a) and pool.free_block_count() == 4
        assert pool.prepare_append(a, 1)[0] != 0  # not while swapped out
        rc, plan, slots_b, _ = pool.prepare_append(b, 64)  # takes every device block, the ones a had included
        assert rc == 0 and pool.commit_append(plan) == 0 and pool.free_block_count() == 0
        fill(pool, slots_b, seed=4)
        assert pool.swap_in(a) != 0 and pool.is_swapped(a)  # no room, no sequence of the same size to trade with
        assert pool.release_seq(b) == 0
        assert pool.swap_in(a) == 0 and not pool.is_swapped(a)
        got_k, got_v = read(pool, slots_of(pool, a, 40, bs))
        assert torch.equal(got_k, want_k) and torch.equal(got_v, want_v)
        ctx.synchronize()
        assert np.array_equal(table_on_device(pool), books(pool, 3, 4))
    finally:
        pool.close()


def test_swap_in_by_exchange(ctx):
    bs = 16
    pool = KvPool(ctx, max_seqs=2, max_seq_len=32, block_size=bs, num_blocks=2, num_swap_blocks=2, num_layers=1,
                  num_kv_heads=2, head_dim=128, deterministic=True)
    try:
        a, b = pool.acquire_seq()[1], pool.acquire_seq()[1]
        rc, plan, slots_a, _ = pool.prepare_append(a, 32)
        assert pool.commit_append(plan) == 0
        a_k, a_v = fill(pool, slots_a, seed=5)
        assert pool.swap_out(a) == 0
        rc, plan, slots_b, _ = pool.prepare_append(b, 32)
        assert rc == 0 and pool.commit_append(plan) == 0 and pool.free_block_count() == 0
        b_k, b_v = fill(pool, slots_b, seed=6)
        assert pool.swap_in(a) == 0  # pool full: a and b trade places
        assert not pool.is_swapped(a) and pool.is_swapped(b) and pool.free_block_count() == 0
        got_k, got_v = read(pool, slots_of(pool, a, 32, bs))
        assert torch.equal(got_k, a_k) and torch.equal(got_v, a_v)
        assert pool.swap_in(b) == 0 and pool.is_swapped(a)  # and back
        got_k, got_v = read(pool, slots_of(pool, b, 32, bs))
        assert torch.equal(got_k, b_k) and torch.equal(got_v, b_v)
        ctx.synchronize()
        assert np.array_equal(table_on_device(pool), books(pool, 2, 2))
    finally:
        pool.close()


def test_attention_on_pool_managed_blocks(ctx, oracle):
    """Three sequences grow by interleaved appends (so their blocks interleave in the pool), one is released and its
    blocks are reused; every step's attention output matches the oracle run on the pool's own table."""
    rng = np.random.default_rng(0)
    bs, L, hq, hkv, hd = 16, 2, 8, 2, 64
    pool = KvPool(ctx, max_seqs=4, max_seq_len=80, block_size=bs, num_blocks=12, num_layers=L, num_kv_heads=hkv, head_dim=hd)
    try:
        kv_k, kv_v, table = pool.tensors()
        ref_k = np.zeros(tuple(kv_k.shape), dtype=np.float16)
        ref_v = np.zeros_like(ref_k)
        seqs = [pool.acquire_seq()[1] for _ in range(3)]
        schedule = [(0, 18), (1, 7), (2, 30), (0, 1), (1, 1), (2, 1), (0, 14), (1, 20)]
        for step, (which, n) in enumerate(schedule):
            if step == 6:  # the third sequence leaves, a new one takes over its blocks
                assert pool.release_seq(seqs[2]) == 0
                seqs[2] = pool.acquire_seq()[1]
            seq = seqs[which]
            rc, plan, slots, start = pool.prepare_append(seq, n)
            assert rc == 0
            meta = np.stack([np.full(n, seq), start + np.arange(n), np.array(slots), np.zeros(n)], axis=1).astype(np.uint32)
            q = rng.normal(0, 1, (n, hq, hd)).astype(np.float32)
            k_new = rng.normal(0, 1, (n, hkv, hd)).astype(np.float32)
            v_new = rng.normal(0, 1, (n, hkv, hd)).astype(np.float32)
            host_table = books(pool, 4, 5)
            for layer in range(L):
                got = ctx.paged_attention(torch.from_numpy(meta).cuda(), torch.from_numpy(q.reshape(n, -1)).cuda(),
                                          torch.from_numpy(k_new.reshape(n, -1)).cuda(),
                                          torch.from_numpy(v_new.reshape(n, -1)).cuda(), kv_k, kv_v, table, layer, hq, hkv,
                                          hd, bs, hd ** -0.5).cpu().numpy().reshape(n, hq, hd)
                want = oracle.paged_attention(meta, q, k_new, v_new, ref_k, ref_v, host_table, layer, bs, hd ** -0.5)
                assert np.max(np.abs(got - want)) <= 2e-5, (step, layer)
            assert pool.commit_append(plan) == 0
        ctx.synchronize()
        used = host_table[host_table != INVALID]
        assert np.array_equal(kv_k.cpu().numpy()[used].view(np.uint16), ref_k[used].view(np.uint16))
    finally:
        pool.close()
