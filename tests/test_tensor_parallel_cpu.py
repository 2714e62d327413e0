"""Host logic of the tensor-/expert-parallel layer on CPU: two gloo ranks, the arithmetic of each shard done by
the CPU oracle standing in for the CUDA library, the sharded result compared with the unsharded operator."""
from __future__ import annotations

import os
import tempfile

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from marmot_b200 import tensor_parallel as tp
from marmot_b200.runtime import BLOCK_BYTES, KIND_Q4_K, KIND_Q6_K, KIND_Q8_0, row_bytes
from tests.util import TOL_FP32, max_rel_err, random_blocks


def test_shard_range_covers_everything():
    for n, world, g in [(4096, 8, 1), (14336, 8, 256), (56, 8, 1), (10, 4, 1), (3, 8, 1), (128256, 8, 32)]:
        spans = [tp.shard_range(n, world, r, g) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= g and all(s % g == 0 for s in sizes)
    with pytest.raises(ValueError):
        tp.shard_range(100, 2, 0, 256)


@pytest.mark.parametrize("kind", [KIND_Q4_K, KIND_Q6_K, KIND_Q8_0])
def test_shards_are_the_right_bytes(kind):
    rng = np.random.default_rng(kind)
    F, K, world = 12, 1024, 4
    W = random_blocks(kind, F, K, rng)
    rb, bb = row_bytes(kind, K), BLOCK_BYTES[kind]
    rows = W.reshape(F, rb)
    got = np.concatenate([tp.shard_rows(W, kind, F, K, world, r)[0] for r in range(world)])
    assert np.array_equal(got, W)  # row shards concatenate back to the matrix
    bv = K // (rb // bb)
    for r in range(world):
        shard, k_lo, k_hi = tp.shard_k(W, kind, F, K, world, r, granule=bv)
        assert (k_lo, k_hi) == (r * K // world, (r + 1) * K // world)
        per_row = shard.reshape(F, -1)
        assert per_row.shape[1] == row_bytes(kind, k_hi - k_lo)
        b_lo = k_lo // bv
        assert np.array_equal(per_row, rows[:, b_lo * bb:b_lo * bb + per_row.shape[1]])
    # default granule: every shard's rows are 16-byte multiples, shards cover K, sizes differ by at most one granule
    g = tp.k_granule(kind, K)
    spans = [tp.shard_k(W, kind, F, K, world, r)[1:] for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == K and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert all((hi - lo) % g == 0 for lo, hi in spans)
    if kind != KIND_Q6_K:  # Q6_K needs K % 2048 == 0 for 16-byte shard rows (checked below on a wider matrix)
        assert all(row_bytes(kind, hi - lo) % 16 == 0 for lo, hi in spans)
    else:
        W6 = random_blocks(kind, 2, 14336, rng)
        spans6 = [tp.shard_k(W6, kind, 2, 14336, 8, r)[1:] for r in range(8)]
        assert [hi - lo for lo, hi in spans6] == [2048] * 7 + [0]
        assert all(row_bytes(kind, hi - lo) % 16 == 0 for lo, hi in spans6)
    with pytest.raises(ValueError):
        tp.shard_k(W, kind, F, 1000, world, 0)
    assert tp.k_granule(KIND_Q6_K, 14336) == 2048 and tp.k_granule(KIND_Q6_K, 1024) == 256
    assert tp.k_granule(KIND_Q4_K, 4096) == 256 and tp.k_granule(KIND_Q8_0, 4096) == 256


class OracleBackend:
    """Same call surface as marmot_b200.Context, computed by the CPU oracle (tests only)."""

    def __init__(self):
        from oracle import build_oracle
        from oracle.bindings import Oracle

        build_oracle.build()
        self.oracle = Oracle()

    def upload(self, a):
        return np.ascontiguousarray(a, dtype=np.uint8)

    def linear(self, kind, x, w, F):
        return torch.from_numpy(self.oracle.linear(kind, np.ascontiguousarray(x.numpy()), w, F, threads=2))

    def moe_experts_local(self, kinds, hidden, gate, up, down, ids, wts, FF, E, e_lo, e_cnt, out=None):
        ids, wts = ids.numpy(), wts.numpy()
        s = np.zeros(len(wts), dtype=np.float32)
        for j in range(wts.shape[1]):  # same summation order as the operator
            s = s + wts[:, j]
        norm = np.where(s > np.finfo(np.float32).tiny, np.float32(1.0) / s, np.float32(0.0)).astype(np.float32)
        w = (wts * norm[:, None]).astype(np.float32)
        local = (ids >= e_lo) & (ids < e_lo + e_cnt)
        w = np.where(local, w, np.float32(0.0)).astype(np.float32)
        lid = np.where(local, ids - e_lo, 0).astype(np.int32)
        y = self.oracle.moe_experts(kinds, hidden.numpy(), gate, up, down, lid, w, FF, e_cnt, policy=0, threads=2)
        return torch.from_numpy(y)


def _worker(rank: int, world: int, store: str, q):
    os.environ["OMP_NUM_THREADS"] = "2"
    dist.init_process_group("gloo", init_method=f"file://{store}", rank=rank, world_size=world)
    try:
        group = tp.Group(rank, world, dist)
        be = OracleBackend()
        rng = np.random.default_rng(42)  # the same weights and inputs on every rank
        res = {}
        for kind in (KIND_Q4_K, KIND_Q6_K, KIND_Q8_0):
            T, K, F = 3, 1024, 72
            W = random_blocks(kind, F, K, rng)
            x = rng.normal(0, 1, (T, K)).astype(np.float32)
            want = be.oracle.linear(kind, x, W, F)
            col = tp.ColumnParallelLinear(be, group, kind, W, F, K, granule=8)
            y_col = col(torch.from_numpy(x), gather=True).numpy()
            res[f"col{kind}"] = bool(np.array_equal(y_col, want))  # a row split changes no arithmetic
            row = tp.RowParallelLinear(be, group, kind, W, F, K)
            y_row = row(torch.from_numpy(x)).numpy()
            res[f"row{kind}"] = float(max_rel_err(y_row, want))
        # column-parallel feeding row-parallel without a gather in between (the FFN pattern)
        T, H, FF = 4, 512, 1024
        Wup, Wdown = random_blocks(KIND_Q4_K, FF, H, rng, d_sigma=0.002), random_blocks(KIND_Q6_K, H, FF, rng)
        x = rng.normal(0, 1, (T, H)).astype(np.float32)
        mid_full = be.oracle.linear(KIND_Q4_K, x, Wup, FF)
        want = be.oracle.linear(KIND_Q6_K, mid_full, Wdown, H)
        up = tp.ColumnParallelLinear(be, group, KIND_Q4_K, Wup, FF, H, granule=256)
        down = tp.RowParallelLinear(be, group, KIND_Q6_K, Wdown, H, FF)
        res["ffn"] = float(max_rel_err(down(up(torch.from_numpy(x))).numpy(), want))
        # expert parallel
        T, H, FF, E, k = 9, 256, 512, 4, 2
        gate = np.concatenate([random_blocks(KIND_Q4_K, FF, H, rng, d_sigma=0.0005) for _ in range(E)])
        upw = np.concatenate([random_blocks(KIND_Q4_K, FF, H, rng, d_sigma=0.0005) for _ in range(E)])
        dwn = np.concatenate([random_blocks(KIND_Q6_K, H, FF, rng) for _ in range(E)])
        hidden = rng.normal(0, 1, (T, H)).astype(np.float32)
        ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
        wts = rng.uniform(0.1, 1.0, (T, k)).astype(np.float32)
        kinds = (KIND_Q4_K, KIND_Q4_K, KIND_Q6_K)
        want = be.oracle.moe_experts(kinds, hidden, gate, upw, dwn, ids, wts, FF, E)
        moe = tp.ExpertParallelMoE(be, group, kinds, gate, upw, dwn, H, FF, E)
        got = moe(torch.from_numpy(hidden), torch.from_numpy(ids), torch.from_numpy(wts)).numpy()
        res["moe"] = float(max_rel_err(got, want))
        res["handles"] = group.exchange_bytes(bytes([rank]) * 4) == [bytes([r]) * 4 for r in range(world)]
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


def test_two_ranks_match_the_unsharded_operator():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        store = os.path.join(d, "store")
        procs = [ctx.Process(target=_worker, args=(r, world, store, q)) for r in range(world)]
        for p in procs:
            p.start()
        results = dict(q.get(timeout=240) for _ in range(world))
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    for rank in range(world):
        res = results[rank]
        for kind in (KIND_Q4_K, KIND_Q6_K, KIND_Q8_0):
            assert res[f"col{kind}"], (rank, kind)
            assert res[f"row{kind}"] <= TOL_FP32, (rank, kind, res[f"row{kind}"])  # only the f32 sum order changes
        assert res["ffn"] <= TOL_FP32, res["ffn"]
        assert res["moe"] <= 1e-5, res["moe"]
        assert res["handles"]
