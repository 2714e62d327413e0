"""The books of the CUDA KV-cache pool (no storage: ctx = None) against the reference's own pool on seeded random
schedules, and against traces the reference produced (tests/golden/kv_pool_traces.json) where it is not available."""
from __future__ import annotations

import json

import pytest

from marmot_b200.runtime import KvPool
from tests.conftest import GOLDEN_DIR
from tests.kv_pool_ref import drive

CONFIGS = {
    "tight": dict(max_seqs=4, max_seq_len=96, block_size=16, num_blocks=10, num_swap_blocks=8, deterministic=False),
    "tight_deterministic": dict(max_seqs=4, max_seq_len=96, block_size=16, num_blocks=10, num_swap_blocks=8, deterministic=True),
    "roomy": dict(max_seqs=6, max_seq_len=64, block_size=8, num_blocks=40, num_swap_blocks=0, deterministic=False),
    "swap_exchange": dict(max_seqs=3, max_seq_len=32, block_size=16, num_blocks=4, num_swap_blocks=6, deterministic=True),
}


def run(pool, name, seed, steps=250):
    c = CONFIGS[name]
    return drive(pool, seed, steps, max_seqs=c["max_seqs"], max_seq_len=c["max_seq_len"], block_size=c["block_size"],
                 swap=c["num_swap_blocks"] > 0)


def as_json(trace):
    return json.loads(json.dumps(trace))


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("seed", [1, 2])
def test_books_match_reference_traces(name, seed):
    golden = json.loads((GOLDEN_DIR / "kv_pool_traces.json").read_text())
    pool = KvPool(None, **CONFIGS[name])
    try:
        assert as_json(run(pool, name, seed)) == golden[f"{name}/{seed}"]
    finally:
        pool.close()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_books_match_reference_live(reference_lib, name):
    """A longer schedule, live against the reference library when it is built here."""
    from oracle import build_ref
    from tests.kv_pool_ref import RefKvPool

    if not build_ref.KV_POOL_LIB.exists():
        pytest.skip("oracle/_ref/libmarmot_ref_kvpool.so not built (needs the reference checkout)")
    theirs = RefKvPool(reference_lib, **CONFIGS[name])
    ours = KvPool(None, **CONFIGS[name])
    try:
        a, b = run(ours, name, 99, steps=1500), run(theirs, name, 99, steps=1500)
        assert len(a) == len(b)
        for i, (x, y) in enumerate(zip(a, b)):
            assert x == y, (i, x, y)
    finally:
        ours.close()
        theirs.close()


def test_argument_checks():
    with pytest.raises(Exception):
        KvPool(None, max_seqs=1, max_seq_len=32, block_size=12, num_blocks=4)  # not a power of two
    with pytest.raises(Exception):
        KvPool(None, max_seqs=0, max_seq_len=32, block_size=16, num_blocks=4)
    pool = KvPool(None, max_seqs=1, max_seq_len=32, block_size=16, num_blocks=1)
    try:
        rc, seq = pool.acquire_seq()
        assert (rc, seq) == (0, 0)
        assert pool.acquire_seq()[0] != 0  # no slot left
        rc, plan, slots, start = pool.prepare_append(seq, 16)
        assert rc == 0 and slots == list(range(16)) and start == 0
        assert pool.prepare_append(seq, 1)[0] != 0  # a plan is pending
        assert pool.release_seq(seq) != 0
        assert pool.commit_append(plan) == 0 and pool.seq_len(seq) == 16
        assert pool.commit_append(plan) != 0  # not twice
        assert pool.prepare_append(seq, 1)[0] != 0 and pool.free_block_count() == 0  # out of blocks, books unchanged
        assert pool.prepare_append(seq, 40)[0] != 0  # beyond max_seq_len
        assert pool.swap_out(seq) != 0  # swap not configured
        assert pool.block_generation(0) == 1 and pool.total_block_count() == 1
        with pytest.raises(Exception):
            pool.tensors()  # books only
        assert pool.release_seq(seq) == 0 and pool.free_block_count() == 1
    finally:
        pool.close()
