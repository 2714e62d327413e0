"""The decoder-operator oracle (oracle/marmot_oracle_decoder.c) pinned against the reference library's own CPU
operators (marmot_rmsnorm, marmot_rope, marmot_swiglu, marmot_paged_attention) and against fixtures generated from
them (tests/golden/decoder_cases.npz)."""
from __future__ import annotations

import numpy as np
import pytest

from tests.conftest import GOLDEN_DIR


def attention_case(rng, T_new, ctx_lens, hq, hkv, hd, block_size, n_layers, layer, kv_dtype, prefill_first=0):
    """Sequences with ctx_lens[i] tokens already cached (filled with random K/V) plus new tokens: the first
    `prefill_first` sequences get T_new tokens each (a prefill chunk), the others one token (decode)."""
    n_seq = len(ctx_lens)
    max_blocks = (max(ctx_lens) + T_new + block_size - 1) // block_size + 1
    n_blocks = n_seq * max_blocks + 3
    perm = rng.permutation(n_blocks)  # physical blocks in scrambled order
    table = np.full((n_seq, max_blocks), 0xFFFFFFFF, dtype=np.uint32)
    pool_shape = (n_blocks, n_layers, hkv, block_size, hd)
    kv_k = rng.normal(0, 1, pool_shape).astype(kv_dtype)
    kv_v = rng.normal(0, 1, pool_shape).astype(kv_dtype)
    meta = []
    nxt = 0
    for s, L in enumerate(ctx_lens):
        new = T_new if s < prefill_first else 1
        for b in range((L + new + block_size - 1) // block_size):
            table[s, b] = perm[nxt]
            nxt += 1
        for j in range(new):
            pos = L + j
            kv_slot = int(table[s, pos // block_size]) * block_size + pos % block_size
            meta.append((s, pos, kv_slot, 0))
    meta = np.array(meta, dtype=np.uint32)
    T = len(meta)
    q = rng.normal(0, 1, (T, hq, hd)).astype(np.float32)
    k_new = rng.normal(0, 1, (T, hkv, hd)).astype(np.float32)
    v_new = rng.normal(0, 1, (T, hkv, hd)).astype(np.float32)
    return dict(meta=meta, q=q, k_new=k_new, v_new=v_new, kv_k=kv_k, kv_v=kv_v, table=table, layer=layer,
                block_size=block_size, scale=float(1.0 / np.sqrt(hd)))


ATTENTION_CASES = {
    "decode_gqa_f32": dict(T_new=1, ctx_lens=[5, 40, 17], hq=8, hkv=2, hd=64, block_size=16, n_layers=2, layer=1, kv_dtype=np.float32),
    "decode_mha_f16": dict(T_new=1, ctx_lens=[0, 33], hq=4, hkv=4, hd=128, block_size=16, n_layers=1, layer=0, kv_dtype=np.float16),
    "prefill_chunk_f16": dict(T_new=9, ctx_lens=[20, 3], hq=8, hkv=4, hd=64, block_size=16, n_layers=3, layer=2, kv_dtype=np.float16, prefill_first=1),
    "long_context_f16": dict(T_new=1, ctx_lens=[300], hq=4, hkv=1, hd=128, block_size=16, n_layers=1, layer=0, kv_dtype=np.float16),
}


@pytest.fixture(scope="module")
def reference_one_thread():
    """The reference's pthread fallback returns an uninitialised status from its error-collecting parallel-for when it
    splits paged attention over several threads (src/backends/cpu/runtime/dispatch.c:485-560); one thread avoids it."""
    from oracle.bindings import REF_LIB, Reference

    if not REF_LIB.exists():
        pytest.skip("oracle/_ref/libmarmot_ref.so not built (needs the reference checkout)")
    ref = Reference(threads=1)
    yield ref
    ref.close()


def run_attention(impl, case, **kw):
    kv_k, kv_v = case["kv_k"].copy(), case["kv_v"].copy()
    res = impl.paged_attention(case["meta"], case["q"], case["k_new"], case["v_new"], kv_k, kv_v, case["table"],
                               case["layer"], case["block_size"], case["scale"], **kw)
    if isinstance(res, tuple):
        return res
    return res, kv_k, kv_v


def test_rmsnorm_rope_swiglu_match_reference(oracle, reference_lib):
    rng = np.random.default_rng(5)
    x = rng.normal(0, 2, (7, 320)).astype(np.float32)
    w = rng.normal(1, 0.1, 320).astype(np.float32)
    res = rng.normal(0, 1, (7, 320)).astype(np.float32)
    for r in (None, res):
        assert np.array_equal(oracle.rmsnorm(x, w, 1e-5, residual=r), reference_lib.rmsnorm(x, w, 1e-5, residual=r))
    pos = np.array([0, 1, 2, 17, 511, 4095, 123], dtype=np.int32)
    for hd, theta, neox in [(64, 10000.0, False), (128, 500000.0, False), (64, 10000.0, True)]:
        xr = rng.normal(0, 1, (7, hd)).astype(np.float32)
        got, want = oracle.rope(xr, pos, theta, 1.0, neox), reference_lib.rope(xr, pos, theta, 1.0, neox)
        assert np.max(np.abs(got - want)) <= 1e-6  # sinf/cosf of the same libm; the sin-cos cache changes nothing
    a, b = rng.normal(0, 3, 1000).astype(np.float32), rng.normal(0, 1, 1000).astype(np.float32)
    assert np.array_equal(oracle.swiglu(a, b), reference_lib.swiglu(a, b))


@pytest.mark.parametrize("name", sorted(ATTENTION_CASES))
def test_paged_attention_matches_reference(oracle, reference_one_thread, name):
    case = attention_case(np.random.default_rng(sum(map(ord, name))), **ATTENTION_CASES[name])
    # the library built here is the scalar flavour, whose f32 -> f16 conversion truncates
    got, gk, gv = run_attention(oracle, case, kv_truncate=True)
    want, wk, wv = run_attention(reference_one_thread, case)
    assert np.array_equal(gk.view(np.uint8), wk.view(np.uint8)) and np.array_equal(gv.view(np.uint8), wv.view(np.uint8))
    assert np.max(np.abs(got - want)) <= 2e-6


def test_decoder_goldens(oracle):
    """Fixtures written by tests/golden/make_golden.py from the reference library: they travel where it cannot."""
    g = np.load(GOLDEN_DIR / "decoder_cases.npz")
    assert np.array_equal(oracle.rmsnorm(g["rms_x"], g["rms_w"], 1e-5, residual=g["rms_res"]), g["rms_out"])
    assert np.max(np.abs(oracle.rope(g["rope_x"], g["rope_pos"], 500000.0) - g["rope_out"])) <= 1e-6
    assert np.array_equal(oracle.swiglu(g["glu_a"], g["glu_b"]), g["glu_out"])
    for name in sorted(ATTENTION_CASES):
        case = {k[len(name) + 1:]: g[k] for k in g.files if k.startswith(name + ".")}
        case = dict(case, layer=int(case["layer"]), block_size=int(case["block_size"]), scale=float(case["scale"]))
        got, gk, gv = run_attention(oracle, case, kv_truncate=True)
        assert np.max(np.abs(got - case["out"])) <= 2e-6
        assert np.array_equal(gk.view(np.uint8), case["kv_k_after"].view(np.uint8))


def test_embedding_and_argmax(oracle):
    from oracle.bindings import KIND_Q4_K
    from tests.util import random_blocks

    rng = np.random.default_rng(2)
    table = random_blocks(KIND_Q4_K, 50, 512, rng)
    ids = np.array([3, 49, 0, 3], dtype=np.int32)
    full = oracle.dequantize(KIND_Q4_K, table, 50 * 512).reshape(50, 512)
    assert np.array_equal(oracle.embedding_gather(KIND_Q4_K, table, 512, ids), full[ids])
    x = rng.normal(0, 1, (5, 100)).astype(np.float32)
    x[2, 7] = x[2, 50] = 99.0
    assert np.array_equal(oracle.argmax(x), np.argmax(x, axis=1).astype(np.int32))
