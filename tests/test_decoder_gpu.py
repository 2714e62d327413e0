"""Decoder operators on the GPU (through the C ABI) against the CPU oracle and the committed reference fixtures.
Floating-point kernels: RMSNorm / RoPE / SwiGLU within 1e-5 relative (parallel sums, device sincosf/expf), attention
within 2e-5 absolute on outputs of order one; the KV pool bytes, the embedding gather and argmax are exact."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from marmot_b200 import KIND_Q4_K, KIND_Q6_K, KIND_Q8_0, Context
from tests.conftest import GOLDEN_DIR
from tests.test_oracle_decoder import ATTENTION_CASES, attention_case
from tests.util import random_blocks

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = Context(0)
    yield c
    c.close()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel(got, want):
    return float(np.max(np.abs(got - want)) / max(float(np.max(np.abs(want))), 1e-30))


@pytest.mark.parametrize("rows,n", [(1, 2048), (7, 4096), (64, 320), (3, 5)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm(ctx, oracle, rows, n, with_res):
    rng = np.random.default_rng(rows * n)
    x = rng.normal(0, 2, (rows, n)).astype(np.float32)
    w = rng.normal(1, 0.1, n).astype(np.float32)
    res = rng.normal(0, 1, (rows, n)).astype(np.float32) if with_res else None
    got = ctx.rmsnorm(dev(x), dev(w), 1e-5, residual=dev(res) if with_res else None).cpu().numpy()
    assert rel(got, oracle.rmsnorm(x, w, 1e-5, residual=res)) <= 1e-5
    got = ctx.rmsnorm(dev(x), None, 1e-6, weight_offset=0.0).cpu().numpy()
    assert rel(got, oracle.rmsnorm(x, None, 1e-6)) <= 1e-5


@pytest.mark.parametrize("heads,hd,theta,neox", [(32, 64, 10000.0, False), (8, 128, 500000.0, False), (4, 64, 10000.0, True)])
def test_rope(ctx, oracle, heads, hd, theta, neox):
    rng = np.random.default_rng(heads + hd)
    pos = np.array([0, 1, 17, 511, 4095], dtype=np.int32)
    T = len(pos)
    x = rng.normal(0, 1, (T, heads * hd)).astype(np.float32)
    got = ctx.rope(dev(x), dev(pos), heads, hd, theta, 1.0, neox).cpu().numpy()
    want = oracle.rope(x.reshape(T * heads, hd), np.repeat(pos, heads), theta, 1.0, neox).reshape(T, heads * hd)
    assert np.max(np.abs(got - want)) <= 2e-5  # angles up to 4095 rad: one ulp of the angle is 2.4e-4 * 2^-... per term
    xd = dev(x)
    ctx.rope(xd, dev(pos), heads, hd, theta, 1.0, neox, out=xd)  # in place
    assert np.array_equal(xd.cpu().numpy(), got)


@pytest.mark.parametrize("rows,n", [(1, 2048), (64, 4096), (5, 37)])
def test_add_rmsnorm_is_add_then_rmsnorm(ctx, oracle, rows, n):
    rng = np.random.default_rng(rows + n)
    x = rng.normal(0, 2, (rows, n)).astype(np.float32)
    delta = rng.normal(0, 1, (rows, n)).astype(np.float32)
    w = rng.normal(1, 0.1, n).astype(np.float32)
    xd, h = dev(x), torch.empty((rows, n), dtype=torch.float32, device="cuda")
    ctx.add_rmsnorm(xd, dev(delta), dev(w), 1e-5, xd, h)  # residual stream updated in place
    assert np.array_equal(xd.cpu().numpy(), x + delta)
    assert rel(h.cpu().numpy(), oracle.rmsnorm(x + delta, w, 1e-5)) <= 1e-5
    # the very bits of the two separate operators
    two = ctx.rmsnorm(ctx.add(dev(x), dev(delta)), dev(w), 1e-5)
    assert torch.equal(h, two)


@pytest.mark.parametrize("hq,hkv,hd,neox", [(32, 4, 64, False), (32, 8, 128, False), (4, 4, 64, True)])
def test_rope_qk_is_two_ropes(ctx, hq, hkv, hd, neox):
    rng = np.random.default_rng(hq + hd)
    pos = dev(np.array([0, 3, 100, 2047], dtype=np.int32))
    q = dev(rng.normal(0, 1, (4, hq * hd)).astype(np.float32))
    k = dev(rng.normal(0, 1, (4, hkv * hd)).astype(np.float32))
    want_q = ctx.rope(q, pos, hq, hd, 500000.0, 1.0, neox)
    want_k = ctx.rope(k, pos, hkv, hd, 500000.0, 1.0, neox)
    ctx.rope_qk(q, k, pos, hq, hkv, hd, 500000.0, 1.0, neox)
    assert torch.equal(q, want_q) and torch.equal(k, want_k)


def test_swiglu_add_argmax_embedding(ctx, oracle):
    rng = np.random.default_rng(3)
    a, b = rng.normal(0, 3, 5000).astype(np.float32), rng.normal(0, 1, 5000).astype(np.float32)
    assert rel(ctx.swiglu(dev(a), dev(b)).cpu().numpy(), oracle.swiglu(a, b)) <= 1e-6
    assert np.array_equal(ctx.add(dev(a), dev(b)).cpu().numpy(), a + b)
    x = rng.normal(0, 1, (6, 32000)).astype(np.float32)
    x[2, 7] = x[2, 31999] = 99.0
    x[4, :] = -np.inf
    assert np.array_equal(ctx.argmax(dev(x)).cpu().numpy(), oracle.argmax(x))
    # one long row: many slices, the maximum twice (in different slices), called twice (the tickets return to zero)
    y = rng.normal(0, 1, (1, 128256)).astype(np.float32)
    y[0, 70001] = y[0, 127000] = 50.0
    for _ in range(2):
        assert int(ctx.argmax(dev(y)).item()) == 70001
    for kind in (KIND_Q4_K, KIND_Q6_K, KIND_Q8_0):
        table = random_blocks(kind, 40, 512, rng)
        ids = np.array([3, 39, 0, 3, 17], dtype=np.int32)
        got = ctx.embedding_gather(kind, ctx.upload(table), 512, dev(ids)).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), oracle.embedding_gather(kind, table, 512, ids).view(np.uint32))


def run_gpu_attention(ctx, case):
    q = case["q"]
    T, hq, hd = q.shape
    hkv = case["k_new"].shape[1]
    kv_k, kv_v = dev(case["kv_k"]), dev(case["kv_v"])
    out = ctx.paged_attention(dev(case["meta"]), dev(q.reshape(T, hq * hd)), dev(case["k_new"].reshape(T, hkv * hd)),
                              dev(case["v_new"].reshape(T, hkv * hd)), kv_k, kv_v, dev(case["table"]),
                              int(case["layer"]), hq, hkv, hd, int(case["block_size"]), float(case["scale"]))
    return out.cpu().numpy().reshape(T, hq, hd), kv_k.cpu().numpy(), kv_v.cpu().numpy()


@pytest.mark.parametrize("name", sorted(ATTENTION_CASES))
def test_paged_attention_vs_oracle(ctx, oracle, name):
    case = attention_case(np.random.default_rng(sum(map(ord, name))), **ATTENTION_CASES[name])
    got, gk, gv = run_gpu_attention(ctx, case)
    wk, wv = case["kv_k"].copy(), case["kv_v"].copy()
    want = oracle.paged_attention(case["meta"], case["q"], case["k_new"], case["v_new"], wk, wv, case["table"],
                                  case["layer"], case["block_size"], case["scale"])  # round-to-nearest f16 pool
    assert np.array_equal(gk.view(np.uint8), wk.view(np.uint8)) and np.array_equal(gv.view(np.uint8), wv.view(np.uint8))
    assert np.max(np.abs(got - want)) <= 2e-5


def test_paged_attention_vs_reference_fixture(ctx):
    """f32 pool: the pool bytes and the reference library's own output (fixture) must be reproduced."""
    g = np.load(GOLDEN_DIR / "decoder_cases.npz")
    name = "decode_gqa_f32"
    case = {k[len(name) + 1:]: g[k] for k in g.files if k.startswith(name + ".")}
    got, gk, _ = run_gpu_attention(ctx, case)
    assert np.array_equal(gk.view(np.uint8), case["kv_k_after"].view(np.uint8))
    assert np.max(np.abs(got - case["out"])) <= 2e-5


def test_paged_attention_full_size_properties(ctx):
    """BASELINE config-4 sizes (64 sequences, contexts up to 4096, 32/8 heads of 128, f16 pool): softmax weights are a
    convex combination, so with V == 1 everywhere the output is exactly 1 up to rounding, and with one dominant key
    the output is that key's value row."""
    rng = np.random.default_rng(8)
    n_seq, hq, hkv, hd, bs = 64, 32, 8, 128, 16
    ctx_lens = rng.integers(256, 4096, n_seq)
    max_blocks = 4096 // bs + 1
    n_blocks = int(sum((l + 1 + bs - 1) // bs for l in ctx_lens))
    table = np.full((n_seq, max_blocks), 0xFFFFFFFF, dtype=np.uint32)
    nxt, meta = 0, []
    for s, L in enumerate(ctx_lens):
        nb = (L + 1 + bs - 1) // bs
        table[s, :nb] = np.arange(nxt, nxt + nb)
        nxt += nb
        meta.append((s, L, int(table[s, L // bs]) * bs + L % bs, 0))
    meta = np.array(meta, dtype=np.uint32)
    kv_k = torch.randn((n_blocks, 1, hkv, bs, hd), device="cuda").half()
    kv_v = torch.ones((n_blocks, 1, hkv, bs, hd), device="cuda", dtype=torch.float16)
    q = torch.randn((n_seq, hq * hd), device="cuda")
    k_new = torch.randn((n_seq, hkv * hd), device="cuda")
    v_new = torch.ones((n_seq, hkv * hd), device="cuda")
    out = ctx.paged_attention(dev(meta), q, k_new, v_new, kv_k, kv_v, dev(table), 0, hq, hkv, hd, bs, hd ** -0.5)
    assert float((out - 1.0).abs().max()) <= 1e-5
    # one dominant key: the new token's own key, made huge and aligned with q
    k_dom = (q.view(n_seq, hkv, hq // hkv, hd)[:, :, 0, :] * 50.0).reshape(n_seq, hkv * hd)
    v_mark = torch.randn((n_seq, hkv * hd), device="cuda")
    out = ctx.paged_attention(dev(meta), q, k_dom, v_mark, kv_k, kv_v, dev(table), 0, hq, hkv, hd, bs, hd ** -0.5)
    got = out.view(n_seq, hkv, hq // hkv, hd)[:, :, 0, :].reshape(n_seq, hkv * hd)
    assert float((got - v_mark.half().float()).abs().max()) <= 1e-3


@pytest.mark.parametrize("n_seq,hq,hkv,hd,lo,hi,neox", [(64, 32, 8, 128, 256, 4096, False), (1, 32, 4, 64, 0, 1, False),
                                                        (5, 4, 4, 64, 100, 300, True), (3, 8, 2, 128, 126, 130, False)])
def test_decode_attention_in_one_launch_equals_the_three_steps(ctx, n_seq, hq, hkv, hd, lo, hi, neox):
    """RoPE + append + attention + chunk merge as one kernel (f16 pool) against rope_qk, then paged_attention: the
    same arithmetic in the same order, so outputs and pools agree bit for bit -- contexts inside one 128-position
    chunk (the CTA writes the result itself), across many chunks (last-arriver merge), at a chunk boundary, and twice in
    a row on one context (the tickets are back at zero)."""
    rng = np.random.default_rng(n_seq * 31 + hd)
    bs = 16
    ctx_lens = rng.integers(lo, hi, n_seq)
    max_blocks = hi // bs + 2
    n_blocks = int(sum((l + 1 + bs - 1) // bs for l in ctx_lens))
    table = np.full((n_seq, max_blocks), 0xFFFFFFFF, dtype=np.uint32)
    nxt, meta = 0, []
    for s, L in enumerate(ctx_lens):
        nb = (L + 1 + bs - 1) // bs
        table[s, :nb] = np.arange(nxt, nxt + nb)
        nxt += nb
        meta.append((s, L, int(table[s, L // bs]) * bs + L % bs, 0))
    meta = np.array(meta, dtype=np.uint32)
    pool_k = torch.randn((n_blocks, 2, hkv, bs, hd), device="cuda").half()
    pool_v = torch.randn((n_blocks, 2, hkv, bs, hd), device="cuda").half()
    q = torch.randn((n_seq, hq * hd), device="cuda")
    k_new = torch.randn((n_seq, hkv * hd), device="cuda")
    v_new = torch.randn((n_seq, hkv * hd), device="cuda")
    pos = dev(ctx_lens.astype(np.int32))
    theta = 500000.0
    for _ in range(2):
        k1, v1 = pool_k.clone(), pool_v.clone()
        l0 = ctx.launch_count()
        rope = ctx.rope_table(pos, hd, theta) if _ == 0 else None  # with the caller's table, then with its own
        got = ctx.paged_attention_decode(dev(meta), q.clone(), k_new.clone(), v_new, k1, v1, dev(table), 1, hq, hkv, hd, bs,
                                         hd ** -0.5, pos, theta, neox=neox, rope_table=rope)
        assert ctx.launch_count() - l0 == (3 if n_seq == 64 else 2)  # the table, the attention, at many CTAs a merge kernel
        k2, v2 = pool_k.clone(), pool_v.clone()
        q2, kn2 = q.clone(), k_new.clone()
        ctx.rope_qk(q2, kn2, pos, hq, hkv, hd, theta, neox=neox)
        want = ctx.paged_attention(dev(meta), q2, kn2, v_new, k2, v2, dev(table), 1, hq, hkv, hd, bs, hd ** -0.5)
        assert torch.equal(k1, k2) and torch.equal(v1, v2)
        assert torch.equal(got, want)


def test_graph_capture_replays_a_call_sequence(ctx, oracle):
    """A short chain (RMSNorm -> Q4_K linear -> add -> argmax) recorded once through the C ABI's own capture and replayed
    on new input contents; the calls that wait for the device refuse to be captured and leave the capture intact."""
    from marmot_b200.runtime import MarmotCudaError

    rng = np.random.default_rng(21)
    T, K, F = 3, 1024, 256
    w = ctx.upload(random_blocks(KIND_Q4_K, F, K, rng))
    norm_w = dev(rng.normal(1, 0.1, K).astype(np.float32))
    x = dev(rng.normal(0, 1, (T, K)).astype(np.float32))
    res = dev(rng.normal(0, 1, (T, F)).astype(np.float32))
    h, y = torch.empty_like(x), torch.empty((T, F), dtype=torch.float32, device="cuda")
    pick = torch.empty(T, dtype=torch.int32, device="cuda")

    def chain():
        ctx.rmsnorm(x, norm_w, 1e-5, out=h)
        ctx.linear(KIND_Q4_K, h, w, F, out=y)
        ctx.add(y, res, out=y)
        ctx.argmax(y, out=pick)

    chain()  # sizes the workspace
    ctx.synchronize()
    want_first = y.clone()
    with pytest.raises(MarmotCudaError, match="default stream"):
        ctx.graph_capture_begin()  # the fixture's context rides torch's default stream, which cannot be captured
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    ctx.set_stream(stream.cuda_stream)
    try:
        with torch.cuda.stream(stream):
            _capture_and_replay(ctx, chain, rng, x, y, pick, w, want_first, K, F)
    finally:
        ctx.set_stream(0)


def _capture_and_replay(ctx, chain, rng, x, y, pick, w, want_first, K, F):
    from marmot_b200.runtime import MarmotCudaError

    ctx.graph_capture_begin()
    chain()
    with pytest.raises(MarmotCudaError):
        ctx.synchronize()  # refused, and the capture goes on
    with pytest.raises(MarmotCudaError):
        ctx.linear_host(KIND_Q4_K, np.zeros((1, K), dtype=np.float32), w, F)
    graph = ctx.graph_capture_end()
    y.zero_()
    graph.launch()
    ctx.synchronize()
    assert torch.equal(y, want_first)
    x.copy_(dev(rng.normal(0, 1, tuple(x.shape)).astype(np.float32)))  # new contents, same buffers
    graph.launch()
    ctx.synchronize()
    got, got_pick = y.clone(), pick.clone()
    chain()
    ctx.synchronize()
    assert torch.equal(got, y) and torch.equal(got_pick, pick)
    graph.close()
    with pytest.raises(MarmotCudaError):
        ctx.graph_capture_end()  # nothing in progress
    # a call that needs more workspace than any before it cannot be captured: it says so instead of breaking the capture
    big = dev(rng.normal(0, 1, (48, 4096)).astype(np.float32))
    wb = ctx.upload(random_blocks(KIND_Q4_K, 64, 4096, rng))
    ctx.graph_capture_begin()
    with pytest.raises(MarmotCudaError, match="before capturing"):
        ctx.linear(KIND_Q4_K, big, wb, 64)
    ctx.lib.mcu_graph_capture_end.argtypes = [__import__("ctypes").c_void_p, __import__("ctypes").c_void_p]
    assert ctx.lib.mcu_graph_capture_end(ctx.handle, None) == 0  # discard
    ctx.linear(KIND_Q4_K, big, wb, 64)  # fine outside a capture
    ctx.synchronize()
