"""The drop-in path end to end: marmot's own public API on `marmot_init(MARMOT_BACKEND_CUDA)`.

marmot_b200/libmarmot_b200.so is marmot's core and CPU backend plus this package's CUDA backend, built by
marmot_b200/host/build_marmot.py from a marmot checkout: the kernel-DSL code generator emits the CUDA query function,
the `marmot_cuda_*_exec` dispatch wrappers and the bytecode tables from host/kernels/*.def, and the three per-backend
switch statements of the core get their CUDA case.  Every call below goes the way a marmot user's call goes:
public API -> op signature -> generated `marmot_cuda_query_kernel` -> one-instruction bytecode program -> generated
exec wrapper -> cuda_backend.c -> C ABI -> sm_100a kernel, with host tensors in and results read back through
`marmot_tensor_copy_to_host_buffer`.  The checker is the CPU context of the same library (the reference's own code).
"""
from __future__ import annotations

import os

import numpy as np
import pytest

from marmot_b200.marmot_api import (BACKEND_CPU, BACKEND_CUDA, FULL_LIB, POLICY_RENORMALIZE_SELECTED,
                                    POLICY_SOFTMAX_SELECTED, MarmotLibrary)
from marmot_b200.runtime import KIND_Q4_K, KIND_Q6_K, KIND_Q8_0
from tests.util import TOL_FP32, TOL_MMA, TOL_MOE, cosine, max_rel_err, random_blocks

pytestmark = pytest.mark.gpu

KIND_Q8_K = 12


@pytest.fixture(scope="module")
def libs():
    if not FULL_LIB.exists():
        pytest.skip("libmarmot_b200.so not built (marmot_b200/host/build_marmot.py needs a marmot checkout)")
    cpu = MarmotLibrary(FULL_LIB, BACKEND_CPU, threads=1)
    cuda = MarmotLibrary(FULL_LIB, BACKEND_CUDA)
    yield cpu, cuda
    cuda.close()
    cpu.close()


@pytest.mark.parametrize("kind", [KIND_Q4_K, KIND_Q6_K, KIND_Q8_0])
@pytest.mark.parametrize("T,K,F", [(1, 4096, 512), (5, 1024, 96), (40, 2048, 640), (200, 512, 256)])
def test_marmot_linear(libs, kind, T, K, F):
    cpu, cuda = libs
    rng = np.random.default_rng(T * 7 + kind)
    W = random_blocks(kind, F, K, rng)
    x = rng.normal(0, 1, (T, K)).astype(np.float32)
    got, want = cuda.linear(kind, x, W, F), cpu.linear(kind, x, W, F)
    err = max_rel_err(got, want)
    assert err <= (TOL_FP32 if T <= 8 else TOL_MMA), err
    assert cosine(got, want) >= 0.999


@pytest.mark.parametrize("kind", [KIND_Q4_K, KIND_Q6_K, KIND_Q8_0])
@pytest.mark.parametrize("T,K,F,half_out", [(1, 4096, 256, False), (6, 1024, 96, True), (20, 512, 64, False)])
def test_marmot_linear_with_float16_activations(libs, kind, T, K, F, half_out):
    """FLOAT16 inputs take the reference's unpacked branch (no Q8 packing, f32 arithmetic per weight value): the CUDA
    context against the CPU context, f32 and f16 outputs."""
    cpu, cuda = libs
    rng = np.random.default_rng(T + kind + K)
    W = random_blocks(kind, F, K, rng)
    x16 = rng.normal(0, 1, (T, K)).astype(np.float16)
    got = cuda.linear_f16(kind, x16, W, F, half_out).astype(np.float32)
    want = cpu.linear_f16(kind, x16, W, F, half_out).astype(np.float32)
    if half_out:
        ok = np.isfinite(want)
        assert np.max(np.abs(got - want)[ok] / np.maximum(np.abs(want[ok]), 1.0)) <= 2e-3  # one f16 place
    else:
        assert max_rel_err(got, want) <= 2e-5


@pytest.mark.parametrize("kind", [KIND_Q4_K, KIND_Q6_K, KIND_Q8_0])
def test_marmot_dequantize_is_bit_exact(libs, kind):
    cpu, cuda = libs
    rng = np.random.default_rng(kind)
    n = 7 * 1024
    blocks = random_blocks(kind, 7, 1024, rng)
    got, want = cuda.dequantize(kind, blocks, n), cpu.dequantize(kind, blocks, n)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_marmot_topk_and_moe_experts(libs):
    cpu, cuda = libs
    rng = np.random.default_rng(9)
    H, FF, E, k = 512, 1024, 8, 2
    kinds = (KIND_Q4_K, KIND_Q4_K, KIND_Q6_K)
    gate = random_blocks(kinds[0], E * FF, H, rng, d_sigma=0.0005)
    up = random_blocks(kinds[1], E * FF, H, rng, d_sigma=0.0005)
    down = random_blocks(kinds[2], E * H, FF, rng, d_sigma=0.00005)
    for T, tol in ((3, TOL_FP32 * 5), (160, TOL_MOE)):  # per-expert decode launches / grouped tensor-core launches
        hidden = rng.normal(0, 1, (T, H)).astype(np.float32)
        logits = rng.normal(0, 1, (T, E)).astype(np.float32)
        probs = np.exp(logits) / np.exp(logits).sum(axis=1, keepdims=True)
        vals, ids = cuda.topk(probs.astype(np.float32), k)
        ref_vals, ref_ids = cpu.topk(probs.astype(np.float32), k)
        assert np.array_equal(ids, ref_ids) and np.array_equal(vals, ref_vals)
        for policy in (POLICY_RENORMALIZE_SELECTED, POLICY_SOFTMAX_SELECTED):
            got = cuda.moe_experts(kinds, hidden, gate, up, down, ids, vals, FF, E, policy=policy)
            # A fresh CPU context per comparison: the reference's CPU backend keeps packed-weight caches keyed by
            # host address and is not told when a tensor's memory is freed, so expert tensors that land on addresses
            # an earlier call used for other weights would be served stale data (seen here: cosine 0.42 against the
            # oracle after a 3-token call followed by a 160-token call).
            fresh = MarmotLibrary(FULL_LIB, BACKEND_CPU, threads=1)
            want = fresh.moe_experts(kinds, hidden, gate, up, down, ref_ids, ref_vals, FF, E, policy=policy)
            fresh.close()
            assert cosine(got, want) >= 0.999
            assert max_rel_err(got, want) <= tol, (T, policy, max_rel_err(got, want))


@pytest.mark.parametrize("name,kind,act,act_kind,nb", [("q4_k", KIND_Q4_K, "q8_k", KIND_Q8_K, 1),
                                                      ("q6_k", KIND_Q6_K, "q8_k", KIND_Q8_K, 1),
                                                      ("q8_0", KIND_Q8_0, "q8_0", KIND_Q8_0, 8)])
def test_marmot_vec_dot_on_the_reference_goldens(libs, llama_goldens, name, kind, act, act_kind, nb):
    cpu, cuda = libs
    w, a = llama_goldens[f"vec_dot_{name}_weights"], llama_goldens[f"vec_dot_{act}_activations"]
    got = cuda.vec_dot(kind, act_kind, w, a, nb)
    exp = float(llama_goldens[f"vec_dot_{name}_{act}_expected"][0])
    assert abs(got - exp) <= abs(exp) * 2e-5 + 1e-5  # the bound of tests/backend/test_vec_dot.c:135-156
    want = cpu.vec_dot(kind, act_kind, w, a, nb)
    assert abs(got - want) <= abs(want) * 2e-6 + 1e-6


def test_decoder_operators_through_the_public_api(libs):
    """marmot_rmsnorm, marmot_rope, marmot_swiglu and marmot_paged_attention on the CUDA context against the CPU
    context of the same library."""
    cpu, cuda = libs
    rng = np.random.default_rng(17)
    T, d, hq, hkv, hd, bs = 6, 512, 8, 2, 64, 16
    x = rng.normal(0, 1, (T, d)).astype(np.float32)
    w = rng.normal(1, 0.1, d).astype(np.float32)
    res = rng.normal(0, 1, (T, d)).astype(np.float32)
    assert max_rel_err(cuda.rmsnorm(x, w, 1e-5), cpu.rmsnorm(x, w, 1e-5)) <= 2e-6
    assert max_rel_err(cuda.rmsnorm(x, w, 1e-5, residual=res), cpu.rmsnorm(x, w, 1e-5, residual=res)) <= 2e-6
    q = rng.normal(0, 1, (T * hq, hd)).astype(np.float32)
    pos = np.repeat(np.arange(3, 3 + T, dtype=np.int32), hq)
    for neox in (False, True):
        assert max_rel_err(cuda.rope(q, pos, 500000.0, neox=neox), cpu.rope(q, pos, 500000.0, neox=neox)) <= 2e-5
    a, b = rng.normal(0, 2, (T, d)).astype(np.float32), rng.normal(0, 1, (T, d)).astype(np.float32)
    assert max_rel_err(cuda.swiglu(a, b), cpu.swiglu(a, b)) <= 2e-6
    # paged attention: a prefill chunk of T tokens of sequence slot 1 appended at positions 0..T-1
    n_blocks, layers = 4, 2
    table = np.full((2, 2), 0xFFFFFFFF, dtype=np.uint32)
    table[1] = [2, 0]
    meta = np.stack([np.ones(T), np.arange(T), 2 * bs + np.arange(T), np.zeros(T)], axis=1).astype(np.uint32)
    qh = rng.normal(0, 1, (T, hq, hd)).astype(np.float32)
    kn, vn = rng.normal(0, 1, (T, hkv, hd)).astype(np.float32), rng.normal(0, 1, (T, hkv, hd)).astype(np.float32)
    for kv_dtype, tol in ((np.float32, 2e-5), (np.float16, 3e-3)):
        pool_k = np.zeros((n_blocks, layers, hkv, bs, hd), dtype=kv_dtype)
        pool_v = np.zeros_like(pool_k)
        # one thread: the reference's parallel-for returns an uninitialised status from this operator on several
        got, gk, gv = cuda.paged_attention(meta, qh, kn, vn, pool_k, pool_v, table, 1, bs, hd ** -0.5)
        want, wk, wv = cpu.paged_attention(meta, qh, kn, vn, pool_k, pool_v, table, 1, bs, hd ** -0.5)
        assert max_rel_err(got, want) <= tol, (kv_dtype, max_rel_err(got, want))
        if kv_dtype == np.float32:
            assert np.array_equal(gk, wk) and np.array_equal(gv, wv)
        else:  # the scalar build of the reference truncates to f16 where the CUDA path rounds to nearest even
            assert np.max(np.abs(gk.astype(np.float32) - wk.astype(np.float32))) <= 2e-3


def test_unsupported_signatures_are_refused_not_computed_on_the_host(libs):
    """A block format without a CUDA kernel is answered "unsupported" at query time: the call fails, nothing falls
    back to host arithmetic."""
    _, cuda = libs
    rng = np.random.default_rng(1)
    K, F = 256, 8
    q4_0 = rng.integers(0, 256, F * (K // 32) * 18, dtype=np.uint8)  # Q4_0: 18 bytes per 32 values
    q4_0.reshape(-1, 18)[:, 1] = 0x1C  # finite fp16 scales
    with pytest.raises(RuntimeError):
        cuda.linear(1, rng.normal(0, 1, (1, K)).astype(np.float32), q4_0, F)  # MARMOT_QUANT_KIND_Q4_0


def test_graph_batch_hooks(libs):
    """marmot_graph_batch_begin / _end (what the graph executor brackets a bytecode program with) around resident
    operands: the operators inside only enqueue work; the results are there when the tensors are read afterwards."""
    cpu, cuda = libs
    rng = np.random.default_rng(3)
    K, F = 1024, 256
    W = random_blocks(KIND_Q4_K, F, K, rng)
    run = cuda.linear_resident(KIND_Q4_K, W, F, K, T=2)
    x = rng.normal(0, 1, (2, K)).astype(np.float32)
    want = cpu.linear(KIND_Q4_K, x, W, F)
    assert max_rel_err(run(x).copy(), want) <= TOL_FP32
    tw, tx, to = run.tensors
    L = cuda.lib
    assert L.marmot_graph_batch_begin(cuda.ctx) == 0
    assert L.marmot_linear(cuda.ctx, tx, tw, None, to) == 0
    assert L.marmot_linear(cuda.ctx, tx, tw, None, to) == 0
    assert L.marmot_graph_batch_end(cuda.ctx, True) == 0
    assert max_rel_err(cuda._read(to, (2, F), np.float32), want) <= TOL_FP32
    # an abandoned batch (commit == false) leaves the context usable
    assert L.marmot_graph_batch_begin(cuda.ctx) == 0
    assert L.marmot_linear(cuda.ctx, tx, tw, None, to) == 0
    assert L.marmot_graph_batch_end(cuda.ctx, False) == 0
    assert max_rel_err(run(x).copy(), want) <= TOL_FP32


def test_graph_batch_recorded_into_a_cuda_graph():
    """With MARMOT_CUDA_GRAPH_BATCH=capture the outermost batch is recorded with mcu_graph_capture_begin / _end and
    launched once at its end; an operand that is not resident fails the batch instead of breaking the capture."""
    if not FULL_LIB.exists():
        pytest.skip("libmarmot_b200.so not built")
    os.environ["MARMOT_CUDA_GRAPH_BATCH"] = "capture"
    try:
        cuda = MarmotLibrary(FULL_LIB, BACKEND_CUDA)
    finally:
        del os.environ["MARMOT_CUDA_GRAPH_BATCH"]
    cpu = MarmotLibrary(FULL_LIB, BACKEND_CPU)
    try:
        rng = np.random.default_rng(4)
        K, F = 2048, 512
        W = random_blocks(KIND_Q6_K, F, K, rng)
        run = cuda.linear_resident(KIND_Q6_K, W, F, K, T=1)
        x = rng.normal(0, 1, (1, K)).astype(np.float32)
        want = cpu.linear(KIND_Q6_K, x, W, F)
        assert max_rel_err(run(x).copy(), want) <= TOL_FP32  # unbatched once: operands resident, workspace warm
        tw, tx, to = run.tensors
        L = cuda.lib
        x2 = rng.normal(0, 1, (1, K)).astype(np.float32)
        want2 = cpu.linear(KIND_Q6_K, x2, W, F)
        assert L.marmot_tensor_copy_from_host_buffer(cuda.ctx, tx, x2.ctypes.data, x2.nbytes) == 0
        assert L.marmot_tensor_to_device(cuda.ctx, tx) == 0
        assert L.marmot_graph_batch_begin(cuda.ctx) == 0
        assert L.marmot_linear(cuda.ctx, tx, tw, None, to) == 0
        assert L.marmot_graph_batch_end(cuda.ctx, True) == 0
        assert max_rel_err(cuda._read(to, (1, F), np.float32), want2) <= TOL_FP32
        # a weight whose host copy is the current one needs an upload, which cannot be recorded: the operator is
        # refused and the batch is abandoned cleanly
        W3 = random_blocks(KIND_Q6_K, F, K, rng)
        tw3 = cuda._qtensor((F, K), KIND_Q6_K, W3)
        assert L.marmot_tensor_to_host(cuda.ctx, tw3) == 0
        assert L.marmot_graph_batch_begin(cuda.ctx) == 0
        assert L.marmot_linear(cuda.ctx, tx, tw3, None, to) != 0
        assert L.marmot_graph_batch_end(cuda.ctx, False) == 0
        assert max_rel_err(cuda.linear(KIND_Q6_K, x2, W3, F), cpu.linear(KIND_Q6_K, x2, W3, F)) <= TOL_FP32
        L.marmot_tensor_destroy(tw3)
    finally:
        cuda.close()
        cpu.close()
