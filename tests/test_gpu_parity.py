"""Parity of the CUDA path (through the C ABI) against the CPU oracle, the reference's golden vectors
and fixtures produced by the reference library.  Integer / bit-level work is compared exactly;
matmul outputs within the tolerances in tests/util.py."""
from __future__ import annotations

import numpy as np
import pytest

from tests.util import (BLOCK_VALUES, KIND_Q4_K, KIND_Q6_K, KIND_Q8_0, KINDS, TOL_FP32, TOL_MMA, TOL_MOE, cosine, max_rel_err,
                        random_blocks, row_bytes, unpack_q8_0, unpack_q8_k, unsplit_q8_k)

pytestmark = pytest.mark.gpu

NAMES = ["q4_k", "q6_k", "q8_0"]


@pytest.fixture(scope="module")
def ctx():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from marmot_b200 import Context

    c = Context(0)
    yield c
    c.close()


def dev(ctx, a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).to("cuda:0")


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


# ---------------------------------------------------------------- dequantize (bit-exact)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("rows,K", [(1, 256), (3, 768), (64, 4096)])
def test_dequantize_bit_exact(ctx, oracle, name, rows, K):
    kind = KINDS[name]
    rng = np.random.default_rng(rows * 1000 + K)
    W = random_blocks(kind, rows, K, rng)
    n = rows * K
    got = ctx.dequantize(kind, ctx.upload(W), n).cpu().numpy()
    assert np.array_equal(bits(got), bits(oracle.dequantize(kind, W, n)))


@pytest.mark.parametrize("name", NAMES)
def test_dequantize_ragged_tail_and_golden(ctx, oracle, llama_goldens, name):
    kind = KINDS[name]
    rng = np.random.default_rng(5)
    W = random_blocks(kind, 1, 2 * BLOCK_VALUES[kind], rng)
    n = 2 * BLOCK_VALUES[kind] - 7  # count not a multiple of the block size
    got = ctx.dequantize(kind, ctx.upload(W), n).cpu().numpy()
    assert np.array_equal(bits(got), bits(oracle.dequantize(kind, W, n)))
    exp = llama_goldens[f"llama_{name}_dequant"]
    got = ctx.dequantize(kind, ctx.upload(llama_goldens[f"llama_{name}"]), exp.size).cpu().numpy()
    assert np.max(np.abs(got - exp)) <= 5e-4  # tolerance of tests/backend/test_backend_quantization.c


# ---------------------------------------------------------------- activation packers (bit-exact)
@pytest.mark.parametrize("T,K", [(1, 256), (3, 700), (5, 4096), (2, 31)])
def test_quantize_activations_q8_k_bit_exact(ctx, oracle, T, K):
    rng = np.random.default_rng(T * 31 + K)
    x = rng.normal(0, 1, (T, K)).astype(np.float32)
    x[0, : min(K, 256)] = 0.0  # an all-zero block
    if K > 300:
        x[T - 1, 260] = -x[T - 1, 270] if x[T - 1, 270] != 0 else 1.0
        x[T - 1, 260:272] = np.float32(3.5)  # ties on |x|: the first one decides the sign
        x[T - 1, 265] = np.float32(-3.5)
    qs, d, bs = ctx.quantize_activations(KIND_Q4_K, dev(ctx, x))
    nb = (K + 255) // 256
    ref = np.concatenate([oracle.pack_q8_k(x[t]) for t in range(T)])
    rq, rd, rb = unpack_q8_k(ref, T, nb)
    assert np.array_equal(unsplit_q8_k(qs.cpu().numpy()), rq)
    assert np.array_equal(bits(d.cpu().numpy()), bits(rd))
    assert np.array_equal(bs.cpu().numpy(), rb)


@pytest.mark.parametrize("T,K", [(1, 32), (4, 100), (3, 4096)])
def test_quantize_activations_q8_0_bit_exact(ctx, oracle, T, K):
    rng = np.random.default_rng(T * 77 + K)
    x = rng.normal(0, 1, (T, K)).astype(np.float32)
    x[0, :32] = 0.0
    x[T - 1, :8] = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5, -126.5], dtype=np.float32)  # round half away
    if K >= 8:
        x[T - 1, 7 if K < 32 else 31] = np.float32(127.0)  # makes the scale exactly 1
    qs, d, _ = ctx.quantize_activations(KIND_Q8_0, dev(ctx, x))
    nb = (K + 31) // 32
    ref = np.concatenate([oracle.pack_q8_0(x[t]) for t in range(T)])
    rq, rd = unpack_q8_0(ref, T, nb)
    assert np.array_equal(qs.cpu().numpy(), rq)
    assert np.array_equal(bits(d.cpu().numpy()), bits(rd))


# ---------------------------------------------------------------- linear
SHAPES = [(1, 256, 1), (1, 4096, 64), (2, 768, 13), (3, 1024, 40), (5, 2304, 9), (8, 512, 33), (9, 512, 17),
          (17, 1280, 24), (33, 256, 65)]


@pytest.fixture(params=["auto", "plain"])
def variant(request, ctx):
    """Decode kernels: the shared-memory streaming variant (picked automatically when the shape allows)
    and the plain-load variant."""
    from marmot_b200.runtime import REGIME_AUTO, REGIME_GEMV_PLAIN

    ctx.set_regime(REGIME_GEMV_PLAIN if request.param == "plain" else REGIME_AUTO)
    yield request.param
    ctx.set_regime(REGIME_AUTO)


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("T,K,F", SHAPES + [(4, 14336, 40), (7, 2048, 296), (1, 4096, 1184)])
def test_linear_vs_oracle(ctx, oracle, variant, name, T, K, F):
    kind = KINDS[name]
    rng = np.random.default_rng(kind * 1000003 + T * 100003 + K * 101 + F)
    W = random_blocks(kind, F, K, rng)
    x = rng.normal(0, 1, (T, K)).astype(np.float32)
    got = ctx.linear(kind, dev(ctx, x), ctx.upload(W), F).cpu().numpy()
    ctx.synchronize()
    ref = oracle.linear(kind, x, W, F)
    # more than eight tokens go to the tensor-core kernel unless the plain decode kernels are forced
    tol = TOL_MMA if (T > 8 and variant == "auto") else TOL_FP32
    assert max_rel_err(got, ref) <= tol
    assert cosine(got, ref) >= 0.999


GEMM_SHAPES = [(9, 96, 17), (16, 512, 200), (33, 768, 130), (64, 4096, 256), (130, 1024, 384), (300, 2048, 640),
               (512, 4096, 512), (64, 14336, 128), (1, 256, 5)]


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("T,K,F", GEMM_SHAPES)
def test_gemm_tensor_core_vs_oracle(ctx, oracle, name, T, K, F):
    """tcgen05 kernel forced for every shape: fp16 operands, f32 accumulation in tensor memory."""
    from marmot_b200.runtime import REGIME_AUTO, REGIME_GEMM

    kind = KINDS[name]
    if kind != KIND_Q8_0 and K % 256:
        K = (K + 255) // 256 * 256
    rng = np.random.default_rng(kind * 7919 + T * 131 + K + F)
    W = random_blocks(kind, F, K, rng)
    x = rng.normal(0, 1, (T, K)).astype(np.float32)
    bias = rng.normal(0, 1, F).astype(np.float32)
    ctx.set_regime(REGIME_GEMM)
    try:
        got = ctx.linear(kind, dev(ctx, x), ctx.upload(W), F, bias=dev(ctx, bias)).cpu().numpy()
        ctx.synchronize()
    finally:
        ctx.set_regime(REGIME_AUTO)
    ref = oracle.linear(kind, x, W, F, bias=bias)
    assert max_rel_err(got, ref) <= TOL_MMA
    assert cosine(got, ref) >= 0.999


def test_register_operand_kernel_on_q4_k():
    """Q6_K takes the register-operand (mma.sync) kernel for 8 < T <= 64 by default; Q4_K only behind a switch that is
    read once per process, so its parity cases run in a child process with the switch set."""
    import os
    import subprocess
    import sys

    from pathlib import Path

    REPO_ROOT = Path(__file__).resolve().parents[1]
    env = {**os.environ, "MARMOT_CUDA_GEMM_WARP_Q4K": "1"}
    r = subprocess.run([sys.executable, "-m", "pytest", "tests/test_gpu_parity.py", "-x", "-q", "-k",
                        "(test_gemm_tensor_core_vs_oracle or test_dual_output_equals_two_singles) and q4_k"],
                       cwd=REPO_ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]


def test_config_q8_0_prefill_gemm_full_size(ctx, oracle):
    """Q8_0 prefill GEMM, 512 tokens x K = 4096 x F = 14336, with the benchmark's value distributions."""
    kind, T, K, F = KIND_Q8_0, 512, 4096, 14336
    rng = np.random.default_rng(0xB201)
    W = random_blocks(kind, F, K, rng)
    x = rng.normal(0, 1, (T, K)).astype(np.float32)
    got = ctx.linear(kind, dev(ctx, x), ctx.upload(W), F).cpu().numpy()
    ctx.synchronize()
    ref = oracle.linear(kind, x, W, F)
    assert max_rel_err(got, ref) <= TOL_MMA and cosine(got, ref) >= 0.999


@pytest.mark.parametrize("name", NAMES)
def test_linear_ragged_k_strided_input_and_bias(ctx, oracle, variant, name):
    kind = KINDS[name]
    bv = BLOCK_VALUES[kind]
    T, K, F = 3, 2 * bv + bv // 2 + 3, 11  # K not a multiple of the block size
    rng = np.random.default_rng(11)
    W = random_blocks(kind, F, K, rng)
    xfull = rng.normal(0, 1, (T, K + 5)).astype(np.float32)
    x = xfull[:, :K]
    bias = rng.normal(0, 1, F).astype(np.float32)
    xd = dev(ctx, xfull)[:, :K]  # row stride K+5
    got = ctx.linear(kind, xd, ctx.upload(W), F, bias=dev(ctx, bias)).cpu().numpy()
    ref = oracle.linear(kind, np.ascontiguousarray(x), W, F, bias=bias)
    assert max_rel_err(got, ref) <= TOL_FP32


@pytest.mark.parametrize("name", NAMES)
def test_linear_llama_golden(ctx, llama_goldens, name):
    T, K, F = (int(v) for v in llama_goldens[f"matmul_{name}_dims"])
    x = llama_goldens[f"matmul_{name}_input_f32"].reshape(T, K)
    got = ctx.linear(KINDS[name], dev(ctx, x), ctx.upload(llama_goldens[f"matmul_{name}_weight"]), F).cpu().numpy()
    exp = llama_goldens[f"matmul_{name}_output_from_f32"].reshape(T, F)
    # the reference's own tolerance, tests/backend/test_matmul_quantized.c:163-166
    assert np.all(np.abs(got - exp) <= np.abs(exp) * 5e-5 + 2e-5)


@pytest.mark.parametrize("name,act,nb", [("q4_k", "q8_k", 1), ("q6_k", "q8_k", 1), ("q8_0", "q8_0", 8)])
def test_vec_dot_llama_golden(ctx, oracle, llama_goldens, name, act, nb):
    """The row dot on pre-quantized activation blocks against the reference's llama.cpp golden vectors, at the
    reference's own tolerance (tests/backend/test_vec_dot.c:135-156), and against the oracle."""
    w, a = llama_goldens[f"vec_dot_{name}_weights"], llama_goldens[f"vec_dot_{act}_activations"]
    got = ctx.vec_dot_host(KINDS[name], w, a, nb)
    exp = float(llama_goldens[f"vec_dot_{name}_{act}_expected"][0])
    assert abs(got - exp) <= abs(exp) * 2e-5 + 1e-5
    ref = oracle.vec_dot(KINDS[name], w, a, nb)
    assert abs(got - ref) <= abs(ref) * 2e-6 + 1e-6
    assert ctx.vec_dot_host(KINDS[name], w, a, 0) == 0.0  # as cpu_vec_dot: nothing to do


def test_vec_dot_long_row(ctx, oracle):
    """A 4096-value row: activations packed by the oracle into the reference's Q8_K / Q8_0 block structs."""
    rng = np.random.default_rng(11)
    K = 4096
    x = rng.normal(0, 1, K).astype(np.float32)
    for kind in (KIND_Q4_K, KIND_Q6_K, KIND_Q8_0):
        W = random_blocks(kind, 1, K, rng)
        acts = oracle.pack_q8_0(x) if kind == KIND_Q8_0 else oracle.pack_q8_k(x)
        nb = K // (32 if kind == KIND_Q8_0 else 256)
        got = ctx.vec_dot_host(kind, W, acts, nb)
        want = oracle.vec_dot(kind, W, acts, nb)
        assert abs(got - want) <= abs(want) * 2e-5 + 1e-5


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("case", [0, 1, 2])
def test_linear_reference_fixture(ctx, ref_cases, name, case):
    kind = KINDS[name]
    x, W = ref_cases[f"{name}_{case}_x"], ref_cases[f"{name}_{case}_w"]
    T, K = x.shape
    F = W.size // row_bytes(kind, K)
    wd = ctx.upload(W)
    deq = ctx.dequantize(kind, wd, F * K).cpu().numpy()
    assert np.array_equal(bits(deq), bits(ref_cases[f"{name}_{case}_deq"]))
    got = ctx.linear(kind, dev(ctx, x), wd, F).cpu().numpy()
    assert max_rel_err(got, ref_cases[f"{name}_{case}_y"]) <= (TOL_MMA if T > 8 else TOL_FP32)


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("T", [1, 4, 12])
def test_dual_output_equals_two_singles(ctx, variant, name, T):
    # tests/backend/test_matmul_quantized.c:202-298: dual-output == two single calls
    kind = KINDS[name]
    K, F = 1024, 48
    rng = np.random.default_rng(T)
    Wa, Wb = ctx.upload(random_blocks(kind, F, K, rng)), ctx.upload(random_blocks(kind, F, K, rng))
    x = dev(ctx, rng.normal(0, 1, (T, K)).astype(np.float32))
    oa, ob = ctx.linear_dual(kind, x, Wa, Wb, F)
    assert np.array_equal(bits(oa.cpu().numpy()), bits(ctx.linear(kind, x, Wa, F).cpu().numpy()))
    assert np.array_equal(bits(ob.cpu().numpy()), bits(ctx.linear(kind, x, Wb, F).cpu().numpy()))


def test_linear_host_buffers(ctx, oracle):
    kind, T, K, F = KIND_Q4_K, 2, 1024, 96
    rng = np.random.default_rng(3)
    W = random_blocks(kind, F, K, rng)
    x = rng.normal(0, 1, (T, K)).astype(np.float32)
    bias = rng.normal(0, 1, F).astype(np.float32)
    got = ctx.linear_host(kind, x, ctx.upload(W), F, bias_host=bias)
    assert max_rel_err(got, oracle.linear(kind, x, W, F, bias=bias)) <= TOL_FP32


@pytest.mark.parametrize("T,strided", [(1, False), (3, True), (12, False)])
def test_linear_host_pinned_buffers_equal_staged_copies(ctx, T, strided):
    """A page-locked result buffer is written in place by the decode kernels (T <= 8); the result must be the very bits
    of the staged-copy path, which pageable buffers take."""
    import torch

    kind, K, F = KIND_Q4_K, 2048, 264
    rng = np.random.default_rng(T)
    w = ctx.upload(random_blocks(kind, F, K, rng))
    ld = K + 64 if strided else K
    x_pin = torch.zeros((T, ld), dtype=torch.float32).pin_memory()
    x_pin[:, :K] = torch.from_numpy(rng.normal(0, 1, (T, K)).astype(np.float32))
    out_pin = torch.full((T, F), np.nan, dtype=torch.float32).pin_memory()
    x_np = x_pin.numpy()[:, :K]  # a view: same page-locked memory, row stride ld
    got = ctx.linear_host(kind, x_np, w, F, out_host=out_pin.numpy())
    want = ctx.linear_host(kind, np.ascontiguousarray(x_np), w, F)  # pageable copies
    assert np.array_equal(bits(got), bits(want))


def test_config_q4k_gemv_full_size(ctx, oracle):
    """The single-token Q4_K GEMV at 4096 x 4096 with the benchmark's value distributions."""
    kind, T, K, F = KIND_Q4_K, 1, 4096, 4096
    rng = np.random.default_rng(0xB200)
    W = random_blocks(kind, F, K, rng)
    x = rng.normal(0, 1, (T, K)).astype(np.float32)
    got = ctx.linear(kind, dev(ctx, x), ctx.upload(W), F).cpu().numpy()
    ref = oracle.linear(kind, x, W, F)
    assert max_rel_err(got, ref) <= TOL_FP32 and cosine(got, ref) >= 0.999


def test_linearity_in_the_dequantised_weights(ctx):
    """Size-independent property: the matmul is linear in the output rows, so stacking two weight
    matrices stacks the outputs (checked bit for bit)."""
    kind, T, K, F = KIND_Q6_K, 4, 2048, 256
    rng = np.random.default_rng(9)
    Wa, Wb = random_blocks(kind, F, K, rng), random_blocks(kind, F, K, rng)
    x = dev(ctx, rng.normal(0, 1, (T, K)).astype(np.float32))
    both = ctx.linear(kind, x, ctx.upload(np.concatenate([Wa, Wb])), 2 * F).cpu().numpy()
    a = ctx.linear(kind, x, ctx.upload(Wa), F).cpu().numpy()
    b = ctx.linear(kind, x, ctx.upload(Wb), F).cpu().numpy()
    assert np.array_equal(bits(both[:, :F]), bits(a)) and np.array_equal(bits(both[:, F:]), bits(b))


def test_zero_sized_inputs(ctx):
    import torch

    x = torch.empty((0, 256), dtype=torch.float32, device="cuda:0")
    W = ctx.upload(random_blocks(KIND_Q4_K, 4, 256, np.random.default_rng(0)))
    assert ctx.linear(KIND_Q4_K, x, W, 4).shape == (0, 4)


def test_error_codes(ctx):
    import torch
    from marmot_b200 import MarmotCudaError

    x = torch.zeros((1, 256), dtype=torch.float32, device="cuda:0")
    W = ctx.upload(random_blocks(KIND_Q4_K, 4, 256, np.random.default_rng(0)))
    lib = ctx.lib
    # Q5_1 (kind 4) has no CUDA kernel: reported as not implemented, never computed some other way
    assert lib.mcu_linear(ctx.handle, 4, x.data_ptr(), 256, W.data_ptr(), 1, 256, 4, None, x.data_ptr(), 4) == -8
    with pytest.raises(MarmotCudaError) as e:
        ctx.dequantize(4, W, 256)
    assert e.value.code == -8
    assert lib.mcu_linear(ctx.handle, KIND_Q4_K, None, 256, W.data_ptr(), 1, 256, 4, None, x.data_ptr(), 4) == -1
    assert lib.mcu_linear(ctx.handle, KIND_Q4_K, x.data_ptr(), 100, W.data_ptr(), 1, 256, 4, None, x.data_ptr(), 4) == -7
    # a misaligned Q4_K weight pointer is rejected rather than read with vector loads
    assert lib.mcu_linear(ctx.handle, KIND_Q4_K, x.data_ptr(), 256, W.data_ptr() + 2, 1, 256, 1, None, x.data_ptr(), 4) == -1


# ---------------------------------------------------------------- MoE
def test_topk_matches_oracle_with_ties(ctx, oracle):
    rng = np.random.default_rng(1)
    x = rng.integers(0, 4, (257, 8)).astype(np.float32)  # many ties
    vals, idx = ctx.topk(dev(ctx, x), 3)
    rv, ri = oracle.topk(x, 3)
    assert np.array_equal(idx.cpu().numpy(), ri) and np.array_equal(bits(vals.cpu().numpy()), bits(rv))


def _moe_case(rng, T, H, FF, E, k, kinds):
    hid = rng.normal(0, 1, (T, H)).astype(np.float32)
    # small block scales keep the synthetic expert weights at a realistic magnitude (|w| < 1)
    gate = np.concatenate([random_blocks(kinds[0], FF, H, rng, d_sigma=0.0005) for _ in range(E)])
    up = np.concatenate([random_blocks(kinds[1], FF, H, rng, d_sigma=0.0005) for _ in range(E)])
    down = np.concatenate([random_blocks(kinds[2], H, FF, rng, d_sigma=0.0005) for _ in range(E)])
    logits = rng.normal(0, 1, (T, E)).astype(np.float32)
    p = np.exp(logits - logits.max(1, keepdims=True))
    p = (p / p.sum(1, keepdims=True)).astype(np.float32)
    return hid, gate, up, down, p


@pytest.mark.parametrize("T,k,policy,scale", [(37, 2, 2, 1.0), (3, 2, 2, 1.0), (20, 3, 0, 0.5), (9, 1, 2, 1.0)])
def test_moe_experts_vs_oracle(ctx, oracle, T, k, policy, scale):
    H, FF, E = 256, 512, 4
    kinds = (KIND_Q4_K, KIND_Q4_K, KIND_Q6_K)
    rng = np.random.default_rng(T * 10 + k)
    hid, gate, up, down, p = _moe_case(rng, T, H, FF, E, k, kinds)
    vals, ids = oracle.topk(p, k)
    ref = oracle.moe_experts(kinds, hid, gate, up, down, ids, vals, FF, E, weights_scale=scale, policy=policy)
    got = ctx.moe_experts(kinds, dev(ctx, hid), ctx.upload(gate), ctx.upload(up), ctx.upload(down), dev(ctx, ids),
                          dev(ctx, vals), FF, E, weights_scale=scale, policy=policy).cpu().numpy()
    # experts that receive more than eight routes run on the tensor-core kernel
    assert max_rel_err(got, ref) <= TOL_MOE and cosine(got, ref) >= 0.999


@pytest.mark.parametrize("kinds", [(KIND_Q4_K, KIND_Q4_K, KIND_Q6_K), (KIND_Q8_0, KIND_Q8_0, KIND_Q4_K)])
def test_moe_grouped_path_vs_oracle(ctx, oracle, kinds):
    """256 routes or more take the grouped launches (one per projection over all experts, sized from the device-resident
    counts, nothing read back): against the oracle, against the per-expert path's tolerance, for an expert nobody
    selects, for a local expert range, and recorded into a CUDA graph."""
    H, FF, E, T, k = 256, 2048, 5, 150, 2  # Q6_K rows of 2048 values are a multiple of 16 bytes, as the tensor map needs
    rng = np.random.default_rng(12)
    hid, gate, up, down, p = _moe_case(rng, T, H, FF, E, k, kinds)
    p[:, 3] = 0.0  # expert 3 receives no route
    vals, ids = oracle.topk(p, k)
    ref = oracle.moe_experts(kinds, hid, gate, up, down, ids, vals, FF, E)
    gd, ud, dd = ctx.upload(gate), ctx.upload(up), ctx.upload(down)
    hd_, idd, vd = dev(ctx, hid), dev(ctx, ids), dev(ctx, vals)
    launches = ctx.launch_count()
    got = ctx.moe_experts(kinds, hd_, gd, ud, dd, idd, vd, FF, E)
    assert ctx.launch_count() - launches == 3 + 6  # route (3 kernels) + stage, gate, up, stage, down, combine
    ctx.synchronize()
    got = got.cpu().numpy()
    assert max_rel_err(got, ref) <= TOL_MOE and cosine(got, ref) >= 0.999
    # experts [1, 4) only: the other experts' routes contribute nothing
    sl = lambda w, rows, K, kind: w.reshape(E, -1)[1:4].reshape(-1)
    part = ctx.moe_experts_local(kinds, hd_, ctx.upload(sl(gate, FF, H, kinds[0])), ctx.upload(sl(up, FF, H, kinds[1])),
                                 ctx.upload(sl(down, H, FF, kinds[2])), idd, vd, FF, E, 1, 3)
    rest = ctx.moe_experts_local(kinds, hd_, ctx.upload(gate.reshape(E, -1)[0:1].reshape(-1)),
                                 ctx.upload(up.reshape(E, -1)[0:1].reshape(-1)),
                                 ctx.upload(down.reshape(E, -1)[0:1].reshape(-1)), idd, vd, FF, E, 0, 1)
    last = ctx.moe_experts_local(kinds, hd_, ctx.upload(gate.reshape(E, -1)[4:5].reshape(-1)),
                                 ctx.upload(up.reshape(E, -1)[4:5].reshape(-1)),
                                 ctx.upload(down.reshape(E, -1)[4:5].reshape(-1)), idd, vd, FF, E, 4, 1)
    ctx.synchronize()
    total = (part + rest + last).cpu().numpy()
    assert max_rel_err(total, got) <= 1e-5  # the same products, summed per rank first
    # an out-of-range expert id is found on the device and reported at the next synchronize
    from marmot_b200 import MarmotCudaError

    bad = ids.copy()
    bad[7, 1] = E + 2
    ctx.moe_experts(kinds, hd_, gd, ud, dd, dev(ctx, bad), vd, FF, E)
    with pytest.raises(MarmotCudaError) as e:
        ctx.synchronize()
    assert e.value.code == -1
    ctx.synchronize()  # reported once


def test_moe_grouped_path_records_into_a_graph(ctx):
    """With 256 routes or more nothing is read back, so the whole expert block can be captured once and replayed on new
    token contents and new routing; a small batch, which eagerly reads its group sizes back, takes the grouped launches
    too while it is being recorded."""
    import torch

    from marmot_b200 import MarmotCudaError

    H, FF, E, T, k = 256, 512, 4, 160, 2
    kinds = (KIND_Q4_K, KIND_Q4_K, KIND_Q8_0)
    rng = np.random.default_rng(31)
    hid, gate, up, down, p = _moe_case(rng, T, H, FF, E, k, kinds)
    gd, ud, dd = ctx.upload(gate), ctx.upload(up), ctx.upload(down)
    hd_ = dev(ctx, hid)
    order = np.argsort(-p, axis=1)[:, :k].astype(np.int32)
    idd, vd = dev(ctx, order), dev(ctx, np.take_along_axis(p, order, 1))
    out = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    run = lambda: ctx.moe_experts_local(kinds, hd_, gd, ud, dd, idd, vd, FF, E, 0, E, out=out)
    run()  # sizes the workspace
    ctx.synchronize()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    ctx.set_stream(stream.cuda_stream)
    try:
        with torch.cuda.stream(stream):
            ctx.graph_capture_begin()
            run()
            small = torch.zeros((8, H), dtype=torch.float32, device="cuda")
            ctx.moe_experts_local(kinds, hd_[:8], gd, ud, dd, idd[:8], vd[:8], FF, E, 0, E, out=small)
            graph = ctx.graph_capture_end()
            hd_.copy_(dev(ctx, rng.normal(0, 1, (T, H)).astype(np.float32)))
            idd.copy_(dev(ctx, ((order + 1) % E).astype(np.int32)))
            out.zero_()
            graph.launch()
            ctx.synchronize()
            replayed = out.clone()
            run()
            ctx.synchronize()
            assert torch.equal(replayed, out)
            # the small call: recorded on the tensor-core path, eager on the per-expert GEMV path
            eager = ctx.moe_experts_local(kinds, hd_[:8], gd, ud, dd, idd[:8], vd[:8], FF, E, 0, E)
            ctx.synchronize()
            assert max_rel_err(small.cpu().numpy(), eager.cpu().numpy()) <= TOL_MOE
            graph.close()
    finally:
        ctx.set_stream(0)


def test_moe_reference_fixture(ctx, ref_cases):
    T, H, FF, E, k = (int(v) for v in ref_cases["moe_dims"])
    kinds = (KIND_Q4_K, KIND_Q4_K, KIND_Q6_K)
    got = ctx.moe_experts(kinds, dev(ctx, ref_cases["moe_hidden"]), ctx.upload(ref_cases["moe_gate"]),
                          ctx.upload(ref_cases["moe_up"]), ctx.upload(ref_cases["moe_down"]),
                          dev(ctx, ref_cases["moe_ids"]), dev(ctx, ref_cases["moe_weights"]), FF, E).cpu().numpy()
    assert max_rel_err(got, ref_cases["moe_out_renorm"]) <= TOL_MOE


def test_moe_duplicate_routes_and_unused_experts(ctx, oracle):
    # tests/backend/test_backend_moe.c: duplicate expert ids for one token; experts nobody selects
    H, FF, E, k, T = 256, 256, 6, 2, 5
    kinds = (KIND_Q8_0, KIND_Q8_0, KIND_Q8_0)
    rng = np.random.default_rng(2)
    hid, gate, up, down, _ = _moe_case(rng, T, H, FF, E, k, kinds)
    ids = np.array([[1, 1], [4, 1], [1, 4], [4, 4], [1, 4]], dtype=np.int32)
    wts = rng.uniform(0.1, 1.0, (T, k)).astype(np.float32)
    ref = oracle.moe_experts(kinds, hid, gate, up, down, ids, wts, FF, E)
    got = ctx.moe_experts(kinds, dev(ctx, hid), ctx.upload(gate), ctx.upload(up), ctx.upload(down), dev(ctx, ids),
                          dev(ctx, wts), FF, E).cpu().numpy()
    assert max_rel_err(got, ref) <= TOL_FP32
    from marmot_b200 import MarmotCudaError

    bad = ids.copy()
    bad[0, 0] = E
    with pytest.raises(MarmotCudaError) as e:
        ctx.moe_experts(kinds, dev(ctx, hid), ctx.upload(gate), ctx.upload(up), ctx.upload(down), dev(ctx, bad),
                        dev(ctx, wts), FF, E)
    assert e.value.code == -1


# ---- few tokens on integer tensor-core instructions (csrc/gemm_i8.cu) ----
@pytest.mark.parametrize("name", ["q4_k", "q6_k"])
@pytest.mark.parametrize("T,K,F", [(2, 4096, 4096), (5, 2048, 200), (8, 4096, 1024), (9, 2048, 333), (16, 4096, 14336),
                                   (33, 2048, 64), (64, 4096, 4096), (64, 14336, 512), (3, 2048 + 256 * 5, 96)])
def test_integer_mma_matmul_vs_oracle(ctx, oracle, name, T, K, F):
    """2..64 tokens take the mma.sync s8 kernel: exact integer sub-block dots, so the result must sit at the
    fp32-accumulate tolerance whatever the token count; row groups that span several CTAs (and several row groups in
    one CTA), a ragged last row group, bias, and a strided input are all in the list."""
    import torch

    kind = KINDS[name]
    if kind == KINDS["q6_k"] and (K // 256) % 8:
        K = (K // 2048 + 1) * 2048  # Q6_K rows must be 16-byte multiples for the tensor map
    rng = np.random.default_rng(T * 131 + F)
    W = random_blocks(kind, F, K, rng)
    ldx = K + 8
    xbuf = rng.normal(0, 1, (T, ldx)).astype(np.float32)
    x = xbuf[:, :K]
    bias = rng.normal(0, 1, F).astype(np.float32)
    xd = torch.from_numpy(xbuf).cuda()[:, :K]
    l0 = ctx.launch_count()
    ctx.set_regime(4)  # REGIME_I8MMA: this kernel for every token count it covers, not only where it is the fastest
    try:
        got = ctx.linear(kind, xd, ctx.upload(W), F, bias=torch.from_numpy(bias).cuda()).cpu().numpy()
    finally:
        ctx.set_regime(0)
    assert ctx.launch_count() - l0 == 2  # the activation packer and the matmul
    want = oracle.linear(kind, np.ascontiguousarray(x), W, F, bias=bias)
    err = max_rel_err(got, want)
    assert err <= TOL_FP32, err
    assert err <= 2e-5, err  # in practice: only the order of the per-block f32 terms differs


@pytest.mark.parametrize("T", [4, 40])
def test_integer_mma_dual_output(ctx, oracle, T):
    import torch

    K, F = 4096, 1408
    rng = np.random.default_rng(T)
    Wa, Wb = random_blocks(KINDS["q4_k"], F, K, rng), random_blocks(KINDS["q4_k"], F, K, rng)
    x = rng.normal(0, 1, (T, K)).astype(np.float32)
    a = torch.empty((T, F), dtype=torch.float32, device="cuda")
    b = torch.empty((T, F), dtype=torch.float32, device="cuda")
    ctx.set_regime(4)
    try:
        ctx.linear_dual(KINDS["q4_k"], torch.from_numpy(x).cuda(), ctx.upload(Wa), ctx.upload(Wb), F, out_a=a, out_b=b)
        assert max_rel_err(a.cpu().numpy(), oracle.linear(KINDS["q4_k"], x, Wa, F)) <= 2e-5
        assert max_rel_err(b.cpu().numpy(), oracle.linear(KINDS["q4_k"], x, Wb, F)) <= 2e-5
        # twice more on the same context: the tickets were left at zero
        for _ in range(2):
            ctx.linear_dual(KINDS["q4_k"], torch.from_numpy(x).cuda(), ctx.upload(Wa), ctx.upload(Wb), F, out_a=a, out_b=b)
        assert max_rel_err(b.cpu().numpy(), oracle.linear(KINDS["q4_k"], x, Wb, F)) <= 2e-5
    finally:
        ctx.set_regime(0)


# ---- several weights over one activation read, with the layer's elementwise step as prologue (mcu_linear_multi) ----
def _multi_case(rng, names, T, K, Fs, ldx=None):
    import torch

    ldx = ldx or K
    kinds = [KINDS[n] for n in names]
    Ws = [random_blocks(k, F, K, rng) for k, F in zip(kinds, Fs)]
    xbuf = rng.normal(0, 1, (T, ldx)).astype(np.float32)
    xd = torch.from_numpy(xbuf).cuda()[:, :K]
    outs = [torch.full((T, F + 5), 7.0, dtype=torch.float32, device="cuda") for F in Fs]  # wider rows: ldo > F
    return kinds, Ws, np.ascontiguousarray(xbuf[:, :K]), xd, outs


@pytest.mark.parametrize("names,T,K,Fs", [
    (("q4_k", "q4_k", "q6_k"), 1, 2048, (2048, 256, 256)),   # q / k / v of a 1.1B decoder, mixed kinds
    (("q4_k", "q4_k"), 1, 2048, (5632, 5632)),                # gate / up
    (("q6_k",), 3, 2048, (777,)),
    (("q4_k", "q6_k", "q4_k", "q6_k"), 8, 1024, (96, 40, 8, 300)),
    (("q8_0", "q8_0", "q8_0"), 2, 1024, (512, 64, 64)),
    (("q4_k", "q4_k", "q4_k"), 1, 4096, (4096, 1024, 1024)),  # q / k / v of an 8B decoder
])
@pytest.mark.parametrize("with_aux", [True, False])
def test_linear_multi_add_rmsnorm_prologue(ctx, oracle, names, T, K, Fs, with_aux):
    """x' = x + aux, h = rms_norm(x') * w and every matmul of h in ONE launch: results against the oracle's add,
    rms_norm and linear; x' must come back exactly; the padding of wider output rows must stay untouched."""
    import torch

    rng = np.random.default_rng(T * 7919 + K + sum(Fs) + with_aux)
    kinds, Ws, x, xd, outs = _multi_case(rng, names, T, K, Fs)
    aux = rng.normal(0, 1, (T, K)).astype(np.float32) if with_aux else None
    w = rng.normal(1, 0.2, K).astype(np.float32)
    x_out = torch.zeros((T, K), dtype=torch.float32, device="cuda")
    jobs = [(k, ctx.upload(W), F, o[:, :F]) for k, W, F, o in zip(kinds, Ws, Fs, outs)]
    l0 = ctx.launch_count()
    ctx.linear_multi(xd, jobs, ("add_rmsnorm", torch.from_numpy(aux).cuda() if with_aux else None,
                                torch.from_numpy(w).cuda(), 1e-5, 0.0, x_out))
    ctx.synchronize()
    assert ctx.launch_count() - l0 == 1
    xs = (x + aux).astype(np.float32) if with_aux else x
    assert np.array_equal(x_out.cpu().numpy(), xs)
    h = oracle.rmsnorm(xs, w, 1e-5)
    for k, W, F, o in zip(kinds, Ws, Fs, outs):
        got = o.cpu().numpy()
        assert max_rel_err(got[:, :F], oracle.linear(k, h, W, F)) <= TOL_FP32
        assert np.all(got[:, F:] == 7.0)


@pytest.mark.parametrize("name,T,K,F", [("q6_k", 1, 5632, 2048), ("q4_k", 4, 5632, 2048), ("q8_0", 2, 1408, 96),
                                        ("q4_k", 1, 14336, 4096)])
def test_linear_multi_swiglu_prologue(ctx, oracle, name, T, K, F):
    """The down projection reads silu(gate) * up directly."""
    import torch

    rng = np.random.default_rng(T + K + F)
    kinds, Ws, gate, gd, outs = _multi_case(rng, (name,), T, K, (F,), ldx=K + 4)
    up = rng.normal(0, 1, (T, K)).astype(np.float32)
    l0 = ctx.launch_count()
    ctx.linear_multi(gd, [(kinds[0], ctx.upload(Ws[0]), F, outs[0][:, :F])], ("swiglu", torch.from_numpy(up).cuda()))
    ctx.synchronize()
    assert ctx.launch_count() - l0 == 1
    want = oracle.linear(kinds[0], oracle.swiglu(gate, up), Ws[0], F)
    assert max_rel_err(outs[0].cpu().numpy()[:, :F], want) <= TOL_FP32


def test_linear_multi_unaligned_rows_and_no_norm_weight(ctx, oracle):
    """Row strides and K that rule out 16-byte loads, K not a multiple of the block, no norm weight, no x_out."""
    import torch

    T, K, F = 3, 701, 48  # 48 Q6_K rows of 630 bytes: a whole number of 16-byte pieces, as the bulk copies need
    rng = np.random.default_rng(5)
    kinds, Ws, x, xd, outs = _multi_case(rng, ("q4_k", "q6_k"), T, K, (F, F), ldx=K + 1)
    auxbuf = rng.normal(0, 1, (T, K + 3)).astype(np.float32)
    ctx.linear_multi(xd, [(k, ctx.upload(W), F, o[:, :F]) for k, W, o in zip(kinds, Ws, outs)],
                     ("add_rmsnorm", torch.from_numpy(auxbuf).cuda()[:, :K], None, 1e-6, 0.0, None))
    h = oracle.rmsnorm((x + auxbuf[:, :K]).astype(np.float32), np.ones(K, dtype=np.float32), 1e-6)
    for k, W, o in zip(kinds, Ws, outs):
        assert max_rel_err(o.cpu().numpy()[:, :F], oracle.linear(k, h, W, F)) <= TOL_FP32


def test_linear_multi_large_matrices_at_a_handful_of_tokens(ctx, oracle):
    """Five to eight tokens over tens of megabytes of K-quant weights: the prologue runs as a kernel of its own and the
    matmuls take the integer-MMA regime (the dp4a kernel is bound by its dots there); same results as the oracle."""
    import torch

    T, K, F = 6, 4096, 5632  # 2 x 5632 x 2304 B = 26 MB
    rng = np.random.default_rng(606)
    kinds, Ws, x, xd, outs = _multi_case(rng, ("q4_k", "q4_k"), T, K, (F, F))
    aux = rng.normal(0, 1, (T, K)).astype(np.float32)
    w = rng.normal(1, 0.2, K).astype(np.float32)
    x_out = torch.zeros((T, K), dtype=torch.float32, device="cuda")
    jobs = [(k, ctx.upload(W), F, o[:, :F]) for k, W, o in zip(kinds, Ws, outs)]
    l0 = ctx.launch_count()
    ctx.linear_multi(xd, jobs, ("add_rmsnorm", torch.from_numpy(aux).cuda(), torch.from_numpy(w).cuda(), 1e-5, 0.0, x_out))
    ctx.synchronize()
    assert ctx.launch_count() - l0 > 1  # not the one-launch form
    xs = (x + aux).astype(np.float32)
    assert np.array_equal(x_out.cpu().numpy(), xs)
    h = oracle.rmsnorm(xs, w, 1e-5)
    for k, W, o in zip(kinds, Ws, outs):
        got = o.cpu().numpy()
        assert max_rel_err(got[:, :F], oracle.linear(k, h, W, F)) <= TOL_FP32
        assert np.all(got[:, F:] == 7.0)


def test_linear_multi_swiglu_over_a_large_matrix_at_a_handful_of_tokens(ctx, oracle):
    """The down projection of an 8B model for six tokens: SwiGLU as a kernel of its own, the matmul on the integer MMAs."""
    import torch

    T, K, F = 6, 14336, 4096  # 33 MB of Q4_K
    rng = np.random.default_rng(607)
    kinds, Ws, gate, gd, outs = _multi_case(rng, ("q4_k",), T, K, (F,))
    up = rng.normal(0, 1, (T, K)).astype(np.float32)
    l0 = ctx.launch_count()
    ctx.linear_multi(gd, [(kinds[0], ctx.upload(Ws[0]), F, outs[0][:, :F])], ("swiglu", torch.from_numpy(up).cuda()))
    ctx.synchronize()
    assert ctx.launch_count() - l0 > 1
    want = oracle.linear(kinds[0], oracle.swiglu(gate, up), Ws[0], F)
    got = outs[0].cpu().numpy()
    assert max_rel_err(got[:, :F], want) <= TOL_FP32
    assert np.all(got[:, F:] == 7.0)


def test_linear_multi_general_form(ctx, oracle):
    """More than eight tokens, or kinds that do not share an activation format: the prologue runs as its own kernel,
    the matmuls follow; same results."""
    import torch

    for names, T in ((("q4_k", "q4_k", "q6_k"), 12), (("q8_0", "q4_k"), 2)):
        K, Fs = 1024, (128, 128, 72)[:len(names)]
        rng = np.random.default_rng(T)
        kinds, Ws, x, xd, outs = _multi_case(rng, names, T, K, Fs)
        aux = rng.normal(0, 1, (T, K)).astype(np.float32)
        w = rng.normal(1, 0.2, K).astype(np.float32)
        x_out = torch.zeros((T, K), dtype=torch.float32, device="cuda")
        l0 = ctx.launch_count()
        ctx.linear_multi(xd, [(k, ctx.upload(W), F, o[:, :F]) for k, W, F, o in zip(kinds, Ws, Fs, outs)],
                         ("add_rmsnorm", torch.from_numpy(aux).cuda(), torch.from_numpy(w).cuda(), 1e-5, 0.0, x_out))
        assert ctx.launch_count() - l0 > 1
        xs = (x + aux).astype(np.float32)
        assert np.array_equal(x_out.cpu().numpy(), xs)
        h = oracle.rmsnorm(xs, w, 1e-5)
        for k, W, F, o in zip(kinds, Ws, Fs, outs):
            tol = TOL_MMA if T > 8 else TOL_FP32
            assert max_rel_err(o.cpu().numpy()[:, :F], oracle.linear(k, h, W, F)) <= tol


def test_linear_multi_without_prologue_equals_singles(ctx):
    import torch

    rng = np.random.default_rng(11)
    T, K, Fs = 2, 2048, (300, 64, 1000)
    kinds, Ws, x, xd, outs = _multi_case(rng, ("q4_k", "q6_k", "q4_k"), T, K, Fs)
    wd = [ctx.upload(W) for W in Ws]
    ctx.linear_multi(xd, [(k, w, F, o[:, :F]) for k, w, F, o in zip(kinds, wd, Fs, outs)])
    for k, w, F, o in zip(kinds, wd, Fs, outs):
        single = ctx.linear(k, xd, w, F)
        assert torch.equal(single, o[:, :F])  # same kernel, same arithmetic: bit for bit


def test_linear_multi_refusals(ctx):
    import torch
    from marmot_b200.runtime import MarmotCudaError

    x = torch.zeros((1, 256), device="cuda")
    out = torch.zeros((1, 8), device="cuda")
    w = ctx.upload(np.zeros((8, 144), dtype=np.uint8))
    with pytest.raises(MarmotCudaError):  # x_out may not be the input: other CTAs still read it
        ctx.linear_multi(x, [(KIND_Q4_K, w, 8, out)], ("add_rmsnorm", None, None, 1e-5, 0.0, x))
    with pytest.raises(MarmotCudaError):
        ctx.linear_multi(x, [(KIND_Q4_K, w, 8, out)] * 5)
    with pytest.raises(MarmotCudaError):
        ctx.linear_multi(x, [(1, w, 8, out)])  # Q4_0: no CUDA kernel


@pytest.mark.parametrize("names,T,K,Fs", [(("q4_k", "q4_k"), 64, 4096, (1408, 1408)), (("q4_k", "q6_k", "q4_k"), 33, 2048, (256, 128, 512)),
                                          (("q8_0",), 40, 1024, (256,))])
def test_linear_multi_tensor_core_form_with_prologues(ctx, oracle, names, T, K, Fs):
    """More than sixteen tokens: the prologue rides in the fp16 staging kernel and matmuls of one block-format class
    share one staging launch.  add + RMSNorm, then SwiGLU on the first job's shape."""
    import torch

    rng = np.random.default_rng(T + K)
    kinds, Ws, x, xd, outs = _multi_case(rng, names, T, K, Fs)
    aux = rng.normal(0, 1, (T, K)).astype(np.float32)
    w = rng.normal(1, 0.2, K).astype(np.float32)
    x_out = torch.zeros((T, K), dtype=torch.float32, device="cuda")
    wd = [ctx.upload(W) for W in Ws]
    l0 = ctx.launch_count()
    ctx.linear_multi(xd, [(k, wdev, F, o[:, :F]) for k, wdev, F, o in zip(kinds, wd, Fs, outs)],
                     ("add_rmsnorm", torch.from_numpy(aux).cuda(), torch.from_numpy(w).cuda(), 1e-5, 0.0, x_out))
    n_launch = ctx.launch_count() - l0
    xs = (x + aux).astype(np.float32)
    assert np.array_equal(x_out.cpu().numpy(), xs)
    h = oracle.rmsnorm(xs, w, 1e-5)
    for k, W, F, o in zip(kinds, Ws, Fs, outs):
        got = o.cpu().numpy()
        assert max_rel_err(got[:, :F], oracle.linear(k, h, W, F)) <= TOL_MMA
        assert np.all(got[:, F:] == 7.0)
    if len(set(kinds)) == 1 and len(kinds) == 2:
        assert n_launch <= 3  # one staging launch, one dual matmul (plus a split-K reduction at most)
    up = rng.normal(0, 1, (T, K)).astype(np.float32)
    ctx.linear_multi(xd, [(kinds[0], wd[0], Fs[0], outs[0][:, :Fs[0]])], ("swiglu", torch.from_numpy(up).cuda()))
    want = oracle.linear(kinds[0], oracle.swiglu(x, up), Ws[0], Fs[0])
    assert max_rel_err(outs[0].cpu().numpy()[:, :Fs[0]], want) <= TOL_MMA


# ---- float16 activations (mcu_linear_f16): the reference's no-packing branch ----
@pytest.mark.parametrize("name", NAMES)
def test_linear_f16_llama_golden(ctx, llama_goldens, name):
    import torch

    kind = KINDS[name]
    N, K, M = (int(v) for v in llama_goldens[f"matmul_{name}_dims"])
    x16 = llama_goldens[f"matmul_{name}_input_f16"].view(np.float16).reshape(N, K)
    want = llama_goldens[f"matmul_{name}_output_from_f16"].reshape(N, M)
    got = ctx.linear_f16(kind, torch.from_numpy(x16.copy()).cuda(), ctx.upload(llama_goldens[f"matmul_{name}_weight"]), M)
    assert max_rel_err(got.cpu().numpy(), want) <= 1e-5


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("T,K,F", [(1, 4096, 64), (3, 700, 13), (12, 2048, 40), (64, 1024, 9)])
def test_linear_f16_vs_oracle(ctx, oracle, name, T, K, F):
    """Against the oracle's restatement of cpu_vec_dot_*_f16 (one running f32 sum per output; here the sum is a
    shuffle tree): ragged K, strided rows, bias, f16 output."""
    import torch

    kind = KINDS[name]
    rng = np.random.default_rng(T * 31 + K + F)
    W = random_blocks(kind, F, K, rng)
    xbuf = rng.normal(0, 1, (T, K + 3)).astype(np.float16)
    x16 = np.ascontiguousarray(xbuf[:, :K])
    bias = rng.normal(0, 1, F).astype(np.float32)
    wd = ctx.upload(W)
    xd = torch.from_numpy(xbuf).cuda()[:, :K]
    got = ctx.linear_f16(kind, xd, wd, F, bias=torch.from_numpy(bias).cuda()).cpu().numpy()
    want = oracle.linear_f16(kind, x16, W, F, bias=bias)
    assert max_rel_err(got, want) <= TOL_FP32
    assert max_rel_err(got, want) <= 2e-5  # in practice: the order of the f32 additions
    half = ctx.linear_f16(kind, xd, wd, F, out_dtype=torch.float16).cpu().numpy().astype(np.float32)
    plain = oracle.linear_f16(kind, x16, W, F)
    finite = np.abs(plain) < 6e4
    assert np.max(np.abs(half - plain)[finite] / np.maximum(np.abs(plain[finite]), 1.0)) <= 2e-3  # one f16 rounding
