"""Pin the CPU oracle: the reference's own golden vectors, fixtures produced by
the reference library, and (when its library is present) the reference itself."""
from __future__ import annotations

import numpy as np
import pytest

from oracle.bindings import (KIND_BY_NAME, KIND_Q4_K, KIND_Q6_K, KIND_Q8_0, POLICY_RENORMALIZE_SELECTED,
                             POLICY_SOFTMAX_SELECTED, row_bytes)

NAMES = ["q4_k", "q6_k", "q8_0"]


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("name", NAMES)
def test_matmul_llama_golden(oracle, llama_goldens, name):
    # tests/backend/test_matmul_quantized.c:120-182: |d| <= |exp|*5e-5 + 2e-5
    T, K, F = (int(v) for v in llama_goldens[f"matmul_{name}_dims"])
    x = llama_goldens[f"matmul_{name}_input_f32"].reshape(T, K)
    y = oracle.linear(KIND_BY_NAME[name], x, llama_goldens[f"matmul_{name}_weight"], F)
    exp = llama_goldens[f"matmul_{name}_output_from_f32"].reshape(T, F)
    assert np.all(np.abs(y - exp) <= np.abs(exp) * 5e-5 + 2e-5)


@pytest.mark.parametrize("name,act,nb", [("q4_k", "q8_k", 1), ("q6_k", "q8_k", 1), ("q8_0", "q8_0", 8)])
def test_vec_dot_llama_golden(oracle, llama_goldens, name, act, nb):
    # tests/backend/test_vec_dot.c:135-156: |d| <= |exp|*2e-5 + 1e-5
    got = oracle.vec_dot(KIND_BY_NAME[name], llama_goldens[f"vec_dot_{name}_weights"],
                         llama_goldens[f"vec_dot_{act}_activations"], nb)
    exp = float(llama_goldens[f"vec_dot_{name}_{act}_expected"][0])
    assert abs(got - exp) <= abs(exp) * 2e-5 + 1e-5


@pytest.mark.parametrize("name", NAMES)
def test_dequant_llama_golden(oracle, llama_goldens, name):
    # tests/backend/test_backend_quantization.c:209-340: dequant golden within 5e-4
    exp = llama_goldens[f"llama_{name}_dequant"]
    got = oracle.dequantize(KIND_BY_NAME[name], llama_goldens[f"llama_{name}"], exp.size)
    assert np.max(np.abs(got - exp)) <= 5e-4


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("case", [0, 1, 2])
def test_reference_fixture_bit_exact(oracle, ref_cases, name, case):
    kind = KIND_BY_NAME[name]
    x, W = ref_cases[f"{name}_{case}_x"], ref_cases[f"{name}_{case}_w"]
    T, K = x.shape
    F = W.size // row_bytes(kind, K)
    assert np.array_equal(bits(oracle.dequantize(kind, W, F * K)), bits(ref_cases[f"{name}_{case}_deq"]))
    assert np.array_equal(bits(oracle.linear(kind, x, W, F)), bits(ref_cases[f"{name}_{case}_y"]))


def test_reference_fixture_moe(oracle, ref_cases):
    T, H, FF, E, k = (int(v) for v in ref_cases["moe_dims"])
    kinds = (KIND_Q4_K, KIND_Q4_K, KIND_Q6_K)
    args = (ref_cases["moe_hidden"], ref_cases["moe_gate"], ref_cases["moe_up"], ref_cases["moe_down"])
    ids, wts = ref_cases["moe_ids"], ref_cases["moe_weights"]
    vals, idx = oracle.topk(ref_cases["moe_probs"], k)
    assert np.array_equal(idx, ids) and np.array_equal(bits(vals), bits(wts))
    a = oracle.moe_experts(kinds, *args, ids, wts, FF, E, policy=POLICY_RENORMALIZE_SELECTED)
    assert np.array_equal(bits(a), bits(ref_cases["moe_out_renorm"]))
    b = oracle.moe_experts(kinds, *args, ids, wts, FF, E, policy=POLICY_SOFTMAX_SELECTED, weights_scale=0.5)
    assert np.array_equal(bits(b), bits(ref_cases["moe_out_softmax"]))
    c = oracle.moe_experts(kinds, args[0][:3], *args[1:], ids[:3], wts[:3], FF, E)
    assert np.array_equal(bits(c), bits(ref_cases["moe_out_decode"]))


def test_topk_ties_prefer_lower_index(oracle):
    # tests/backend/test_backend_moe.c:127-181
    x = np.array([[1.0, 3.0, 3.0, 2.0, 3.0], [0.5, 0.5, 0.5, 0.5, 0.5]], dtype=np.float32)
    vals, idx = oracle.topk(x, 3)
    assert idx.tolist() == [[1, 2, 4], [0, 1, 2]]
    assert vals.tolist() == [[3.0, 3.0, 3.0], [0.5, 0.5, 0.5]]


def test_pack_edge_cases(oracle):
    # all-zero block -> d = 0 and zero quants; ragged tail is zero padded (matmul_quant_pack.c:121-126,159-166)
    x = np.zeros(300, dtype=np.float32)
    x[256:] = np.linspace(-1, 1, 44, dtype=np.float32)
    blk = oracle.pack_q8_k(x)
    assert blk.size == 2 * 292 and not blk[:292].any()
    qs = blk[292 + 4: 292 + 4 + 256].view(np.int8)
    assert not qs[44:].any() and int(np.abs(qs).max()) == 127
    b0 = oracle.pack_q8_0(np.zeros(40, dtype=np.float32))
    assert b0[:2].view(np.float16)[0] == np.float16(1.0) and not b0[2:34].any()


@pytest.mark.parametrize("name", NAMES)
def test_against_reference_library_live(oracle, reference_lib, name):
    """Seeded random shapes, oracle vs the reference backend in this process: bit for bit."""
    kind = KIND_BY_NAME[name]
    rng = np.random.default_rng(7)
    bv = 32 if kind == KIND_Q8_0 else 256
    for T, K, F in [(1, bv, 1), (2, bv * 3, 5), (17, bv * 8, 19), (16, 4096, 24)]:
        W = reference_lib.quantize(kind, rng.normal(0, 0.02, (F, K)).astype(np.float32))
        x = rng.normal(0, 1, (T, K)).astype(np.float32)
        assert np.array_equal(bits(reference_lib.dequantize(kind, W, F * K)), bits(oracle.dequantize(kind, W, F * K)))
        assert np.array_equal(bits(reference_lib.linear(kind, x, W, F)), bits(oracle.linear(kind, x, W, F)))


@pytest.mark.parametrize("name", ["q4_k", "q6_k", "q8_0"])
def test_linear_f16_oracle_against_the_reference_goldens(oracle, llama_goldens, name):
    """The f16-activation matmul restated from cpu_vec_dot_*_f16 reproduces g_matmul_*_output_from_f16 (bit for bit
    for Q4_K and Q8_0; the Q6_K golden differs in the last place, as the reference library's own output does)."""
    from tests.util import KINDS

    N, K, M = (int(v) for v in llama_goldens[f"matmul_{name}_dims"])
    x16 = llama_goldens[f"matmul_{name}_input_f16"].view(np.uint16).reshape(N, K)
    got = oracle.linear_f16(KINDS[name], x16, llama_goldens[f"matmul_{name}_weight"], M)
    want = llama_goldens[f"matmul_{name}_output_from_f16"].reshape(N, M)
    if name == "q6_k":
        assert np.max(np.abs(got - want) / np.abs(want)) <= 1e-6
    else:
        assert np.array_equal(got, want)
