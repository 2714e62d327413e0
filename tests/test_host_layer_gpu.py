"""The C23 host layer (marmot_b200/host/cuda_backend.c) driven with real marmot tensors.

libmarmot_ref.so (the reference CPU backend, built by oracle/build_ref.py) supplies the marmot tensor API
and is the checker; libmarmot_cuda_backend.so is the layer under test.  Each case runs the reference operator
on the CPU context and the cuda_* implementation function on the same tensors' values, then compares.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np
import pytest

from oracle.bindings import (DT_F32, DT_I8, DT_I32, DT_U8, FFN_SWIGLU, KIND_Q4_K, KIND_Q6_K, KIND_Q8_0,
                             POLICY_RENORMALIZE_SELECTED, REF_LIB, Reference, _MoeDesc, _Tensor, _TopkDesc)
from tests.util import TOL_FP32, TOL_MMA, TOL_MOE, cosine, max_rel_err, random_blocks

pytestmark = pytest.mark.gpu

BACKEND_LIB = Path(__file__).resolve().parents[1] / "marmot_b200" / "libmarmot_cuda_backend.so"
TP = C.POINTER(_Tensor)


class _Ops(C.Structure):
    """struct marmot_device_ops, include/marmot/device.h:42-66."""
    _fields_ = [
        ("init", C.CFUNCTYPE(C.c_int, C.POINTER(C.c_void_p))),
        ("destroy", C.CFUNCTYPE(None, C.c_void_p)),
        ("configure", C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p)),
        ("alloc", C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p))),
        ("free", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p)),
        ("memcpy_to_device", C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t)),
        ("memcpy_from_device", C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t)),
        ("synchronize", C.CFUNCTYPE(C.c_int, C.c_void_p)),
        ("allocator_usage", C.c_void_p),
        ("graph_batch_begin", C.c_void_p),
        ("graph_batch_end", C.c_void_p),
        ("on_host_ptr_freed", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p)),
        ("on_host_range_freed", C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_size_t)),
    ]


class Backend:
    def __init__(self, ref: Reference):
        self.ref = ref
        C.CDLL(str(REF_LIB), mode=C.RTLD_GLOBAL)  # marmot_* helpers the layer calls
        self.lib = L = C.CDLL(str(BACKEND_LIB))
        L.marmot_get_cuda_ops.restype = C.POINTER(_Ops)
        self.ops = L.marmot_get_cuda_ops().contents
        for n in ("q4_k", "q6_k", "q8_0"):
            getattr(L, f"cuda_matmul_quantized_{n}").argtypes = [C.c_void_p, TP, TP, C.c_void_p, TP]
            getattr(L, f"cuda_dequantize_{n}").argtypes = [C.c_void_p, TP, TP]
        L.cuda_matmul_quantized_dual_output.argtypes = [C.c_void_p, TP, TP, TP, TP, TP]
        L.cuda_moe_experts_impl.argtypes = [C.c_void_p, C.POINTER(_MoeDesc)]
        L.cuda_topk_impl.argtypes = [C.c_void_p, C.POINTER(_TopkDesc)]
        ctx = C.c_void_p()
        rc = self.ops.init(C.byref(ctx))
        assert rc == 0 and ctx.value, ref.lib.marmot_get_last_error_detail()
        self.ctx = ctx

    def close(self):
        self.ops.destroy(self.ctx)

    def fetch(self, t, shape, dtype) -> np.ndarray:
        """What marmot_tensor_to_host does for a device-resident tensor (src/core/tensor/transfer.c:36-62)."""
        s = t.contents
        assert s.memory_location == 1 and s.needs_sync  # MARMOT_MEMORY_DEVICE, written by the backend
        nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
        assert self.ops.memcpy_from_device(self.ctx, s.data, s.data, nbytes) == 0
        return np.ctypeslib.as_array(C.cast(s.data, C.POINTER(C.c_uint8)), (nbytes,)).view(dtype).reshape(shape).copy()

    def check(self, rc, what):
        if rc != 0:
            detail = self.ref.lib.marmot_get_last_error_detail()
            raise RuntimeError(f"{what} failed ({rc}): {detail.decode() if detail else ''}")


@pytest.fixture(scope="module")
def backend(reference_lib):
    if not BACKEND_LIB.exists():
        pytest.fail(f"{BACKEND_LIB} missing: run marmot_b200/host/build_host.py with a marmot checkout")
    b = Backend(reference_lib)
    yield b
    b.close()


NAMES = {KIND_Q4_K: "q4_k", KIND_Q6_K: "q6_k", KIND_Q8_0: "q8_0"}


@pytest.mark.parametrize("kind", [KIND_Q4_K, KIND_Q6_K, KIND_Q8_0])
@pytest.mark.parametrize("T,K,F", [(1, 1024, 384), (5, 512, 96), (40, 1024, 256)])
def test_matmul_through_marmot_tensors(backend, kind, T, K, F):
    ref = backend.ref
    rng = np.random.default_rng(kind * 1000 + T)
    W = random_blocks(kind, F, K, rng)
    x = rng.normal(0, 1, (T, K)).astype(np.float32)
    want = ref.linear(kind, x, W, F)
    tx, tw, to = ref._tensor((T, K), DT_F32, x), ref._qtensor((F, K), kind, W), ref._tensor((T, F), DT_F32)
    try:
        fn = getattr(backend.lib, f"cuda_matmul_quantized_{NAMES[kind]}")
        backend.check(fn(backend.ctx, tx, tw, None, to), "cuda_matmul_quantized")
        got = backend.fetch(to, (T, F), np.float32)
        # second call: weights already resident (no upload), same result
        backend.check(fn(backend.ctx, tx, tw, None, to), "cuda_matmul_quantized")
        again = backend.fetch(to, (T, F), np.float32)
    finally:
        for t in (to, tw, tx):
            backend.ops.on_host_ptr_freed(backend.ctx, t.contents.data)
            ref.lib.marmot_tensor_destroy(t)
    tol = TOL_FP32 if T <= 8 else TOL_MMA
    assert max_rel_err(got, want) <= tol
    assert np.array_equal(got, again)


def test_matmul_rejects_what_it_cannot_run(backend):
    ref = backend.ref
    rng = np.random.default_rng(1)
    W = random_blocks(KIND_Q4_K, 8, 256, rng)
    tx = ref._tensor((2, 256), DT_F32, rng.normal(0, 1, (2, 256)).astype(np.float32))
    tw = ref._qtensor((8, 256), KIND_Q4_K, W)
    to = ref._tensor((2, 9), DT_F32)  # wrong feature count
    try:
        assert backend.lib.cuda_matmul_quantized_q4_k(backend.ctx, tx, tw, None, to) != 0
        assert backend.lib.cuda_matmul_quantized_q6_k(backend.ctx, tx, tw, None, to) != 0
        assert backend.lib.cuda_matmul_quantized_q4_k(backend.ctx, None, tw, None, to) != 0
    finally:
        for t in (to, tw, tx):
            ref.lib.marmot_tensor_destroy(t)


def test_dual_output(backend):
    ref = backend.ref
    rng = np.random.default_rng(7)
    T, K, F = 3, 512, 160
    Wa, Wb = random_blocks(KIND_Q4_K, F, K, rng), random_blocks(KIND_Q4_K, F, K, rng)
    x = rng.normal(0, 1, (T, K)).astype(np.float32)
    tx = ref._tensor((T, K), DT_F32, x)
    ta, tb = ref._qtensor((F, K), KIND_Q4_K, Wa), ref._qtensor((F, K), KIND_Q4_K, Wb)
    oa, ob = ref._tensor((T, F), DT_F32), ref._tensor((T, F), DT_F32)
    try:
        backend.check(backend.lib.cuda_matmul_quantized_dual_output(backend.ctx, tx, ta, tb, oa, ob), "dual")
        ga, gb = backend.fetch(oa, (T, F), np.float32), backend.fetch(ob, (T, F), np.float32)
    finally:
        for t in (ob, oa, tb, ta, tx):
            backend.ops.on_host_ptr_freed(backend.ctx, t.contents.data)
            ref.lib.marmot_tensor_destroy(t)
    assert max_rel_err(ga, ref.linear(KIND_Q4_K, x, Wa, F)) <= TOL_FP32
    assert max_rel_err(gb, ref.linear(KIND_Q4_K, x, Wb, F)) <= TOL_FP32


@pytest.mark.parametrize("kind,rows,cols", [(KIND_Q4_K, 6, 512), (KIND_Q6_K, 3, 256), (KIND_Q8_0, 5, 96),
                                            (KIND_Q8_0, 5, 80), (KIND_Q4_K, 2, 300)])
def test_dequantize_bit_exact(backend, kind, rows, cols):
    """cols that are not a whole number of blocks: every row is padded to whole blocks in the input
    (src/backends/cpu/quantization/ops/quantize_core.c:299-330)."""
    ref = backend.ref
    rng = np.random.default_rng(kind)
    W = random_blocks(kind, rows, cols, rng)
    store_dt = DT_I8 if kind == KIND_Q8_0 else DT_U8
    ti, to = ref._tensor((W.nbytes,), store_dt, W), ref._tensor((rows, cols), DT_F32)
    tc = ref._tensor((rows, cols), DT_F32)
    try:
        ref._check(getattr(ref.lib, f"marmot_dequantize_{NAMES[kind]}")(ref.ctx, ti, tc), "marmot_dequantize")
        want = ref._read(tc, (rows, cols), np.float32)
        fn = getattr(backend.lib, f"cuda_dequantize_{NAMES[kind]}")
        backend.check(fn(backend.ctx, ti, to), "cuda_dequantize")
        got = backend.fetch(to, (rows, cols), np.float32)
    finally:
        for t in (tc, to, ti):
            backend.ops.on_host_ptr_freed(backend.ctx, t.contents.data)
            ref.lib.marmot_tensor_destroy(t)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_topk(backend):
    ref = backend.ref
    rng = np.random.default_rng(3)
    rows, cols, k = 33, 8, 2
    x = rng.normal(0, 1, (rows, cols)).astype(np.float32)
    x[4, :] = 0.5  # ties go to the lower index
    tx, tv, ti = ref._tensor((rows, cols), DT_F32, x), ref._tensor((rows, k), DT_F32), ref._tensor((rows, k), DT_I32)
    try:
        desc = _TopkDesc(tx, tv, ti, -1, k)
        backend.check(backend.lib.cuda_topk_impl(backend.ctx, C.byref(desc)), "cuda_topk_impl")
        vals, idx = backend.fetch(tv, (rows, k), np.float32), backend.fetch(ti, (rows, k), np.int32)
    finally:
        for t in (ti, tv, tx):
            backend.ops.on_host_ptr_freed(backend.ctx, t.contents.data)
            ref.lib.marmot_tensor_destroy(t)
    order = np.argsort(-x, axis=1, kind="stable")[:, :k]
    assert np.array_equal(idx, order.astype(np.int32))
    assert np.array_equal(vals, np.take_along_axis(x, order, 1))


def test_moe_experts(backend):
    ref = backend.ref
    rng = np.random.default_rng(11)
    T, H, FF, E, k = 24, 256, 512, 4, 2
    gate = np.concatenate([random_blocks(KIND_Q4_K, FF, H, rng, d_sigma=0.0005) for _ in range(E)])
    up = np.concatenate([random_blocks(KIND_Q4_K, FF, H, rng, d_sigma=0.0005) for _ in range(E)])
    down = np.concatenate([random_blocks(KIND_Q6_K, H, FF, rng) for _ in range(E)])
    hidden = rng.normal(0, 1, (T, H)).astype(np.float32)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    wts = rng.uniform(0.1, 1.0, (T, k)).astype(np.float32)
    kinds = (KIND_Q4_K, KIND_Q4_K, KIND_Q6_K)
    want = ref.moe_experts(kinds, hidden, gate, up, down, ids, wts, FF, E)
    th = ref._tensor((T, H), DT_F32, hidden)
    tg, tu = ref._expert_tensor(kinds[0], gate, FF, H, E), ref._expert_tensor(kinds[1], up, FF, H, E)
    td = ref._expert_tensor(kinds[2], down, H, FF, E)
    ti, tw, to = ref._tensor((T, k), DT_I32, ids), ref._tensor((T, k), DT_F32, wts), ref._tensor((T, H), DT_F32)
    try:
        desc = _MoeDesc(th, tg, tu, td, ti, tw, to, FFN_SWIGLU, 1.0, POLICY_RENORMALIZE_SELECTED)
        backend.check(backend.lib.cuda_moe_experts_impl(backend.ctx, C.byref(desc)), "cuda_moe_experts_impl")
        got = backend.fetch(to, (T, H), np.float32)
    finally:
        for t in (to, tw, ti, td, tu, tg, th):
            backend.ops.on_host_ptr_freed(backend.ctx, t.contents.data)
            ref.lib.marmot_tensor_destroy(t)
    assert max_rel_err(got, want) <= TOL_MOE
    assert cosine(got, want) >= 0.999


class _VecDotDesc(C.Structure):
    """struct marmot_vec_dot_descriptor, include/marmot/ops_types.h:136-143."""
    _fields_ = [("weights", C.c_void_p), ("activations", C.c_void_p), ("num_blocks", C.c_size_t),
                ("weight_kind", C.c_int), ("activation_kind", C.c_int), ("layout", C.c_int)]


@pytest.mark.parametrize("name,kind,act,act_kind,nb", [("q4_k", KIND_Q4_K, "q8_k", 12, 1), ("q6_k", KIND_Q6_K, "q8_k", 12, 1),
                                                      ("q8_0", KIND_Q8_0, "q8_0", KIND_Q8_0, 8)])
def test_vec_dot_llama_golden(backend, llama_goldens, name, kind, act, act_kind, nb):
    """cuda_vec_dot on the reference's llama.cpp golden vectors, at the tolerance of tests/backend/test_vec_dot.c:135-156,
    and against the reference's own cpu_vec_dot through the public marmot_vec_dot."""
    L = backend.lib
    L.cuda_vec_dot.argtypes = [C.c_void_p, C.POINTER(_VecDotDesc), C.POINTER(C.c_float)]
    w = np.ascontiguousarray(llama_goldens[f"vec_dot_{name}_weights"], dtype=np.uint8)
    a = np.ascontiguousarray(llama_goldens[f"vec_dot_{act}_activations"], dtype=np.uint8)
    desc = _VecDotDesc(w.ctypes.data, a.ctypes.data, nb, kind, act_kind, 1)  # MARMOT_QUANT_LAYOUT_GGUF
    out = C.c_float(-1.0)
    assert L.cuda_vec_dot(backend.ctx, C.byref(desc), C.byref(out)) == 0
    exp = float(llama_goldens[f"vec_dot_{name}_{act}_expected"][0])
    assert abs(out.value - exp) <= abs(exp) * 2e-5 + 1e-5
    ref = backend.ref.lib
    ref.marmot_vec_dot.argtypes = [C.c_void_p, C.POINTER(_VecDotDesc), C.POINTER(C.c_float)]
    want = C.c_float(-1.0)
    assert ref.marmot_vec_dot(backend.ref.ctx, C.byref(desc), C.byref(want)) == 0
    assert abs(out.value - want.value) <= abs(want.value) * 2e-6 + 1e-6
    # the reference's argument checks
    bad = _VecDotDesc(w.ctypes.data, a.ctypes.data, nb, kind, KIND_Q4_K, 1)
    assert L.cuda_vec_dot(backend.ctx, C.byref(bad), C.byref(out)) != 0  # activation kind mismatch
    empty = _VecDotDesc(w.ctypes.data, a.ctypes.data, 0, kind, act_kind, 1)
    assert L.cuda_vec_dot(backend.ctx, C.byref(empty), C.byref(out)) == 0 and out.value == 0.0
