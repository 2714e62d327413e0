"""ctypes binding of marmot's public C API (include/marmot/*.h): contexts, tensors and the operators on the quantized
matmul path, for any libmarmot and any backend it was built with.

With marmot_b200/libmarmot_b200.so (host/build_marmot.py: marmot's core + CPU backend + this package's CUDA backend)
`MarmotLibrary(backend=BACKEND_CUDA)` is the drop-in path a marmot user takes: `marmot_init(MARMOT_BACKEND_CUDA)`,
host tensors in, `marmot_linear` / `marmot_moe_experts` / ... through marmot's own dispatch, results read back with
`marmot_tensor_copy_to_host_buffer`.  The same class over the CPU backend gives the reference arithmetic.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

from .runtime import KIND_Q4_K, KIND_Q6_K, KIND_Q8_0, row_bytes

PKG = Path(__file__).resolve().parent
FULL_LIB = PKG / "libmarmot_b200.so"

BACKEND_CPU, BACKEND_METAL, BACKEND_CUDA = 0, 1, 2
POLICY_SOFTMAX_SELECTED, POLICY_RENORMALIZE_SELECTED = 0, 2
FFN_SWIGLU, FFN_GEGLU = 0, 2


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)



MAX_DIMS = 8
DT_F32, DT_F16, DT_I32, DT_I8, DT_U8 = 0, 1, 3, 5, 6


class _Shape(C.Structure):
    _fields_ = [("ndim", C.c_size_t), ("shape", C.c_size_t * MAX_DIMS), ("strides", C.c_size_t * MAX_DIMS)]


class _Tensor(C.Structure):
    """struct marmot_tensor, include/marmot/tensor.h:20-38."""
    _fields_ = [
        ("shape", _Shape), ("dtype", C.c_int), ("data", C.c_void_p), ("capacity_bytes", C.c_size_t),
        ("owns_data", C.c_bool), ("quant_params", C.c_void_p), ("quant_kind", C.c_int), ("quant_layout", C.c_int),
        ("backend", C.c_int), ("ctx", C.c_void_p), ("memory_location", C.c_int), ("needs_sync", C.c_bool),
        ("packed_data", C.c_void_p), ("packed_src_data", C.c_void_p), ("packed_bytes", C.c_size_t),
        ("packed_row_bytes", C.c_size_t), ("packed_rows", C.c_size_t),
    ]


class _MoeDesc(C.Structure):
    """struct marmot_moe_experts_desc, include/marmot/ops_types.h:203-214."""
    _fields_ = [
        ("hidden_states", C.POINTER(_Tensor)), ("gate_exps", C.POINTER(_Tensor)), ("up_exps", C.POINTER(_Tensor)),
        ("down_exps", C.POINTER(_Tensor)), ("topk_ids", C.POINTER(_Tensor)), ("topk_weights", C.POINTER(_Tensor)),
        ("out", C.POINTER(_Tensor)), ("ffn_type", C.c_int), ("weights_scale", C.c_float),
        ("router_weight_policy", C.c_int),
    ]


class _TopkDesc(C.Structure):
    _fields_ = [("x", C.POINTER(_Tensor)), ("values_out", C.POINTER(_Tensor)), ("indices_out", C.POINTER(_Tensor)),
                ("axis", C.c_int32), ("k", C.c_uint32)]


class _RmsnormDesc(C.Structure):
    """struct marmot_rmsnorm_desc, include/marmot/ops_types.h:181-187."""
    _fields_ = [("x", C.POINTER(_Tensor)), ("residual", C.POINTER(_Tensor)), ("weight", C.POINTER(_Tensor)),
                ("out", C.POINTER(_Tensor)), ("eps", C.c_float)]


class _RopeParams(C.Structure):
    """struct marmot_rope_params, include/marmot/ops_types.h:98-112."""
    _fields_ = [("positions", C.POINTER(_Tensor)), ("scaling_type", C.c_int), ("rope_type", C.c_int),
                ("theta", C.c_float), ("freq_scale", C.c_float), ("ext_factor", C.c_float), ("attn_factor", C.c_float),
                ("beta_fast", C.c_float), ("beta_slow", C.c_float), ("orig_ctx_len", C.c_uint32),
                ("head_dim", C.c_uint32), ("apply_to_q", C.c_bool), ("apply_to_k", C.c_bool)]


class _PagedAttentionDesc(C.Structure):
    """marmot_paged_attention_desc_t, include/marmot/ops/paged_attention.h:32-56."""
    _fields_ = [("struct_size", C.c_uint32), ("struct_version", C.c_uint32), ("flags", C.c_uint64),
                ("token_count", C.c_uint32), ("layer_idx", C.c_uint32), ("num_q_heads", C.c_uint32),
                ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("block_size", C.c_uint32),
                ("scale", C.c_float), ("token_meta", C.POINTER(_Tensor)), ("q", C.POINTER(_Tensor)),
                ("k_new", C.POINTER(_Tensor)), ("v_new", C.POINTER(_Tensor)), ("kv_k", C.POINTER(_Tensor)),
                ("kv_v", C.POINTER(_Tensor)), ("block_table", C.POINTER(_Tensor)), ("out", C.POINTER(_Tensor)),
                ("pnext", C.c_void_p), ("reserved", C.c_uint64 * 4)]


DT_U32 = 8


class _VecDotDesc(C.Structure):
    """struct marmot_vec_dot_descriptor, include/marmot/ops_types.h:136-143."""
    _fields_ = [("weights", C.c_void_p), ("activations", C.c_void_p), ("num_blocks", C.c_size_t),
                ("weight_kind", C.c_int), ("activation_kind", C.c_int), ("layout", C.c_int)]


class MarmotLibrary:
    """One marmot context of `backend` in the library at `path`, driven through marmot's public C API."""

    def __init__(self, path: Path = FULL_LIB, backend: int = BACKEND_CUDA, threads: int | None = None):
        path = Path(path)
        if not path.exists():
            raise FileNotFoundError(f"{path} missing: build it from a marmot checkout first")
        self.backend = backend
        if threads is not None:
            os.environ["MARMOT_NUM_THREADS"] = str(threads)
        self.lib = L = C.CDLL(str(path))
        TP = C.POINTER(_Tensor)
        L.marmot_init.restype = C.c_void_p
        L.marmot_init.argtypes = [C.c_int]
        L.marmot_destroy.argtypes = [C.c_void_p]
        L.marmot_tensor_create.restype = TP
        L.marmot_tensor_create.argtypes = [C.c_void_p, C.POINTER(C.c_size_t), C.c_size_t, C.c_int]
        L.marmot_tensor_create_quantized.restype = TP
        L.marmot_tensor_create_quantized.argtypes = [C.c_void_p, C.POINTER(C.c_size_t), C.c_size_t, C.c_int]
        L.marmot_tensor_destroy.argtypes = [TP]
        L.marmot_tensor_copy_from_host_buffer.argtypes = [C.c_void_p, TP, C.c_void_p, C.c_size_t]
        L.marmot_tensor_copy_to_host_buffer.argtypes = [C.c_void_p, TP, C.c_void_p, C.c_size_t]
        L.marmot_tensor_size_bytes.restype = C.c_size_t
        L.marmot_tensor_size_bytes.argtypes = [TP]
        L.marmot_linear.argtypes = [C.c_void_p, TP, TP, C.c_void_p, TP]
        L.marmot_moe_experts.argtypes = [C.c_void_p, C.POINTER(_MoeDesc)]
        L.marmot_get_last_error_detail.restype = C.c_char_p
        for n in ("q4_k", "q6_k", "q8_0"):
            getattr(L, f"marmot_quantize_{n}").argtypes = [C.c_void_p, TP, TP]
            getattr(L, f"marmot_dequantize_{n}").argtypes = [C.c_void_p, TP, TP]
        L.marmot_rmsnorm.argtypes = [C.c_void_p, C.POINTER(_RmsnormDesc)]
        L.marmot_rope.argtypes = [C.c_void_p, TP, C.POINTER(_RopeParams), TP]
        L.marmot_swiglu.argtypes = [C.c_void_p, TP, TP, TP]
        L.marmot_paged_attention.argtypes = [C.c_void_p, C.POINTER(_PagedAttentionDesc)]
        L.marmot_topk.argtypes = [C.c_void_p, C.POINTER(_TopkDesc)]
        L.marmot_vec_dot.argtypes = [C.c_void_p, C.POINTER(_VecDotDesc), C.POINTER(C.c_float)]
        L.marmot_tensor_to_device.argtypes = [C.c_void_p, TP]
        L.marmot_tensor_to_host.argtypes = [C.c_void_p, TP]
        L.marmot_graph_batch_begin.argtypes = [C.c_void_p]
        L.marmot_graph_batch_end.argtypes = [C.c_void_p, C.c_bool]
        self.ctx = L.marmot_init(backend)
        if not self.ctx:
            detail = L.marmot_get_last_error_detail()
            raise RuntimeError(f"marmot_init({backend}) failed: {detail.decode() if detail else ''}")

    def close(self):
        if self.ctx:
            self.lib.marmot_destroy(self.ctx)
            self.ctx = None

    def _check(self, rc, what):
        if rc != 0:
            detail = self.lib.marmot_get_last_error_detail()
            raise RuntimeError(f"{what} failed ({rc}): {detail.decode() if detail else ''}")

    def _tensor(self, shape, dtype, src: np.ndarray | None = None):
        arr = (C.c_size_t * len(shape))(*shape)
        t = self.lib.marmot_tensor_create(self.ctx, arr, len(shape), dtype)
        assert t, "tensor_create"
        if src is not None:
            src = np.ascontiguousarray(src)
            self._check(self.lib.marmot_tensor_copy_from_host_buffer(self.ctx, t, _p(src), src.nbytes), "copy_from")
        return t

    def _qtensor(self, shape, kind, blocks: np.ndarray):
        arr = (C.c_size_t * len(shape))(*shape)
        t = self.lib.marmot_tensor_create_quantized(self.ctx, arr, len(shape), kind)
        assert t, "tensor_create_quantized"
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        assert self.lib.marmot_tensor_size_bytes(t) == blocks.nbytes, (self.lib.marmot_tensor_size_bytes(t), blocks.nbytes)
        self._check(self.lib.marmot_tensor_copy_from_host_buffer(self.ctx, t, _p(blocks), blocks.nbytes), "copy_from")
        return t

    def _read(self, t, shape, dtype) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        self._check(self.lib.marmot_tensor_copy_to_host_buffer(self.ctx, t, _p(out), out.nbytes), "copy_to")
        return out

    def linear(self, kind: int, x: np.ndarray, W: np.ndarray, F: int) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        T, K = x.shape
        tx = self._tensor((T, K), DT_F32, x)
        tw = self._qtensor((F, K), kind, W)
        to = self._tensor((T, F), DT_F32)
        try:
            self._check(self.lib.marmot_linear(self.ctx, tx, tw, None, to), "marmot_linear")
            return self._read(to, (T, F), np.float32)
        finally:
            for t in (to, tw, tx):
                self.lib.marmot_tensor_destroy(t)

    def linear_f16(self, kind: int, x16: np.ndarray, W: np.ndarray, F: int, half_out: bool = False) -> np.ndarray:
        """marmot_linear with FLOAT16 activations [T, K] (float16 array); FLOAT32 result, or FLOAT16 with half_out."""
        x16 = np.ascontiguousarray(x16, dtype=np.float16)
        T, K = x16.shape
        tx = self._tensor((T, K), DT_F16, x16)
        tw = self._qtensor((F, K), kind, W)
        to = self._tensor((T, F), DT_F16 if half_out else DT_F32)
        try:
            self._check(self.lib.marmot_linear(self.ctx, tx, tw, None, to), "marmot_linear")
            return self._read(to, (T, F), np.float16 if half_out else np.float32)
        finally:
            for t in (to, tw, tx):
                self.lib.marmot_tensor_destroy(t)

    def quantize(self, kind: int, w: np.ndarray) -> np.ndarray:
        """Row-wise weight quantisation: w [rows, K] f32 -> packed rows (uint8)."""
        w = np.ascontiguousarray(w, dtype=np.float32)
        rows, K = w.shape
        rb = row_bytes(kind, K)
        name = {KIND_Q4_K: "q4_k", KIND_Q6_K: "q6_k", KIND_Q8_0: "q8_0"}[kind]
        fn = getattr(self.lib, f"marmot_quantize_{name}")
        store_dt = DT_I8 if kind == KIND_Q8_0 else DT_U8
        out = np.empty((rows, rb), dtype=np.uint8)
        tin = self._tensor((K,), DT_F32)
        tq = self._tensor((rb,), store_dt)
        try:
            for r in range(rows):
                self._check(self.lib.marmot_tensor_copy_from_host_buffer(self.ctx, tin, _p(w[r]), K * 4), "copy_from")
                self._check(fn(self.ctx, tin, tq), f"quantize_{name}")
                self._check(self.lib.marmot_tensor_copy_to_host_buffer(self.ctx, tq, _p(out[r]), rb), "copy_to")
        finally:
            self.lib.marmot_tensor_destroy(tq)
            self.lib.marmot_tensor_destroy(tin)
        return out.reshape(-1)

    def dequantize(self, kind: int, blocks: np.ndarray, n_values: int) -> np.ndarray:
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        name = {KIND_Q4_K: "q4_k", KIND_Q6_K: "q6_k", KIND_Q8_0: "q8_0"}[kind]
        store_dt = DT_I8 if kind == KIND_Q8_0 else DT_U8
        tq = self._tensor((blocks.nbytes,), store_dt, blocks)
        to = self._tensor((n_values,), DT_F32)
        try:
            self._check(getattr(self.lib, f"marmot_dequantize_{name}")(self.ctx, tq, to), f"dequantize_{name}")
            return self._read(to, (n_values,), np.float32)
        finally:
            self.lib.marmot_tensor_destroy(to)
            self.lib.marmot_tensor_destroy(tq)

    # ---- decoder operators ----
    def rmsnorm(self, x, weight, eps: float, residual=None) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        tx, to = self._tensor(x.shape, DT_F32, x), self._tensor(x.shape, DT_F32)
        tw = self._tensor((x.shape[1],), DT_F32, np.ascontiguousarray(weight, dtype=np.float32)) if weight is not None else None
        tr = self._tensor(x.shape, DT_F32, np.ascontiguousarray(residual, dtype=np.float32)) if residual is not None else None
        try:
            desc = _RmsnormDesc(tx, tr, tw, to, eps)
            self._check(self.lib.marmot_rmsnorm(self.ctx, C.byref(desc)), "marmot_rmsnorm")
            return self._read(to, x.shape, np.float32)
        finally:
            for t in (to, tx, tw, tr):
                if t is not None:
                    self.lib.marmot_tensor_destroy(t)

    def rope(self, x, positions, theta: float = 10000.0, freq_scale: float = 1.0, neox: bool = False) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        pos = np.ascontiguousarray(positions, dtype=np.int32)
        tx, to = self._tensor(x.shape, DT_F32, x), self._tensor(x.shape, DT_F32)
        tp = self._tensor(pos.shape, DT_I32, pos)
        try:
            params = _RopeParams(tp, 1 if freq_scale != 1.0 else 0, 1 if neox else 0, theta, freq_scale, 0.0, 1.0, 32.0,
                                 1.0, 0, x.shape[1], True, True)
            self._check(self.lib.marmot_rope(self.ctx, tx, C.byref(params), to), "marmot_rope")
            return self._read(to, x.shape, np.float32)
        finally:
            for t in (tp, to, tx):
                self.lib.marmot_tensor_destroy(t)

    def swiglu(self, a, b) -> np.ndarray:
        a = np.ascontiguousarray(a, dtype=np.float32)
        b = np.ascontiguousarray(b, dtype=np.float32)
        ta, tb, to = self._tensor(a.shape, DT_F32, a), self._tensor(a.shape, DT_F32, b), self._tensor(a.shape, DT_F32)
        try:
            self._check(self.lib.marmot_swiglu(self.ctx, ta, tb, to), "marmot_swiglu")
            return self._read(to, a.shape, np.float32)
        finally:
            for t in (to, tb, ta):
                self.lib.marmot_tensor_destroy(t)

    def paged_attention(self, token_meta, q, k_new, v_new, kv_k, kv_v, block_table, layer: int, block_size: int,
                        scale: float):
        """Returns (out, kv_k, kv_v) with the pools after the call."""
        meta = np.ascontiguousarray(token_meta, dtype=np.uint32)
        table = np.ascontiguousarray(block_table, dtype=np.uint32)
        q = np.ascontiguousarray(q, dtype=np.float32)
        kv_dt = DT_F16 if kv_k.dtype == np.float16 else DT_F32
        T, hq, hd = q.shape
        tm, tt = self._tensor(meta.shape, DT_U32, meta), self._tensor(table.shape, DT_U32, table)
        tq, tk, tv = self._tensor(q.shape, DT_F32, q), self._tensor(k_new.shape, DT_F32, k_new), self._tensor(v_new.shape, DT_F32, v_new)
        pk, pv = self._tensor(kv_k.shape, kv_dt, kv_k), self._tensor(kv_v.shape, kv_dt, kv_v)
        to = self._tensor(q.shape, DT_F32)
        try:
            desc = _PagedAttentionDesc(C.sizeof(_PagedAttentionDesc), 1, 0, T, layer, hq, k_new.shape[1], hd, block_size,
                                       scale, tm, tq, tk, tv, pk, pv, tt, to, None, (C.c_uint64 * 4)())
            self._check(self.lib.marmot_paged_attention(self.ctx, C.byref(desc)), "marmot_paged_attention")
            return (self._read(to, q.shape, np.float32), self._read(pk, kv_k.shape, kv_k.dtype),
                    self._read(pv, kv_v.shape, kv_v.dtype))
        finally:
            for t in (to, pv, pk, tv, tk, tq, tt, tm):
                self.lib.marmot_tensor_destroy(t)

    def vec_dot(self, weight_kind: int, activation_kind: int, weights: np.ndarray, activations: np.ndarray,
                num_blocks: int) -> float:
        """One quantized weight row against one pre-quantized activation row (host pointers, as marmot_vec_dot takes
        them); num_blocks in the descriptor's convention."""
        w = np.ascontiguousarray(weights, dtype=np.uint8)
        a = np.ascontiguousarray(activations, dtype=np.uint8)
        desc = _VecDotDesc(w.ctypes.data, a.ctypes.data, num_blocks, weight_kind, activation_kind, 1)
        out = C.c_float()
        self._check(self.lib.marmot_vec_dot(self.ctx, C.byref(desc), C.byref(out)), "marmot_vec_dot")
        return float(out.value)

    def linear_resident(self, kind: int, W: np.ndarray, F: int, K: int, T: int = 1):
        """A weight made resident once and reusable input / output tensors, for repeated calls (what a model holds):
        returns run(x) -> np.ndarray [T, F], each call going through marmot_linear with host activations in and the
        result copied to host memory."""
        tw = self._qtensor((F, K), kind, W)
        self._check(self.lib.marmot_tensor_to_device(self.ctx, tw), "marmot_tensor_to_device")
        tx, to = self._tensor((T, K), DT_F32), self._tensor((T, F), DT_F32)
        out = np.empty((T, F), dtype=np.float32)
        keep = (tw, tx, to)

        out_p, out_bytes = _p(out), out.nbytes
        lib, ctx, check = self.lib, self.ctx, self._check
        in_bytes = T * K * 4

        def run(x: np.ndarray) -> np.ndarray:
            # x: C-contiguous float32 [T, K]; its address is taken without building a ctypes view of the array (that
            # alone costs several microseconds per call, as much as the upload)
            assert x.nbytes == in_bytes and x.dtype == np.float32 and x.flags.c_contiguous
            check(lib.marmot_tensor_copy_from_host_buffer(ctx, tx, C.c_void_p(x.__array_interface__["data"][0]), in_bytes), "copy_from")
            check(lib.marmot_linear(ctx, tx, tw, None, to), "marmot_linear")
            check(lib.marmot_tensor_copy_to_host_buffer(ctx, to, out_p, out_bytes), "copy_to")
            return out

        run.tensors = keep
        return run

    def topk(self, x: np.ndarray, k: int):
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, cols = x.shape
        tx = self._tensor((rows, cols), DT_F32, x)
        tv, ti = self._tensor((rows, k), DT_F32), self._tensor((rows, k), DT_I32)
        try:
            desc = _TopkDesc(tx, tv, ti, -1, k)
            self._check(self.lib.marmot_topk(self.ctx, C.byref(desc)), "marmot_topk")
            return self._read(tv, (rows, k), np.float32), self._read(ti, (rows, k), np.int32)
        finally:
            for t in (ti, tv, tx):
                self.lib.marmot_tensor_destroy(t)

    def _expert_tensor(self, kind: int, blocks: np.ndarray, rows: int, cols: int, experts: int):
        """3-D expert weight in GGUF ne order {cols, rows, experts}, as tests/backend/test_backend_moe.c:77-124."""
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        store_dt = DT_I8 if kind == KIND_Q8_0 else DT_U8
        t = self._tensor((blocks.nbytes,), store_dt, blocks)
        s = t.contents
        s.shape.ndim = 3
        s.shape.shape[0], s.shape.shape[1], s.shape.shape[2] = cols, rows, experts
        s.shape.strides[2], s.shape.strides[1], s.shape.strides[0] = 1, experts, rows * experts
        s.quant_kind = kind
        s.quant_layout = 1  # MARMOT_QUANT_LAYOUT_GGUF
        return t

    def moe_experts(self, kinds, hidden, gate, up, down, topk_ids, topk_weights, FF: int, E: int,
                    ffn_type: int = FFN_SWIGLU, weights_scale: float = 1.0,
                    policy: int = POLICY_RENORMALIZE_SELECTED) -> np.ndarray:
        hidden = np.ascontiguousarray(hidden, dtype=np.float32)
        ids = np.ascontiguousarray(topk_ids, dtype=np.int32)
        wts = np.ascontiguousarray(topk_weights, dtype=np.float32)
        T, H = hidden.shape
        k = ids.shape[1]
        th = self._tensor((T, H), DT_F32, hidden)
        tg = self._expert_tensor(kinds[0], gate, FF, H, E)
        tu = self._expert_tensor(kinds[1], up, FF, H, E)
        td = self._expert_tensor(kinds[2], down, H, FF, E)
        ti = self._tensor((T, k), DT_I32, ids)
        tw = self._tensor((T, k), DT_F32, wts)
        to = self._tensor((T, H), DT_F32)
        desc = _MoeDesc(th, tg, tu, td, ti, tw, to, ffn_type, weights_scale, policy)
        try:
            self._check(self.lib.marmot_moe_experts(self.ctx, C.byref(desc)), "marmot_moe_experts")
            return self._read(to, (T, H), np.float32)
        finally:
            for t in (to, tw, ti, td, tu, tg, th):
                self.lib.marmot_tensor_destroy(t)
