"""ctypes bindings for the two CPU checkers.  TEST INFRASTRUCTURE ONLY.

* ``Oracle``     -> oracle/libmarmot_oracle.so, the plain-C restatement.
* ``Reference``  -> oracle/_ref/libmarmot_ref.so, the reference's own CPU
  backend compiled from its sources (marmot_init(CPU) -> marmot_linear /
  marmot_moe_experts / marmot_quantize_* / marmot_dequantize_*).

Only tests, the smoke check and the CPU-baseline legs of the benchmark import
this module; nothing under marmot_b200/ does.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ORACLE_LIB = HERE / "libmarmot_oracle.so"
REF_LIB = HERE / "_ref" / "libmarmot_ref.so"

KIND_Q8_0, KIND_Q4_K, KIND_Q6_K = 5, 9, 11
KIND_BY_NAME = {"q8_0": KIND_Q8_0, "q4_k": KIND_Q4_K, "q6_k": KIND_Q6_K}
BLOCK_VALUES = {KIND_Q8_0: 32, KIND_Q4_K: 256, KIND_Q6_K: 256}
BLOCK_BYTES = {KIND_Q8_0: 34, KIND_Q4_K: 144, KIND_Q6_K: 210}
POLICY_SOFTMAX_SELECTED, POLICY_RENORMALIZE_SELECTED = 0, 2
FFN_SWIGLU, FFN_GEGLU = 0, 2


def row_bytes(kind: int, K: int) -> int:
    bv = BLOCK_VALUES[kind]
    return (K + bv - 1) // bv * BLOCK_BYTES[kind]


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class Oracle:
    def __init__(self, path: Path = ORACLE_LIB):
        if not path.exists():
            raise FileNotFoundError(f"{path} missing: run oracle/build_oracle.py")
        self.lib = L = C.CDLL(str(path))
        L.mo_dequantize.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
        L.mo_pack_q8_k_f32.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
        L.mo_pack_q8_0_f32.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
        for n in ("mo_vec_dot_q4_k_q8_k", "mo_vec_dot_q6_k_q8_k", "mo_vec_dot_q8_0_q8_0"):
            f = getattr(L, n)
            f.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
            f.restype = C.c_float
        L.mo_linear.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
        L.mo_linear_f16.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                    C.c_void_p, C.c_void_p, C.c_size_t]
        L.mo_topk.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p]
        L.mo_moe_experts.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                     C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.c_size_t, C.c_int, C.c_float, C.c_int, C.c_void_p, C.c_int]
        vp, sz, f32 = C.c_void_p, C.c_size_t, C.c_float
        L.mo_rmsnorm_f32.argtypes = [vp, vp, vp, sz, sz, f32, f32, vp]
        L.mo_rope_f32.argtypes = [vp, vp, sz, sz, f32, f32, C.c_int, vp]
        L.mo_swiglu_f32.argtypes = [vp, vp, sz, vp]
        L.mo_paged_attention_f32.argtypes = [vp, sz, vp, vp, vp, vp, vp, C.c_int, C.c_int, vp, sz, sz, sz, sz, sz, sz, sz, f32, vp]
        L.mo_embedding_gather.argtypes = [C.c_int, vp, sz, vp, sz, vp]
        L.mo_argmax_f32.argtypes = [vp, sz, sz, vp]

    def dequantize(self, kind: int, blocks: np.ndarray, n_values: int) -> np.ndarray:
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        out = np.empty(n_values, dtype=np.float32)
        assert self.lib.mo_dequantize(kind, _p(blocks), n_values, _p(out)) == 0
        return out

    def pack_q8_k(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.zeros(((x.size + 255) // 256) * 292, dtype=np.uint8)
        self.lib.mo_pack_q8_k_f32(_p(x), x.size, _p(out))
        return out

    def pack_q8_0(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.zeros(((x.size + 31) // 32) * 34, dtype=np.uint8)
        self.lib.mo_pack_q8_0_f32(_p(x), x.size, _p(out))
        return out

    def vec_dot(self, kind: int, w: np.ndarray, a: np.ndarray, n_blocks: int) -> float:
        fn = {KIND_Q4_K: self.lib.mo_vec_dot_q4_k_q8_k, KIND_Q6_K: self.lib.mo_vec_dot_q6_k_q8_k,
              KIND_Q8_0: self.lib.mo_vec_dot_q8_0_q8_0}[kind]
        w = np.ascontiguousarray(w, dtype=np.uint8)
        a = np.ascontiguousarray(a, dtype=np.uint8)
        return float(fn(_p(w), _p(a), n_blocks))

    def linear(self, kind: int, x: np.ndarray, W: np.ndarray, F: int, bias: np.ndarray | None = None,
               threads: int | None = None) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        W = np.ascontiguousarray(W, dtype=np.uint8)
        T, K = x.shape
        assert W.size == F * row_bytes(kind, K), (W.size, F, K)
        out = np.empty((T, F), dtype=np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        rc = self.lib.mo_linear(kind, _p(x), K, _p(W), T, K, F, None if b is None else _p(b), _p(out), F,
                                threads or os.cpu_count() or 1)
        assert rc == 0
        return out

    def linear_f16(self, kind: int, x16: np.ndarray, W: np.ndarray, F: int, bias: np.ndarray | None = None) -> np.ndarray:
        """x16 [T, K] float16 (or its uint16 bits): the reference's f16-activation matmul, f32 out."""
        x16 = np.ascontiguousarray(x16).view(np.uint16)
        T, K = x16.shape
        W = np.ascontiguousarray(W, dtype=np.uint8)
        out = np.empty((T, F), dtype=np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        rc = self.lib.mo_linear_f16(kind, _p(x16), K, _p(W), T, K, F, None if b is None else _p(b), _p(out), F)
        assert rc == 0
        return out

    def topk(self, x: np.ndarray, k: int):
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, cols = x.shape
        vals = np.empty((rows, k), dtype=np.float32)
        idx = np.empty((rows, k), dtype=np.int32)
        self.lib.mo_topk(_p(x), rows, cols, cols, k, _p(vals), _p(idx))
        return vals, idx

    def moe_experts(self, kinds, hidden, gate, up, down, topk_ids, topk_weights, FF: int, E: int,
                    ffn_type: int = FFN_SWIGLU, weights_scale: float = 1.0,
                    policy: int = POLICY_RENORMALIZE_SELECTED, threads: int | None = None) -> np.ndarray:
        hidden = np.ascontiguousarray(hidden, dtype=np.float32)
        ids = np.ascontiguousarray(topk_ids, dtype=np.int32)
        wts = np.ascontiguousarray(topk_weights, dtype=np.float32)
        T, H = hidden.shape
        k = ids.shape[1]
        out = np.empty((T, H), dtype=np.float32)
        gate, up, down = (np.ascontiguousarray(a, dtype=np.uint8) for a in (gate, up, down))
        rc = self.lib.mo_moe_experts(kinds[0], kinds[1], kinds[2], _p(hidden), T, H, FF, E, _p(gate), _p(up), _p(down),
                                     _p(ids), _p(wts), k, ffn_type, weights_scale, policy, _p(out),
                                     threads or os.cpu_count() or 1)
        assert rc == 0, rc
        return out


    # ---- decoder operators (marmot_oracle_decoder.c) ----
    def rmsnorm(self, x, weight, eps: float, residual=None, weight_offset: float = 0.0) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, n = x.shape
        out = np.empty_like(x)
        res = None if residual is None else np.ascontiguousarray(residual, dtype=np.float32)
        w = None if weight is None else np.ascontiguousarray(weight, dtype=np.float32)
        self.lib.mo_rmsnorm_f32(_p(x), _p(res) if res is not None else None, _p(w) if w is not None else None, rows, n,
                                C.c_float(eps), C.c_float(weight_offset), _p(out))
        return out

    def rope(self, x, positions, theta: float = 10000.0, freq_scale: float = 1.0, neox: bool = False) -> np.ndarray:
        """x [rows, dim], one position per row."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        pos = np.ascontiguousarray(positions, dtype=np.int32)
        out = np.empty_like(x)
        self.lib.mo_rope_f32(_p(x), _p(pos), x.shape[0], x.shape[1], C.c_float(theta), C.c_float(freq_scale),
                             1 if neox else 0, _p(out))
        return out

    def swiglu(self, a, b) -> np.ndarray:
        a = np.ascontiguousarray(a, dtype=np.float32)
        b = np.ascontiguousarray(b, dtype=np.float32)
        out = np.empty_like(a)
        self.lib.mo_swiglu_f32(_p(a), _p(b), a.size, _p(out))
        return out

    def paged_attention(self, token_meta, q, k_new, v_new, kv_k, kv_v, block_table, layer: int, block_size: int,
                        scale: float, kv_truncate: bool = False) -> np.ndarray:
        """q [T, Hq, hd], k_new/v_new [T, Hkv, hd], pool [blocks, layers, Hkv, block_size, hd] f32 or f16 (updated in
        place), token_meta [T, 4] u32, block_table [seqs, max_blocks] u32.  kv_truncate: write an f16 pool with the
        truncating conversion of the reference's scalar build instead of round-to-nearest-even."""
        meta = np.ascontiguousarray(token_meta, dtype=np.uint32)
        q = np.ascontiguousarray(q, dtype=np.float32)
        k_new = np.ascontiguousarray(k_new, dtype=np.float32)
        v_new = np.ascontiguousarray(v_new, dtype=np.float32)
        table = np.ascontiguousarray(block_table, dtype=np.uint32)
        assert kv_k.flags.c_contiguous and kv_v.flags.c_contiguous and kv_k.dtype in (np.float32, np.float16)
        T, hq, hd = q.shape
        out = np.empty_like(q)
        rc = self.lib.mo_paged_attention_f32(
            _p(meta), T, _p(q), _p(k_new), _p(v_new), _p(kv_k), _p(kv_v), 1 if kv_k.dtype == np.float16 else 0,
            1 if kv_truncate else 0, _p(table), table.shape[1], kv_k.shape[1], layer, hq, k_new.shape[1], hd, block_size, C.c_float(scale), _p(out))
        assert rc == 0, rc
        return out

    def embedding_gather(self, kind: int, table: np.ndarray, dim: int, ids) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        table = np.ascontiguousarray(table, dtype=np.uint8)
        out = np.empty((len(ids), dim), dtype=np.float32)
        assert self.lib.mo_embedding_gather(kind, _p(table), dim, _p(ids), len(ids), _p(out)) == 0
        return out

    def argmax(self, x) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(x.shape[0], dtype=np.int32)
        self.lib.mo_argmax_f32(_p(x), x.shape[0], x.shape[1], _p(out))
        return out


# ---------------------------------------------------------------------------
# The reference library itself: marmot's public C API (bound once, in the package) over the CPU backend of the
# library built from the reference checkout
# ---------------------------------------------------------------------------
import sys as _sys

if str(HERE.parent) not in _sys.path:
    _sys.path.insert(0, str(HERE.parent))

from marmot_b200.marmot_api import (DT_F16, DT_F32, DT_I8, DT_I32, DT_U8, DT_U32, MarmotLibrary,  # noqa: E402,F401
                                    _MoeDesc, _PagedAttentionDesc, _RmsnormDesc, _RopeParams, _Tensor, _TopkDesc)


class Reference(MarmotLibrary):
    """The reference CPU backend, driven through its public C API."""

    def __init__(self, path: Path = REF_LIB, threads: int | None = None):
        if not Path(path).exists():
            raise FileNotFoundError(f"{path} missing: run oracle/build_ref.py on a machine with the reference tree")
        super().__init__(path, backend=0, threads=threads)
