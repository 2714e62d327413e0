"""ctypes binding of libmarmot_cuda.so.  Plumbing only: device buffers are torch tensors, every
operation is one call through the C ABI declared in include/marmot_cuda.h."""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libmarmot_cuda.so"

KIND_Q8_0, KIND_Q4_K, KIND_Q6_K = 5, 9, 11
KIND_BY_NAME = {"q8_0": KIND_Q8_0, "q4_k": KIND_Q4_K, "q6_k": KIND_Q6_K}
BLOCK_VALUES = {KIND_Q8_0: 32, KIND_Q4_K: 256, KIND_Q6_K: 256}
BLOCK_BYTES = {KIND_Q8_0: 34, KIND_Q4_K: 144, KIND_Q6_K: 210}
REGIME_AUTO, REGIME_GEMV, REGIME_GEMM, REGIME_GEMV_PLAIN, REGIME_I8MMA = 0, 1, 2, 3, 4
ROUTER_SOFTMAX_SELECTED, ROUTER_RENORMALIZE_SELECTED = 0, 2
FFN_SWIGLU, FFN_GEGLU = 0, 2

# Every symbol include/marmot_cuda.h declares.
EXPORTS = (
    "mcu_context_create", "mcu_context_destroy", "mcu_context_set_stream", "mcu_context_get_stream",
    "mcu_context_set_regime", "mcu_synchronize", "mcu_last_error_message", "mcu_kernel_launch_count",
    "mcu_malloc", "mcu_free", "mcu_memcpy_to_device", "mcu_memcpy_to_host", "mcu_row_bytes", "mcu_dequantize",
    "mcu_quantize_activations", "mcu_linear", "mcu_linear_dual", "mcu_linear_multi", "mcu_linear_f16", "mcu_linear_host", "mcu_topk", "mcu_moe_experts",
    "mcu_linear_static_scratch", "mcu_moe_experts_local", "mcu_moe_experts_ep", "mcu_peer_moe_combine", "mcu_peer_comm_capacity", "mcu_peer_comm_rank", "mcu_peer_comm_world", "mcu_moe_last_buffers", "mcu_peer_comm_create", "mcu_peer_comm_export",
    "mcu_peer_comm_connect", "mcu_peer_comm_staging", "mcu_peer_allreduce", "mcu_peer_comm_destroy",
    "mcu_linear_allreduce", "mcu_peer_comm_set_fused", "mcu_peer_comm_set_one_slot", "mcu_rmsnorm", "mcu_rope", "mcu_swiglu", "mcu_add", "mcu_argmax",
    "mcu_embedding_gather", "mcu_paged_attention", "mcu_paged_attention_decode", "mcu_rope_table", "mcu_decode_plan_create", "mcu_decode_plan_run",
    "mcu_decode_plan_destroy", "mcu_decode_plan_phase_times", "mcu_add_rmsnorm", "mcu_rope_qk", "mcu_device_caps", "mcu_vec_dot_host",
    "mcu_kv_pool_options_init", "mcu_kv_pool_create", "mcu_kv_pool_destroy", "mcu_kv_pool_acquire_seq",
    "mcu_kv_pool_release_seq", "mcu_kv_pool_prepare_append", "mcu_kv_pool_commit_append", "mcu_kv_pool_abort_append",
    "mcu_kv_pool_prepare_prefix_attach", "mcu_kv_pool_commit_prefix_attach", "mcu_kv_pool_abort_prefix_attach",
    "mcu_kv_pool_get_pointers", "mcu_kv_pool_free_block_count", "mcu_kv_pool_total_block_count", "mcu_kv_pool_seq_len",
    "mcu_kv_pool_block_id", "mcu_kv_pool_block_generation", "mcu_kv_pool_set_block_retained", "mcu_kv_pool_swap_out_seq",
    "mcu_kv_pool_swap_in_seq", "mcu_kv_pool_is_seq_swapped",
    "mcu_graph_capture_begin", "mcu_graph_capture_end", "mcu_graph_launch", "mcu_graph_destroy",
    "mcu_gguf_open", "mcu_gguf_close", "mcu_gguf_tensor_count", "mcu_gguf_find_tensor", "mcu_gguf_tensor_info",
    "mcu_gguf_meta_u64", "mcu_gguf_meta_f64", "mcu_gguf_meta_str", "mcu_gguf_upload",
)


PROLOGUE_NONE, PROLOGUE_ADD_RMSNORM, PROLOGUE_SWIGLU = 0, 1, 2


class LinearJob(C.Structure):
    """mcu_linear_job_t"""
    _fields_ = [("kind", C.c_int), ("w_dev", C.c_void_p), ("F", C.c_size_t), ("bias_dev", C.c_void_p),
                ("out_dev", C.c_void_p), ("ldo", C.c_size_t)]


class Prologue(C.Structure):
    """mcu_prologue_t"""
    _fields_ = [("op", C.c_int), ("aux_dev", C.c_void_p), ("ld_aux", C.c_size_t), ("norm_weight_dev", C.c_void_p),
                ("eps", C.c_float), ("weight_offset", C.c_float), ("x_out_dev", C.c_void_p), ("ld_x_out", C.c_size_t)]


class DecodeLayer(C.Structure):
    """mcu_decode_layer_t"""
    _fields_ = [(n, C.c_int) for n in ("kind_q", "kind_k", "kind_v", "kind_o", "kind_gate", "kind_up", "kind_down")] + \
               [(n, C.c_void_p) for n in ("wq", "wk", "wv", "wo", "gate", "up", "down", "attn_norm", "ffn_norm")]


class DecodePlanDesc(C.Structure):
    """mcu_decode_plan_desc_t"""
    _fields_ = [(n, C.c_size_t) for n in ("n_layers", "d", "ffn", "n_q_heads", "n_kv_heads", "head_dim", "vocab")] + \
               [("rms_eps", C.c_float), ("attn_scale", C.c_float), ("rope_type", C.c_int), ("layers", C.POINTER(DecodeLayer)),
                ("out_norm", C.c_void_p), ("kind_output", C.c_int), ("output", C.c_void_p)] + \
               [(n, C.c_void_p) for n in ("x0", "x1", "q", "k", "v", "att", "proj", "gate", "up", "logits", "token_meta",
                                          "block_table")] + \
               [("max_blocks_per_seq", C.c_size_t), ("kv_k", C.c_void_p), ("kv_v", C.c_void_p), ("kv_dtype", C.c_int),
                ("block_size", C.c_size_t), ("rope_table", C.c_void_p)]


class DecodePlan:
    """mcu_decode_plan: one decode step of one token as a single persistent kernel; every pointer is fixed at creation
    (the tensors named in the description must stay alive and in place)."""

    def __init__(self, ctx: "Context", desc: DecodePlanDesc, keep):
        self.ctx, self._keep = ctx, keep
        h = C.c_void_p()
        ctx._check(ctx.lib.mcu_decode_plan_create(ctx.handle, C.byref(desc), C.byref(h)))
        self.handle = h

    def run(self):
        self.ctx._check(self.ctx.lib.mcu_decode_plan_run(self.handle))

    def phase_times(self):
        """Nanosecond stamps of the last run: the start of every phase, then the end."""
        n = C.c_size_t()
        self.ctx._check(self.ctx.lib.mcu_decode_plan_phase_times(self.handle, None, 0, C.byref(n)))
        buf = (C.c_ulonglong * n.value)()
        self.ctx._check(self.ctx.lib.mcu_decode_plan_phase_times(self.handle, buf, n.value, C.byref(n)))
        return list(buf)

    def close(self):
        if self.handle:
            self.ctx.lib.mcu_decode_plan_destroy(self.handle)
            self.handle = None


class MarmotCudaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"marmot_cuda error {code}: {message}")
        self.code = code


def row_bytes(kind: int, K: int) -> int:
    bv = BLOCK_VALUES[kind]
    return (K + bv - 1) // bv * BLOCK_BYTES[kind]


_lib = None


def load_library() -> C.CDLL:
    """Load libmarmot_cuda.so; there is no fallback if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = Path(os.environ.get("MARMOT_CUDA_LIB") or LIB_PATH)  # another build of the library, for A/B measurements
    if not path.exists():
        raise FileNotFoundError(
            f"{path} is missing: build it with `python -m marmot_b200.build` (needs nvcc); "
            "marmot_b200 has no CPU or PyTorch fallback"
        )
    L = C.CDLL(str(path))
    vp, sz, i32, f32 = C.c_void_p, C.c_size_t, C.c_int, C.c_float
    L.mcu_context_create.argtypes = [i32, C.POINTER(vp)]
    L.mcu_context_destroy.argtypes = [vp]
    L.mcu_context_destroy.restype = None
    L.mcu_context_set_stream.argtypes = [vp, vp]
    L.mcu_context_get_stream.argtypes = [vp]
    L.mcu_context_get_stream.restype = vp
    L.mcu_context_set_regime.argtypes = [vp, i32]
    L.mcu_synchronize.argtypes = [vp]
    L.mcu_last_error_message.restype = C.c_char_p
    L.mcu_kernel_launch_count.argtypes = [vp]
    L.mcu_kernel_launch_count.restype = C.c_uint64
    L.mcu_malloc.argtypes = [vp, sz, C.POINTER(vp)]
    L.mcu_free.argtypes = [vp, vp]
    L.mcu_memcpy_to_device.argtypes = [vp, vp, vp, sz]
    L.mcu_memcpy_to_host.argtypes = [vp, vp, vp, sz]
    L.mcu_row_bytes.argtypes = [i32, sz]
    L.mcu_row_bytes.restype = sz
    L.mcu_dequantize.argtypes = [vp, i32, vp, sz, vp]
    L.mcu_quantize_activations.argtypes = [vp, i32, vp, sz, sz, sz, vp, vp, vp]
    L.mcu_linear.argtypes = [vp, i32, vp, sz, vp, sz, sz, sz, vp, vp, sz]
    L.mcu_linear_dual.argtypes = [vp, i32, vp, sz, vp, vp, sz, sz, sz, vp, vp, sz]
    L.mcu_linear_host.argtypes = [vp, i32, vp, sz, vp, sz, sz, sz, vp, vp, sz]
    L.mcu_linear_multi.argtypes = [vp, vp, sz, sz, sz, vp, vp, sz]
    L.mcu_linear_f16.argtypes = [vp, i32, vp, sz, vp, sz, sz, sz, vp, vp, sz, i32]
    L.mcu_linear_static_scratch.argtypes = [vp, i32, vp, sz, vp, sz, sz, sz, vp, vp, sz]
    L.mcu_topk.argtypes = [vp, vp, sz, sz, sz, sz, vp, vp]
    L.mcu_vec_dot_host.argtypes = [vp, i32, vp, vp, sz, vp]
    L.mcu_moe_experts.argtypes = [vp, i32, i32, i32, vp, sz, sz, sz, sz, vp, vp, vp, vp, vp, sz, i32, f32, i32, vp]
    L.mcu_moe_experts_local.argtypes = [vp, i32, i32, i32, vp, sz, sz, sz, sz, sz, sz, vp, vp, vp, vp, vp, sz, i32, f32,
                                        i32, vp]
    L.mcu_moe_last_buffers.argtypes = [vp, vp]
    L.mcu_moe_experts_ep.argtypes = [vp, vp, i32, i32, i32, vp, sz, sz, sz, sz, vp, vp, vp, vp, vp, vp, sz, i32, f32, i32, vp]
    L.mcu_peer_comm_capacity.argtypes = [vp]
    L.mcu_peer_comm_capacity.restype = sz
    L.mcu_peer_comm_create.argtypes = [vp, i32, i32, sz, C.POINTER(vp)]
    L.mcu_peer_comm_export.argtypes = [vp, vp]
    L.mcu_peer_comm_connect.argtypes = [vp, vp]
    L.mcu_peer_comm_staging.argtypes = [vp]
    L.mcu_peer_comm_staging.restype = vp
    L.mcu_peer_allreduce.argtypes = [vp, sz, vp]
    L.mcu_peer_comm_destroy.argtypes = [vp]
    L.mcu_peer_comm_destroy.restype = None
    L.mcu_linear_allreduce.argtypes = [vp, vp, i32, vp, sz, vp, sz, sz, sz, vp]
    L.mcu_peer_comm_set_fused.argtypes = [vp, i32]
    L.mcu_peer_comm_set_one_slot.argtypes = [vp, i32]
    L.mcu_rmsnorm.argtypes = [vp, vp, vp, vp, sz, sz, f32, f32, vp]
    L.mcu_rope.argtypes = [vp, vp, sz, vp, sz, sz, sz, f32, f32, i32, vp, sz]
    L.mcu_swiglu.argtypes = [vp, vp, vp, sz, vp]
    L.mcu_add_rmsnorm.argtypes = [vp, vp, vp, vp, sz, sz, f32, f32, vp, vp]
    L.mcu_rope_qk.argtypes = [vp, vp, sz, sz, vp, sz, sz, vp, sz, sz, f32, f32, i32]
    L.mcu_add.argtypes = [vp, vp, vp, sz, vp]
    L.mcu_argmax.argtypes = [vp, vp, sz, sz, vp]
    L.mcu_embedding_gather.argtypes = [vp, i32, vp, sz, vp, sz, vp]
    L.mcu_paged_attention.argtypes = [vp, vp, sz, vp, vp, vp, vp, vp, i32, vp, sz, sz, sz, sz, sz, sz, sz, f32, vp]
    L.mcu_paged_attention_decode.argtypes = [vp, vp, sz, vp, vp, vp, vp, vp, i32, vp, sz, sz, sz, sz, sz, sz, sz, f32, vp, f32,
                                             f32, i32, vp, vp]
    L.mcu_rope_table.argtypes = [vp, vp, sz, sz, f32, f32, vp]
    L.mcu_decode_plan_create.argtypes = [vp, vp, C.POINTER(vp)]
    L.mcu_decode_plan_run.argtypes = [vp]
    L.mcu_decode_plan_destroy.argtypes = [vp]
    L.mcu_decode_plan_phase_times.argtypes = [vp, vp, sz, vp]
    L.mcu_decode_plan_destroy.restype = None
    _lib = L
    return L


def _ptr(t) -> int:
    return 0 if t is None else int(t.data_ptr())


class Context:
    """One mcu_context_t on one device.  Tensors passed in must live on that device."""

    def __init__(self, device: int = 0, use_torch_stream: bool = True):
        import torch

        self.torch = torch
        self.lib = load_library()
        self.device = device
        h = C.c_void_p()
        self._check(self.lib.mcu_context_create(device, C.byref(h)))
        self.handle = h
        if use_torch_stream:
            with torch.cuda.device(device):
                # torch reports the legacy default stream as handle 0, which this ABI reads as
                # "use the context's own stream"; cudaStreamLegacy (0x1) names it explicitly.
                stream = torch.cuda.current_stream().cuda_stream or 1
            self._check(self.lib.mcu_context_set_stream(self.handle, C.c_void_p(stream)))

    def close(self):
        if getattr(self, "handle", None):
            self.lib.mcu_context_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc != 0:
            raise MarmotCudaError(rc, self.lib.mcu_last_error_message().decode())

    # -- helpers -----------------------------------------------------------
    def upload(self, host: np.ndarray):
        """Host bytes -> device tensor (uint8), the one-time residency step for weights."""
        t = self.torch.from_numpy(np.ascontiguousarray(host).view(np.uint8).reshape(-1))
        return t.to(f"cuda:{self.device}")

    def set_stream(self, cuda_stream: int):
        """Run on the given cudaStream_t handle (0 is mapped to cudaStreamLegacy)."""
        self._check(self.lib.mcu_context_set_stream(self.handle, C.c_void_p(cuda_stream or 1)))

    def set_regime(self, regime: int):
        self._check(self.lib.mcu_context_set_regime(self.handle, regime))

    def synchronize(self):
        self._check(self.lib.mcu_synchronize(self.handle))

    def launch_count(self) -> int:
        return int(self.lib.mcu_kernel_launch_count(self.handle))

    # -- operations ----------------------------------------------------------
    def dequantize(self, kind: int, blocks, n_values: int):
        out = self.torch.empty(n_values, dtype=self.torch.float32, device=blocks.device)
        self._check(self.lib.mcu_dequantize(self.handle, kind, _ptr(blocks), n_values, _ptr(out)))
        return out

    def quantize_activations(self, weight_kind: int, x):
        T, K = x.shape
        bv = BLOCK_VALUES[weight_kind]
        nb = (K + bv - 1) // bv
        tc = self.torch
        qs = tc.empty((T, nb * bv), dtype=tc.int8, device=x.device)
        d = tc.empty((T, nb), dtype=tc.float32, device=x.device)
        bs = tc.empty((T, nb * 16), dtype=tc.int16, device=x.device) if weight_kind != KIND_Q8_0 else None
        self._check(self.lib.mcu_quantize_activations(self.handle, weight_kind, _ptr(x), x.stride(0), T, K, _ptr(qs),
                                                      _ptr(d), _ptr(bs)))
        return qs, d, bs

    def linear(self, kind: int, x, w, F: int, bias=None, out=None):
        T, K = x.shape
        assert x.stride(1) == 1 and w.numel() * w.element_size() >= F * row_bytes(kind, K)
        if out is None:
            out = self.torch.empty((T, F), dtype=self.torch.float32, device=x.device)
        self._check(self.lib.mcu_linear(self.handle, kind, _ptr(x), x.stride(0), _ptr(w), T, K, F, _ptr(bias), _ptr(out),
                                        out.stride(0)))
        return out

    def linear_dual(self, kind: int, x, w_a, w_b, F: int, out_a=None, out_b=None):
        T, K = x.shape
        tc = self.torch
        oa = out_a if out_a is not None else tc.empty((T, F), dtype=tc.float32, device=x.device)
        ob = out_b if out_b is not None else tc.empty((T, F), dtype=tc.float32, device=x.device)
        self._check(self.lib.mcu_linear_dual(self.handle, kind, _ptr(x), x.stride(0), _ptr(w_a), _ptr(w_b), T, K, F,
                                             _ptr(oa), _ptr(ob), F))
        return oa, ob

    def linear_f16(self, kind: int, x16, w, F: int, bias=None, out_dtype=None):
        """float16 activations [T, K] (no packing, f32 arithmetic on weight values formed as the reference's f16 row
        dots form them); float32 out unless out_dtype is torch.float16."""
        T, K = x16.shape
        tc = self.torch
        assert x16.dtype == tc.float16
        half_out = out_dtype == tc.float16
        out = tc.empty((T, F), dtype=tc.float16 if half_out else tc.float32, device=x16.device)
        self._check(self.lib.mcu_linear_f16(self.handle, kind, _ptr(x16), x16.stride(0), _ptr(w), T, K, F,
                                            _ptr(bias) if bias is not None else None, _ptr(out), F, 1 if half_out else 0))
        return out

    def linear_multi(self, x, jobs, prologue=None):
        """Several weights over one activation read: jobs = [(kind, w, F, out), ...] (1..4, out [T, F] or wider rows),
        prologue = None, ("add_rmsnorm", aux or None, norm_weight or None, eps, weight_offset, x_out or None) or
        ("swiglu", up).  One launch for up to eight tokens on the streaming path."""
        T, K = x.shape
        arr = (LinearJob * len(jobs))()
        for slot, (kind, w, F, out) in zip(arr, jobs):
            slot.kind, slot.w_dev, slot.F, slot.bias_dev, slot.out_dev, slot.ldo = kind, _ptr(w), F, None, _ptr(out), out.stride(0)
        pro = None
        if prologue is not None:
            pro = Prologue()
            if prologue[0] == "add_rmsnorm":
                _, aux, weight, eps, w_off, x_out = prologue
                pro.op = PROLOGUE_ADD_RMSNORM
                pro.aux_dev, pro.ld_aux = (_ptr(aux), aux.stride(0)) if aux is not None else (None, 0)
                pro.norm_weight_dev = _ptr(weight) if weight is not None else None
                pro.eps, pro.weight_offset = eps, w_off
                pro.x_out_dev, pro.ld_x_out = (_ptr(x_out), x_out.stride(0)) if x_out is not None else (None, 0)
            elif prologue[0] == "swiglu":
                pro.op = PROLOGUE_SWIGLU
                pro.aux_dev, pro.ld_aux = _ptr(prologue[1]), prologue[1].stride(0)
            else:
                raise ValueError(f"unknown prologue {prologue[0]!r}")
        self._check(self.lib.mcu_linear_multi(self.handle, _ptr(x), x.stride(0), T, K,
                                              C.byref(pro) if pro is not None else None, arr, len(jobs)))

    def linear_host(self, kind: int, x_host: np.ndarray, w, F: int, bias_host: np.ndarray | None = None,
                    out_host: np.ndarray | None = None) -> np.ndarray:
        """Host activations in, host result out; weights device resident."""
        T, K = x_host.shape
        if out_host is None:
            out_host = np.empty((T, F), dtype=np.float32)
        bp = None if bias_host is None else bias_host.ctypes.data
        self._check(self.lib.mcu_linear_host(self.handle, kind, x_host.ctypes.data, x_host.strides[0] // 4, _ptr(w), T, K,
                                             F, bp, out_host.ctypes.data, out_host.strides[0] // 4))
        return out_host

    def graph_capture_begin(self) -> None:
        """Start recording the calls made on this context (they are not run); see graph_capture_end."""
        self.lib.mcu_graph_capture_begin.argtypes = [C.c_void_p]
        self._check(self.lib.mcu_graph_capture_begin(self.handle))

    def graph_capture_end(self) -> "Graph":
        self.lib.mcu_graph_capture_end.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
        h = C.c_void_p()
        self._check(self.lib.mcu_graph_capture_end(self.handle, C.byref(h)))
        return Graph(self, h)

    def vec_dot_host(self, kind: int, weights: np.ndarray, activations: np.ndarray, num_blocks: int) -> float:
        """One weight row times one pre-quantized activation row (reference block structs as uint8 arrays)."""
        w = np.ascontiguousarray(weights, dtype=np.uint8)
        a = np.ascontiguousarray(activations, dtype=np.uint8)
        out = C.c_float(0.0)
        self._check(self.lib.mcu_vec_dot_host(self.handle, kind, w.ctypes.data, a.ctypes.data, num_blocks, C.byref(out)))
        return float(out.value)

    def topk(self, x, k: int):
        rows, cols = x.shape
        tc = self.torch
        vals = tc.empty((rows, k), dtype=tc.float32, device=x.device)
        idx = tc.empty((rows, k), dtype=tc.int32, device=x.device)
        self._check(self.lib.mcu_topk(self.handle, _ptr(x), rows, cols, x.stride(0), k, _ptr(vals), _ptr(idx)))
        return vals, idx

    def moe_experts(self, kinds, hidden, gate, up, down, topk_ids, topk_weights, FF: int, E: int,
                    ffn_type: int = FFN_SWIGLU, weights_scale: float = 1.0, policy: int = ROUTER_RENORMALIZE_SELECTED):
        T, H = hidden.shape
        k = topk_ids.shape[1]
        out = self.torch.empty((T, H), dtype=self.torch.float32, device=hidden.device)
        self._check(self.lib.mcu_moe_experts(self.handle, kinds[0], kinds[1], kinds[2], _ptr(hidden), T, H, FF, E,
                                             _ptr(gate), _ptr(up), _ptr(down), _ptr(topk_ids), _ptr(topk_weights), k,
                                             ffn_type, weights_scale, policy, _ptr(out)))
        return out

    # ---- decoder operators ----
    def rmsnorm(self, x, weight, eps: float, residual=None, weight_offset: float = 0.0, out=None):
        rows, n = x.shape
        if out is None:
            out = self.torch.empty_like(x)
        self._check(self.lib.mcu_rmsnorm(self.handle, _ptr(x), _ptr(residual), _ptr(weight), rows, n, eps, weight_offset,
                                         _ptr(out)))
        return out

    def rope(self, x, positions, n_heads: int, head_dim: int, theta: float = 10000.0, freq_scale: float = 1.0,
             neox: bool = False, out=None):
        """x [T, n_heads*head_dim] (row stride allowed), positions int32 [T]; out may alias x."""
        T = x.shape[0]
        if out is None:
            out = self.torch.empty((T, n_heads * head_dim), dtype=self.torch.float32, device=x.device)
        self._check(self.lib.mcu_rope(self.handle, _ptr(x), x.stride(0), _ptr(positions), T, n_heads, head_dim, theta,
                                      freq_scale, 1 if neox else 0, _ptr(out), out.stride(0)))
        return out

    def add_rmsnorm(self, x, delta, weight, eps: float, x_out, h_out, weight_offset: float = 0.0):
        """x_out = x + delta; h_out = rmsnorm(x_out) * weight (x_out may be x)."""
        rows, n = x.shape
        self._check(self.lib.mcu_add_rmsnorm(self.handle, _ptr(x), _ptr(delta), _ptr(weight), rows, n, eps, weight_offset,
                                             _ptr(x_out), _ptr(h_out)))
        return x_out, h_out

    def rope_qk(self, q, k, positions, n_q_heads: int, n_k_heads: int, head_dim: int, theta: float = 10000.0,
                freq_scale: float = 1.0, neox: bool = False):
        """RoPE in place on q [T, n_q_heads*head_dim] and k [T, n_k_heads*head_dim]."""
        self._check(self.lib.mcu_rope_qk(self.handle, _ptr(q), q.stride(0), n_q_heads, _ptr(k), k.stride(0), n_k_heads,
                                         _ptr(positions), q.shape[0], head_dim, theta, freq_scale, 1 if neox else 0))
        return q, k

    def swiglu(self, gate, up, out=None):
        if out is None:
            out = self.torch.empty_like(gate)
        self._check(self.lib.mcu_swiglu(self.handle, _ptr(gate), _ptr(up), gate.numel(), _ptr(out)))
        return out

    def add(self, a, b, out=None):
        if out is None:
            out = self.torch.empty_like(a)
        self._check(self.lib.mcu_add(self.handle, _ptr(a), _ptr(b), a.numel(), _ptr(out)))
        return out

    def argmax(self, x, out=None):
        rows, n = x.shape
        if out is None:
            out = self.torch.empty((rows,), dtype=self.torch.int32, device=x.device)
        self._check(self.lib.mcu_argmax(self.handle, _ptr(x), rows, n, _ptr(out)))
        return out

    def embedding_gather(self, kind: int, table, dim: int, ids, out=None):
        T = ids.shape[0]
        if out is None:
            out = self.torch.empty((T, dim), dtype=self.torch.float32, device=ids.device)
        self._check(self.lib.mcu_embedding_gather(self.handle, kind, _ptr(table), dim, _ptr(ids), T, _ptr(out)))
        return out

    def paged_attention(self, token_meta, q, k_new, v_new, kv_k, kv_v, block_table, layer: int, n_q_heads: int,
                        n_kv_heads: int, head_dim: int, block_size: int, scale: float, out=None):
        """q [T, n_q_heads*head_dim], k_new/v_new [T, n_kv_heads*head_dim] (contiguous); the pool tensors
        [blocks, layers, kv_heads, block_size, head_dim] (float32 or float16) are updated in place."""
        T = q.shape[0]
        if out is None:
            out = self.torch.empty_like(q)
        kv_dtype = 1 if kv_k.dtype == self.torch.float16 else 0
        self._check(self.lib.mcu_paged_attention(
            self.handle, _ptr(token_meta), T, _ptr(q), _ptr(k_new), _ptr(v_new), _ptr(kv_k), _ptr(kv_v), kv_dtype,
            _ptr(block_table), block_table.shape[1], kv_k.shape[1], layer, n_q_heads, n_kv_heads, head_dim, block_size,
            scale, _ptr(out)))
        return out

    def rope_table(self, positions, head_dim: int, theta: float, freq_scale: float = 1.0, out=None):
        """[T, head_dim/2, 2] float32 {cos, sin} of position * frequency: the rotation every layer of a step applies."""
        T = positions.shape[0]
        if out is None:
            out = self.torch.empty((T, head_dim // 2, 2), dtype=self.torch.float32, device=positions.device)
        self._check(self.lib.mcu_rope_table(self.handle, _ptr(positions), T, head_dim, theta, freq_scale, _ptr(out)))
        return out

    def paged_attention_decode(self, token_meta, q, k_new, v_new, kv_k, kv_v, block_table, layer: int, n_q_heads: int,
                               n_kv_heads: int, head_dim: int, block_size: int, scale: float, positions, rope_theta: float,
                               rope_freq_scale: float = 1.0, neox: bool = False, rope_table=None, out=None):
        """A decode step's RoPE + append + attention + chunk merge (one launch on float16 pools).  q / k_new are the
        projections before RoPE and may be rotated in place; at most one token per sequence in the call.  rope_table:
        what rope_table() made for these positions (shared by the layers of a step); None computes one per call."""
        T = q.shape[0]
        if out is None:
            out = self.torch.empty_like(q)
        kv_dtype = 1 if kv_k.dtype == self.torch.float16 else 0
        self._check(self.lib.mcu_paged_attention_decode(
            self.handle, _ptr(token_meta), T, _ptr(q), _ptr(k_new), _ptr(v_new), _ptr(kv_k), _ptr(kv_v), kv_dtype,
            _ptr(block_table), block_table.shape[1], kv_k.shape[1], layer, n_q_heads, n_kv_heads, head_dim, block_size,
            scale, _ptr(positions), rope_theta, rope_freq_scale, 1 if neox else 0,
            _ptr(rope_table) if rope_table is not None else None, _ptr(out)))
        return out

    def moe_last_buffers(self, T: int, k: int, H: int, FF: int) -> dict:
        """Views of the intermediates the last MoE call left in the workspace (see mcu_moe_last_buffers): for checking
        the operator stage by stage.  Synchronizes first."""
        b = _MoeBuffers()
        self.synchronize()
        self._check(self.lib.mcu_moe_last_buffers(self.handle, C.byref(b)))
        view = lambda ptr, shape, ts="<f4": _tensor_from_ptr(self.torch, ptr, shape, self.device, ts)
        r, E = int(b.routes), int(b.experts)
        assert r == T * k
        return {"offsets": view(b.offsets, (E + 1,), "<i4"), "sorted_tok": view(b.sorted_tok, (r,), "<i4"),
                "sorted_w": view(b.sorted_w, (r,)), "route_pos": view(b.route_pos, (r,), "<i4"),
                "gate_out": view(b.gate_out, (r, FF)), "up_out": view(b.up_out, (r, FF)),
                "route_down": view(b.route_down, (r, H)), "grouped": bool(b.grouped)}

    def moe_experts_local(self, kinds, hidden, gate, up, down, topk_ids, topk_weights, FF: int, E: int,
                          expert_begin: int, expert_count: int, ffn_type: int = FFN_SWIGLU,
                          weights_scale: float = 1.0, policy: int = ROUTER_RENORMALIZE_SELECTED, out=None):
        """This rank's share of the MoE output: gate/up/down hold experts [expert_begin, +expert_count) only."""
        T, H = hidden.shape
        k = topk_ids.shape[1]
        if out is None:
            out = self.torch.empty((T, H), dtype=self.torch.float32, device=hidden.device)
        self._check(self.lib.mcu_moe_experts_local(
            self.handle, kinds[0], kinds[1], kinds[2], _ptr(hidden), T, H, FF, E, expert_begin, expert_count,
            _ptr(gate), _ptr(up), _ptr(down), _ptr(topk_ids), _ptr(topk_weights), k, ffn_type, weights_scale, policy,
            _ptr(out)))
        return out


class PeerComm:
    """mcu_peer_comm: staging buffers mapped across the ranks of one box and the one-shot all-reduce kernel.
    `exchange(handle_bytes) -> list of every rank's handle bytes in rank order` is the host transport
    (torch.distributed.all_gather_object in tensor_parallel.py)."""

    def __init__(self, ctx: "Context", rank: int, world: int, max_bytes: int, exchange):
        self.ctx, self.rank, self.world, self.max_bytes = ctx, rank, world, max_bytes
        h = C.c_void_p()
        ctx._check(ctx.lib.mcu_peer_comm_create(ctx.handle, rank, world, max_bytes, C.byref(h)))
        self.handle = h
        mine = C.create_string_buffer(64)
        ctx._check(ctx.lib.mcu_peer_comm_export(h, mine))
        handles = exchange(bytes(mine.raw))
        assert len(handles) == world and all(len(x) == 64 for x in handles)
        ctx._check(ctx.lib.mcu_peer_comm_connect(h, C.create_string_buffer(b"".join(handles), 64 * world)))

    def set_fused(self, enabled: bool):
        """One-kernel form of linear_allreduce (matmul epilogue + all-reduce); every rank must choose the same."""
        self.ctx._check(self.ctx.lib.mcu_peer_comm_set_fused(self.handle, 1 if enabled else 0))

    def set_one_slot(self, enabled: bool):
        """One staging slot and a closing "finished reading" exchange per collective: a captured CUDA graph may then hold
        any number of collectives (an even number with the default two slots); every rank must choose the same."""
        self.ctx._check(self.ctx.lib.mcu_peer_comm_set_one_slot(self.handle, 1 if enabled else 0))

    def staging(self, shape):
        """The buffer the next all-reduce sums, as a float32 torch tensor of `shape` (a view, no copy)."""
        n = int(np.prod(shape))
        assert n * 4 <= self.max_bytes
        ptr = self.ctx.lib.mcu_peer_comm_staging(self.handle)
        return _tensor_from_ptr(self.ctx.torch, ptr, shape, self.ctx.device)

    def allreduce(self, n_floats: int, out):
        self.ctx._check(self.ctx.lib.mcu_peer_allreduce(self.handle, n_floats, _ptr(out)))
        return out

    def linear_allreduce(self, kind: int, x, w, F: int, out=None):
        T, K = x.shape
        if out is None:
            out = self.ctx.torch.empty((T, F), dtype=self.ctx.torch.float32, device=x.device)
        self.ctx._check(self.ctx.lib.mcu_linear_allreduce(self.ctx.handle, self.handle, kind, _ptr(x), x.stride(0),
                                                          _ptr(w), T, K, F, _ptr(out)))
        return out

    def moe_experts_ep(self, kinds, hidden, gate, up, down, topk_ids, topk_weights, FF: int, E: int, expert_bounds,
                       ffn_type: int = FFN_SWIGLU, weights_scale: float = 1.0, policy: int = ROUTER_RENORMALIZE_SELECTED,
                       out=None):
        """Expert-parallel MoE FFN: this rank holds the experts [expert_bounds[rank], expert_bounds[rank + 1]); the
        routed rows return to the owners of their tokens over peer memory and the token slices are gathered (see
        mcu_moe_experts_ep).  Raises MarmotCudaError with code NOT_IMPLEMENTED for shapes off the grouped path."""
        T, H = hidden.shape
        k = topk_ids.shape[1]
        if out is None:
            out = self.ctx.torch.empty((T, H), dtype=self.ctx.torch.float32, device=hidden.device)
        bounds = (C.c_int32 * (self.world + 1))(*[int(b) for b in expert_bounds])
        self.ctx._check(self.ctx.lib.mcu_moe_experts_ep(
            self.ctx.handle, self.handle, kinds[0], kinds[1], kinds[2], _ptr(hidden), T, H, FF, E, bounds, _ptr(gate),
            _ptr(up), _ptr(down), _ptr(topk_ids), _ptr(topk_weights), k, ffn_type, weights_scale, policy, _ptr(out)))
        return out

    def close(self):
        if self.handle:
            self.ctx.lib.mcu_peer_comm_destroy(self.handle)
            self.handle = None


def _tensor_from_ptr(torch, ptr: int, shape, device_index: int, typestr: str = "<f4"):
    """torch view (float32 unless `typestr` says otherwise) of device memory owned by the library (CUDA array
    interface)."""

    class _Ext:
        pass

    e = _Ext()
    e.__cuda_array_interface__ = {"shape": tuple(int(v) for v in shape), "typestr": typestr, "data": (int(ptr), False),
                                  "version": 2}
    return torch.as_tensor(e, device=torch.device("cuda", device_index))


class _MoeBuffers(C.Structure):
    """struct mcu_moe_buffers, include/marmot_cuda.h."""
    _fields_ = [("offsets", C.c_void_p), ("sorted_tok", C.c_void_p), ("sorted_w", C.c_void_p), ("route_pos", C.c_void_p),
                ("gate_out", C.c_void_p), ("up_out", C.c_void_p), ("route_down", C.c_void_p), ("routes", C.c_size_t),
                ("experts", C.c_size_t), ("grouped", C.c_int)]


class Graph:
    """A recorded sequence of calls (marmot_cuda.h: mcu_graph_*); launch() replays it on the context's stream."""

    def __init__(self, ctx: "Context", handle):
        self.ctx, self.handle = ctx, handle
        ctx.lib.mcu_graph_launch.argtypes = [C.c_void_p]
        ctx.lib.mcu_graph_destroy.argtypes = [C.c_void_p]
        ctx.lib.mcu_graph_destroy.restype = None

    def launch(self) -> None:
        self.ctx._check(self.ctx.lib.mcu_graph_launch(self.handle))

    def close(self) -> None:
        if self.handle:
            self.ctx.lib.mcu_graph_destroy(self.handle)
            self.handle = None


class _KvPoolOptions(C.Structure):
    """struct mcu_kv_pool_options."""
    _fields_ = [("flags", C.c_uint64), ("max_seqs", C.c_size_t), ("max_seq_len", C.c_size_t), ("block_size", C.c_size_t),
                ("num_blocks", C.c_size_t), ("num_swap_blocks", C.c_size_t), ("num_layers", C.c_size_t),
                ("num_kv_heads", C.c_size_t), ("head_dim", C.c_size_t), ("kv_dtype", C.c_int)]


class _KvAppendPlan(C.Structure):
    _fields_ = [("seq", C.c_uint32), ("token_count", C.c_size_t), ("cookie", C.c_uint64)]


class _KvPrefixPlan(C.Structure):
    _fields_ = [("seq", C.c_uint32), ("num_blocks", C.c_size_t), ("prefix_len", C.c_size_t), ("cookie", C.c_uint64)]


class KvPool:
    """The paged KV-cache pool (marmot_cuda.h: mcu_kv_pool_*).  `ctx=None` keeps books only (no GPU needed).
    Methods return the library's status code (0 = success) next to their outputs, as the reference API does."""

    def __init__(self, ctx: "Context | None", *, max_seqs: int, max_seq_len: int, block_size: int, num_blocks: int,
                 num_swap_blocks: int = 0, num_layers: int = 1, num_kv_heads: int = 1, head_dim: int = 64,
                 kv_f16: bool = True, deterministic: bool = False, lib=None):
        self.lib = L = lib or (ctx.lib if ctx is not None else load_library())
        self.ctx = ctx
        vp, sz, u32 = C.c_void_p, C.c_size_t, C.c_uint32
        L.mcu_kv_pool_create.argtypes = [vp, C.POINTER(_KvPoolOptions), C.POINTER(vp)]
        L.mcu_kv_pool_destroy.argtypes = [vp]
        L.mcu_kv_pool_destroy.restype = None
        L.mcu_kv_pool_acquire_seq.argtypes = [vp, C.POINTER(u32)]
        L.mcu_kv_pool_release_seq.argtypes = [vp, u32]
        L.mcu_kv_pool_prepare_append.argtypes = [vp, u32, sz, C.POINTER(_KvAppendPlan), C.POINTER(u32), C.POINTER(sz)]
        L.mcu_kv_pool_commit_append.argtypes = [vp, C.POINTER(_KvAppendPlan)]
        L.mcu_kv_pool_abort_append.argtypes = [vp, C.POINTER(_KvAppendPlan)]
        L.mcu_kv_pool_abort_append.restype = None
        L.mcu_kv_pool_prepare_prefix_attach.argtypes = [vp, u32, C.POINTER(u32), sz, sz, C.POINTER(_KvPrefixPlan)]
        L.mcu_kv_pool_commit_prefix_attach.argtypes = [vp, C.POINTER(_KvPrefixPlan)]
        L.mcu_kv_pool_abort_prefix_attach.argtypes = [vp, C.POINTER(_KvPrefixPlan)]
        L.mcu_kv_pool_abort_prefix_attach.restype = None
        L.mcu_kv_pool_get_pointers.argtypes = [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(sz)]
        for name in ("free_block_count", "total_block_count"):
            getattr(L, f"mcu_kv_pool_{name}").argtypes = [vp]
            getattr(L, f"mcu_kv_pool_{name}").restype = sz
        L.mcu_kv_pool_seq_len.argtypes = [vp, u32]
        L.mcu_kv_pool_seq_len.restype = sz
        L.mcu_kv_pool_block_id.argtypes = [vp, u32, sz]
        L.mcu_kv_pool_block_id.restype = u32
        L.mcu_kv_pool_block_generation.argtypes = [vp, u32]
        L.mcu_kv_pool_block_generation.restype = u32
        L.mcu_kv_pool_set_block_retained.argtypes = [vp, u32, C.c_int]
        L.mcu_kv_pool_set_block_retained.restype = None
        L.mcu_kv_pool_swap_out_seq.argtypes = [vp, u32]
        L.mcu_kv_pool_swap_in_seq.argtypes = [vp, u32]
        L.mcu_kv_pool_is_seq_swapped.argtypes = [vp, u32, C.POINTER(C.c_int)]
        opts = _KvPoolOptions(1 if deterministic else 0, max_seqs, max_seq_len, block_size, num_blocks, num_swap_blocks,
                              num_layers, num_kv_heads, head_dim, 1 if kv_f16 else 0)
        self.shape = (num_blocks, num_layers, num_kv_heads, block_size, head_dim)
        self.kv_f16 = kv_f16
        self.max_seqs = max_seqs
        h = vp()
        rc = L.mcu_kv_pool_create(ctx.handle if ctx is not None else None, C.byref(opts), C.byref(h))
        if rc != 0:
            raise MarmotCudaError(rc, L.mcu_last_error_message().decode())
        self.handle = h

    def close(self):
        if self.handle:
            self.lib.mcu_kv_pool_destroy(self.handle)
            self.handle = None

    def acquire_seq(self):
        seq = C.c_uint32(0xFFFFFFFF)
        rc = self.lib.mcu_kv_pool_acquire_seq(self.handle, C.byref(seq))
        return rc, seq.value

    def release_seq(self, seq: int) -> int:
        return self.lib.mcu_kv_pool_release_seq(self.handle, seq)

    def prepare_append(self, seq: int, n: int):
        plan = _KvAppendPlan()
        slots = (C.c_uint32 * max(n, 1))()
        start = C.c_size_t(0)
        rc = self.lib.mcu_kv_pool_prepare_append(self.handle, seq, n, C.byref(plan), slots, C.byref(start))
        return rc, plan, list(slots[:n]) if rc == 0 else [], start.value

    def commit_append(self, plan) -> int:
        return self.lib.mcu_kv_pool_commit_append(self.handle, C.byref(plan))

    def abort_append(self, plan) -> None:
        self.lib.mcu_kv_pool_abort_append(self.handle, C.byref(plan))

    def prepare_prefix_attach(self, seq: int, block_ids, prefix_len: int):
        plan = _KvPrefixPlan()
        ids = (C.c_uint32 * max(len(block_ids), 1))(*block_ids)
        rc = self.lib.mcu_kv_pool_prepare_prefix_attach(self.handle, seq, ids, len(block_ids), prefix_len, C.byref(plan))
        return rc, plan

    def commit_prefix_attach(self, plan) -> int:
        return self.lib.mcu_kv_pool_commit_prefix_attach(self.handle, C.byref(plan))

    def abort_prefix_attach(self, plan) -> None:
        self.lib.mcu_kv_pool_abort_prefix_attach(self.handle, C.byref(plan))

    def free_block_count(self) -> int:
        return self.lib.mcu_kv_pool_free_block_count(self.handle)

    def total_block_count(self) -> int:
        return self.lib.mcu_kv_pool_total_block_count(self.handle)

    def seq_len(self, seq: int) -> int:
        return self.lib.mcu_kv_pool_seq_len(self.handle, seq)

    def block_id(self, seq: int, logical: int) -> int:
        return self.lib.mcu_kv_pool_block_id(self.handle, seq, logical)

    def block_generation(self, block: int) -> int:
        return self.lib.mcu_kv_pool_block_generation(self.handle, block)

    def set_block_retained(self, block: int, keep: bool) -> None:
        self.lib.mcu_kv_pool_set_block_retained(self.handle, block, 1 if keep else 0)

    def swap_out(self, seq: int) -> int:
        return self.lib.mcu_kv_pool_swap_out_seq(self.handle, seq)

    def swap_in(self, seq: int) -> int:
        return self.lib.mcu_kv_pool_swap_in_seq(self.handle, seq)

    def is_swapped(self, seq: int) -> bool:
        out = C.c_int(0)
        self.lib.mcu_kv_pool_is_seq_swapped(self.handle, seq, C.byref(out))
        return bool(out.value)

    def tensors(self):
        """(kv_k, kv_v, block_table) as torch tensors over the pool's device memory (no copy)."""
        import torch

        k, v, t, mb = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_size_t()
        self.lib.mcu_kv_pool_get_pointers(self.handle, C.byref(k), C.byref(v), C.byref(t), C.byref(mb))
        if not k.value:
            raise MarmotCudaError(-1, "the pool keeps books only: it has no storage")
        dev = torch.device("cuda", self.ctx.device)
        dt = torch.float16 if self.kv_f16 else torch.float32

        def view(ptr, shape, dtype):
            n = int(np.prod(shape))
            holder = type("_Cai", (), {"__cuda_array_interface__": {
                "shape": (n,), "typestr": {torch.float16: "<f2", torch.float32: "<f4", torch.int32: "<i4"}[dtype],
                "data": (ptr, False), "version": 2}})()
            return torch.as_tensor(holder, device=dev).view(shape)

        return (view(k.value, self.shape, dt), view(v.value, self.shape, dt),
                view(t.value, (self.max_seqs, mb.value), torch.int32))
