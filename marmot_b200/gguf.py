"""GGUF model files -> a device-resident, optionally tensor-parallel decoder.

`GgufFile` wraps the library's reader (marmot_cuda.h: mcu_gguf_*; the file is memory-mapped and indexed in C++, the
payloads travel from the mapping to the device without a host copy).  `load_llama_decoder` reads the hyper-parameters
the reference's builder reads (src/graph/gguf/architecture.cpp: `<arch>.block_count`, `.embedding_length`,
`.feed_forward_length`, `.attention.head_count`, `.attention.head_count_kv`, `.rope.freq_base`,
`.attention.layer_norm_rms_epsilon`) and the tensors of a Llama-family model (`token_embd`, `blk.N.attn_{q,k,v,output}`,
`blk.N.ffn_{gate,up,down}`, `blk.N.{attn,ffn}_norm`, `output_norm`, `output`; a missing `output` falls back to the
embedding table), and uploads this rank's share of each: heads, FFN rows and vocabulary rows as row ranges,
`attn_output` and `ffn_down` as K ranges (one strided copy each).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from .runtime import KIND_Q4_K, KIND_Q6_K, KIND_Q8_0, MarmotCudaError, load_library, row_bytes


class _TensorInfo(C.Structure):
    """struct mcu_gguf_tensor_info."""
    _fields_ = [("name", C.c_char_p), ("ggml_type", C.c_uint32), ("kind", C.c_int), ("n_dims", C.c_uint32),
                ("dims", C.c_uint64 * 4), ("nbytes", C.c_size_t), ("data", C.c_void_p)]


class GgufFile:
    def __init__(self, path: str, lib=None):
        self.lib = L = lib or load_library()
        vp = C.c_void_p
        L.mcu_gguf_open.argtypes = [C.c_char_p, C.POINTER(vp)]
        L.mcu_gguf_close.argtypes = [vp]
        L.mcu_gguf_close.restype = None
        L.mcu_gguf_tensor_count.argtypes = [vp]
        L.mcu_gguf_tensor_count.restype = C.c_size_t
        L.mcu_gguf_find_tensor.argtypes = [vp, C.c_char_p]
        L.mcu_gguf_tensor_info.argtypes = [vp, C.c_size_t, C.POINTER(_TensorInfo)]
        L.mcu_gguf_meta_u64.argtypes = [vp, C.c_char_p, C.POINTER(C.c_uint64)]
        L.mcu_gguf_meta_f64.argtypes = [vp, C.c_char_p, C.POINTER(C.c_double)]
        L.mcu_gguf_meta_str.argtypes = [vp, C.c_char_p, C.POINTER(C.c_char_p), C.POINTER(C.c_size_t)]
        L.mcu_gguf_upload.argtypes = [vp, vp, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, vp]
        h = vp()
        rc = L.mcu_gguf_open(str(path).encode(), C.byref(h))
        if rc != 0:
            raise MarmotCudaError(rc, L.mcu_last_error_message().decode())
        self.handle = h

    def close(self):
        if self.handle:
            self.lib.mcu_gguf_close(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __len__(self):
        return self.lib.mcu_gguf_tensor_count(self.handle)

    def find(self, name: str) -> int:
        return self.lib.mcu_gguf_find_tensor(self.handle, name.encode())

    def info(self, index: int) -> dict:
        t = _TensorInfo()
        rc = self.lib.mcu_gguf_tensor_info(self.handle, index, C.byref(t))
        if rc != 0:
            raise MarmotCudaError(rc, self.lib.mcu_last_error_message().decode())
        return {"name": t.name.decode(), "ggml_type": t.ggml_type, "kind": t.kind, "dims": tuple(t.dims[:t.n_dims]),
                "nbytes": t.nbytes, "data": t.data}

    def tensor_bytes(self, index: int) -> np.ndarray:
        """The tensor's payload as a uint8 view of the mapping (valid while the file is open)."""
        i = self.info(index)
        return np.ctypeslib.as_array(C.cast(i["data"], C.POINTER(C.c_uint8)), shape=(i["nbytes"],))

    def meta_int(self, key: str, default=None) -> int:
        out = C.c_uint64()
        if self.lib.mcu_gguf_meta_u64(self.handle, key.encode(), C.byref(out)) != 0:
            if default is None:
                raise KeyError(key)
            return default
        return int(out.value)

    def meta_float(self, key: str, default=None) -> float:
        out = C.c_double()
        if self.lib.mcu_gguf_meta_f64(self.handle, key.encode(), C.byref(out)) != 0:
            if default is None:
                raise KeyError(key)
            return default
        return float(out.value)

    def meta_str(self, key: str, default=None) -> str:
        out, n = C.c_char_p(), C.c_size_t()
        if self.lib.mcu_gguf_meta_str(self.handle, key.encode(), C.byref(out), C.byref(n)) != 0:
            if default is None:
                raise KeyError(key)
            return default
        return out.value[:n.value].decode()

    def upload(self, ctx, index: int, rows=None, k_range=None):
        """This tensor, or rows [lo, hi) x values [k_lo, k_hi) of it, as a packed device tensor (uint8 for block
        formats, float32 for F32)."""
        torch = ctx.torch
        i = self.info(index)
        K = i["dims"][0]
        n_rows = int(np.prod(i["dims"][1:])) if len(i["dims"]) > 1 else 1
        lo, hi = rows if rows is not None else (0, n_rows)
        k_lo, k_hi = k_range if k_range is not None else (0, K)
        if i["ggml_type"] == 0:
            per_row = 4 * (k_hi - k_lo)
        elif i["kind"] >= 0:
            per_row = row_bytes(i["kind"], k_hi - k_lo)
        else:
            raise MarmotCudaError(-1, f"{i['name']}: ggml type {i['ggml_type']} has no CUDA kernel")
        out = torch.empty(max((hi - lo) * per_row, 1), dtype=torch.uint8, device=torch.device("cuda", ctx.device))
        rc = self.lib.mcu_gguf_upload(ctx.handle, self.handle, index, lo, hi, k_lo, k_hi, out.data_ptr())
        if rc != 0:
            raise MarmotCudaError(rc, self.lib.mcu_last_error_message().decode())
        out = out[:(hi - lo) * per_row]
        return out.view(torch.float32) if i["ggml_type"] == 0 else out


# Architectures whose layer is exactly what `decoder.Decoder` computes: interleaved-pair ("NORM") RoPE, no attention
# bias, no q/k norm.  The reference picks these traits per architecture (src/graph/gguf/architecture.cpp:12-143):
# qwen2 / qwen3 / phi3 / gemma rotate half-split pairs ("NEOX"), qwen2 adds attention biases, qwen3 normalises q and k.
SUPPORTED_ARCHITECTURES = ("llama", "mistral")


def decoder_shape_from_gguf(f: "GgufFile"):
    """The hyper-parameters the reference's graph builder reads (src/graph/gguf/graph_builder.cpp) as a DecoderShape.
    Files of an architecture whose layer differs from the Llama layer are refused rather than decoded wrongly."""
    from .decoder import DecoderShape

    arch = f.meta_str("general.architecture", "llama")
    if arch not in SUPPORTED_ARCHITECTURES:
        raise MarmotCudaError(-1, f"architecture '{arch}' is not supported by the CUDA decoder "
                                  f"(supported: {', '.join(SUPPORTED_ARCHITECTURES)}): its RoPE pairing, attention "
                                  "biases or q/k normalisation differ from the Llama layer")
    n_heads = f.meta_int(f"{arch}.attention.head_count")
    d = f.meta_int(f"{arch}.embedding_length")
    emb = f.info(f.find("token_embd.weight"))
    q0 = f.find("blk.0.attn_q.weight")  # without an explicit key length the query projection tells the head size
    hd_default = int(f.info(q0)["dims"][1]) // n_heads if q0 >= 0 else d // n_heads
    return DecoderShape(
        layers=f.meta_int(f"{arch}.block_count"), d=d, ffn=f.meta_int(f"{arch}.feed_forward_length"),
        n_heads=n_heads, n_kv_heads=f.meta_int(f"{arch}.attention.head_count_kv", n_heads),
        head_dim=f.meta_int(f"{arch}.attention.key_length", hd_default), vocab=int(emb["dims"][1]),
        rope_theta=f.meta_float(f"{arch}.rope.freq_base", 10000.0),
        rms_eps=f.meta_float(f"{arch}.attention.layer_norm_rms_epsilon", 1e-5))


def load_llama_decoder(path: str, ctx, max_seqs: int, max_ctx: int, block_size: int = 16, kv_dtype=None, group=None,
                       comm=None, kv_pool=None):
    """A `decoder.Decoder` over the weights of a Llama-family GGUF file; with `group` / `comm` this rank's
    tensor-parallel share (see decoder.Decoder)."""
    from . import tensor_parallel as tp
    from .decoder import Decoder

    group = group or tp.Group()
    world, rank = group.world, group.rank
    with GgufFile(path, lib=ctx.lib) as f:
        shape = decoder_shape_from_gguf(f)
        hd = shape.head_dim
        if world > 1 and (shape.n_heads % world or shape.n_kv_heads % world):
            raise ValueError("heads must divide over the ranks")
        q_rows = tp.shard_range(shape.n_heads * hd, world, rank, shape.n_heads * hd // world)
        kv_rows = tp.shard_range(shape.n_kv_heads * hd, world, rank, shape.n_kv_heads * hd // world)
        ffn_rows = tp.shard_range(shape.ffn, world, rank, 2048) if world > 1 else (0, shape.ffn)
        vocab_rows = tp.shard_range(shape.vocab, world, rank, 32) if world > 1 else (0, shape.vocab)

        def need(name):
            idx = f.find(name)
            if idx < 0:
                raise KeyError(f"{path}: tensor {name} is missing")
            return idx

        def matrix(name, rows=None, k_range=None):
            idx = need(name)
            info = f.info(idx)
            if info["kind"] < 0:
                raise MarmotCudaError(-1, f"{name}: ggml type {info['ggml_type']} has no CUDA kernel (Q4_K, Q6_K, Q8_0 do)")
            if rows is not None and rows[0] == rows[1] or k_range is not None and k_range[0] == k_range[1]:
                return None, info["kind"]
            return f.upload(ctx, idx, rows, k_range), info["kind"]

        def vector(name):
            idx = need(name)
            if f.info(idx)["ggml_type"] != 0:
                raise MarmotCudaError(-1, f"{name}: norm weights must be F32")
            return f.upload(ctx, idx)

        weights, kinds = {}, {}
        for i in range(shape.layers):
            b = f"blk.{i}."
            for ours, theirs, rows, k_range in (
                    ("wq", "attn_q", q_rows, None), ("wk", "attn_k", kv_rows, None), ("wv", "attn_v", kv_rows, None),
                    ("wo", "attn_output", None, q_rows), ("gate", "ffn_gate", ffn_rows, None),
                    ("up", "ffn_up", ffn_rows, None), ("down", "ffn_down", None, ffn_rows)):
                weights[f"l{i}.{ours}"], kinds[f"l{i}.{ours}"] = matrix(b + theirs + ".weight", rows, k_range)
            weights[f"l{i}.attn_norm"] = vector(b + "attn_norm.weight")
            weights[f"l{i}.ffn_norm"] = vector(b + "ffn_norm.weight")
        weights["tok_embd"], kinds["tok_embd"] = matrix("token_embd.weight")
        out_name = "output.weight" if f.find("output.weight") >= 0 else "token_embd.weight"
        weights["output"], kinds["output"] = matrix(out_name, vocab_rows)
        weights["out_norm"] = vector("output_norm.weight")
        ctx.synchronize()  # the uploads read the mapping, which closes with the file
    return Decoder(ctx, shape, max_seqs=max_seqs, max_ctx=max_ctx, block_size=block_size, kv_dtype=kv_dtype,
                   device_weights=weights, kinds=kinds, group=group if world > 1 else None, comm=comm, kv_pool=kv_pool)
