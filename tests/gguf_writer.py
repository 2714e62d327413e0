"""A minimal GGUF v3 writer for tests: metadata (u32 / f32 / string / string arrays) and tensors with raw payloads,
laid out as llama.cpp writes them (little endian, tensor data aligned to general.alignment)."""
from __future__ import annotations

import struct

import numpy as np

GGML_F32, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K = 0, 8, 12, 14
KIND_TO_GGML = {5: GGML_Q8_0, 9: GGML_Q4_K, 11: GGML_Q6_K}


def _string(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _value(v) -> bytes:
    if isinstance(v, bool):
        return struct.pack("<IB", 7, int(v))
    if isinstance(v, int):
        return struct.pack("<II", 4, v)
    if isinstance(v, float):
        return struct.pack("<If", 6, v)
    if isinstance(v, str):
        return struct.pack("<I", 8) + _string(v)
    if isinstance(v, (list, tuple)) and all(isinstance(x, str) for x in v):
        return struct.pack("<IIQ", 9, 8, len(v)) + b"".join(_string(x) for x in v)
    if isinstance(v, np.ndarray) and v.dtype == np.int32:
        return struct.pack("<IIQ", 9, 5, v.size) + v.tobytes()
    raise TypeError(type(v))


def write_gguf(path, metadata: dict, tensors: list, alignment: int = 32, version: int = 3) -> None:
    """tensors: (name, ggml_type, dims innermost-first, payload bytes-like)."""
    meta = dict(metadata)
    meta.setdefault("general.alignment", alignment)
    head = struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(meta))
    for k, v in meta.items():
        head += _string(k) + _value(v)
    offset, infos, blobs = 0, b"", []
    for name, ggml_type, dims, payload in tensors:
        payload = np.ascontiguousarray(payload).view(np.uint8).reshape(-1)
        infos += _string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", ggml_type, offset)
        blobs.append((offset, payload))
        offset = (offset + payload.size + alignment - 1) // alignment * alignment
    start = (len(head) + len(infos) + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(head + infos)
        f.write(b"\0" * (start - len(head) - len(infos)))
        for off, payload in blobs:
            f.seek(start + off)
            f.write(payload.tobytes())
        f.truncate(start + offset)


def write_llama(path, shape, weights: dict, kinds: dict | None = None, tie_output: bool = False) -> None:
    """A Llama-family file from the `weights` dict of tests (names as in marmot_b200.decoder)."""
    from marmot_b200.decoder import LAYER_WEIGHTS

    default = {n: k for n, k, _, _ in LAYER_WEIGHTS}
    default.update(tok_embd=9, output=11)
    kind = lambda name: (kinds or {}).get(name, default[name.split(".")[-1]])
    meta = {"general.architecture": "llama", "general.name": "synthetic", "llama.block_count": shape.layers,
            "llama.embedding_length": shape.d, "llama.feed_forward_length": shape.ffn,
            "llama.attention.head_count": shape.n_heads, "llama.attention.head_count_kv": shape.n_kv_heads,
            "llama.rope.freq_base": float(shape.rope_theta), "llama.attention.layer_norm_rms_epsilon": float(shape.rms_eps),
            "llama.context_length": 2048, "tokenizer.ggml.tokens": [f"t{i}" for i in range(8)]}
    names = {"wq": "attn_q", "wk": "attn_k", "wv": "attn_v", "wo": "attn_output", "gate": "ffn_gate", "up": "ffn_up",
             "down": "ffn_down"}
    tensors = [("token_embd.weight", KIND_TO_GGML[kind("tok_embd")], (shape.d, shape.vocab), weights["tok_embd"])]
    for i in range(shape.layers):
        for ours, kdefault, rows, cols in LAYER_WEIGHTS:
            tensors.append((f"blk.{i}.{names[ours]}.weight", KIND_TO_GGML[kind(f"l{i}.{ours}")], (cols(shape), rows(shape)),
                            weights[f"l{i}.{ours}"]))
        tensors.append((f"blk.{i}.attn_norm.weight", GGML_F32, (shape.d,), weights[f"l{i}.attn_norm"].astype(np.float32)))
        tensors.append((f"blk.{i}.ffn_norm.weight", GGML_F32, (shape.d,), weights[f"l{i}.ffn_norm"].astype(np.float32)))
    tensors.append(("output_norm.weight", GGML_F32, (shape.d,), weights["out_norm"].astype(np.float32)))
    if not tie_output:
        tensors.append(("output.weight", KIND_TO_GGML[kind("output")], (shape.d, shape.vocab), weights["output"]))
    write_gguf(path, meta, tensors)
