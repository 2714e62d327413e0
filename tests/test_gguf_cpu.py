"""The GGUF reader on files written by tests/gguf_writer.py: header, metadata of every scalar kind, tensor directory,
payload addresses; malformed files are refused."""
from __future__ import annotations

import struct

import numpy as np
import pytest

from marmot_b200.gguf import GgufFile
from marmot_b200.runtime import KIND_Q4_K, KIND_Q6_K, KIND_Q8_0, MarmotCudaError
from tests.gguf_writer import GGML_F32, GGML_Q4_K, GGML_Q6_K, GGML_Q8_0, write_gguf
from tests.util import random_blocks


@pytest.mark.parametrize("alignment,version", [(32, 3), (64, 3), (32, 2)])
def test_directory_metadata_and_payloads(tmp_path, alignment, version):
    rng = np.random.default_rng(alignment + version)
    a = random_blocks(KIND_Q4_K, 6, 512, rng)
    b = random_blocks(KIND_Q6_K, 3, 256, rng)
    c = random_blocks(KIND_Q8_0, 5, 96, rng)
    v = rng.normal(0, 1, 7).astype(np.float32)
    path = tmp_path / "m.gguf"
    write_gguf(path, {"general.architecture": "llama", "llama.block_count": 22, "llama.rope.freq_base": 500000.0,
                      "flag": True, "tokenizer.ggml.tokens": ["a", "bc", "def"],
                      "tokenizer.ggml.token_type": np.arange(5, dtype=np.int32)},
               [("a.weight", GGML_Q4_K, (512, 6), a), ("b.weight", GGML_Q6_K, (256, 3), b),
                ("c.weight", GGML_Q8_0, (96, 5), c), ("v.weight", GGML_F32, (7,), v)], alignment=alignment, version=version)
    with GgufFile(path) as f:
        assert len(f) == 4
        assert f.meta_str("general.architecture") == "llama" and f.meta_int("llama.block_count") == 22
        assert f.meta_float("llama.rope.freq_base") == 500000.0 and f.meta_int("flag") == 1
        assert f.meta_int("tokenizer.ggml.tokens") == 3 and f.meta_int("tokenizer.ggml.token_type") == 5  # array lengths
        assert f.meta_int("general.alignment") == alignment
        assert f.meta_int("missing", default=-1) == -1 and f.meta_float("llama.block_count") == 22.0
        with pytest.raises(KeyError):
            f.meta_str("llama.block_count")  # not a string
        for name, kind, dims, want in (("a.weight", KIND_Q4_K, (512, 6), a), ("b.weight", KIND_Q6_K, (256, 3), b),
                                       ("c.weight", KIND_Q8_0, (96, 5), c)):
            i = f.find(name)
            info = f.info(i)
            assert info["kind"] == kind and info["dims"] == dims and info["nbytes"] == want.size
            assert info["data"] % alignment == 0
            assert np.array_equal(f.tensor_bytes(i), want)
        i = f.find("v.weight")
        assert f.info(i)["kind"] == -1 and np.array_equal(f.tensor_bytes(i).view(np.float32), v)
        assert f.find("nope") == -1


def test_malformed_files_are_refused(tmp_path):
    good = tmp_path / "g.gguf"
    write_gguf(good, {"general.architecture": "llama"}, [("a.weight", GGML_F32, (4,), np.ones(4, dtype=np.float32))])
    raw = good.read_bytes()
    cases = {"magic": b"GGML" + raw[4:], "version": raw[:4] + struct.pack("<I", 1) + raw[8:], "truncated": raw[:-24],
             "tiny": raw[:10], "counts": raw[:8] + struct.pack("<Q", 1 << 40) + raw[16:]}
    for name, data in cases.items():
        p = tmp_path / f"{name}.gguf"
        p.write_bytes(data)
        with pytest.raises(MarmotCudaError):
            GgufFile(p)
    with pytest.raises(MarmotCudaError):
        GgufFile(tmp_path / "absent.gguf")


def test_crafted_directories_are_refused(tmp_path):
    """Sizes in the tensor directory come from the file: products that wrap, rows that are not whole blocks and
    odd alignments must be refused at open, before any row range is computed from them."""
    blocks = random_blocks(KIND_Q4_K, 1, 256, np.random.default_rng(0))
    cases = {
        "wrapping_dims": dict(tensors=[("a.weight", GGML_Q4_K, (256, (1 << 56) + 1), blocks)]),
        "huge_dims": dict(tensors=[("a.weight", GGML_Q4_K, (256, 1 << 50), blocks)]),
        "partial_block_rows": dict(tensors=[("a.weight", GGML_Q4_K, (128, 2), blocks)]),
        "odd_alignment": dict(tensors=[("a.weight", GGML_Q4_K, (256, 1), blocks)], alignment=48),
        "huge_alignment": dict(tensors=[("a.weight", GGML_Q4_K, (256, 1), blocks)], alignment=1 << 30),
    }
    for name, kw in cases.items():
        p = tmp_path / f"{name}.gguf"
        meta = {"general.architecture": "llama"}
        if name == "huge_alignment":  # written with a sane layout, the metadata value alone is absurd
            meta["general.alignment"] = kw.pop("alignment")
        write_gguf(p, meta, **kw)
        with pytest.raises(MarmotCudaError):
            GgufFile(p)
    # an array whose byte length wraps
    good = tmp_path / "arr.gguf"
    write_gguf(good, {"general.architecture": "llama", "arr": np.arange(4, dtype=np.int32)},
               [("a.weight", GGML_Q4_K, (256, 1), blocks)])
    raw = bytearray(good.read_bytes())
    at = raw.find(b"arr") + 3 + 4 + 4  # key, value type (array), element type
    raw[at:at + 8] = struct.pack("<Q", (1 << 62) + 1)
    bad = tmp_path / "arr_bad.gguf"
    bad.write_bytes(bytes(raw))
    with pytest.raises(MarmotCudaError):
        GgufFile(bad)


def test_unsupported_architectures_are_refused(tmp_path):
    """A qwen2 / phi3 file has the same tensor names but another layer (half-split RoPE pairs, attention biases, q/k
    norm); decoding it with the Llama layer would give wrong logits without any error, so the loader refuses it."""
    from marmot_b200.gguf import decoder_shape_from_gguf

    emb = random_blocks(KIND_Q4_K, 8, 256, np.random.default_rng(1))
    for arch, ok in (("llama", True), ("mistral", True), ("qwen2", False), ("phi3", False), ("gemma", False), ("qwen3", False)):
        p = tmp_path / f"{arch}.gguf"
        write_gguf(p, {"general.architecture": arch, f"{arch}.block_count": 2, f"{arch}.embedding_length": 256,
                       f"{arch}.feed_forward_length": 512, f"{arch}.attention.head_count": 4,
                       f"{arch}.attention.head_count_kv": 2}, [("token_embd.weight", GGML_Q4_K, (256, 8), emb)])
        with GgufFile(p) as f:
            if ok:
                shape = decoder_shape_from_gguf(f)
                assert (shape.layers, shape.d, shape.ffn, shape.n_heads, shape.n_kv_heads, shape.head_dim, shape.vocab) == \
                    (2, 256, 512, 4, 2, 64, 8)
            else:
                with pytest.raises(MarmotCudaError, match=arch):
                    decoder_shape_from_gguf(f)
