"""The decoder step of marmot_b200.decoder.Decoder restated on the CPU oracle (tests only)."""
from __future__ import annotations

import numpy as np

from marmot_b200.decoder import LAYER_WEIGHTS, DecoderShape
from marmot_b200.runtime import KIND_Q4_K, KIND_Q6_K

DEFAULT_KINDS = {n: k for n, k, _, _ in LAYER_WEIGHTS}


def oracle_step(oracle, shape: DecoderShape, weights: dict, ids, meta, positions, kv_k, kv_v, block_table,
                block_size: int, capture: list | None = None, kinds: dict | None = None, last_only: bool = False,
                perturb: float = 0.0):
    """The same step on the CPU oracle: returns logits; kv_k / kv_v are updated in place.

    `capture`, when a list, receives one dict per layer with every intermediate of the layer (the input of each
    operator and its output), so that a test can hand the oracle's input of a stage to the GPU operator and compare
    the outputs of that stage alone.  `last_only` computes the logits of the last token only.  `perturb` scales every
    element of the embedded tokens by 1 +- perturb (seeded signs): the oracle against its own perturbed run shows how
    far a rounding-level difference travels through the re-quantised activations of the following matmuls."""
    s = shape
    T = len(ids)
    hq, hkv, hd = s.n_heads, s.n_kv_heads, s.head_dim
    kind = lambda name: (kinds or {}).get(name, DEFAULT_KINDS.get(name.split(".")[-1], KIND_Q4_K))
    x = oracle.embedding_gather((kinds or {}).get("tok_embd", KIND_Q4_K), weights["tok_embd"], s.d, ids)
    if perturb:
        signs = np.random.default_rng(12345).choice(np.array([-1.0, 1.0], dtype=np.float32), size=x.shape)
        x = (x * (np.float32(1.0) + np.float32(perturb) * signs)).astype(np.float32)
    pos = np.asarray(positions, dtype=np.int32)
    for i in range(s.layers):
        w = lambda n: weights[f"l{i}.{n}"]
        st = {"x_in": x}
        h = oracle.rmsnorm(x, w("attn_norm"), s.rms_eps)
        q = oracle.linear(kind(f"l{i}.wq"), h, w("wq"), hq * hd)
        k = oracle.linear(kind(f"l{i}.wk"), h, w("wk"), hkv * hd)
        v = oracle.linear(kind(f"l{i}.wv"), h, w("wv"), hkv * hd)
        st.update(h=h, q=q, k=k, v=v)
        q = oracle.rope(q.reshape(T * hq, hd), np.repeat(pos, hq), s.rope_theta).reshape(T, hq, hd)
        k = oracle.rope(k.reshape(T * hkv, hd), np.repeat(pos, hkv), s.rope_theta).reshape(T, hkv, hd)
        st.update(q_rope=q.reshape(T, hq * hd), k_rope=k.reshape(T, hkv * hd))
        att = oracle.paged_attention(meta, q, k, v.reshape(T, hkv, hd), kv_k, kv_v, block_table, i, block_size,
                                     float(hd) ** -0.5).reshape(T, hq * hd)
        proj = oracle.linear(kind(f"l{i}.wo"), att, w("wo"), s.d)
        x = x + proj
        h2 = oracle.rmsnorm(x, w("ffn_norm"), s.rms_eps)
        gate = oracle.linear(kind(f"l{i}.gate"), h2, w("gate"), s.ffn)
        up = oracle.linear(kind(f"l{i}.up"), h2, w("up"), s.ffn)
        g = oracle.swiglu(gate, up)
        down = oracle.linear(kind(f"l{i}.down"), g, w("down"), s.d)
        st.update(att=att, proj=proj, x_mid=x, h2=h2, gate=gate, up=up, glu=g, down=down)
        x = x + down
        st["x_out"] = x
        if capture is not None:
            capture.append(st)
    if last_only:
        x = x[-1:]
    h = oracle.rmsnorm(x, weights["out_norm"], s.rms_eps)
    return oracle.linear((kinds or {}).get("output", KIND_Q6_K), h, weights["output"], s.vocab)
