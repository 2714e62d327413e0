"""The decoder step of marmot_b200.decoder.Decoder restated on the CPU oracle (tests only)."""
from __future__ import annotations

import numpy as np

from marmot_b200.decoder import DecoderShape
from marmot_b200.runtime import KIND_Q4_K, KIND_Q6_K


def oracle_step(oracle, shape: DecoderShape, weights: dict, ids, meta, positions, kv_k, kv_v, block_table,
                block_size: int):
    """The same step on the CPU oracle (tests only): returns logits; kv_k / kv_v are updated in place."""
    s = shape
    T = len(ids)
    hq, hkv, hd = s.n_heads, s.n_kv_heads, s.head_dim
    x = oracle.embedding_gather(KIND_Q4_K, weights["tok_embd"], s.d, ids)
    pos = np.asarray(positions, dtype=np.int32)
    for i in range(s.layers):
        w = lambda n: weights[f"l{i}.{n}"]
        h = oracle.rmsnorm(x, w("attn_norm"), s.rms_eps)
        q = oracle.linear(KIND_Q4_K, h, w("wq"), hq * hd)
        k = oracle.linear(KIND_Q4_K, h, w("wk"), hkv * hd)
        v = oracle.linear(KIND_Q6_K, h, w("wv"), hkv * hd)
        q = oracle.rope(q.reshape(T * hq, hd), np.repeat(pos, hq), s.rope_theta).reshape(T, hq, hd)
        k = oracle.rope(k.reshape(T * hkv, hd), np.repeat(pos, hkv), s.rope_theta).reshape(T, hkv, hd)
        att = oracle.paged_attention(meta, q, k, v.reshape(T, hkv, hd), kv_k, kv_v, block_table, i, block_size,
                                     float(hd) ** -0.5).reshape(T, hq * hd)
        x = x + oracle.linear(KIND_Q4_K, att, w("wo"), s.d)
        h = oracle.rmsnorm(x, w("ffn_norm"), s.rms_eps)
        g = oracle.swiglu(oracle.linear(KIND_Q4_K, h, w("gate"), s.ffn), oracle.linear(KIND_Q4_K, h, w("up"), s.ffn))
        x = x + oracle.linear(KIND_Q6_K, g, w("down"), s.d)
    h = oracle.rmsnorm(x, weights["out_norm"], s.rms_eps)
    return oracle.linear(KIND_Q6_K, h, weights["output"], s.vocab)
