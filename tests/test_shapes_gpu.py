"""Parity at the shapes the benchmark configurations name, against the CPU oracle:

* the TinyLlama-1.1B shape as a whole model (22 layers, d = 2048, FFN 5632, 32 query / 4 KV heads of 64, vocabulary
  32000, Q4_K_M mix, f16 paged KV, block 16): a 128-token prompt prefilled in one call, then greedy decode steps;
* a four-layer slice of the Llama-3-8B shape (d = 4096, FFN 14336, 32 / 8 heads of 128, theta 5e5) decoding 64
  sequences with ragged contexts in one step, every operator of every layer also checked on its own with the
  oracle's input of that stage;
* the Mixtral-8x7B-shape expert FFN (8 experts, top-2, d = 4096, FFN 14336, Q4_K) on 256 tokens (grouped launches)
  and on 3 tokens (per-expert decode launches), stage by stage and end to end, both router weight policies.

Weights are random-init N(0, 0.02) quantised into blocks (marmot_b200.synthetic.quantize_rows); the same bytes go to
the GPU and to the oracle.  Each test prints the errors it measured (run with -s to see them).  Every operator is
held to the path's stated tolerance with the oracle's own input of that stage: 2e-3 for the integer-dot kernels, 1e-2
for the tensor-core kernels.

Whole-model logits are a different matter.  Every matmul re-quantises its input to 8 bits, and a rounding-level
difference in that input flips a few quantised values by one step (1/127 of a block's largest value): a relative
difference d becomes about sqrt(0.025 * d) after the next matmul, so ANY difference - a different summation order
is enough - reaches the quantisation noise floor of about 1e-2 within five matmuls, whatever its size at the start,
and then accumulates slowly with depth.  The tests therefore run the oracle a second time with its embedded tokens
perturbed by one part in a million and hold the GPU to that yardstick: its logits must be as close to the oracle's as
the oracle's own perturbed run is (minus a small margin), and at least 0.999 where the yardstick itself is.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from marmot_b200 import Context
from marmot_b200.decoder import LAYER_WEIGHTS, TINYLLAMA_1B, Decoder, DecoderShape
from marmot_b200.runtime import KIND_Q4_K, KIND_Q6_K
from marmot_b200.synthetic import normal_blocks
from tests.decoder_ref import oracle_step
from tests.util import TOL_FP32, TOL_MMA, TOL_MOE, cosine, max_rel_err

pytestmark = pytest.mark.gpu

SIGMA = 0.02


def model_weights(shape: DecoderShape, seed: int) -> dict:
    """Host byte arrays of a whole random-init model in the Q4_K_M mix; norm weights are ones."""
    gen = torch.Generator().manual_seed(seed)
    w = {}
    for i in range(shape.layers):
        for name, kind, rows, cols in LAYER_WEIGHTS:
            w[f"l{i}.{name}"] = normal_blocks(torch, kind, rows(shape), cols(shape), "cpu", gen, SIGMA).numpy()
        w[f"l{i}.attn_norm"] = np.ones(shape.d, dtype=np.float32)
        w[f"l{i}.ffn_norm"] = np.ones(shape.d, dtype=np.float32)
    w["tok_embd"] = normal_blocks(torch, KIND_Q4_K, shape.vocab, shape.d, "cpu", gen, SIGMA).numpy()
    w["output"] = normal_blocks(torch, KIND_Q6_K, shape.vocab, shape.d, "cpu", gen, SIGMA).numpy()
    w["out_norm"] = np.ones(shape.d, dtype=np.float32)
    return w


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def check_layer_stages(ctx, dec: Decoder, layer: int, st: dict, meta, pos, pool_k, pool_v, tol_linear: float, report: dict):
    """Every operator of one layer on the GPU with the oracle's input of that stage; `pool_k` / `pool_v` are device
    copies of the KV pool as it was before the step.  Worst error per operator kind goes to `report`."""
    s, kd, lw = dec.local, dec.kinds, dec.layers[layer]
    hq, hkv, hd = s.n_heads, s.n_kv_heads, s.head_dim
    T = st["x_in"].shape[0]

    def note(name, got, want, tol):
        err = max_rel_err(got.cpu().numpy(), want)
        report[name] = max(report.get(name, 0.0), err)
        assert err <= tol, (layer, name, err, tol)

    note("rmsnorm", ctx.rmsnorm(dev(st["x_in"]), lw["attn_norm"], s.rms_eps), st["h"], 1e-5)
    h = dev(st["h"])
    note("wq", ctx.linear(kd[f"l{layer}.wq"], h, lw["wq"], hq * hd), st["q"], tol_linear)
    note("wk", ctx.linear(kd[f"l{layer}.wk"], h, lw["wk"], hkv * hd), st["k"], tol_linear)
    note("wv", ctx.linear(kd[f"l{layer}.wv"], h, lw["wv"], hkv * hd), st["v"], tol_linear)
    q, k = dev(st["q"]), dev(st["k"])
    ctx.rope_qk(q, k, pos, hq, hkv, hd, s.rope_theta)
    note("rope_q", q, st["q_rope"], 2e-5)
    note("rope_k", k, st["k_rope"], 2e-5)
    att = ctx.paged_attention(meta, dev(st["q_rope"]), dev(st["k_rope"]), dev(st["v"]), pool_k, pool_v, dec.block_table,
                              layer, hq, hkv, hd, dec.block_size, float(hd) ** -0.5)
    note("attention", att, st["att"], 1e-4)
    note("wo", ctx.linear(kd[f"l{layer}.wo"], dev(st["att"]), lw["wo"], s.d), st["proj"], tol_linear)
    x_mid, h2 = torch.empty((T, s.d), device="cuda"), torch.empty((T, s.d), device="cuda")
    ctx.add_rmsnorm(dev(st["x_in"]), dev(st["proj"]), lw["ffn_norm"], s.rms_eps, x_mid, h2)
    note("add_rmsnorm_x", x_mid, st["x_mid"], 1e-6)
    note("add_rmsnorm_h", h2, st["h2"], 1e-5)
    gate, up = torch.empty((T, s.ffn), device="cuda"), torch.empty((T, s.ffn), device="cuda")
    ctx.linear_dual(kd[f"l{layer}.gate"], dev(st["h2"]), lw["gate"], lw["up"], s.ffn, out_a=gate, out_b=up)
    note("gate", gate, st["gate"], tol_linear)
    note("up", up, st["up"], tol_linear)
    note("swiglu", ctx.swiglu(dev(st["gate"]), dev(st["up"])), st["glu"], 1e-5)
    note("down", ctx.linear(kd[f"l{layer}.down"], dev(st["glu"]), lw["down"], s.d), st["down"], tol_linear)


def test_tinyllama_shape_prefill_then_greedy_decode(oracle):
    shape = TINYLLAMA_1B
    n_prompt, n_decode = 128, 16
    weights = model_weights(shape, 11)
    ctx = Context(0)
    try:
        dec = Decoder(ctx, shape, max_seqs=1, max_ctx=n_prompt + n_decode + 16, block_size=16, kv_dtype=torch.float16,
                      weights=weights)
        kv_k = np.zeros(tuple(dec.kv_k.shape), dtype=np.float16)
        kv_v = np.zeros_like(kv_k)
        table = dec.block_table.cpu().numpy()
        rng = np.random.default_rng(3)
        ids = rng.integers(0, shape.vocab, n_prompt).astype(np.int32)
        pos = np.arange(n_prompt, dtype=np.int32)
        cosines, errors, agree, first_miss = [], [], 0, None
        report = {}
        # the yardstick: the oracle's prefill against itself with the embedded tokens perturbed by 1e-6
        yk, yv = np.zeros_like(kv_k), np.zeros_like(kv_v)
        yard = oracle_step(oracle, shape, weights, ids, dec.token_meta([0] * n_prompt, pos), pos, yk, yv, table, 16,
                           last_only=True, perturb=1e-6)
        del yk, yv
        for step in range(1 + n_decode):
            meta = dec.token_meta([0] * len(ids), pos)
            if step == 1:  # the first decode step also operator by operator, on two layers (GEMV regime)
                kv0_k, kv0_v = dev(kv_k), dev(kv_v)
                cap = []
            else:
                cap = None
            got = dec.step(dev(ids), dev(meta), dev(pos), decode=step > 0)[-1:].cpu().numpy()
            want = oracle_step(oracle, shape, weights, ids, meta, pos, kv_k, kv_v, table, 16, capture=cap, last_only=True)
            if cap is not None:
                for layer in (0, shape.layers - 1):
                    check_layer_stages(ctx, dec, layer, cap[layer], dev(meta), dev(pos), kv0_k, kv0_v, TOL_FP32, report)
                del kv0_k, kv0_v, cap
            cosines.append(cosine(got, want))
            errors.append(max_rel_err(got, want))
            if step == 0:
                first_want = want
            if step > 0:
                same = int(np.argmax(got[0])) == int(np.argmax(want[0]))
                agree += same
                if not same and first_miss is None:
                    first_miss = step - 1
            # both sides continue from the oracle's token: one flipped near-tie cannot derail the comparison, and up
            # to the first disagreement this is exactly the free-running greedy sequence of both
            nxt = int(np.argmax(want[0]))
            ids = np.array([nxt], dtype=np.int32)
            pos = np.array([pos[-1] + 1], dtype=np.int32)
        yard_cos = cosine(yard, first_want)
        print(f"\nTinyLlama shape: prefill logit cosine {cosines[0]:.6f} (max rel err {errors[0]:.2e}); decode cosine min "
              f"{min(cosines[1:]):.6f}, max rel err {max(errors[1:]):.2e}; oracle against its own 1e-6-perturbed run: "
              f"{yard_cos:.6f}; greedy tokens agreeing {agree}/{n_decode} (first difference at step {first_miss}); "
              "per-operator worst errors at decode: " + ", ".join(f"{k} {v:.1e}" for k, v in report.items()))
        assert min(cosines) >= min(0.999, yard_cos - 1e-3), (cosines, yard_cos)
        assert agree >= n_decode // 2, (agree, first_miss)
    finally:
        ctx.close()


def test_llama3_8b_shape_layer_slice_batched_decode(oracle):
    shape = DecoderShape(layers=4, d=4096, ffn=14336, n_heads=32, n_kv_heads=8, head_dim=128, vocab=16384,
                         rope_theta=500000.0)
    n_seq, max_ctx = 64, 640
    weights = model_weights(shape, 12)
    rng = np.random.default_rng(4)
    ctx = Context(0)
    try:
        dec = Decoder(ctx, shape, max_seqs=n_seq, max_ctx=max_ctx, block_size=16, kv_dtype=torch.float16, weights=weights)
        # contexts already in the pool: values of the size real K / V rows have (order one)
        kv_k = rng.standard_normal(tuple(dec.kv_k.shape), dtype=np.float32).astype(np.float16)
        kv_v = rng.standard_normal(tuple(dec.kv_v.shape), dtype=np.float32).astype(np.float16)
        dec.kv_k.copy_(torch.from_numpy(kv_k))
        dec.kv_v.copy_(torch.from_numpy(kv_v))
        pool0_k, pool0_v = dec.kv_k.clone(), dec.kv_v.clone()
        table = dec.block_table.cpu().numpy()
        ctx_len = rng.integers(64, 601, n_seq).astype(np.int32)
        ids = rng.integers(0, shape.vocab, n_seq).astype(np.int32)
        meta = dec.token_meta(np.arange(n_seq), ctx_len)
        got = dec.step(dev(ids), dev(meta), dev(ctx_len), decode=True).cpu().numpy()
        cap = []
        yk, yv = kv_k.copy(), kv_v.copy()
        want = oracle_step(oracle, shape, weights, ids, meta, ctx_len, kv_k, kv_v, table, 16, capture=cap)
        yard_cos = cosine(oracle_step(oracle, shape, weights, ids, meta, ctx_len, yk, yv, table, 16, perturb=1e-6), want)
        del yk, yv
        cos, err = cosine(got, want), max_rel_err(got, want)
        # the K / V rows the step appended: same f16 rounding on both sides, inputs differ by the matmul error
        # (layer 0 only: its inputs are identical on both sides; deeper layers inherit the noise described above)
        p0 = pool0_k[:, 0].cpu().numpy().astype(np.float32)
        new_k = dec.kv_k[:, 0].cpu().numpy().astype(np.float32) - p0
        ref_k = kv_k[:, 0].astype(np.float32) - p0
        err_pool = float(np.max(np.abs(new_k - ref_k)) / max(np.max(np.abs(ref_k)), 1e-30))
        report = {}
        for layer in range(shape.layers):  # (the attention stage appends into pool0 itself)
            check_layer_stages(ctx, dec, layer, cap[layer], dev(meta), dev(ctx_len), pool0_k, pool0_v, TOL_MMA, report)
        print(f"\nLlama-3-8B-shape slice, 64 sequences, contexts {ctx_len.min()}..{ctx_len.max()}: logit cosine {cos:.6f}, "
              f"max rel err {err:.2e} (oracle against its own 1e-6-perturbed run: {yard_cos:.6f}), K rows appended by "
              f"layer 0 {err_pool:.2e}; per-operator worst errors with the oracle's stage inputs: "
              + ", ".join(f"{k} {v:.1e}" for k, v in report.items()))
        assert cos >= min(0.999, yard_cos - 1e-3), (cos, yard_cos)
        assert err_pool <= TOL_MMA, err_pool
    finally:
        ctx.close()


def _silu_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    g = gate.astype(np.float32)
    return (g / (np.float32(1.0) + np.exp(-g, dtype=np.float32)) * up.astype(np.float32)).astype(np.float32)


@pytest.fixture(scope="module")
def mixtral_experts():
    """Gate / up / down of the 8 experts (792 MB of Q4_K blocks), drawn once for the module."""
    H, FF, E = 4096, 14336, 8
    gen = torch.Generator().manual_seed(21)
    return tuple(normal_blocks(torch, KIND_Q4_K, rows, K, "cpu", gen, SIGMA).numpy()
                 for rows, K in ((E * FF, H), (E * FF, H), (E * H, FF)))


@pytest.mark.parametrize("T,policy", [(256, 2), (256, 0), (3, 2), (3, 0)])
def test_mixtral_shape_expert_ffn(oracle, mixtral_experts, T, policy):
    H, FF, E, k = 4096, 14336, 8, 2
    gate, up, down = mixtral_experts
    rng = np.random.default_rng(100 + T)
    hidden = rng.normal(0, 1, (T, H)).astype(np.float32)
    logits = rng.normal(0, 1, (T, E)).astype(np.float32)
    probs = np.exp(logits - logits.max(axis=1, keepdims=True))
    probs = (probs / probs.sum(axis=1, keepdims=True)).astype(np.float32)
    kinds = (KIND_Q4_K,) * 3
    ctx = Context(0)
    try:
        vals, ids = ctx.topk(dev(probs), k)
        ref_vals, ref_ids = oracle.topk(probs, k)
        assert np.array_equal(ids.cpu().numpy(), ref_ids) and np.array_equal(vals.cpu().numpy(), ref_vals)
        g_dev, u_dev, d_dev = ctx.upload(gate), ctx.upload(up), ctx.upload(down)
        got = ctx.moe_experts(kinds, dev(hidden), g_dev, u_dev, d_dev, ids, vals, FF, E, policy=policy)
        got = got.cpu().numpy()
        want = oracle.moe_experts(kinds, hidden, gate, up, down, ref_ids, ref_vals, FF, E, policy=policy)
        cos, err = cosine(got, want), max_rel_err(got, want)
        bufs = ctx.moe_last_buffers(T, k, H, FF)
        grouped = bufs["grouped"]
        assert grouped == (T * k >= 256)
        # stage by stage, in sorted-route order: each GPU stage against the oracle applied to the GPU's own input of
        # that stage, so a stage's bound is not loosened by what came before it
        offsets = bufs["offsets"].cpu().numpy()
        sorted_tok = bufs["sorted_tok"].cpu().numpy()
        assert offsets[E] == T * k and np.all(np.diff(offsets) >= 0)
        flat_ids = ref_ids.reshape(-1)
        for e in range(E):  # the stable scatter: expert-major, route order inside an expert
            assert np.array_equal(sorted_tok[offsets[e]:offsets[e + 1]], np.nonzero(flat_ids == e)[0] // k)
        gate_out, up_out = bufs["gate_out"].cpu().numpy(), bufs["up_out"].cpu().numpy()
        route_down = bufs["route_down"].cpu().numpy()
        tol = TOL_MMA if grouped else TOL_FP32
        stage = {"gate": 0.0, "up": 0.0, "down": 0.0}
        gb, db = FF * (H // 256) * 144, H * (FF // 256) * 144
        for e in range(E):
            lo, hi = int(offsets[e]), int(offsets[e + 1])
            if hi == lo:
                continue
            rows = hidden[sorted_tok[lo:hi]]
            want_gate = oracle.linear(KIND_Q4_K, rows, gate[e * gb:(e + 1) * gb], FF)
            want_up = oracle.linear(KIND_Q4_K, rows, up[e * gb:(e + 1) * gb], FF)
            if grouped:  # gate_out is the plain projection, the GLU is applied by the down projection's prologue
                stage["gate"] = max(stage["gate"], max_rel_err(gate_out[lo:hi], want_gate))
                glu = _silu_mul(gate_out[lo:hi], up_out[lo:hi])
            else:        # gate_out already holds act(gate) * up
                stage["gate"] = max(stage["gate"], max_rel_err(gate_out[lo:hi], _silu_mul(want_gate, want_up)))
                glu = gate_out[lo:hi]
            stage["up"] = max(stage["up"], max_rel_err(up_out[lo:hi], want_up))
            want_down = oracle.linear(KIND_Q4_K, glu, down[e * db:(e + 1) * db], H)
            stage["down"] = max(stage["down"], max_rel_err(route_down[lo:hi], want_down))
        # the weighted combine from the GPU's own down rows, in route order
        w_sorted, route_pos = bufs["sorted_w"].cpu().numpy(), bufs["route_pos"].cpu().numpy().reshape(T, k)
        comb = np.zeros((T, H), dtype=np.float32)
        for t in range(T):
            for p in sorted(route_pos[t]):
                comb[t] = comb[t] + w_sorted[p] * route_down[p]
        stage["combine"] = max_rel_err(got, comb)
        print(f"\nMixtral-shape expert FFN, T={T}, policy={policy}, {'grouped' if grouped else 'per-expert'} launches: "
              f"end to end cosine {cos:.6f}, max rel err {err:.2e}; per stage " +
              ", ".join(f"{n} {v:.1e}" for n, v in stage.items()))
        for name in ("gate", "up", "down"):
            assert stage[name] <= tol, (name, stage[name])
        assert stage["combine"] <= 1e-6, stage["combine"]
        assert cos >= 0.999, cos
        # end to end the second matmul sees a re-quantised intermediate: a rounding flip there is 1/127 of a block's
        # largest value, so a first-stage difference d arrives as about sqrt(0.025 * d).  The root-mean-square
        # difference is held to the tensor-core tolerance, single elements to the reference's own bound between its
        # backends for this operator (tests/backend/test_backend_moe.c:901,1052).
        rms_rel = float(np.linalg.norm(got.astype(np.float64) - want) / np.linalg.norm(want.astype(np.float64)))
        print(f"  end to end relative rms difference {rms_rel:.2e}")
        assert rms_rel <= (TOL_MMA if grouped else TOL_FP32), rms_rel
        assert err <= TOL_MOE, err
    finally:
        ctx.close()
