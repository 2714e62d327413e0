"""A whole Llama-shape decoder step through the C ABI against the same op sequence on the CPU oracle: prefill of a
short prompt, then greedy decode steps that read the KV pool the earlier calls wrote."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from marmot_b200 import Context
from marmot_b200.decoder import LAYER_WEIGHTS, Decoder, DecoderShape
from marmot_b200.runtime import KIND_Q4_K, KIND_Q6_K
from tests.decoder_ref import oracle_step
from tests.util import TOL_FP32, TOL_MMA, cosine, max_rel_err, random_blocks

pytestmark = pytest.mark.gpu

SHAPE = DecoderShape(layers=2, d=256, ffn=512, n_heads=4, n_kv_heads=2, head_dim=64, vocab=512, rope_theta=10000.0)


def make_weights(rng, SHAPE=SHAPE, kinds=None):
    """Block scales small enough that activations stay of order one (weight std about 1/sqrt(K)), as in a trained
    model: with the default block-space scales the attention scores reach the thousands, the softmax saturates and a
    1e-3 perturbation of a score flips whole attention rows."""
    sig = 0.0003
    w = {}
    for i in range(SHAPE.layers):
        for name, kind, rows, cols in LAYER_WEIGHTS:
            kind = (kinds or {}).get(f"l{i}.{name}", kind)
            w[f"l{i}.{name}"] = random_blocks(kind, rows(SHAPE), cols(SHAPE), rng, d_sigma=sig)
        w[f"l{i}.attn_norm"] = rng.normal(1, 0.1, SHAPE.d).astype(np.float32)
        w[f"l{i}.ffn_norm"] = rng.normal(1, 0.1, SHAPE.d).astype(np.float32)
    w["tok_embd"] = random_blocks(KIND_Q4_K, SHAPE.vocab, SHAPE.d, rng, d_sigma=0.003)
    w["output"] = random_blocks(KIND_Q6_K, SHAPE.vocab, SHAPE.d, rng, d_sigma=sig)
    w["out_norm"] = rng.normal(1, 0.1, SHAPE.d).astype(np.float32)
    return w


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("prompt_len,kv_dtype", [(5, torch.float32), (5, torch.float16), (12, torch.float16)])
def test_prefill_then_greedy_decode(oracle, prompt_len, kv_dtype, fused):
    """fused: the decode steps run as Decoder.step(decode=True): one persistent kernel per one-token step on a float16
    pool (five launches per layer otherwise)."""
    rng = np.random.default_rng(prompt_len)
    weights = make_weights(rng)
    ctx = Context(0)
    dec = Decoder(ctx, SHAPE, max_seqs=2, max_ctx=64, block_size=16, kv_dtype=kv_dtype, weights=weights)
    np_kv = np.float16 if kv_dtype == torch.float16 else np.float32
    kv_k = np.zeros(tuple(dec.kv_k.shape), dtype=np_kv)
    kv_v = np.zeros_like(kv_k)
    table = dec.block_table.cpu().numpy()
    seq = 1  # not the first sequence slot: the block table matters
    ids = rng.integers(0, SHAPE.vocab, prompt_len).astype(np.int32)
    pos = np.arange(prompt_len, dtype=np.int32)
    # several matmuls in sequence, each re-quantising its input: the tensor-core prefill (1e-3 per matmul) compounds
    # the model-level bar for that path is the logit cosine; the element-wise bound below is a sanity limit
    tol = TOL_FP32 * 5 if prompt_len <= 8 else 0.25
    for step in range(4):
        meta = dec.token_meta([seq] * len(ids), pos)
        l0 = ctx.launch_count()
        got = dec.step(torch.from_numpy(ids).cuda(), torch.from_numpy(meta).cuda(), torch.from_numpy(pos).cuda(),
                       decode=fused and step > 0)
        if fused and step > 0 and kv_dtype == torch.float16:
            assert ctx.launch_count() - l0 == 3  # embedding gather, RoPE table, the persistent step kernel
        got = got.cpu().numpy()
        want = oracle_step(oracle, SHAPE, weights, ids, meta, pos, kv_k, kv_v, table, 16)
        assert cosine(got, want) >= 0.999, (step, cosine(got, want))
        assert max_rel_err(got, want) <= tol, (step, max_rel_err(got, want))
        nxt = int(np.argmax(want[-1]))
        assert int(ctx.argmax(torch.from_numpy(got[-1:]).cuda()).item()) == int(np.argmax(got[-1]))
        # both sides continue from the oracle's token so that one flipped near-tie cannot derail the comparison
        ids = np.array([nxt], dtype=np.int32)
        pos = np.array([pos[-1] + 1], dtype=np.int32)  # (after a tensor-core prefill the pool carries its rounding)
    # the pools agree after the run (f16: same rounding; small differences come from the matmuls feeding K and V)
    ref_k = kv_k.astype(np.float32)
    err_k = float(np.max(np.abs(dec.kv_k.cpu().numpy().astype(np.float32) - ref_k)) / np.max(np.abs(ref_k)))
    assert err_k <= (5e-3 if prompt_len <= 8 else 0.1), err_k
    ctx.close()


def test_decode_with_pool_managed_cache_equals_static_cache():
    """Two sequences prefill and decode in turns; one decoder keeps the static one-range-per-sequence cache, the other
    takes blocks, table and kv slots from a KvPool in which the two sequences' blocks interleave.  Same logits, bit
    for bit: only where the K/V rows live differs."""
    from marmot_b200.runtime import KvPool

    rng = np.random.default_rng(77)
    weights = make_weights(rng)
    ctx = Context(0)
    pool = KvPool(ctx, max_seqs=2, max_seq_len=64, block_size=16, num_blocks=8, num_layers=SHAPE.layers,
                  num_kv_heads=SHAPE.n_kv_heads, head_dim=SHAPE.head_dim)
    try:
        static = Decoder(ctx, SHAPE, max_seqs=2, max_ctx=64, weights=weights)
        pooled = Decoder(ctx, SHAPE, max_seqs=2, max_ctx=64, weights=weights, kv_pool=pool)
        seqs = [pool.acquire_seq()[1], pool.acquire_seq()[1]]
        lengths = [0, 0]
        for which, n in [(0, 9), (1, 20), (0, 1), (1, 1), (0, 12), (1, 1), (0, 1)]:
            ids = torch.from_numpy(rng.integers(0, SHAPE.vocab, n).astype(np.int32)).cuda()
            pos_np = np.arange(lengths[which], lengths[which] + n, dtype=np.int32)
            pos = torch.from_numpy(pos_np).cuda()
            rc, plan, slots, start = pool.prepare_append(seqs[which], n)
            assert rc == 0 and start == lengths[which]
            want = static.step(ids, torch.from_numpy(static.token_meta([which] * n, pos_np)).cuda(), pos).clone()
            got = pooled.step(ids, torch.from_numpy(pooled.token_meta([seqs[which]] * n, pos_np, kv_slots=slots)).cuda(), pos)
            assert torch.equal(got, want), (which, n)
            assert pool.commit_append(plan) == 0
            lengths[which] += n
        assert pool.block_id(seqs[0], 1) != pool.block_id(seqs[0], 0) + 1  # the blocks did interleave
    finally:
        pool.close()
        ctx.close()


@pytest.mark.parametrize("tie_output", [False, True])
def test_decoder_loaded_from_gguf_equals_direct_weights(tmp_path, tie_output):
    """A synthetic Llama-family GGUF file (Q4_K_M-like mix: attn_v and ffn_down alternate between Q6_K and Q4_K by
    layer) loaded through the library's reader gives the very logits of the same weights handed over as arrays."""
    from marmot_b200.gguf import load_llama_decoder
    from tests.gguf_writer import write_llama

    rng = np.random.default_rng(5)
    kinds = {"l1.wv": KIND_Q4_K, "l1.down": KIND_Q4_K, "l0.wq": KIND_Q6_K}
    if tie_output:
        kinds["output"] = KIND_Q4_K  # the embedding table doubles as the output projection
    weights = make_weights(rng)
    for name, kind in kinds.items():
        if name == "output":
            continue
        _, _, rows, cols = next(w for w in LAYER_WEIGHTS if w[0] == name.split(".")[1])
        weights[name] = random_blocks(kind, rows(SHAPE), cols(SHAPE), rng, d_sigma=0.0003)
    if tie_output:
        weights["output"] = weights["tok_embd"]
    path = tmp_path / "llama.gguf"
    write_llama(path, SHAPE, weights, kinds, tie_output=tie_output)
    ctx = Context(0)
    try:
        direct = Decoder(ctx, SHAPE, max_seqs=2, max_ctx=64, weights=weights, kinds=kinds)
        loaded = load_llama_decoder(str(path), ctx, max_seqs=2, max_ctx=64)
        import dataclasses

        got_shape, want_shape = dataclasses.asdict(loaded.shape), dataclasses.asdict(SHAPE)
        for key in ("rope_theta", "rms_eps"):  # stored as f32 in the file
            assert np.float32(got_shape.pop(key)) == np.float32(want_shape.pop(key))
        assert got_shape == want_shape
        assert loaded.kinds["l1.wv"] == KIND_Q4_K and loaded.kinds["l0.wv"] == KIND_Q6_K
        for n, start in ((7, 0), (1, 7), (12, 8)):
            ids = torch.from_numpy(rng.integers(0, SHAPE.vocab, n).astype(np.int32)).cuda()
            pos_np = np.arange(start, start + n, dtype=np.int32)
            meta = torch.from_numpy(direct.token_meta([1] * n, pos_np)).cuda()
            pos = torch.from_numpy(pos_np).cuda()
            assert torch.equal(loaded.step(ids, meta, pos), direct.step(ids, meta, pos))
    finally:
        ctx.close()


@pytest.mark.parametrize("prompt_len", [3, 40])
def test_one_token_step_kernel_matches_the_five_launch_layer(monkeypatch, prompt_len):
    """Decoder.step(decode=True) for one token runs ONE persistent kernel (mcu_decode_plan); with the diagnostic switch it
    runs five launches per layer.  Same weights, same prompt: the matmuls share their device functions, the attention is
    f32 in one and split-f16 MMAs in the other, so logits agree to rounding, the greedy tokens are the same, and the
    K/V rows both wrote into their pools agree (bit for bit in the first layer).  Contexts inside one 32-position tile and across two; also replayed
    from a CUDA graph."""
    rng = np.random.default_rng(prompt_len)
    weights = make_weights(rng)
    ctx = Context(0)
    try:
        decs = [Decoder(ctx, SHAPE, max_seqs=2, max_ctx=64, block_size=16, kv_dtype=torch.float16, weights=weights) for _ in range(2)]
        ids = torch.from_numpy(rng.integers(0, SHAPE.vocab, prompt_len).astype(np.int32)).cuda()
        pos_np = np.arange(prompt_len, dtype=np.int32)
        for d in decs:
            d.step(ids, torch.from_numpy(d.token_meta([1] * prompt_len, pos_np)).cuda(), torch.from_numpy(pos_np).cuda())
        tok = torch.tensor([7], dtype=torch.int32, device="cuda")
        for step in range(8):
            p = np.array([prompt_len + step], dtype=np.int32)
            meta, pos = torch.from_numpy(decs[0].token_meta([1], p)).cuda(), torch.from_numpy(p).cuda()
            l0 = ctx.launch_count()
            got = decs[0].step(tok, meta, pos, decode=True).clone()
            assert ctx.launch_count() - l0 == 3
            monkeypatch.setenv("MARMOT_DECODER_NO_STEP_KERNEL", "1")
            want = decs[1].step(tok, meta, pos, decode=True).clone()
            monkeypatch.delenv("MARMOT_DECODER_NO_STEP_KERNEL")
            ctx.synchronize()
            assert max_rel_err(got.cpu().numpy(), want.cpu().numpy()) <= 1e-4, step
            assert int(got.argmax()) == int(want.argmax())
            tok = want.argmax(dim=1).to(torch.int32)
        # layer 0's rows come from identical arithmetic; deeper layers inherit the attention's last-place differences,
        # which an f16 rounding can turn into one unit in the last place
        for a, b in ((decs[0].kv_k, decs[1].kv_k), (decs[0].kv_v, decs[1].kv_v)):
            assert torch.equal(a[:, 0], b[:, 0])
            assert float((a.float() - b.float()).abs().max()) <= 2e-3 * float(b.float().abs().max())
        # the same plan from a CUDA graph: fixed tensors, new contents
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        ctx.set_stream(stream.cuda_stream)
        p = np.array([prompt_len + 8], dtype=np.int32)
        meta, pos = torch.from_numpy(decs[0].token_meta([1], p)).cuda(), torch.from_numpy(p).cuda()
        logits = torch.empty((1, SHAPE.vocab), dtype=torch.float32, device="cuda")
        with torch.cuda.stream(stream):
            decs[0].step(tok, meta, pos, logits_out=logits, decode=True)  # builds the plan for these tensors
            torch.cuda.synchronize()
            eager = logits.clone()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                decs[0].step(tok, meta, pos, logits_out=logits, decode=True)
            logits.zero_()
            g.replay()
            torch.cuda.synchronize()
            assert torch.equal(logits, eager)  # same position, same pool rows rewritten with the same values
        ctx.synchronize()
        ctx.set_stream(0)
    finally:
        ctx.close()


@pytest.mark.parametrize("shape,ctx_len", [
    # head_dim 128, four query heads on one KV head, FFN of six blocks
    (DecoderShape(layers=2, d=512, ffn=1536, n_heads=4, n_kv_heads=1, head_dim=128, vocab=512, rope_theta=500000.0), 70),
    # the row lengths of an 8B model: 16 blocks of hidden size (more blocks than consumer warps), 32 / 8 heads of 128
    (DecoderShape(layers=1, d=4096, ffn=4352, n_heads=32, n_kv_heads=8, head_dim=128, vocab=256, rope_theta=500000.0), 33),
    # eight query heads per KV head at head_dim 64, a context of more tiles than attention warps (16 > 15)
    (DecoderShape(layers=1, d=512, ffn=768, n_heads=8, n_kv_heads=1, head_dim=64, vocab=256, rope_theta=10000.0), 500),
    # other block formats per tensor: an up projection in Q6_K (gate and up as two jobs, SwiGLU as down's prologue),
    # down in Q4_K with rows of three blocks, v in Q4_K
    (DecoderShape(layers=2, d=256, ffn=768, n_heads=4, n_kv_heads=2, head_dim=64, vocab=512, rope_theta=10000.0), 21),
])
def test_one_token_step_kernel_on_other_shapes(monkeypatch, shape, ctx_len):
    """The persistent decode-step kernel against the five-launch layer on shapes that take its other code paths."""
    rng = np.random.default_rng(shape.d + ctx_len)
    kinds = {"l0.up": KIND_Q6_K, "l1.down": KIND_Q4_K, "l0.wv": KIND_Q4_K, "l1.gate": KIND_Q6_K} if ctx_len == 21 else None
    weights = make_weights(rng, shape, kinds)
    ctx = Context(0)
    try:
        decs = [Decoder(ctx, shape, max_seqs=1, max_ctx=ctx_len + 16, block_size=16, kv_dtype=torch.float16, weights=weights,
                        kinds=kinds) for _ in range(2)]
        n = min(ctx_len, 96)  # a prompt, then the pool filled up to ctx_len with the same random rows in both decoders
        ids = torch.from_numpy(rng.integers(0, shape.vocab, n).astype(np.int32)).cuda()
        pos_np = np.arange(n, dtype=np.int32)
        for d in decs:
            d.step(ids, torch.from_numpy(d.token_meta([0] * n, pos_np)).cuda(), torch.from_numpy(pos_np).cuda())
        fill_k = (torch.randn(decs[0].kv_k.shape, device="cuda") * 0.5).half()
        fill_v = (torch.randn(decs[0].kv_v.shape, device="cuda") * 0.5).half()
        blocks_done = n // 16  # whole blocks the prompt wrote stay as they are
        for d in decs:
            d.kv_k[blocks_done + 1:] = fill_k[blocks_done + 1:]
            d.kv_v[blocks_done + 1:] = fill_v[blocks_done + 1:]
        tok = torch.tensor([3], dtype=torch.int32, device="cuda")
        for step in range(3):
            p = np.array([ctx_len + step], dtype=np.int32)
            meta, pos = torch.from_numpy(decs[0].token_meta([0], p)).cuda(), torch.from_numpy(p).cuda()
            l0 = ctx.launch_count()
            got = decs[0].step(tok, meta, pos, decode=True).clone()
            assert ctx.launch_count() - l0 == 3  # embedding gather, RoPE table, the persistent kernel
            monkeypatch.setenv("MARMOT_DECODER_NO_STEP_KERNEL", "1")
            want = decs[1].step(tok, meta, pos, decode=True).clone()
            monkeypatch.delenv("MARMOT_DECODER_NO_STEP_KERNEL")
            ctx.synchronize()
            assert max_rel_err(got.cpu().numpy(), want.cpu().numpy()) <= 2e-4, step
            assert int(got.argmax()) == int(want.argmax())
            tok = want.argmax(dim=1).to(torch.int32)
        for a, b in ((decs[0].kv_k, decs[1].kv_k), (decs[0].kv_v, decs[1].kv_v)):
            assert torch.equal(a[:, 0], b[:, 0])
    finally:
        ctx.close()


def test_step_kernel_barrier_wait_runs_out_and_the_context_stays_usable(monkeypatch):
    """Failure detection without a GPU fault: a host-side hook makes one CTA skip one arrival at the grid barrier, so the
    other CTAs' bounded waits run out (a short limit for the test); the kernel returns with the error flag set, the next
    synchronize reports it, and the same context and decoder then run the step correctly."""
    from marmot_b200.runtime import MarmotCudaError

    rng = np.random.default_rng(77)
    weights = make_weights(rng)
    ctx = Context(0)
    try:
        decs = [Decoder(ctx, SHAPE, max_seqs=1, max_ctx=64, block_size=16, kv_dtype=torch.float16, weights=weights) for _ in range(2)]
        n = 5
        ids = torch.from_numpy(rng.integers(0, SHAPE.vocab, n).astype(np.int32)).cuda()
        pos_np = np.arange(n, dtype=np.int32)
        for d in decs:
            d.step(ids, torch.from_numpy(d.token_meta([0] * n, pos_np)).cuda(), torch.from_numpy(pos_np).cuda())
        ctx.synchronize()
        tok = torch.tensor([9], dtype=torch.int32, device="cuda")
        p = np.array([n], dtype=np.int32)
        meta, pos = torch.from_numpy(decs[0].token_meta([0], p)).cuda(), torch.from_numpy(p).cuda()
        monkeypatch.setenv("MARMOT_DECODE_PLAN_SPIN_LIMIT", str(1 << 15))
        monkeypatch.setenv("MARMOT_DECODE_PLAN_TEST_SKIP_ARRIVE", "3")  # after the fourth phase (gate/up of layer 0)
        decs[0].step(tok, meta, pos, decode=True)
        with pytest.raises(MarmotCudaError, match="timed out"):
            ctx.synchronize()
        monkeypatch.delenv("MARMOT_DECODE_PLAN_SPIN_LIMIT")
        monkeypatch.delenv("MARMOT_DECODE_PLAN_TEST_SKIP_ARRIVE")
        for plan in decs[0]._plans.values():  # a plan keeps the hooks it was created with
            if plan is not None:
                plan.close()
        decs[0]._plans.clear()
        got = decs[0].step(tok, meta, pos, decode=True).clone()
        ctx.synchronize()
        monkeypatch.setenv("MARMOT_DECODER_NO_STEP_KERNEL", "1")
        want = decs[1].step(tok, meta, pos, decode=True).clone()
        ctx.synchronize()
        assert max_rel_err(got.cpu().numpy(), want.cpu().numpy()) <= 1e-4
        assert int(got.argmax()) == int(want.argmax())
    finally:
        ctx.close()
