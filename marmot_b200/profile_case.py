"""Run one quantized-linear shape (or one paged-attention decode step) a few times through the C ABI: the small,
self-ending command that a profiler (ncu) or a quick timing wraps.

    python -m marmot_b200.profile_case --kind q4_k -T 1 -K 4096 -F 4096 --copies 16 --iters 3
    python -m marmot_b200.profile_case --op attention --seqs 64 --ctx 2048 --layers 4 --iters 2 --time
    python -m marmot_b200.profile_case --op attention --decode --seqs 1 --ctx 250 --q-heads 32 --kv-heads 4 --head-dim 64
    python -m marmot_b200.profile_case --op layer --layers 22 --iters 2 --time      (the decode step's five kernels)
    python -m marmot_b200.profile_case --op step --ctx 250 --iters 3 --time         (one-token step: the persistent kernel)

The weights rotate over ``--copies`` distinct matrices so that a memory-bound kernel reads from HBM rather
than from L2.  With ``--time`` the calls are also captured in a CUDA graph and replayed, and the average
device time per call is printed (a number taken under a profiler means nothing).
"""
from __future__ import annotations

import argparse

import numpy as np

from .runtime import KIND_BY_NAME, KIND_Q4_K, KIND_Q6_K, Context, row_bytes
from .synthetic import synthetic_blocks, synthetic_blocks_device

REGIMES = {"auto": 0, "gemv": 1, "gemm": 2, "gemv_plain": 3, "i8mma": 4}


def attention_case(args) -> None:
    """Decode-step attention: `seqs` sequences of `ctx` cached positions each, one new token per sequence, the layers of
    the pool visited in turn (so that consecutive calls read different memory).  Pool bytes read per call:
    2 (K and V) * seqs * (ctx + 1) * kv_heads * head_dim * element size."""
    import torch

    dev = torch.device("cuda", 0)
    ctx = Context(0)
    hq, hkv, hd, bs, L = args.q_heads, args.kv_heads, args.head_dim, 16, args.layers
    kv_dtype = torch.float16 if args.kv == "f16" else torch.float32
    per_seq = (args.ctx + 1 + bs - 1) // bs
    n_blocks = args.seqs * per_seq
    gen = torch.Generator(device=dev).manual_seed(0)
    kv_k = torch.randn((n_blocks, L, hkv, bs, hd), device=dev, generator=gen).to(kv_dtype)
    kv_v = torch.randn((n_blocks, L, hkv, bs, hd), device=dev, generator=gen).to(kv_dtype)
    table = torch.arange(n_blocks, dtype=torch.int32, device=dev).view(args.seqs, per_seq).contiguous()
    meta = np.zeros((args.seqs, 4), dtype=np.uint32)
    meta[:, 0] = np.arange(args.seqs)
    meta[:, 1] = args.ctx
    meta[:, 2] = np.arange(args.seqs) * per_seq * bs + args.ctx
    meta = torch.from_numpy(meta.view(np.int32)).to(dev)
    q = torch.randn((args.seqs, hq * hd), device=dev, generator=gen)
    k = torch.randn((args.seqs, hkv * hd), device=dev, generator=gen)
    v = torch.randn((args.seqs, hkv * hd), device=dev, generator=gen)
    out = torch.empty_like(q)

    pos = torch.full((args.seqs,), args.ctx, dtype=torch.int32, device=dev)
    rope = ctx.rope_table(pos, hd, 500000.0)

    def one_pass():
        for layer in range(L):
            if args.decode:  # RoPE + append + attention + merge in one launch (two at many CTAs)
                ctx.paged_attention_decode(meta, q, k, v, kv_k, kv_v, table, layer, hq, hkv, hd, bs, hd ** -0.5, pos,
                                           500000.0, rope_table=rope, out=out)
            else:
                ctx.paged_attention(meta, q, k, v, kv_k, kv_v, table, layer, hq, hkv, hd, bs, hd ** -0.5, out=out)

    stream = torch.cuda.Stream(dev)
    ctx.set_stream(stream.cuda_stream)
    with torch.cuda.stream(stream):
        for _ in range(args.iters):
            one_pass()
    torch.cuda.synchronize()
    nbytes = 2 * args.seqs * (args.ctx + 1) * hkv * hd * kv_k.element_size()
    print(f"attention seqs={args.seqs} ctx={args.ctx} heads={hq}/{hkv}x{hd} kv={args.kv}: {L} layers, {args.iters} passes, "
          f"{ctx.launch_count()} kernel launches, {nbytes} pool bytes per call, pool {2 * kv_k.numel() * kv_k.element_size() >> 20} MiB")
    if args.time:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_pass()
        with torch.cuda.stream(stream):
            for _ in range(3):
                graph.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 10
            e0.record(stream)
            for _ in range(reps):
                graph.replay()
            e1.record(stream)
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (reps * L)
        what = "RoPE + append + attention + merge" if args.decode else "append + attention + merge"
        print(f"{us:.2f} us per call ({what}), {nbytes / us / 1e3:.0f} GB/s of pool bytes")
    ctx.set_stream(0)
    ctx.close()


def moe_case(args) -> None:
    """Expert FFN block: -T tokens, --top-k routes each over --experts experts of shape K (hidden) x F (expert FFN),
    gate/up/down all of --kind; routing is uniform random without repeats.  FLOPs per call: 6 * T * top_k * K * F."""
    import torch

    dev = torch.device("cuda", 0)
    ctx = Context(0)
    kind = KIND_BY_NAME[args.kind]
    E, k, T, H, FF = args.experts, args.top_k, args.T, args.K, args.F
    gen = torch.Generator(device=dev).manual_seed(0)
    gate = synthetic_blocks_device(torch, kind, E * FF, H, dev, gen)
    up = synthetic_blocks_device(torch, kind, E * FF, H, dev, gen)
    down = synthetic_blocks_device(torch, kind, E * H, FF, dev, gen)
    hidden = torch.randn((T, H), device=dev, generator=gen)
    scores = torch.rand((T, E), device=dev, generator=gen)
    vals, ids = torch.topk(scores, k, dim=1)
    ids = ids.to(torch.int32).contiguous()
    vals = (vals / vals.sum(1, keepdim=True)).contiguous()
    out = torch.empty((T, H), dtype=torch.float32, device=dev)
    kinds = (kind, kind, kind)

    def one_pass():
        ctx.moe_experts_local(kinds, hidden, gate, up, down, ids, vals, FF, E, 0, E, out=out)

    stream = torch.cuda.Stream(dev)
    ctx.set_stream(stream.cuda_stream)
    with torch.cuda.stream(stream):
        for _ in range(args.iters):
            one_pass()
    torch.cuda.synchronize()
    flops = 6.0 * T * k * H * FF
    print(f"moe {args.kind} T={T} top_k={k} experts={E} H={H} FF={FF}: {args.iters} calls, {ctx.launch_count()} kernel "
          f"launches, {flops / 1e9:.1f} GFLOP per call")
    if args.time:
        with torch.cuda.stream(stream):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 10
            e0.record(stream)
            for _ in range(reps):
                one_pass()
            e1.record(stream)
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / reps
        print(f"{us:.1f} us per call, {flops / us / 1e6:.1f} TFLOP/s")
    ctx.set_stream(0)
    ctx.close()


def step_case(args) -> None:
    """One-token decode steps of the TinyLlama-1.1B shape (random-init weights, 128-token prompt prefilled, the token at
    position `--ctx`) through Decoder.step: the persistent decode-step kernel.  Prints the kernel's own timeline (CTA 0's
    clock at every phase start; per matmul phase also when the activations were packed and when the rows were done),
    medians over the layers, and with --time the device time per step in CUDA-graph replay."""
    import torch

    from .decoder import TINYLLAMA_1B, Decoder

    dev = torch.device("cuda", 0)
    ctx = Context(0)
    shape = TINYLLAMA_1B
    n_prompt = min(128, args.ctx)
    dec = Decoder(ctx, shape, max_seqs=1, max_ctx=max(args.ctx, n_prompt) + 64, block_size=16, kv_dtype=torch.float16, seed=5)
    stream = torch.cuda.Stream(dev)
    ctx.set_stream(stream.cuda_stream)
    rng = np.random.default_rng(3)
    with torch.cuda.stream(stream):
        ids = torch.from_numpy(rng.integers(0, shape.vocab, n_prompt).astype(np.int32)).to(dev)
        pos = np.arange(n_prompt, dtype=np.int32)
        dec.step(ids, torch.from_numpy(dec.token_meta([0] * n_prompt, pos)).to(dev), torch.from_numpy(pos).to(dev))
        ids = torch.from_numpy(rng.integers(0, shape.vocab, 1).astype(np.int32)).to(dev)
        pos_np = np.asarray([args.ctx], dtype=np.int32)
        pos = torch.from_numpy(pos_np).to(dev)
        meta = torch.from_numpy(dec.token_meta(np.arange(1), pos_np)).to(dev)
        logits = torch.empty((1, dec.local_vocab), dtype=torch.float32, device=dev)

        def one():
            dec.step(ids, meta, pos, logits_out=logits, decode=True)

        l0 = ctx.launch_count()
        one()
        launches = ctx.launch_count() - l0
        for _ in range(max(1, args.iters) - 1):
            one()
        torch.cuda.synchronize()
        plan = next((pl for pl in dec._plans.values() if pl is not None), None)
        print(f"step d={shape.d} ffn={shape.ffn} layers={shape.layers} ctx={args.ctx}: {launches} kernel launches per step, "
              f"{'persistent kernel' if plan is not None else 'five launches per layer'}")
        if plan is not None:
            t = np.array(plan.phase_times(), dtype=np.int64)
            n = (len(t) - 1) // 3
            L = shape.layers
            dur = np.diff(t[:n + 1]) / 1e3
            det = (t[n + 1:].reshape(n, 2) - t[:n, None]) / 1e3
            names = ["q/k/v", "attention", "o proj", "gate/up", "down"]
            per, pk, wk = dur[:5 * L].reshape(L, 5), det[:5 * L, 0].reshape(L, 5), det[:5 * L, 1].reshape(L, 5)
            print("phase        us   packed at   rows done at   (medians over the layers, CTA 0)")
            for i, name in enumerate(names):
                packed = f"{np.median(pk[:, i]):9.2f}" if i != 1 else "        -"
                print(f"{name:10s} {np.median(per[:, i]):5.2f}   {packed}   {np.median(wk[:, i]):9.2f}")
            print(f"{'output':10s} {dur[5 * L]:5.2f}   {det[5 * L, 0]:9.2f}   {det[5 * L, 1]:9.2f}")
            print(f"kernel, first phase start to end: {(t[n] - t[0]) / 1e3:.1f} us")
        if args.time:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                one()
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(100):
                g.replay()
            e1.record(stream)
            torch.cuda.synchronize()
            print(f"{e0.elapsed_time(e1) * 10:.1f} us per step in graph replay")
    ctx.synchronize()
    ctx.set_stream(0)


def layer_case(args) -> None:
    """The five launches of one decoder layer in a fused decode step, TinyLlama-1.1B shape by default (d 2048, FFN 5632,
    32 / 4 heads of 64; Q4_K with Q6_K for v and down), -T tokens of one context length each, `--layers` layers with
    weights of their own in turn: q/k/v with add + RMSNorm prologue, decode attention, o projection, gate/up with
    add + RMSNorm prologue, down with SwiGLU prologue."""
    import torch

    from .synthetic import synthetic_blocks_device

    dev = torch.device("cuda", 0)
    ctx = Context(0)
    d, ffn, hq, hkv, hd, L, T, bs = args.K if args.K != 4096 else 2048, args.F if args.F != 4096 else 5632, 32, 4, 64, args.layers, args.T, 16
    gen = torch.Generator(device=dev).manual_seed(1)
    mk = lambda kind, F, K: [synthetic_blocks_device(torch, kind, F, K, dev, gen) for _ in range(L)]
    wq, wk, wv, wo = mk(KIND_Q4_K, d, d), mk(KIND_Q4_K, hkv * hd, d), mk(KIND_Q6_K, hkv * hd, d), mk(KIND_Q4_K, d, d)
    wg, wu, wd = mk(KIND_Q4_K, ffn, d), mk(KIND_Q4_K, ffn, d), mk(KIND_Q6_K, d, ffn)
    xa, xb = torch.randn((T, d), device=dev, generator=gen), torch.empty((T, d), device=dev)
    nw = torch.ones(d, device=dev)
    q, k, v = (torch.empty((T, n), device=dev) for n in (d, hkv * hd, hkv * hd))
    att, proj = torch.empty((T, d), device=dev), torch.randn((T, d), device=dev, generator=gen) * 0.01
    gate, up = torch.empty((T, ffn), device=dev), torch.empty((T, ffn), device=dev)
    per_seq = (args.ctx + 1 + bs - 1) // bs
    kv_k = (torch.randn((T * per_seq, L, hkv, bs, hd), device=dev, generator=gen) * 0.1).half()
    kv_v = (torch.randn((T * per_seq, L, hkv, bs, hd), device=dev, generator=gen) * 0.1).half()
    table = torch.arange(T * per_seq, dtype=torch.int32, device=dev).view(T, per_seq).contiguous()
    meta = np.zeros((T, 4), dtype=np.uint32)
    meta[:, 0], meta[:, 1], meta[:, 2] = np.arange(T), args.ctx, np.arange(T) * per_seq * bs + args.ctx
    meta = torch.from_numpy(meta.view(np.int32)).to(dev)
    pos = torch.full((T,), args.ctx, dtype=torch.int32, device=dev)
    rope = ctx.rope_table(pos, hd, 10000.0)

    steps = {
        "qkv": lambda i: ctx.linear_multi(xa, [(KIND_Q4_K, wq[i], d, q), (KIND_Q4_K, wk[i], hkv * hd, k),
                                               (KIND_Q6_K, wv[i], hkv * hd, v)], ("add_rmsnorm", proj, nw, 1e-5, 0.0, xb)),
        "attn": lambda i: ctx.paged_attention_decode(meta, q, k, v, kv_k, kv_v, table, i, hq, hkv, hd, bs, hd ** -0.5, pos,
                                                     10000.0, rope_table=rope, out=att),
        "wo": lambda i: ctx.linear(KIND_Q4_K, att, wo[i], d, out=proj),
        "gateup": lambda i: ctx.linear_multi(xb, [(KIND_Q4_K, wg[i], ffn, gate), (KIND_Q4_K, wu[i], ffn, up)],
                                             ("add_rmsnorm", proj, nw, 1e-5, 0.0, xa)),
        "down": lambda i: ctx.linear_multi(gate, [(KIND_Q6_K, wd[i], d, proj)], ("swiglu", up)),
    }
    chosen = [steps[n] for n in (args.only.split(",") if args.only else steps)]  # --only: a chain of one kind of kernel

    def one_pass():
        for i in range(L):
            for step in chosen:
                step(i)

    stream = torch.cuda.Stream(dev)
    ctx.set_stream(stream.cuda_stream)
    with torch.cuda.stream(stream):
        for _ in range(args.iters):
            one_pass()
    torch.cuda.synchronize()
    wbytes = sum(int(w[0].numel()) for w in (wq, wk, wv, wo, wg, wu, wd))
    print(f"layer d={d} ffn={ffn} T={T} ctx={args.ctx}: {L} layers, {args.iters} passes, {ctx.launch_count()} kernel launches, "
          f"{wbytes} weight bytes per layer")
    if args.time:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_pass()
        with torch.cuda.stream(stream):
            for _ in range(3):
                graph.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 20
            e0.record(stream)
            for _ in range(reps):
                graph.replay()
            e1.record(stream)
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (reps * L)
        print(f"{us:.2f} us per layer ({args.only or 'all five launches'}), {wbytes / us / 1e3:.0f} GB/s of the layer's weight bytes")
    ctx.set_stream(0)
    ctx.close()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", default="linear", choices=["linear", "attention", "moe", "layer", "step"])
    ap.add_argument("--only", default="", help="layer: comma-separated subset of qkv,attn,wo,gateup,down")
    ap.add_argument("--decode", action="store_true", help="attention: the one-launch decode form (RoPE + append + merge folded in)")
    ap.add_argument("--experts", type=int, default=8, help="moe: experts")
    ap.add_argument("--top-k", type=int, default=2, help="moe: routes per token")
    ap.add_argument("--seqs", type=int, default=64, help="attention: sequences (one new token each)")
    ap.add_argument("--ctx", type=int, default=2048, help="attention: cached positions per sequence")
    ap.add_argument("--layers", type=int, default=4, help="attention: layers in the pool, visited in turn")
    ap.add_argument("--q-heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--kv", default="f16", choices=["f16", "f32"])
    ap.add_argument("--kind", default="q4_k", choices=sorted(KIND_BY_NAME))
    ap.add_argument("-T", type=int, default=1, help="tokens")
    ap.add_argument("-K", type=int, default=4096, help="reduction length")
    ap.add_argument("-F", type=int, default=4096, help="output features")
    ap.add_argument("--copies", type=int, default=16)
    ap.add_argument("--iters", type=int, default=3, help="passes over the rotation")
    ap.add_argument("--regime", default="auto", choices=sorted(REGIMES))
    ap.add_argument("--time", action="store_true", help="also replay a CUDA graph of one pass and print us per call")
    args = ap.parse_args()
    if args.op == "attention":
        return attention_case(args)
    if args.op == "moe":
        return moe_case(args)
    if args.op == "layer":
        return layer_case(args)
    if args.op == "step":
        return step_case(args)

    import torch

    kind = KIND_BY_NAME[args.kind]
    dev = torch.device("cuda", 0)
    ctx = Context(0)
    ctx.set_regime(REGIMES[args.regime])
    rng = np.random.default_rng(0)
    weights = [ctx.upload(synthetic_blocks(kind, args.F, args.K, rng)) for _ in range(args.copies)]
    x = torch.from_numpy(rng.normal(0, 1, (args.T, args.K)).astype(np.float32)).to(dev)
    out = torch.empty((args.T, args.F), dtype=torch.float32, device=dev)

    def one_pass():
        for w in weights:
            ctx.linear(kind, x, w, args.F, out=out)

    stream = torch.cuda.Stream(dev)
    ctx.set_stream(stream.cuda_stream)
    with torch.cuda.stream(stream):
        for _ in range(args.iters):
            one_pass()
    torch.cuda.synchronize()
    nbytes = args.F * row_bytes(kind, args.K) + 4 * args.T * (args.K + args.F)
    print(f"{args.kind} T={args.T} K={args.K} F={args.F}: {args.copies} weight copies, {args.iters} passes, "
          f"{ctx.launch_count()} kernel launches, {nbytes} algorithmic bytes per call")
    if args.time:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_pass()
        with torch.cuda.stream(stream):
            for _ in range(3):
                graph.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 20
            e0.record(stream)
            for _ in range(reps):
                graph.replay()
            e1.record(stream)
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (reps * args.copies)
        flops = 2.0 * args.T * args.K * args.F
        print(f"{us:.2f} us per call, {nbytes / us / 1e3:.0f} GB/s algorithmic, {flops / us / 1e6:.1f} TFLOP/s")
    ctx.set_stream(0)
    ctx.close()


if __name__ == "__main__":
    main()
