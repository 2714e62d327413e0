"""One rank of the multi-GPU tensor-parallel check (launched by torch.distributed.run from
test_tensor_parallel_gpu.py or by hand).  Every rank builds the same weights, shards them, runs the
column-/row-/expert-parallel layers on its GPU and compares with the unsharded operator on the same GPU.
Rank 0 prints one JSON line per rank; exit code 0 means every check of that rank passed."""
from __future__ import annotations

import json
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from marmot_b200 import Context  # noqa: E402
from marmot_b200 import tensor_parallel as tp  # noqa: E402
from marmot_b200.runtime import KIND_Q4_K, KIND_Q6_K, KIND_Q8_0, MarmotCudaError  # noqa: E402
from tests.util import TOL_FP32, TOL_MMA, TOL_MOE, max_rel_err, random_blocks  # noqa: E402


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ctx = Context(local)
    group = tp.Group(rank, world, dist)
    comm = tp.make_peer_comm(ctx, group, 8 << 20)
    res, ok = {}, True

    def check(name, cond, value=None):
        nonlocal ok
        res[name] = value if value is not None else bool(cond)
        if not cond:
            ok = False

    # the all-reduce kernel alone: fixed summation order, identical on all ranks
    n = 100003
    parts = [np.random.default_rng(100 + r).normal(0, 1, n).astype(np.float32) for r in range(world)]
    want = parts[0].copy()
    for r in range(1, world):
        want = want + parts[r]
    for rep in range(3):  # both parities and a reuse
        comm.staging((n,)).copy_(torch.from_numpy(parts[rank]).to(dev))
        out = torch.empty(n, dtype=torch.float32, device=dev)
        comm.allreduce(n, out)
        ctx.synchronize()
        check(f"allreduce_exact_{rep}", np.array_equal(out.cpu().numpy(), want))

    # a message above the two-phase threshold (reduce-scatter + all-gather in one kernel), ragged length
    n = 800003
    parts = [np.random.default_rng(200 + r).normal(0, 1, n).astype(np.float32) for r in range(world)]
    want = parts[0].copy()
    for r in range(1, world):
        want = want + parts[r]
    for rep in range(3):
        comm.staging((n,)).copy_(torch.from_numpy(parts[rank]).to(dev))
        out = torch.full((n + 5,), 3.0, dtype=torch.float32, device=dev)
        comm.allreduce(n, out)
        ctx.synchronize()
        got = out.cpu().numpy()
        check(f"allreduce_two_phase_exact_{rep}", np.array_equal(got[:n], want) and np.all(got[n:] == 3.0))

    # one-slot mode: a CUDA graph with an ODD number of collectives (small and large), replayed; back to two slots after
    comm.set_one_slot(True)
    stream = torch.cuda.Stream(dev)
    ctx.set_stream(stream.cuda_stream)
    sizes = (100003, 800003, 4099)
    srcs = [torch.from_numpy(np.random.default_rng(300 + 10 * i + rank).normal(0, 1, m).astype(np.float32)).to(dev)
            for i, m in enumerate(sizes)]
    wants = []
    for i, m in enumerate(sizes):
        acc = np.random.default_rng(300 + 10 * i).normal(0, 1, m).astype(np.float32)
        for r in range(1, world):
            acc = acc + np.random.default_rng(300 + 10 * i + r).normal(0, 1, m).astype(np.float32)
        wants.append(acc)
    outs = [torch.zeros(m, dtype=torch.float32, device=dev) for m in sizes]

    def three_collectives():
        for src, o in zip(srcs, outs):
            comm.staging((src.numel(),)).copy_(src)
            comm.allreduce(src.numel(), o)

    with torch.cuda.stream(stream):
        three_collectives()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            three_collectives()
        for rep in range(3):
            for o in outs:
                o.zero_()
            g.replay()
            torch.cuda.synchronize()
            check(f"one_slot_graph_replay_{rep}", all(np.array_equal(o.cpu().numpy(), w) for o, w in zip(outs, wants)))
    ctx.synchronize()
    ctx.set_stream(0)
    comm.set_one_slot(False)
    dist.barrier()

    rng = np.random.default_rng(42)
    for kind in (KIND_Q4_K, KIND_Q6_K, KIND_Q8_0):
        for T in (1, 5, 48):
            K, F = 2048, 384
            W = random_blocks(kind, F, K, rng)
            x = torch.from_numpy(rng.normal(0, 1, (T, K)).astype(np.float32)).to(dev)
            want = ctx.linear(kind, x, ctx.upload(W), F).cpu().numpy()
            tol = TOL_FP32 if T <= 8 else TOL_MMA
            col = tp.ColumnParallelLinear(ctx, group, kind, W, F, K, granule=16)
            y = col(x, gather=True).cpu().numpy()
            check(f"col_{kind}_{T}", max_rel_err(y, want) <= tol, float(max_rel_err(y, want)))
            for name, c in (("nccl", None), ("peer", comm), ("fused", comm)):
                if c is not None:
                    c.set_fused(name == "fused")  # the one-kernel form applies to T = 48 here, else it falls back
                row = tp.RowParallelLinear(ctx, group, kind, W, F, K, comm=c)
                y = row(x)
                ctx.synchronize()
                e = float(max_rel_err(y.cpu().numpy(), want))
                check(f"row_{name}_{kind}_{T}", e <= tol, e)
                gathered = [torch.empty_like(y) for _ in range(world)]
                dist.all_gather(gathered, y)
                if name != "nccl":  # every rank holds the same bits
                    check(f"row_{name}_same_{kind}_{T}", all(torch.equal(g, gathered[0]) for g in gathered))
            comm.set_fused(False)

    T, H, FF, E, k = 40, 512, 1024, 8, 2
    gate = np.concatenate([random_blocks(KIND_Q4_K, FF, H, rng, d_sigma=0.0005) for _ in range(E)])
    up = np.concatenate([random_blocks(KIND_Q4_K, FF, H, rng, d_sigma=0.0005) for _ in range(E)])
    down = np.concatenate([random_blocks(KIND_Q6_K, H, FF, rng) for _ in range(E)])
    hidden = torch.from_numpy(rng.normal(0, 1, (T, H)).astype(np.float32)).to(dev)
    ids = torch.from_numpy(np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)).to(dev)
    wts = torch.from_numpy(rng.uniform(0.1, 1.0, (T, k)).astype(np.float32)).to(dev)
    kinds = (KIND_Q4_K, KIND_Q4_K, KIND_Q6_K)
    want = ctx.moe_experts(kinds, hidden, ctx.upload(gate), ctx.upload(up), ctx.upload(down), ids, wts, FF, E).cpu().numpy()
    for name, c in (("nccl", None), ("peer", comm)):
        moe = tp.ExpertParallelMoE(ctx, group, kinds, gate, up, down, H, FF, E, comm=c)
        y = moe(hidden, ids, wts)
        ctx.synchronize()
        e = float(max_rel_err(y.cpu().numpy(), want))
        check(f"moe_{name}", e <= TOL_MOE, e)
    # 256 routes or more: the grouped launches, which skip the routes of other ranks' experts on the device
    T = 160
    down4 = np.concatenate([random_blocks(KIND_Q4_K, H, FF, rng, d_sigma=0.0005) for _ in range(E)])
    hidden = torch.from_numpy(rng.normal(0, 1, (T, H)).astype(np.float32)).to(dev)
    ids = torch.from_numpy(np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)).to(dev)
    wts = torch.from_numpy(rng.uniform(0.1, 1.0, (T, k)).astype(np.float32)).to(dev)
    kinds = (KIND_Q4_K, KIND_Q4_K, KIND_Q4_K)
    want = ctx.moe_experts(kinds, hidden, ctx.upload(gate), ctx.upload(up), ctx.upload(down4), ids, wts, FF, E).cpu().numpy()
    for name, c in (("nccl", None), ("peer", comm)):
        moe = tp.ExpertParallelMoE(ctx, group, kinds, gate, up, down4, H, FF, E, comm=c)
        y = moe(hidden, ids, wts, exchange=False)
        ctx.synchronize()
        e = float(max_rel_err(y.cpu().numpy(), want))
        check(f"moe_grouped_{name}", e <= 1e-5, e)  # the same products as on one GPU, summed per rank first
    # the routed rows return to the token owners, who combine them in the one-GPU order: the same bits, on every rank,
    # also with a ragged token count and repeated (both parities of the staging slots)
    moe = tp.ExpertParallelMoE(ctx, group, kinds, gate, up, down4, H, FF, E, comm=comm)
    for rep in range(3):
        l0 = ctx.launch_count()
        y = moe(hidden, ids, wts)
        ctx.synchronize()
        check(f"moe_exchange_exact_{rep}", np.array_equal(y.cpu().numpy(), want), float(max_rel_err(y.cpu().numpy(), want)))
        check(f"moe_exchange_launches_{rep}", ctx.launch_count() - l0 == 9, int(ctx.launch_count() - l0))
    T2 = 157
    y = moe(hidden[:T2].contiguous(), ids[:T2].contiguous(), wts[:T2].contiguous())
    ctx.synchronize()
    want2 = ctx.moe_experts(kinds, hidden[:T2].contiguous(), ctx.upload(gate), ctx.upload(up), ctx.upload(down4),
                            ids[:T2].contiguous(), wts[:T2].contiguous(), FF, E).cpu().numpy()
    check("moe_exchange_ragged", np.array_equal(y.cpu().numpy(), want2))

    # a whole decoder step: every rank cuts its share out of the same full-model weights; logits slices and the greedy
    # pick must match the single-GPU decoder on the full weights (only the f32 order of the row-parallel sums differs)
    from marmot_b200.decoder import LAYER_WEIGHTS, Decoder, DecoderShape

    shape = DecoderShape(layers=2, d=512, ffn=4096, n_heads=16, n_kv_heads=8, head_dim=128, vocab=1024)
    wrng = np.random.default_rng(7)
    weights = {}
    for i in range(shape.layers):
        for name, kind, rows, cols in LAYER_WEIGHTS:
            weights[f"l{i}.{name}"] = random_blocks(kind, rows(shape), cols(shape), wrng, d_sigma=0.0003)
        weights[f"l{i}.attn_norm"] = wrng.normal(1, 0.1, shape.d).astype(np.float32)
        weights[f"l{i}.ffn_norm"] = wrng.normal(1, 0.1, shape.d).astype(np.float32)
    weights["tok_embd"] = random_blocks(KIND_Q4_K, shape.vocab, shape.d, wrng, d_sigma=0.003)
    weights["output"] = random_blocks(KIND_Q6_K, shape.vocab, shape.d, wrng, d_sigma=0.0003)
    weights["out_norm"] = wrng.normal(1, 0.1, shape.d).astype(np.float32)
    if shape.n_kv_heads % world == 0:
        one = Decoder(ctx, shape, max_seqs=2, max_ctx=64, weights=weights)
        many = Decoder(ctx, shape, max_seqs=2, max_ctx=64, weights=weights, group=group, comm=comm)
        ids = torch.from_numpy(wrng.integers(0, shape.vocab, 5).astype(np.int32)).to(dev)
        pos_np = np.arange(5, dtype=np.int32)
        for step in range(3):
            pos = torch.from_numpy(pos_np).to(dev)
            meta = torch.from_numpy(one.token_meta([1] * len(pos_np), pos_np)).to(dev)
            want = one.step(ids, meta, pos).clone()
            got = many.step(ids, meta, pos)
            ctx.synchronize()
            e = float(max_rel_err(got.cpu().numpy(), want[:, many.v_lo:many.v_lo + many.local_vocab].cpu().numpy()))
            check(f"decoder_logits_{step}", e <= 5 * TOL_FP32, e)
            pick = torch.empty(len(pos_np), dtype=torch.int32, device=dev)
            many.greedy(got, pick)
            ctx.synchronize()
            check(f"decoder_greedy_{step}", torch.equal(pick.long(), want.argmax(dim=1)))
            ids = pick[-1:].clone()
            pos_np = pos_np[-1:] + 1

    # the same model from a GGUF file: every rank uploads only its share (row ranges, and K ranges as strided copies)
    if shape.n_kv_heads % world == 0:
        import tempfile

        from marmot_b200.gguf import load_llama_decoder
        from tests.gguf_writer import write_llama

        with tempfile.TemporaryDirectory() as d:
            path = os.path.join(d, f"rank{rank}.gguf")
            write_llama(path, shape, weights)
            from_file = load_llama_decoder(path, ctx, max_seqs=2, max_ctx=64, group=group, comm=comm)
        ids = torch.from_numpy(wrng.integers(0, shape.vocab, 6).astype(np.int32)).to(dev)
        pos_np = np.arange(6, dtype=np.int32)
        pos = torch.from_numpy(pos_np).to(dev)
        meta = torch.from_numpy(one.token_meta([0] * 6, pos_np)).to(dev)
        want = many.step(ids, meta, pos).clone()  # shards cut on the host from the same weights
        got = from_file.step(ids, meta, pos)
        ctx.synchronize()
        check("decoder_from_gguf", torch.equal(got, want))

    # a peer that never arrives: the bounded wait gives up and the error reaches the host; nothing hangs
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0 and world > 1:
        out = torch.empty(16, dtype=torch.float32, device=dev)
        comm.staging((16,)).zero_()
        comm.allreduce(16, out)
        try:
            ctx.synchronize()
            check("timeout_reported", False)
        except MarmotCudaError as exc:
            check("timeout_reported", "timed out" in str(exc))
    dist.barrier()
    torch.cuda.synchronize()
    # one writer: lines of several ranks printed at once can interleave in the launcher's pipe
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "ok": ok, **res})
    if rank == 0:
        for item in gathered:
            print(json.dumps(item), flush=True)
    # the communicator's epochs now differ between ranks: it is not used again
    comm.close()
    ctx.close()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
