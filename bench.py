#!/usr/bin/env python3
"""Benchmark of the quantized-matmul hot path.

Workload (default): the single-token Q4_K GEMV, K = 4096, F = 4096, f32 activations drawn from
N(0,1), weights drawn in block space (fp16 d, dmin = |N(0,0.02)|, 6-bit scales / mins and 4-bit
quants uniform).  One *step* is one pass over a rotation of ``--copies`` distinct weight matrices
(default 32 x 9.4 MB = 302 MB, larger than twice the 126 MB L2, so every pass streams from HBM);
each GEMV in the pass is one call of the library's ``mcu_linear``.

Printed on rank 0 as one JSON line:
  value     GB/s of algorithmic bytes (packed weights + x + y = 9 469 952 B per GEMV) over the timed
            region, inputs resident in HBM, summed over ranks
  e2e       the same through the reference's public API on its CUDA context (``marmot_linear`` after
            ``marmot_init(MARMOT_BACKEND_CUDA)`` in libmarmot_b200.so; ``mcu_linear_host`` when that library
            is not built): activations start in host memory and the result lands in host memory inside the
            timed region, weights stay resident
  roofline  the GEMV kernel against the measured HBM copy bandwidth
  cpu_baseline  the reference CPU backend (or the oracle port) on the host cores, bounded sample

``--impl reference`` times the reference's own CPU implementation instead.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

KIND_Q4_K = 9
K_DIM, F_DIM, T_TOK = 4096, 4096, 1
W_BYTES = F_DIM * (K_DIM // 256) * 144
ALG_BYTES = W_BYTES + T_TOK * K_DIM * 4 + T_TOK * F_DIM * 4  # 9 469 952
METRIC = "q4k_gemv_hbm_gbps"
UNIT = "GB/s"
NCU_TRAFFIC_BYTES = 9_504_512  # DRAM bytes of one launch, from the committed ncu capture of this shape
WORKLOAD = "Q4_K GEMV T=1 K=4096 F=4096 (BASELINE config 1), rotation of distinct weight matrices"


def measured_peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def make_weights(seed: int) -> np.ndarray:
    from marmot_b200.synthetic import random_blocks

    return random_blocks(KIND_Q4_K, F_DIM, K_DIM, np.random.default_rng(seed))


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


class CpuGemv:
    """The CPU checker's GEMV on this host (the reference library when present, else the oracle port): one context and
    one set of weight tensors for the whole run, as a model holds them."""

    def __init__(self, copies: int, threads: int):
        from oracle.bindings import REF_LIB, Oracle, Reference

        self.copies, self.threads = copies, threads
        ws = [make_weights(1000 + i) for i in range(copies)]
        x = np.random.default_rng(5).normal(0, 1, (T_TOK, K_DIM)).astype(np.float32)
        if REF_LIB.exists():
            ref = Reference(threads=threads)
            tw = [ref._qtensor((F_DIM, K_DIM), KIND_Q4_K, w) for w in ws]
            tx = ref._tensor((T_TOK, K_DIM), 0, x)
            to = ref._tensor((T_TOK, F_DIM), 0)
            self._keep = (ref, tw, tx, to, ws)
            self.run = lambda i: ref._check(ref.lib.marmot_linear(ref.ctx, tx, tw[i % copies], None, to), "marmot_linear")
            self.kind = "reference"
        else:
            from oracle import build_oracle

            build_oracle.build()
            orc = Oracle()
            self._keep = (orc, ws)
            self.run = lambda i: orc.linear(KIND_Q4_K, x, ws[i % copies], F_DIM, threads=threads)
            self.kind = "port"
        for i in range(max(copies, 8)):  # every weight copy touched, thread pool and caches warm
            self.run(i)

    def seconds(self, n: int, start: int = 0) -> float:
        """Wall time of n GEMVs, rotating over the weight copies."""
        t0 = time.perf_counter()
        for i in range(start, start + n):
            self.run(i)
        return time.perf_counter() - t0


def workload_config(copies: int) -> dict:
    """The workload description both arms print (the driver compares the two dictionaries)."""
    return {"workload": WORKLOAD, "T": T_TOK, "K": K_DIM, "F": F_DIM, "quant": "Q4_K", "weight_copies": copies,
            "l2_policy": f"inputs larger than L2: rotation over {copies * W_BYTES / 1e6:.0f} MB of weights",
            "multi_gpu": "replicas only (independent GEMVs per rank, no collective)"}


def time_other_regimes(ctx, dev):
    """Short CUDA-graph timings of the other regimes of the path (not the headline): large-F GEMVs of the three
    formats (F = 28672, and the 128256-row output projection of the Llama-3 shape), the batched-decode shape and the Q8_0 prefill GEMM of BASELINE config 2.  Each entry is one
    `mcu_linear` call (activation quantisation included), rotating over weight copies larger than L2."""
    import torch

    from marmot_b200.synthetic import synthetic_blocks
    from marmot_b200.runtime import KIND_BY_NAME, row_bytes

    peak_bw, _ = measured_peaks()
    peaks = json.loads((REPO / "MEASURED_PEAKS.json").read_text()) if (REPO / "MEASURED_PEAKS.json").exists() else {}
    peak_tf = float(peaks.get("bf16_tflops", 1590.0))
    out = []
    stream = torch.cuda.Stream(dev)
    ctx.set_stream(stream.cuda_stream)
    rng = np.random.default_rng(11)
    for name, T, K, F, copies in [("q4_k", 1, 4096, 28672, 4), ("q6_k", 1, 4096, 28672, 4), ("q8_0", 1, 4096, 28672, 4),
                                  ("q4_k", 1, 4096, 128256, 2), ("q6_k", 1, 4096, 128256, 1),  # Llama-3 output projection
                                  ("q4_k", 8, 4096, 14336, 8), ("q4_k", 64, 4096, 14336, 4),
                                  ("q8_0", 512, 4096, 14336, 2), ("q4_k", 512, 4096, 14336, 2)]:
        kind = KIND_BY_NAME[name]
        ws = [ctx.upload(synthetic_blocks(kind, F, K, rng)) for _ in range(copies)]
        x = torch.from_numpy(rng.normal(0, 1, (T, K)).astype(np.float32)).to(dev)
        y = torch.empty((T, F), dtype=torch.float32, device=dev)
        with torch.cuda.stream(stream):
            for w in ws:
                ctx.linear(kind, x, w, F, out=y)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for w in ws:
                ctx.linear(kind, x, w, F, out=y)
        reps = 10
        with torch.cuda.stream(stream):
            for _ in range(3):
                g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                g.replay()
            e1.record(stream)
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (reps * copies)
        nbytes = F * row_bytes(kind, K) + 4 * T * (K + F)
        gbs, tf = nbytes / us / 1e3, 2.0 * T * K * F / us / 1e6
        entry = {"quant": name, "T": T, "K": K, "F": F, "us_per_call": round(us, 2), "GBps": round(gbs, 1),
                 "TFLOPs": round(tf, 2)}
        if T <= 64:
            entry["frac_hbm"] = round(gbs / peak_bw, 3)
        else:
            entry["frac_tensor"] = round(tf / peak_tf, 3)
        out.append(entry)
        del g, ws
    ctx.set_stream(0)
    return out


LLAMA8B = {"layers": 32, "d": 4096, "ffn": 14336, "kv": 1024, "vocab": 128256}


def time_tp_decode_matmuls(ctx, dev, rank: int, world: int, dist, T: int = 64):
    """The weight-streaming part of a Llama-3-8B-shape Q4_K_M decode step for T concurrent sequences, tensor
    parallel over `world` GPUs: per layer q/k/v (column-parallel), attention output (row-parallel + all-reduce),
    gate/up (column-parallel, one dual launch), down (row-parallel + all-reduce), and the vocabulary projection once
    per step.  Attention, norms and RoPE are not part of it.  Every rank draws its own shard-shaped random weights
    (distinct per layer, so nothing is re-read from L2); the step is captured in a CUDA graph and replayed."""
    import torch

    from marmot_b200 import tensor_parallel as tp
    from marmot_b200.synthetic import synthetic_blocks_device
    from marmot_b200.runtime import KIND_Q6_K, row_bytes

    m = LLAMA8B
    d, ffn, kv, vocab, L = m["d"], m["ffn"], m["kv"], m["vocab"], m["layers"]
    if d % (256 * world) or kv % world:
        return {"skipped": f"shapes do not divide over {world} ranks"}
    # the FFN width is dealt out in 2048-value granules (the same ranges for gate/up rows and down's K), so that the
    # Q6_K rows of every down shard stay 16-byte multiples; ranks may differ by one granule
    f_lo, f_hi = tp.shard_range(ffn, world, rank, 2048)
    ffn_r = f_hi - f_lo
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    Q4, Q6 = KIND_Q4_K, KIND_Q6_K
    group = tp.Group(rank, world, dist if world > 1 else None)
    comm = tp.make_peer_comm(ctx, group, T * d * 4) if world > 1 else None
    mk = lambda kind, F, K: synthetic_blocks_device(torch, kind, F, K, dev, gen)
    layers, wbytes = [], 0
    for _ in range(L):
        w = {"q": (Q4, mk(Q4, d // world, d), d // world, d), "k": (Q4, mk(Q4, kv // world, d), kv // world, d),
             "v": (Q6, mk(Q6, kv // world, d), kv // world, d), "o": (Q4, mk(Q4, d, d // world), d, d // world),
             "gate": (Q4, mk(Q4, ffn_r, d), ffn_r, d), "up": (Q4, mk(Q4, ffn_r, d), ffn_r, d),
             "down": (Q6, mk(Q6, d, ffn_r), d, ffn_r)}
        wbytes += sum(F * row_bytes(kind, K) for kind, _, F, K in w.values())
        layers.append(w)
    v_lo, v_hi = tp.shard_range(vocab, world, rank, 32)
    head = (Q6, mk(Q6, v_hi - v_lo, d), v_hi - v_lo, d)
    wbytes += head[2] * row_bytes(Q6, d)
    x = torch.randn((T, d), device=dev, generator=gen)
    x_attn = torch.randn((T, d // world), device=dev, generator=gen)
    x_ffn = torch.randn((T, max(ffn_r, 1)), device=dev, generator=gen)
    bufs = {n: torch.empty((T, F), dtype=torch.float32, device=dev)
            for n, F in (("q", d // world), ("k", kv // world), ("v", kv // world), ("o", d), ("gate", max(ffn_r, 1)),
                         ("up", max(ffn_r, 1)), ("down", d), ("head", v_hi - v_lo))}

    ffn_empty_somewhere = any(b == a for a, b in (tp.shard_range(ffn, world, r, 2048) for r in range(world)))

    def row_parallel(entry, xin, out, how):
        kind, wt, F, K = entry
        unfused = ffn_empty_somewhere and K != d // world  # the down projection when some rank has no share of it
        if how in ("peer", "peer_fused") and unfused and K > 0:
            ctx.linear(kind, xin, wt, F, out=comm.staging((T, F)))
            comm.allreduce(T * F, out)
        elif K == 0:  # more ranks than granules: this rank adds zeros
            if how in ("peer", "peer_fused"):
                comm.staging((T, F)).zero_()
                comm.allreduce(T * F, out)
            else:
                out.zero_()
                dist.all_reduce(out)
        elif world == 1:
            ctx.linear(kind, xin, wt, F, out=out)
        elif how in ("peer", "peer_fused"):
            comm.linear_allreduce(kind, xin, wt, F, out=out)
        else:
            ctx.linear(kind, xin, wt, F, out=out)
            dist.all_reduce(out)

    def step(how):
        for w in layers:
            for n in ("q", "k", "v"):
                kind, wt, F, K = w[n]
                ctx.linear(kind, x, wt, F, out=bufs[n])
            row_parallel(w["o"], x_attn, bufs["o"], how)
            if ffn_r > 0:
                ctx.linear_dual(Q4, x, w["gate"][1], w["up"][1], w["gate"][2], out_a=bufs["gate"], out_b=bufs["up"])
            row_parallel(w["down"], x_ffn, bufs["down"], how)
        kind, wt, F, K = head
        ctx.linear(kind, x, wt, F, out=bufs["head"])

    result = {"T": T, "layers": L, "weight_bytes_per_gpu": wbytes, "tensor_parallel": world}
    stream = torch.cuda.Stream(dev)
    ctx.set_stream(stream.cuda_stream)
    for how in (["single"] if world == 1 else ["peer", "peer_fused", "nccl"]):
        try:
            if comm is not None:
                comm.set_fused(how == "peer_fused")  # one kernel for matmul + all-reduce instead of two
            with torch.cuda.stream(stream):
                for _ in range(2):
                    step(how)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            l0 = ctx.launch_count()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                step(how)
            launches = ctx.launch_count() - l0
            reps = 5
            with torch.cuda.stream(stream):
                for _ in range(2):
                    g.replay()
                torch.cuda.synchronize()
                if world > 1:
                    dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(reps):
                    g.replay()
                e1.record(stream)
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / reps
            if world > 1:
                t = torch.tensor([ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            ctx.synchronize()
            result[how] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(T / ms * 1e3, 1),
                           "weight_GBps_per_gpu": round(wbytes / ms / 1e6, 1), "kernel_launches_per_step": int(launches)}
            del g
        except Exception as exc:  # e.g. a collective that cannot be captured
            result[how] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    ctx.set_stream(0)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    if comm is not None:
        comm.close()
    return result


def time_decode(ctx, dev, rank: int = 0, world: int = 1, dist=None, c4_only: bool = False):
    """Decode tokens/s of the Llama-shape decoders of BASELINE configs 3 and 4, random-init weights (N(0, 0.02) quantised
    to the Q4_K_M mix of block formats on the device by marmot_b200.synthetic.normal_blocks),
    fp16 paged KV cache with 16-token blocks, the whole step (embedding gather, 7 matmuls + attention + glue per layer,
    output projection, argmax, position update) captured in one CUDA graph and replayed; greedy sampling stays on the
    device.  Config 3: TinyLlama-1.1B shape, batch 1, 128-token prompt, 256 decoded tokens.  Config 4: Llama-3-8B shape,
    64 sequences with contexts uniform in [256, 4096], one decode step repeated at fixed contexts."""
    import torch

    from marmot_b200 import tensor_parallel as tp
    from marmot_b200.decoder import LLAMA3_8B, TINYLLAMA_1B, Decoder, weight_bytes

    peak_bw, _ = measured_peaks()
    out = {}
    group = tp.Group(rank, world, dist if world > 1 else None)

    def run(shape, n_seq, ctx_lens, n_prompt, n_decode, advance, replicas=False):
        """replicas: every rank holds all weights and decodes its own share of the sequences (no collective)."""
        max_ctx = int(max(ctx_lens)) + n_decode + 16
        total_seq = n_seq
        if replicas:
            ctx_lens = np.asarray(ctx_lens)[rank::world]
            n_seq = len(ctx_lens)
        tpar = world > 1 and not replicas
        comm = tp.make_peer_comm(ctx, group, n_seq * max(shape.d, world) * 4) if tpar else None
        dec = Decoder(ctx, shape, max_seqs=n_seq, max_ctx=max_ctx, block_size=16, kv_dtype=torch.float16, seed=5,
                      group=group if tpar else None, comm=comm)
        stream = torch.cuda.Stream(dev)
        ctx.set_stream(stream.cuda_stream)
        rng = np.random.default_rng(3)
        with torch.cuda.stream(stream):
            if n_prompt > 0:  # prefill the prompt in one call (tensor-core regime)
                ids = torch.from_numpy(rng.integers(0, shape.vocab, n_prompt).astype(np.int32)).to(dev)
                pos = np.arange(n_prompt, dtype=np.int32)
                dec.step(ids, torch.from_numpy(dec.token_meta([0] * n_prompt, pos)).to(dev), torch.from_numpy(pos).to(dev))
            ids = torch.from_numpy(rng.integers(0, shape.vocab, n_seq).astype(np.int32)).to(dev)
            pos_np = np.asarray(ctx_lens, dtype=np.int32)
            pos = torch.from_numpy(pos_np).to(dev)
            meta = torch.from_numpy(dec.token_meta(np.arange(n_seq), pos_np)).to(dev)
            meta_i32 = meta.view(torch.int32)  # torch has no uint32 arithmetic on CUDA; the values stay below 2^31
            logits = torch.empty((n_seq, dec.local_vocab), dtype=torch.float32, device=dev)

            def one_token():
                dec.step(ids, meta, pos, logits_out=logits, decode=True)
                dec.greedy(logits, ids)
                if advance:  # a sequence's blocks are contiguous here, so kv_slot advances with the position
                    pos.add_(1)
                    meta_i32[:, 1:3] += 1

            one_token()
            one_token()  # an even number of eager steps: the communicator's staging parity is what the graph captures
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            l0 = ctx.launch_count()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                one_token()
            launches = ctx.launch_count() - l0
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(n_decode):
                g.replay()
            e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n_decode
        ctx.synchronize()  # reports a peer wait that ran out
        ctx.set_stream(0)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            dist.barrier()
            torch.cuda.synchronize()
            if comm is not None:
                comm.close()
        wb = weight_bytes(dec.local) - dec.local.vocab * row_bytes_q6(dec.local.d) + dec.local_vocab * row_bytes_q6(dec.local.d)
        kv_heads_here = dec.local.n_kv_heads
        mean_ctx = float(np.mean(ctx_lens)) + (n_decode / 2 if advance else 0)
        kvb = n_seq * mean_ctx * shape.layers * kv_heads_here * shape.head_dim * 2 * 2
        return {"ms_per_step": round(ms, 4), "tokens_per_s": round(total_seq / ms * 1e3, 1), "sequences": total_seq,
                "tensor_parallel": world if tpar else 1, "replicas": world if replicas else 1,
                "weight_bytes_per_step_per_gpu": wb, "kv_bytes_per_step_per_gpu": int(kvb),
                "GBps": round((wb + kvb) / ms / 1e6, 1), "frac_hbm": round((wb + kvb) / ms / 1e6 / peak_bw, 3),
                "kernel_launches_per_step": int(launches)}

    def row_bytes_q6(K):
        return (K // 256) * 210

    if world == 1 and not c4_only:
        out["tinyllama_1b_batch1"] = run(TINYLLAMA_1B, 1, [128], 128, 256, True)
        torch.cuda.empty_cache()
    lens = np.random.default_rng(4).integers(256, 4097, 64)
    out["llama3_8b_64seq"] = run(LLAMA3_8B, 64, lens, 0, 20, False)
    torch.cuda.empty_cache()
    if world > 1:  # the same 64 sequences dealt out over replicas of the whole model (it fits one GPU many times over)
        out["llama3_8b_64seq_replicas"] = run(LLAMA3_8B, 64, lens, 0, 20, False, replicas=True)
        torch.cuda.empty_cache()
    return out


def time_moe_c5(ctx, dev, rank: int, world: int, dist):
    """BASELINE config 5: Mixtral-8x7B-shape expert FFN (8 experts, top-2, d=4096, FFN 14336, Q4_K), 2048 tokens,
    softmax top-2 routing of N(0,1) logits; expert parallel over the ranks (contiguous expert ranges, router
    replicated; the routed rows return to the owners of their tokens over peer memory, are combined there in route
    order and the token slices gathered, mcu_moe_experts_ep).  At this size the operator takes its grouped path, whose group
    sizes stay on the device; the calls are timed by the host clock around ten of them with a synchronize at the end."""
    import torch

    from marmot_b200 import tensor_parallel as tp
    from marmot_b200.synthetic import normal_blocks

    T, H, FF, E, k = 2048, 4096, 14336, 8, 2
    if E % world:
        return {"skipped": f"{E} experts do not divide over {world} ranks"}
    e_lo, e_hi = tp.shard_range(E, world, rank)
    n_local = e_hi - e_lo
    gen = torch.Generator(device=dev)
    gen.manual_seed(77)  # the same router inputs on every rank
    hidden = torch.randn((T, H), device=dev, generator=gen)
    probs = torch.softmax(torch.randn((T, E), device=dev, generator=gen), dim=1)
    vals, ids = ctx.topk(probs, k)
    gen.manual_seed(1000 + rank)
    gate = normal_blocks(torch, KIND_Q4_K, n_local * FF, H, dev, gen).reshape(-1)  # random init: N(0, 0.02), quantised
    up = normal_blocks(torch, KIND_Q4_K, n_local * FF, H, dev, gen).reshape(-1)
    down = normal_blocks(torch, KIND_Q4_K, n_local * H, FF, dev, gen).reshape(-1)
    kinds = (KIND_Q4_K,) * 3
    group = tp.Group(rank, world, dist if world > 1 else None)
    # staging slots for the routed rows and the combined token slices: (T * k + T) * H floats
    comm = tp.make_peer_comm(ctx, group, (T * k + T) * H * 4 + 256) if world > 1 else None
    out = torch.empty((T, H), dtype=torch.float32, device=dev)
    bounds = [tp.shard_range(E, world, r)[0] for r in range(world)] + [E]

    def call():
        if world == 1:
            ctx.moe_experts_local(kinds, hidden, gate, up, down, ids, vals, FF, E, 0, E, out=out)
        else:  # routed rows back to the token owners over peer memory, combine, gather the token slices
            comm.moe_experts_ep(kinds, hidden, gate, up, down, ids, vals, FF, E, bounds, out=out)

    for _ in range(3):
        call()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    reps = 10
    t0 = time.perf_counter()
    for _ in range(reps):
        call()
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / reps
    if world > 1:
        t = torch.tensor([dt], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
        dist.barrier()
        torch.cuda.synchronize()
    if comm is not None:
        comm.close()
    flops = T * k * 3 * 2 * H * FF
    peaks = json.loads((REPO / "MEASURED_PEAKS.json").read_text()) if (REPO / "MEASURED_PEAKS.json").exists() else {}
    tf = flops / dt / 1e12
    return {"tokens": T, "experts": E, "top_k": k, "expert_parallel": world, "ms_per_call": round(dt * 1e3, 3),
            "TFLOPs_total": round(tf, 1), "frac_tensor_per_gpu": round(tf / world / float(peaks.get("bf16_tflops", 1590.0)), 3),
            "timing": "host wall clock around 10 calls, max over ranks"}


def run_reference_arm(args, rank: int):
    """The reference's own CPU implementation of the path on all host cores: a step is one rotation over the same
    number of distinct weight matrices as the GPU arm's step."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    copies = args.copies
    cpu = CpuGemv(copies, threads)
    for w in range(args.warmup):
        cpu.seconds(copies, w * copies)
    times = [cpu.seconds(copies, s * copies) for s in range(args.steps)]
    total = sum(times)
    value = args.steps * copies * ALG_BYTES / total / 1e9
    sample = f"{copies} GEMVs per step (one rotation over {copies} weight copies), {threads} host threads, one context"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 dot, f32 scale", "data": "synthetic",
        "config": workload_config(copies),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": cpu.kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--copies", type=int, default=32)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-extra", action="store_true", help="skip the short timings of the other regimes")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    import torch
    import torch.distributed as dist

    from marmot_b200 import Context

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank)
    ctx = Context(local_rank)

    R = args.copies
    weights = [ctx.upload(make_weights(1000 * rank + i)) for i in range(R)]
    rng = np.random.default_rng(7 + rank)
    xs_host = torch.from_numpy(rng.normal(0, 1, (R, T_TOK, K_DIM)).astype(np.float32)).pin_memory()
    xs = xs_host.to(dev)
    outs = torch.empty((R, T_TOK, F_DIM), dtype=torch.float32, device=dev)
    outs_host = torch.empty((R, T_TOK, F_DIM), dtype=torch.float32).pin_memory()

    def step_device():
        for i in range(R):
            ctx.linear(KIND_Q4_K, xs[i], weights[i], F_DIM, out=outs[i])

    xh_np = xs_host.numpy()
    oh_np = outs_host.numpy()

    def step_host():
        for i in range(R):
            ctx.linear_host(KIND_Q4_K, xh_np[i], weights[i], F_DIM, out_host=oh_np[i])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # The device-timed region replays a CUDA graph of one step on a dedicated stream: a 9 MB GEMV lasts a
    # few microseconds, less than the host needs to issue it, so eager launches would time the host.
    stream = torch.cuda.Stream(dev)
    ctx.set_stream(stream.cuda_stream)
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            step_device()
    barrier()
    graph = None
    l0 = ctx.launch_count()
    if not args.no_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step_device()
        launches_per_step = ctx.launch_count() - l0
    else:
        with torch.cuda.stream(stream):
            step_device()
        launches_per_step = ctx.launch_count() - l0
    run_step = graph.replay if graph is not None else step_device

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            run_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            run_step()
        e1.record(stream)
        barrier()
    ms_dev = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_dev], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_dev = float(t.item())
    launches = launches_per_step * args.steps
    clocks = sampler.stop() if sampler else None
    ctx.set_stream(0)  # back to the legacy default stream for the host-buffer path

    # End to end through the reference's own public API on its CUDA context (marmot_init(MARMOT_BACKEND_CUDA) in
    # libmarmot_b200.so: marmot's core with this backend generated into its dispatch): host activations into a marmot
    # tensor, marmot_linear, result read back with marmot_tensor_copy_to_host_buffer, every GEMV; weights resident.
    # Without that library (no marmot checkout at build time) the C ABI's host-buffer entry point stands in.
    e2e_steps = max(3, min(args.steps, 10))
    e2e_api = "mcu_linear_host"
    step_e2e = step_host
    marmot = None
    try:
        from marmot_b200.marmot_api import BACKEND_CUDA, FULL_LIB, MarmotLibrary

        if FULL_LIB.exists():
            os.environ.setdefault("MARMOT_CUDA_DEVICE", str(local_rank))
            marmot = MarmotLibrary(FULL_LIB, BACKEND_CUDA)
            host_w = [make_weights(1000 * rank + i) for i in range(R)]
            runs = [marmot.linear_resident(KIND_Q4_K, host_w[i], F_DIM, K_DIM, T=T_TOK) for i in range(R)]
            del host_w

            def step_marmot():
                for i in range(R):
                    oh_np[i][...] = runs[i](xh_np[i])

            step_e2e, e2e_api = step_marmot, "marmot_linear on marmot_init(MARMOT_BACKEND_CUDA)"
    except Exception as exc:  # the library is optional on the box; say why it was not used
        e2e_api = f"mcu_linear_host (marmot API unavailable: {type(exc).__name__}: {exc})"[:200]
    for _ in range(args.warmup):
        step_e2e()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        step_e2e()
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    if marmot is not None:
        marmot.close()

    tp_section = moe_section = decode_section = sharded = None
    if not args.no_extra:
        tp_section = time_tp_decode_matmuls(ctx, dev, rank, world, dist)
        moe_section = time_moe_c5(ctx, dev, rank, world, dist)
        if LLAMA8B["kv"] // 128 % world == 0:
            decode_section = time_decode(ctx, dev, rank, world, dist)
        if world > 1:
            # The same two sharded workloads on ONE GPU, in this same run (every rank runs its own copy at the same time;
            # rank 0 reports its own), so that the strong-scaling efficiency has its denominator beside it.
            one_moe = time_moe_c5(ctx, dev, 0, 1, None)
            one_dec = time_decode(ctx, dev, 0, 1, None, c4_only=True) if decode_section is not None else None
            sharded = {"n_gpus": world, "timing": "device events (decode) / host wall clock (MoE), max over ranks; N=1 from this run, rank 0"}
            if one_dec is not None:
                a, b = one_dec["llama3_8b_64seq"], decode_section["llama3_8b_64seq"]
                sharded["llama3_8b_64seq_tensor_parallel"] = {
                    "n1_ms_per_step": a["ms_per_step"], "n1_tokens_per_s": a["tokens_per_s"], "ms_per_step": b["ms_per_step"],
                    "tokens_per_s": b["tokens_per_s"], "speedup": round(a["ms_per_step"] / b["ms_per_step"], 3),
                    "strong_scaling_efficiency": round(a["ms_per_step"] / b["ms_per_step"] / world, 3)}
                if "llama3_8b_64seq_replicas" in decode_section:
                    r = decode_section["llama3_8b_64seq_replicas"]
                    sharded["llama3_8b_64seq_replicas"] = {
                        "ms_per_step": r["ms_per_step"], "tokens_per_s": r["tokens_per_s"],
                        "speedup": round(a["ms_per_step"] / r["ms_per_step"], 3),
                        "strong_scaling_efficiency": round(a["ms_per_step"] / r["ms_per_step"] / world, 3)}
            if "ms_per_call" in one_moe and "ms_per_call" in moe_section:
                sharded["moe_mixtral_expert_ffn_expert_parallel"] = {
                    "n1_ms_per_call": one_moe["ms_per_call"], "ms_per_call": moe_section["ms_per_call"],
                    "tokens_per_s": round(moe_section["tokens"] / moe_section["ms_per_call"] * 1e3, 1),
                    "speedup": round(one_moe["ms_per_call"] / moe_section["ms_per_call"], 3),
                    "strong_scaling_efficiency": round(one_moe["ms_per_call"] / moe_section["ms_per_call"] / world, 3)}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    n_gemv = args.steps * R
    value = world * n_gemv * ALG_BYTES / (ms_dev * 1e-3) / 1e9
    e2e_value = world * e2e_steps * R * ALG_BYTES / e2e_s / 1e9
    peak, peak_kind = measured_peaks()
    # dominant kernel: the GEMV; its launches in the region == n_gemv.  Region time / launches is an
    # upper bound of its duration (it includes the small activation-quantisation kernel and launch gaps).
    per_launch_s = ms_dev * 1e-3 / n_gemv
    achieved = ALG_BYTES / per_launch_s / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 dot, f32 scale", "data": "synthetic",
        "config": workload_config(R),
        "launch": "eager" if args.no_graph else "cuda graph of one step, replayed",
        "gpu_launches": int(launches),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": R * T_TOK * K_DIM * 4,
                "d2h_bytes_per_step": R * T_TOK * F_DIM * 4, "steps": e2e_steps,
                "api": e2e_api,
                "note": "weights device resident; per GEMV the activations go host to device and the result comes back to "
                        "host memory inside the timed region, the host waits for each result"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_TRAFFIC_BYTES, "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of "
                     "one launch of this kernel and shape (profiles/gemv_stream_q4k_T1_K4096_F4096.md)",
                     "peak_source": peak_kind, "frac_of_nominal_8TBs": achieved / 8000.0,
                     "algorithmic_bytes": ALG_BYTES, "kernel": "gemv_stream_kernel<Q4_K, T=1, TW=14, TEAMS=1, MINB=2, PRO=none>",
                     "us_per_launch": per_launch_s * 1e6},
        "clocks": clocks,
    }
    if tp_section is not None:
        line["llama8b_decode_matmuls"] = tp_section
    if moe_section is not None:
        line["moe_mixtral_expert_ffn"] = moe_section
    if decode_section is not None:
        line["decode"] = decode_section
    if sharded is not None:
        line["sharded_scaling"] = sharded
    if not args.no_extra and world == 1:
        line["other_regimes"] = time_other_regimes(ctx, dev)
    if not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        cpu = CpuGemv(R, threads)
        iters = 8 * R
        dt = cpu.seconds(iters) / iters
        line["cpu_baseline"] = {"value": ALG_BYTES / dt / 1e9, "unit": UNIT, "cores": threads, "kind": cpu.kind,
                                "sample": f"{iters} GEMVs rotating over {R} weight copies ({dt * 1e3:.3f} ms each), one context"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
