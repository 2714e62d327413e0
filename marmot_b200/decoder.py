"""A Llama-shape decoder step driven through the C ABI: the op sequence the reference's GGUF graph builder emits per
layer (src/graph/gguf/graph_builder.cpp:1454-2400) -- rms_norm, linear q/k/v, rope, paged_attention (KV append inside),
linear o, add, rms_norm, linear gate/up, swiglu, linear down, add; tail rms_norm, linear output -- on random-init
weights of a named shape, quantized in the Q4_K_M mix (Q4_K everywhere, Q6_K for attn_v, ffn_down and output).

Plumbing only: every operator is one call into libmarmot_cuda; torch holds the buffers and replays the CUDA graph.
Used by bench.py (decode tokens/s of BASELINE configs 3 and 4) and by the decode parity test.
"""
from __future__ import annotations

import os

from dataclasses import dataclass

import numpy as np

from .runtime import KIND_Q4_K, KIND_Q6_K, Context, row_bytes


@dataclass
class DecoderShape:
    layers: int
    d: int
    ffn: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    vocab: int
    rope_theta: float = 10000.0
    rms_eps: float = 1e-5


TINYLLAMA_1B = DecoderShape(22, 2048, 5632, 32, 4, 64, 32000, 10000.0)
LLAMA3_8B = DecoderShape(32, 4096, 14336, 32, 8, 128, 128256, 500000.0)

# (name, quant kind, rows, cols as functions of the shape): the Q4_K_M mix
LAYER_WEIGHTS = (
    ("wq", KIND_Q4_K, lambda s: s.n_heads * s.head_dim, lambda s: s.d),
    ("wk", KIND_Q4_K, lambda s: s.n_kv_heads * s.head_dim, lambda s: s.d),
    ("wv", KIND_Q6_K, lambda s: s.n_kv_heads * s.head_dim, lambda s: s.d),
    ("wo", KIND_Q4_K, lambda s: s.d, lambda s: s.n_heads * s.head_dim),
    ("gate", KIND_Q4_K, lambda s: s.ffn, lambda s: s.d),
    ("up", KIND_Q4_K, lambda s: s.ffn, lambda s: s.d),
    ("down", KIND_Q6_K, lambda s: s.d, lambda s: s.ffn),
)


def weight_bytes(shape: DecoderShape) -> int:
    """Packed weight bytes one decode step streams (all layers + output projection; the embedding gather reads rows)."""
    per_layer = sum(rows(shape) * row_bytes(kind, cols(shape)) for _, kind, rows, cols in LAYER_WEIGHTS)
    return shape.layers * per_layer + shape.vocab * row_bytes(KIND_Q6_K, shape.d)


class Decoder:
    """`device_weights` are this rank's shards already on the device (what gguf.load_llama_decoder uploads), with
    `kinds[name]` naming each matrix's block format (a Q4_K_M file mixes Q4_K and Q6_K from layer to layer); otherwise
    weights are given as host byte arrays of the full model (`weights[name]`, per layer `weights[f"l{i}.{name}"]`;
    each rank cuts its own share out of them) or drawn on the device when `weights` is None (timing only).

    Tensor parallel over the ranks of `group` (tensor_parallel.Group) with `comm` (runtime.PeerComm): query and KV
    heads, the FFN width (in 2048-value granules, so that the Q6_K down shards keep 16-byte rows) and the vocabulary
    are dealt out; attention output and ffn_down are row-parallel with one all-reduce each; every rank keeps the
    residual stream, its own slice of the KV pool and finds the global argmax from the ranks' local maxima."""

    def __init__(self, ctx: Context, shape: DecoderShape, max_seqs: int, max_ctx: int, block_size: int = 16,
                 kv_dtype=None, weights: dict | None = None, seed: int = 0, group=None, comm=None, kv_pool=None,
                 device_weights: dict | None = None, kinds: dict | None = None):
        import torch

        from . import tensor_parallel as tp
        from .synthetic import normal_blocks

        self.ctx, self.shape, self.torch = ctx, shape, torch
        self.block_size, self.max_seqs = block_size, max_seqs
        dev = torch.device("cuda", ctx.device)
        self.dev = dev
        self.group = group or tp.Group()
        self.comm = comm
        world, rank = self.group.world, self.group.rank
        full = shape
        f_lo, f_hi, v_lo, v_hi = 0, shape.ffn, 0, shape.vocab
        if world > 1:
            if shape.n_kv_heads % world or shape.n_heads % world or comm is None:
                raise ValueError("heads must divide over the ranks and a PeerComm is needed")
            f_lo, f_hi = tp.shard_range(shape.ffn, world, rank, 2048)
            v_lo, v_hi = tp.shard_range(shape.vocab, world, rank, 32)
            self.v_lo = v_lo
            self.ffn_empty_somewhere = any(b == a for a, b in (tp.shard_range(shape.ffn, world, r, 2048) for r in range(world)))
            shape = DecoderShape(shape.layers, shape.d, f_hi - f_lo, shape.n_heads // world, shape.n_kv_heads // world,
                                 shape.head_dim, shape.vocab, shape.rope_theta, shape.rms_eps)
            self.local_vocab = v_hi - v_lo
        else:
            self.v_lo, self.local_vocab, self.ffn_empty_somewhere = 0, shape.vocab, False
        self.local = shape  # this rank's share of heads / FFN width (d, layers, vocab as in the full shape)
        s = shape
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed + 1000 * rank)

        default_kinds = {n: k for n, k, _, _ in LAYER_WEIGHTS}
        default_kinds.update(tok_embd=KIND_Q4_K, output=KIND_Q6_K)
        self.kinds = {}

        def kind_of(name):
            return (kinds or {}).get(name, default_kinds[name.split(".")[-1]])

        def cut(name, kind, w):
            """This rank's share of a full-model matrix: heads, FFN rows and vocabulary rows are contiguous row ranges;
            the two row-parallel matrices are cut along K (block columns repacked per row)."""
            base = name.split(".")[-1]
            if world == 1 or base == "tok_embd":
                return w
            if base in ("wq", "wk", "wv"):
                F = (full.n_heads if base == "wq" else full.n_kv_heads) * full.head_dim
                return tp.shard_rows(w, kind, F, full.d, world, rank, F // world)[0]
            if base == "wo":
                K = full.n_heads * full.head_dim
                return tp.shard_k(w, kind, full.d, K, world, rank, K // world)[0]
            if base in ("gate", "up"):
                return tp.shard_rows(w, kind, full.ffn, full.d, world, rank, 2048)[0]
            if base == "down":
                return tp.shard_k(w, kind, full.d, full.ffn, world, rank, 2048)[0]
            if base == "output":
                return tp.shard_rows(w, kind, full.vocab, full.d, world, rank, 32)[0]
            raise KeyError(name)

        def mat(name, kind, rows, cols):
            kind = self.kinds[name] = kind_of(name)
            if device_weights is not None:
                return device_weights[name]
            if rows == 0 or cols == 0:
                return None
            if weights is not None:
                return ctx.upload(cut(name, kind, weights[name]))
            return normal_blocks(torch, kind, rows, cols, dev, gen).reshape(-1)  # random init: N(0, 0.02), quantised

        def vec(name, n):
            if device_weights is not None:
                return device_weights[name]
            if weights is not None:
                return torch.from_numpy(np.ascontiguousarray(weights[name], dtype=np.float32)).to(dev)
            return torch.ones(n, dtype=torch.float32, device=dev)

        self.layers = []
        for i in range(s.layers):
            lw = {name: mat(f"l{i}.{name}", kind, rows(s), cols(s)) for name, kind, rows, cols in LAYER_WEIGHTS}
            lw["attn_norm"] = vec(f"l{i}.attn_norm", s.d)
            lw["ffn_norm"] = vec(f"l{i}.ffn_norm", s.d)
            self.layers.append(lw)
        gen.manual_seed(seed)  # the embedding table is replicated: the same on every rank
        self.tok_embd = mat("tok_embd", KIND_Q4_K, s.vocab, s.d)
        gen.manual_seed(seed + 77 + 1000 * rank)
        self.output = mat("output", KIND_Q6_K, self.local_vocab, s.d)
        self.out_norm = vec("out_norm", s.d)

        self.max_blocks = (max_ctx + block_size - 1) // block_size
        self.kv_pool = kv_pool
        if kv_pool is not None:
            # blocks, block table and kv slots come from a runtime.KvPool (the caller plans appends with it and builds
            # token_meta from the slots it hands out): what a serving engine with sequences coming and going does
            self.kv_k, self.kv_v, self.block_table = kv_pool.tensors()
            want = (s.layers, s.n_kv_heads, block_size, s.head_dim)
            if tuple(self.kv_k.shape[1:]) != want:
                raise ValueError(f"KV pool blocks are {tuple(self.kv_k.shape[1:])}, the model needs {want}")
            self.max_blocks = self.block_table.shape[1]
        else:
            n_blocks = max_seqs * self.max_blocks
            kv_dtype = kv_dtype or torch.float16
            pool = (n_blocks, s.layers, s.n_kv_heads, block_size, s.head_dim)
            self.kv_k = torch.zeros(pool, dtype=kv_dtype, device=dev)
            self.kv_v = torch.zeros(pool, dtype=kv_dtype, device=dev)
            # sequence i owns the blocks [i*max_blocks, (i+1)*max_blocks): a static block table
            table = np.arange(n_blocks, dtype=np.uint32).reshape(max_seqs, self.max_blocks)
            self.block_table = torch.from_numpy(table).to(dev)
        self._bufs = {}
        self._plans = {}  # one-token step plans (persistent kernel), per set of caller tensors
        self._side = None

    def _side_contexts(self):
        """Two more contexts on streams of their own (each with its own workspace), for the key and value projections,
        which read the same normalised activations as the query projection and are small enough at decode batch sizes
        that their duration is mostly fixed latency: the three run side by side and rejoin before RoPE.  The fork and
        the join are stream-to-stream waits, so a CUDA-graph capture of the step records them as graph edges."""
        if self._side is None:
            import os

            torch = self.torch
            if os.environ.get("MARMOT_DECODER_SERIAL_QKV"):  # diagnostic switch: one stream, three calls in turn
                self._side = ()
            else:
                streams = [torch.cuda.Stream(self.dev) for _ in range(2)]
                ctxs = [Context(self.ctx.device, use_torch_stream=False) for _ in streams]
                for c, st in zip(ctxs, streams):
                    c.set_stream(st.cuda_stream)
                self._side = (ctxs, streams)
        return self._side

    def _main_stream(self):
        handle = self.ctx.lib.mcu_context_get_stream(self.ctx.handle) or 0
        if handle in (0, 1):  # the legacy default stream
            return self.torch.cuda.default_stream(self.dev)
        return self.torch.cuda.ExternalStream(handle, device=self.dev)

    def _buf(self, name, shape, dtype=None):
        key = (name, tuple(shape))
        if key not in self._bufs:
            self._bufs[key] = self.torch.empty(shape, dtype=dtype or self.torch.float32, device=self.dev)
        return self._bufs[key]

    def token_meta(self, seq_slots, positions, kv_slots=None):
        """[T, 4] u32 rows {seq_slot, pos, kv_slot, flags} for tokens at `positions` of sequences `seq_slots`; with a
        KV pool the kv slots are the ones its prepare_append returned."""
        seq = np.asarray(seq_slots, dtype=np.int64)
        pos = np.asarray(positions, dtype=np.int64)
        if kv_slots is not None:
            return np.stack([seq, pos, np.asarray(kv_slots, dtype=np.int64), np.zeros_like(seq)], axis=1).astype(np.uint32)
        if self.kv_pool is not None:
            raise ValueError("with a KV pool, pass the kv slots that prepare_append returned")
        block = seq * self.max_blocks + pos // self.block_size
        kv_slot = block * self.block_size + pos % self.block_size
        return np.stack([seq, pos, kv_slot, np.zeros_like(seq)], axis=1).astype(np.uint32)

    def _row_parallel(self, kind, x, w, F, out, K):
        """out = all-reduce over the ranks of x @ w.T (this rank's K-slice)."""
        if self.group.world == 1:
            return self.ctx.linear(kind, x, w, F, out=out)
        T = x.shape[0]
        if K == 0:  # this rank has no share of the FFN width: it adds zeros
            self.comm.staging((T, F)).zero_()
            return self.comm.allreduce(T * F, out)
        if self.ffn_empty_somewhere and K == self.local.ffn:  # all ranks must then use the two-kernel form
            self.ctx.linear(kind, x, w, F, out=self.comm.staging((T, F)))
            return self.comm.allreduce(T * F, out)
        return self.comm.linear_allreduce(kind, x, w, F, out=out)

    def greedy(self, logits, ids_out):
        """Global argmax of the ranks' logits slices into ids_out (int32 [T]); two small all-reduces gather the local
        maxima (an even number keeps the communicator's staging parity stable across CUDA-graph replays)."""
        ctx, torch = self.ctx, self.torch
        T = logits.shape[0]
        if self.group.world == 1:
            return ctx.argmax(logits, out=ids_out)
        world, rank = self.group.world, self.group.rank
        local_idx = ctx.argmax(logits, out=self._buf("lidx", (T,), torch.int32))
        local_val = logits.gather(1, local_idx.long().unsqueeze(1)).squeeze(1)
        vals, idxs = self._buf("gvals", (T, world)), self._buf("gidx", (T, world))
        for src, dst in ((local_val, vals), ((local_idx + self.v_lo).float(), idxs)):
            st = self.comm.staging((T, world))
            st.zero_()
            st[:, rank] = src
            self.comm.allreduce(T * world, dst)
        best = vals.argmax(dim=1, keepdim=True)  # ties: the lowest rank, i.e. the lowest vocabulary index
        ids_out.copy_(idxs.gather(1, best).squeeze(1).to(torch.int32))
        return ids_out

    def step(self, ids, meta, positions, logits_out=None, decode=False):
        """One forward pass for T tokens: ids int32 [T], meta u32 [T, 4], positions int32 [T] (device tensors).
        Returns logits [T, vocab] (tensor parallel: this rank's vocabulary slice [T, local_vocab]).

        decode=True promises at most one token per sequence in the call (a decode step): RoPE, the KV append, the
        attention and the merge of its context chunks then run as one kernel, and on one GPU every elementwise step
        (residual add + RMSNorm, SwiGLU) rides in the prologue of the matmul that consumes it -- five launches per layer
        for up to eight tokens."""
        if decode and self.group.world == 1 and ids.shape[0] <= 8:
            return self._step_fused(ids, meta, positions, logits_out)
        ctx, s = self.ctx, self.local
        T = ids.shape[0]
        hq, hkv, hd = s.n_heads, s.n_kv_heads, s.head_dim
        kd = self.kinds
        x = ctx.embedding_gather(kd["tok_embd"], self.tok_embd, s.d, ids, out=self._buf("x", (T, s.d)))
        h = self._buf("h", (T, s.d))
        q, k, v = self._buf("q", (T, hq * hd)), self._buf("k", (T, hkv * hd)), self._buf("v", (T, hkv * hd))
        att, proj = self._buf("att", (T, hq * hd)), self._buf("proj", (T, s.d))
        gate, up = self._buf("gate", (T, max(s.ffn, 1))), self._buf("up", (T, max(s.ffn, 1)))
        scale = float(hd) ** -0.5
        # the residual add that ends a block and the rms_norm that opens the next one run as one kernel
        ctx.rmsnorm(x, self.layers[0]["attn_norm"], s.rms_eps, out=h)
        # up to eight tokens q / k / v are one launch; beyond, three matmuls that run side by side on streams of their own
        side = self._side_contexts() if T > 8 else ()
        fuse_ffn = T > 16 and s.ffn > 0 and not os.environ.get("MARMOT_DECODER_UNFUSED_FFN")  # (diagnostic switch)
        main = self._main_stream() if side else None
        for i, lw in enumerate(self.layers):
            if side:
                (ctx_k, ctx_v), (st_k, st_v) = side
                st_k.wait_stream(main)
                st_v.wait_stream(main)
                ctx_k.linear(kd[f"l{i}.wk"], h, lw["wk"], hkv * hd, out=k)
                ctx_v.linear(kd[f"l{i}.wv"], h, lw["wv"], hkv * hd, out=v)
                ctx.linear(kd[f"l{i}.wq"], h, lw["wq"], hq * hd, out=q)
                main.wait_stream(st_k)
                main.wait_stream(st_v)
            else:
                ctx.linear_multi(h, [(kd[f"l{i}.wq"], lw["wq"], hq * hd, q), (kd[f"l{i}.wk"], lw["wk"], hkv * hd, k),
                                     (kd[f"l{i}.wv"], lw["wv"], hkv * hd, v)])
            if decode:
                if i == 0:
                    rope = ctx.rope_table(positions, hd, s.rope_theta, out=self._buf("rope", (T, hd // 2, 2)))
                ctx.paged_attention_decode(meta, q, k, v, self.kv_k, self.kv_v, self.block_table, i, hq, hkv, hd,
                                           self.block_size, scale, positions, s.rope_theta, rope_table=rope, out=att)
            else:
                ctx.rope_qk(q, k, positions, hq, hkv, hd, s.rope_theta)
                ctx.paged_attention(meta, q, k, v, self.kv_k, self.kv_v, self.block_table, i, hq, hkv, hd, self.block_size,
                                    scale, out=att)
            self._row_parallel(kd[f"l{i}.wo"], att, lw["wo"], s.d, proj, hq * hd)
            if fuse_ffn:
                # the residual add + RMSNorm ride in the staging of gate / up; the sum goes to the other residual buffer
                # (the prologue's output may not be its input)
                x_next = self._buf("x2" if x is self._buf("x", (T, s.d)) else "x", (T, s.d))
                ctx.linear_multi(x, [(kd[f"l{i}.gate"], lw["gate"], s.ffn, gate), (kd[f"l{i}.up"], lw["up"], s.ffn, up)],
                                 ("add_rmsnorm", proj, lw["ffn_norm"], s.rms_eps, 0.0, x_next))
                x = x_next
                # SwiGLU stays a kernel of its own here: inside the staging kernel (one CTA per token) it ran over
                # 14336 values per CTA on 64 CTAs and cost 29 us against 7 + 6 us for the two kernels, measured
                ctx.swiglu(gate, up, out=gate)
                self._row_parallel(kd[f"l{i}.down"], gate, lw["down"], s.d, proj, s.ffn)
            else:
                ctx.add_rmsnorm(x, proj, lw["ffn_norm"], s.rms_eps, x, h)
                if s.ffn > 0:
                    ctx.linear_multi(h, [(kd[f"l{i}.gate"], lw["gate"], s.ffn, gate), (kd[f"l{i}.up"], lw["up"], s.ffn, up)])
                    ctx.swiglu(gate, up, out=gate)
                self._row_parallel(kd[f"l{i}.down"], gate, lw["down"], s.d, proj, s.ffn)
            nxt = self.layers[i + 1]["attn_norm"] if i + 1 < len(self.layers) else self.out_norm
            ctx.add_rmsnorm(x, proj, nxt, s.rms_eps, x, h)
        logits = logits_out if logits_out is not None else self._buf("logits", (T, self.local_vocab))
        ctx.linear(kd["output"], h, self.output, self.local_vocab, out=logits)
        return logits

    def _one_token_plan(self, meta, positions, logits):
        """The persistent-kernel plan for a one-token step on these very tensors (mcu_decode_plan), or None when the
        model does not suit it (formats other than Q4_K / Q6_K, float32 pool, ...).  Plans are kept per tensor set."""
        import ctypes as C

        from .runtime import DecodeLayer, DecodePlan, DecodePlanDesc, MarmotCudaError, _ptr

        if os.environ.get("MARMOT_DECODER_NO_STEP_KERNEL"):  # diagnostic switch: the five-launch layer instead
            return None
        # The kernel's attention gives a query head one CTA: right for the contexts of single-sequence decoding, slower
        # than the five-launch layer's attention once a layer's cache runs to thousands of positions.
        if self.max_blocks * self.block_size > int(os.environ.get("MARMOT_DECODER_STEP_KERNEL_MAX_CTX", "2560")):
            return None
        key = (meta.data_ptr(), positions.data_ptr(), logits.data_ptr())
        if key in self._plans:
            return self._plans[key]
        s, kd = self.local, self.kinds
        hq, hkv, hd = s.n_heads, s.n_kv_heads, s.head_dim
        plan = None
        if self.kv_k.dtype == self.torch.float16 and s.ffn > 0 and hq * hd == s.d:
            L = len(self.layers)
            layers = (DecodeLayer * L)()
            for i, (slot, lw) in enumerate(zip(layers, self.layers)):
                for name in ("q", "k", "v", "o"):
                    setattr(slot, f"kind_{name}", kd[f"l{i}.w{name}"])
                    setattr(slot, f"w{name}", _ptr(lw[f"w{name}"]))
                for name in ("gate", "up", "down"):
                    setattr(slot, f"kind_{name}", kd[f"l{i}.{name}"])
                    setattr(slot, name, _ptr(lw[name]))
                slot.attn_norm, slot.ffn_norm = _ptr(lw["attn_norm"]), _ptr(lw["ffn_norm"])
            buf = lambda name, n: self._buf(name, (1, n))
            rope = self._buf("rope", (1, hd // 2, 2))
            d = DecodePlanDesc()
            d.n_layers, d.d, d.ffn, d.n_q_heads, d.n_kv_heads, d.head_dim, d.vocab = L, s.d, s.ffn, hq, hkv, hd, self.local_vocab
            d.rms_eps, d.attn_scale, d.rope_type = s.rms_eps, float(hd) ** -0.5, 0
            d.layers, d.out_norm, d.kind_output, d.output = layers, _ptr(self.out_norm), kd["output"], _ptr(self.output)
            d.x0, d.x1 = _ptr(buf("x", s.d)), _ptr(buf("x2", s.d))
            d.q, d.k, d.v = _ptr(buf("q", hq * hd)), _ptr(buf("k", hkv * hd)), _ptr(buf("v", hkv * hd))
            d.att, d.proj = _ptr(buf("att", hq * hd)), _ptr(buf("proj", s.d))
            d.gate, d.up, d.logits = _ptr(buf("gate", s.ffn)), _ptr(buf("up", s.ffn)), _ptr(logits)
            d.token_meta, d.block_table, d.max_blocks_per_seq = _ptr(meta), _ptr(self.block_table), self.block_table.shape[1]
            d.kv_k, d.kv_v, d.kv_dtype, d.block_size, d.rope_table = _ptr(self.kv_k), _ptr(self.kv_v), 1, self.block_size, _ptr(rope)
            try:
                plan = DecodePlan(self.ctx, d, keep=(layers, meta, positions, logits))
            except MarmotCudaError as exc:
                if exc.code != -8:  # NOT_IMPLEMENTED: this model takes the five-launch layer
                    raise
        self._plans[key] = plan
        return plan

    def _step_fused(self, ids, meta, positions, logits_out):
        """The decode step with every elementwise operator folded into its consumer (see step).  One token: a single
        persistent kernel walks all layers (mcu_decode_plan; embedding gather and RoPE table before it).  Otherwise five
        launches per layer; the residual stream alternates between two buffers: a prologue reads x and the pending
        projection and stores their sum to the other buffer (the CTAs of one launch all read x, so the sum cannot go
        back in place)."""
        ctx, s = self.ctx, self.local
        T = ids.shape[0]
        if T == 1:
            logits = logits_out if logits_out is not None else self._buf("logits", (1, self.local_vocab))
            plan = self._one_token_plan(meta, positions, logits)
            if plan is not None:
                ctx.embedding_gather(self.kinds["tok_embd"], self.tok_embd, s.d, ids, out=self._buf("x", (1, s.d)))
                ctx.rope_table(positions, s.head_dim, s.rope_theta, out=self._buf("rope", (1, s.head_dim // 2, 2)))
                plan.run()
                return logits
        hq, hkv, hd = s.n_heads, s.n_kv_heads, s.head_dim
        kd = self.kinds
        xs = [self._buf("x", (T, s.d)), self._buf("x2", (T, s.d))]
        cur = 0
        ctx.embedding_gather(kd["tok_embd"], self.tok_embd, s.d, ids, out=xs[0])
        q, k, v = self._buf("q", (T, hq * hd)), self._buf("k", (T, hkv * hd)), self._buf("v", (T, hkv * hd))
        att, proj = self._buf("att", (T, hq * hd)), self._buf("proj", (T, s.d))
        gate, up = self._buf("gate", (T, max(s.ffn, 1))), self._buf("up", (T, max(s.ffn, 1)))
        scale = float(hd) ** -0.5
        pending = None  # the projection not yet added to the residual stream
        rope = ctx.rope_table(positions, hd, s.rope_theta, out=self._buf("rope", (T, hd // 2, 2)))
        for i, lw in enumerate(self.layers):
            ctx.linear_multi(xs[cur], [(kd[f"l{i}.wq"], lw["wq"], hq * hd, q), (kd[f"l{i}.wk"], lw["wk"], hkv * hd, k),
                                       (kd[f"l{i}.wv"], lw["wv"], hkv * hd, v)],
                             ("add_rmsnorm", pending, lw["attn_norm"], s.rms_eps, 0.0, xs[1 - cur] if pending is not None else None))
            if pending is not None:
                cur = 1 - cur
            ctx.paged_attention_decode(meta, q, k, v, self.kv_k, self.kv_v, self.block_table, i, hq, hkv, hd,
                                       self.block_size, scale, positions, s.rope_theta, rope_table=rope, out=att)
            ctx.linear(kd[f"l{i}.wo"], att, lw["wo"], s.d, out=proj)
            pending = proj
            if s.ffn > 0:
                ctx.linear_multi(xs[cur], [(kd[f"l{i}.gate"], lw["gate"], s.ffn, gate), (kd[f"l{i}.up"], lw["up"], s.ffn, up)],
                                 ("add_rmsnorm", pending, lw["ffn_norm"], s.rms_eps, 0.0, xs[1 - cur]))
                cur = 1 - cur
                ctx.linear_multi(gate, [(kd[f"l{i}.down"], lw["down"], s.d, proj)], ("swiglu", up))
                pending = proj
        logits = logits_out if logits_out is not None else self._buf("logits", (T, self.local_vocab))
        ctx.linear_multi(xs[cur], [(kd["output"], self.output, self.local_vocab, logits)],
                         ("add_rmsnorm", pending, self.out_norm, s.rms_eps, 0.0, None))
        return logits
