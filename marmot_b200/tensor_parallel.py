"""Tensor- and expert-parallel sharding of quantized weights over the GPUs of one box (one process per GPU).

The reference engine runs on a single device and only reserves fields for sharding
(include/marmot/graph/kernel_selection.h:18-23: est_comm_us, shardable_axes, device_affinity are always 0),
so this layer has no reference counterpart; its results are checked against the unsharded operator.

Quantized weights are row-major [F, K] matrices of blocks (K/256 super-blocks of 144 or 210 bytes, or K/32
blocks of 34 bytes per row):

* column-parallel (split F: q/k/v, gate/up, vocabulary): a contiguous range of rows, no requantisation;
  every rank holds all of x and produces a slice of the features.
* row-parallel (split K: attention output, ffn_down): every row is cut at block granularity into `world`
  contiguous runs of blocks and each rank's runs are packed into its own contiguous [F, K/world] matrix at
  load.  Activation quantisation is per block along K, so a rank quantises only its K-slice and gets the
  very integers of the unsharded run; the partial results are summed by one all-reduce per output, in a
  fixed rank order.
* expert-parallel: experts are dealt out in contiguous ranges; the router runs replicated, every rank
  computes the routes of its own experts and the outputs are summed by the same all-reduce.

The collective is `torch.distributed.all_reduce` (NCCL on GPUs, gloo in CPU tests) or, with
`allreduce="peer"`, the library's own one-shot peer-memory kernel (marmot_cuda.h: mcu_peer_allreduce).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .runtime import BLOCK_BYTES, BLOCK_VALUES, row_bytes


def shard_range(n: int, world: int, rank: int, granule: int = 1) -> tuple[int, int]:
    """Contiguous [lo, hi) share of n items for `rank`, in whole granules, sizes differing by at most one granule."""
    if n % granule:
        raise ValueError(f"{n} is not a multiple of the granule {granule}")
    units = n // granule
    base, extra = divmod(units, world)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo * granule, hi * granule


def shard_rows(blocks: np.ndarray, kind: int, F: int, K: int, world: int, rank: int, granule: int = 1):
    """Column-parallel shard: rows [lo, hi) of a [F, K] quantized matrix.  Returns (bytes, lo, hi)."""
    rb = row_bytes(kind, K)
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(F, rb)
    lo, hi = shard_range(F, world, rank, granule)
    return np.ascontiguousarray(blocks[lo:hi]).reshape(-1), lo, hi


def k_granule(kind: int, K: int) -> int:
    """Granule (in values) for splitting K: the smallest run of blocks whose bytes are a multiple of 16, so that
    every shard's rows stay 16-byte multiples and the TMA-fed matmul applies (Q4_K: 256, Q6_K: 2048, Q8_0: 256);
    the block size when K is not a multiple of that."""
    bv, bb = BLOCK_VALUES[kind], BLOCK_BYTES[kind]
    blocks = 16 // np.gcd(bb, 16)
    return int(bv * blocks) if K % (bv * blocks) == 0 else bv


def shard_k(blocks: np.ndarray, kind: int, F: int, K: int, world: int, rank: int, granule: int | None = None):
    """Row-parallel shard: for every row the blocks covering K-range [k_lo, k_hi), packed as a contiguous
    [F, k_hi - k_lo] matrix.  Returns (bytes, k_lo, k_hi).  K must be a whole number of blocks; shards are whole
    granules (default k_granule), so they may differ in size by one granule and the last ranks may get none."""
    bv, bb = BLOCK_VALUES[kind], BLOCK_BYTES[kind]
    if K % bv:
        raise ValueError(f"K={K} is not a whole number of {bv}-value blocks")
    nb = K // bv
    g = granule or k_granule(kind, K)
    if g % bv:
        raise ValueError(f"granule {g} is not a whole number of {bv}-value blocks")
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(F, nb, bb)
    k_lo, k_hi = shard_range(K, world, rank, g)
    return np.ascontiguousarray(blocks[:, k_lo // bv:k_hi // bv]).reshape(-1), k_lo, k_hi


def shard_experts(stacked: np.ndarray, E: int, world: int, rank: int):
    """Expert-parallel shard of E stacked per-expert matrices.  Returns (bytes, e_lo, e_hi)."""
    stacked = np.ascontiguousarray(stacked, dtype=np.uint8).reshape(E, -1)
    lo, hi = shard_range(E, world, rank)
    return np.ascontiguousarray(stacked[lo:hi]).reshape(-1), lo, hi


@dataclass
class Group:
    """The ranks of one box.  `dist` is torch.distributed (None for a single rank)."""
    rank: int = 0
    world: int = 1
    dist: object = None

    def all_reduce_(self, t):
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return t

    def all_gather_features(self, t, sizes):
        """Concatenate per-rank feature slices [T, F_r] into [T, sum F_r] (ragged slices allowed)."""
        if self.world == 1:
            return t
        import torch

        width = max(sizes)
        padded = t if t.shape[1] == width else torch.nn.functional.pad(t, (0, width - t.shape[1]))
        parts = [torch.empty_like(padded) for _ in range(self.world)]
        self.dist.all_gather(parts, padded.contiguous())
        return torch.cat([p[:, :n] for p, n in zip(parts, sizes)], dim=1)

    def exchange_bytes(self, payload: bytes):
        if self.world == 1:
            return [payload]
        out = [None] * self.world
        self.dist.all_gather_object(out, payload)
        return out


class ColumnParallelLinear:
    """y[:, lo:hi] = x @ W[lo:hi].T on this rank; `gather=True` returns the full [T, F] on every rank."""

    def __init__(self, backend, group: Group, kind: int, blocks: np.ndarray, F: int, K: int, granule: int = 1):
        self.backend, self.group, self.kind, self.F, self.K = backend, group, kind, F, K
        shard, self.lo, self.hi = shard_rows(blocks, kind, F, K, group.world, group.rank, granule)
        self.sizes = [b - a for a, b in (shard_range(F, group.world, r, granule) for r in range(group.world))]
        self.weight = backend.upload(shard)

    def __call__(self, x, gather: bool = False):
        y = self.backend.linear(self.kind, x, self.weight, self.hi - self.lo)
        return self.group.all_gather_features(y, self.sizes) if gather else y


class RowParallelLinear:
    """y = sum over ranks of x[:, k_lo:k_hi] @ W[:, k_lo:k_hi].T; x may be the full activation (sliced here)
    or already this rank's slice (the output of a column-parallel layer)."""

    def __init__(self, backend, group: Group, kind: int, blocks: np.ndarray, F: int, K: int, comm=None,
                 granule: int | None = None):
        self.backend, self.group, self.kind, self.F, self.K = backend, group, kind, F, K
        shard, self.k_lo, self.k_hi = shard_k(blocks, kind, F, K, group.world, group.rank, granule)
        self.weight = backend.upload(shard) if self.k_hi > self.k_lo else None
        g = granule or k_granule(kind, K)
        spans = [shard_range(K, group.world, r, g) for r in range(group.world)]
        # a rank without a share cannot take part in the fused matmul + all-reduce kernel: then every rank runs the
        # matmul and the all-reduce kernel separately (all ranks must issue the same sequence of collectives)
        self.any_empty = any(hi == lo for lo, hi in spans)
        self.comm = comm  # runtime.PeerComm: the library's own all-reduce instead of torch.distributed

    def __call__(self, x):
        kw = self.k_hi - self.k_lo
        peer = self.comm is not None and self.group.world > 1
        if kw == 0:  # more ranks than granules: this rank contributes zeros
            import torch

            T = x.shape[0]
            if peer:
                self.comm.staging((T, self.F)).zero_()
                return self.comm.allreduce(T * self.F, torch.empty((T, self.F), dtype=torch.float32, device=x.device))
            return self.group.all_reduce_(torch.zeros((T, self.F), dtype=torch.float32, device=x.device))
        xs = x if x.shape[1] == kw else x[:, self.k_lo:self.k_hi]
        if peer and self.any_empty:
            import torch

            T = x.shape[0]
            self.backend.linear(self.kind, xs, self.weight, self.F, out=self.comm.staging((T, self.F)))
            return self.comm.allreduce(T * self.F, torch.empty((T, self.F), dtype=torch.float32, device=x.device))
        if peer:
            return self.comm.linear_allreduce(self.kind, xs, self.weight, self.F)
        y = self.backend.linear(self.kind, xs, self.weight, self.F)
        return self.group.all_reduce_(y)


class ExpertParallelMoE:
    """Mixture-of-experts FFN with the experts dealt out over the ranks; router results are replicated."""

    def __init__(self, backend, group: Group, kinds, gate: np.ndarray, up: np.ndarray, down: np.ndarray, H: int,
                 FF: int, E: int, comm=None):
        self.backend, self.group, self.kinds, self.H, self.FF, self.E = backend, group, tuple(kinds), H, FF, E
        g, self.e_lo, self.e_hi = shard_experts(gate, E, group.world, group.rank)
        u, _, _ = shard_experts(up, E, group.world, group.rank)
        d, _, _ = shard_experts(down, E, group.world, group.rank)
        self.gate, self.up, self.down = backend.upload(g), backend.upload(u), backend.upload(d)
        self.comm = comm

    def __call__(self, hidden, topk_ids, topk_weights, exchange: bool = True, **kw):
        """exchange: with a peer communicator large enough for (T * k + T) * H floats, the routed rows go back to the
        token owners and the token slices are gathered (every rank moves about 1 / world of what the all-reduce of
        whole outputs moves); otherwise, or for shapes off the grouped path, each rank's partial output is summed by an
        all-reduce."""
        T = hidden.shape[0]
        peer = self.comm is not None and self.group.world > 1
        if peer and exchange and (T * topk_ids.shape[1] + T) * self.H * 4 + 256 <= self.comm.max_bytes:
            from .runtime import MarmotCudaError

            bounds = [shard_range(self.E, self.group.world, r)[0] for r in range(self.group.world)] + [self.E]
            try:
                return self.comm.moe_experts_ep(self.kinds, hidden, self.gate, self.up, self.down, topk_ids, topk_weights,
                                                self.FF, self.E, bounds, **kw)
            except MarmotCudaError as exc:
                if exc.code != -8:  # NOT_IMPLEMENTED: every rank gets it for the same shape, and all fall through
                    raise
        out = self.comm.staging((T, self.H)) if peer else None
        y = self.backend.moe_experts_local(self.kinds, hidden, self.gate, self.up, self.down, topk_ids, topk_weights,
                                           self.FF, self.E, self.e_lo, self.e_hi - self.e_lo, out=out, **kw)
        if peer:
            import torch

            res = torch.empty((T, self.H), dtype=torch.float32, device=hidden.device)
            return self.comm.allreduce(T * self.H, res)
        return self.group.all_reduce_(y)


def make_peer_comm(backend, group: Group, max_bytes: int):
    """A PeerComm over the group's ranks; the IPC handles travel through torch.distributed."""
    from .runtime import PeerComm

    return PeerComm(backend, group.rank, group.world, max_bytes, group.exchange_bytes)
