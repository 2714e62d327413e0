"""Seeded synthetic weights in the reference's GGUF block formats, for benchmarks, smoke checks and tests.

No checkpoint travels with the library, so every measurement runs on payloads drawn here.  Two families:

* `random_blocks`: the value distributions the benchmark configurations state (fp16 block scales drawn from
  |N(0, sigma)|, 6-bit sub-block scales / mins and the quants uniform) - every bit pattern of the payload is a
  legal block, so the blocks can be drawn directly without running a weight quantizer.
* `synthetic_blocks` / `synthetic_blocks_device`: uniformly random payload bytes with the exponent of the fp16 block
  scale clamped to a small finite range.  Cheaper to draw (GB-sized models on the GPU in milliseconds); used where
  only the timing matters.  These are NOT quantized N(0, 0.02) weights.
"""
from __future__ import annotations

import numpy as np

KIND_Q8_0, KIND_Q4_K, KIND_Q6_K = 5, 9, 11
BLOCK_VALUES = {KIND_Q8_0: 32, KIND_Q4_K: 256, KIND_Q6_K: 256}
BLOCK_BYTES = {KIND_Q8_0: 34, KIND_Q4_K: 144, KIND_Q6_K: 210}


def random_blocks(kind: int, rows: int, K: int, rng: np.random.Generator, d_sigma: float | None = None) -> np.ndarray:
    """`rows` rows of K values as packed blocks (uint8, row-major): fp16 d / dmin = |N(0, sigma)|, 6-bit scales /
    mins uniform, quants uniform."""
    bv, bb = BLOCK_VALUES[kind], BLOCK_BYTES[kind]
    nb = (K + bv - 1) // bv
    n = rows * nb
    out = np.empty((n, bb), dtype=np.uint8)
    if kind == KIND_Q4_K:
        sigma = 0.02 if d_sigma is None else d_sigma
        out[:, 0:2] = np.abs(rng.normal(0, sigma, n)).astype(np.float16).view(np.uint8).reshape(n, 2)
        out[:, 2:4] = np.abs(rng.normal(0, sigma, n)).astype(np.float16).view(np.uint8).reshape(n, 2)
        out[:, 4:] = rng.integers(0, 256, (n, 140), dtype=np.uint8)  # scales (6-bit fields) + nibbles
    elif kind == KIND_Q6_K:
        sigma = 0.002 if d_sigma is None else d_sigma
        out[:, :192] = rng.integers(0, 256, (n, 192), dtype=np.uint8)
        out[:, 192:208] = rng.integers(-64, 64, (n, 16)).astype(np.int8).view(np.uint8)
        out[:, 208:210] = np.abs(rng.normal(0, sigma, n)).astype(np.float16).view(np.uint8).reshape(n, 2)
    else:
        sigma = 0.01 if d_sigma is None else d_sigma
        out[:, 0:2] = np.abs(rng.normal(0, sigma, n)).astype(np.float16).view(np.uint8).reshape(n, 2)
        out[:, 2:] = rng.integers(-127, 128, (n, 32)).astype(np.int8).view(np.uint8)
    return out.reshape(-1)


def _scale_columns(kind: int):
    """Byte columns holding the high byte of an fp16 block scale."""
    return (1, 3) if kind == KIND_Q4_K else (209,) if kind == KIND_Q6_K else (1,)


def synthetic_blocks(kind: int, rows: int, K: int, rng: np.random.Generator) -> np.ndarray:
    """Random block payloads with finite fp16 scales (high byte 0x1C..0x1F is roughly 0.004..0.008)."""
    nb = (K + BLOCK_VALUES[kind] - 1) // BLOCK_VALUES[kind]
    blocks = rng.integers(0, 256, (rows * nb, BLOCK_BYTES[kind]), dtype=np.uint8)
    scale_hi = rng.integers(0x1C, 0x20, rows * nb, dtype=np.uint8)
    for col in _scale_columns(kind):
        blocks[:, col] = scale_hi
    return blocks.reshape(-1)


def synthetic_blocks_device(torch, kind: int, rows: int, K: int, device, generator=None):
    """The same on the GPU (a uint8 tensor), for weights too large to draw on the host in reasonable time."""
    nb = (K + BLOCK_VALUES[kind] - 1) // BLOCK_VALUES[kind]
    blocks = torch.randint(0, 256, (rows * nb, BLOCK_BYTES[kind]), dtype=torch.uint8, device=device, generator=generator)
    scale_hi = torch.randint(0x1C, 0x20, (rows * nb,), dtype=torch.uint8, device=device, generator=generator)
    for col in _scale_columns(kind):
        blocks[:, col] = scale_hi
    return blocks.reshape(-1)
