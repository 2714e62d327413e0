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


# ---------------------------------------------------------------------------------------------------------------
# Quantising f32 weights into the block formats.  A plain min/max quantiser written with torch tensor operations, so
# that GB-sized random-init models can be quantised on the GPU in well under a second (or on the host for tests).
# It is NOT the reference's weight quantiser (a search over candidate scales, src/backends/cpu/quantization/
# common/kquant_common.h); it produces legal blocks whose dequantised values approximate the input with the
# format's own step, which is what a random-init benchmark model needs.
# ---------------------------------------------------------------------------------------------------------------
def _f16_bytes(torch, x):
    """f32 tensor [n] -> uint8 tensor [n, 2] holding the fp16 bit patterns (little endian)."""
    return x.to(torch.float16).contiguous().view(torch.uint8).reshape(-1, 2)


def quantize_rows(torch, kind: int, w):
    """w [rows, K] f32 (K a multiple of the block size) -> packed blocks, uint8 tensor on w's device."""
    rows, K = w.shape
    bv = BLOCK_VALUES[kind]
    if K % bv:
        raise ValueError("K must be a whole number of blocks")
    n = rows * (K // bv)
    w = w.reshape(n, bv).to(torch.float32)
    out = torch.empty((n, BLOCK_BYTES[kind]), dtype=torch.uint8, device=w.device)
    if kind == KIND_Q8_0:
        d = w.abs().amax(dim=1) / 127.0
        d16 = d.to(torch.float16)
        inv = torch.where(d16 > 0, 1.0 / d16.to(torch.float32), torch.zeros_like(d))
        q = torch.clamp(torch.round(w * inv[:, None]), -127, 127).to(torch.int8)
        out[:, 0:2] = _f16_bytes(torch, d)
        out[:, 2:] = q.view(torch.uint8)
    elif kind == KIND_Q4_K:
        s = w.reshape(n, 8, 32)
        mn = torch.clamp(-s.amin(dim=2), min=0.0)                   # sub-block offsets (value = scale*q - min)
        sc = (s.amax(dim=2) + mn) / 15.0                            # sub-block steps
        d16 = (sc.amax(dim=1) / 63.0).to(torch.float16)
        m16 = (mn.amax(dim=1) / 63.0).to(torch.float16)
        d, dm = d16.to(torch.float32), m16.to(torch.float32)
        isc = torch.where(d[:, None] > 0, torch.clamp(torch.round(sc / d[:, None].clamp(min=1e-30)), 0, 63), torch.zeros_like(sc))
        imn = torch.where(dm[:, None] > 0, torch.clamp(torch.round(mn / dm[:, None].clamp(min=1e-30)), 0, 63), torch.zeros_like(mn))
        step = d[:, None] * isc
        q = torch.where(step[:, :, None] > 0,
                        torch.round((s + (dm[:, None] * imn)[:, :, None]) / step[:, :, None].clamp(min=1e-30)),
                        torch.zeros_like(s))
        q = torch.clamp(q, 0, 15).to(torch.uint8)
        isc, imn = isc.to(torch.uint8), imn.to(torch.uint8)
        out[:, 0:2] = _f16_bytes(torch, d)
        out[:, 2:4] = _f16_bytes(torch, dm)
        # 6-bit (scale, min) pairs packed into 12 bytes, the inverse of get_scale_min_k4
        out[:, 4:8] = (isc[:, 0:4] & 63) | ((isc[:, 4:8] >> 4) << 6)
        out[:, 8:12] = (imn[:, 0:4] & 63) | ((imn[:, 4:8] >> 4) << 6)
        out[:, 12:16] = (isc[:, 4:8] & 15) | ((imn[:, 4:8] & 15) << 4)
        q = q.reshape(n, 4, 2, 32)                                  # [64-value group][low / high nibble][32]
        out[:, 16:] = (q[:, :, 0, :] | (q[:, :, 1, :] << 4)).reshape(n, 128)
    elif kind == KIND_Q6_K:
        s = w.reshape(n, 16, 16)
        amax = s.abs().amax(dim=2)
        sc = amax / 31.0                                            # sub-block steps (values -32..31)
        d16 = (sc.amax(dim=1) / 127.0).to(torch.float16)
        d = d16.to(torch.float32)
        isc = torch.where(d[:, None] > 0, torch.clamp(torch.round(sc / d[:, None].clamp(min=1e-30)), 0, 127), torch.zeros_like(sc))
        step = d[:, None] * isc
        q = torch.where(step[:, :, None] > 0, torch.round(s / step[:, :, None].clamp(min=1e-30)), torch.zeros_like(s))
        q = (torch.clamp(q, -32, 31) + 32).to(torch.uint8).reshape(n, 2, 4, 32)   # [half][32-value run][32]
        lo, hi = q & 15, q >> 4
        # per 128-value half: ql[l] = run0 | run2 << 4, ql[l + 32] = run1 | run3 << 4, qh[l] = two bits of each run
        ql = torch.stack([lo[:, :, 0] | (lo[:, :, 2] << 4), lo[:, :, 1] | (lo[:, :, 3] << 4)], dim=2)  # [n, 2, 2, 32]
        qh = hi[:, :, 0] | (hi[:, :, 1] << 2) | (hi[:, :, 2] << 4) | (hi[:, :, 3] << 6)                # [n, 2, 32]
        out[:, 0:128] = ql.reshape(n, 128)
        out[:, 128:192] = qh.reshape(n, 64)
        out[:, 192:208] = isc.to(torch.int8).view(torch.uint8)
        out[:, 208:210] = _f16_bytes(torch, d)
    else:
        raise ValueError(f"kind {kind}")
    return out.reshape(-1)


def normal_blocks(torch, kind: int, rows: int, K: int, device, generator=None, sigma: float = 0.02, chunk_rows: int = 8192):
    """Random-init weights N(0, sigma) quantised into `kind` blocks, drawn and quantised on `device` in row chunks."""
    parts = []
    for r0 in range(0, rows, chunk_rows):
        r = min(chunk_rows, rows - r0)
        w = torch.randn((r, K), device=device, generator=generator, dtype=torch.float32) * sigma
        parts.append(quantize_rows(torch, kind, w))
    return torch.cat(parts) if len(parts) > 1 else parts[0]
