"""Shared helpers for the parity tests: seeded synthetic tensors in the reference's block formats and
the error metric the tolerances are stated in."""
from __future__ import annotations

import numpy as np

from marmot_b200.synthetic import random_blocks  # noqa: F401  (the tests draw their weights with the product generator)

KIND_Q8_0, KIND_Q4_K, KIND_Q6_K = 5, 9, 11
KINDS = {"q4_k": KIND_Q4_K, "q6_k": KIND_Q6_K, "q8_0": KIND_Q8_0}
BLOCK_VALUES = {KIND_Q8_0: 32, KIND_Q4_K: 256, KIND_Q6_K: 256}
BLOCK_BYTES = {KIND_Q8_0: 34, KIND_Q4_K: 144, KIND_Q6_K: 210}

# fp32-accumulate kernels (activation quantizer emulated exactly): max relative error 2e-3
TOL_FP32 = 2e-3
# tensor-core kernels (fp16 operands, f32 accumulation): max relative error 1e-2
TOL_MMA = 1e-2
# MoE expert FFN: two chained matmuls with a GLU in between, and the intermediate is re-quantized to Q8_K, so a
# 1e-3 perturbation of the first stage flips quantizer roundings of the second stage's input (each flip is
# 1/127 of a block's amax).  The reference's own Q4_K + Q6_K MoE tests accept 8e-2 (decode) and 9e-2 (prefill)
# between its backends for this reason (tests/backend/test_backend_moe.c:901,1052,1147,1173).
TOL_MOE = 8e-2


def row_bytes(kind: int, K: int) -> int:
    bv = BLOCK_VALUES[kind]
    return (K + bv - 1) // bv * BLOCK_BYTES[kind]


def max_rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    """max |got-ref| / max(|ref|, rms(ref)): relative error per element, with the scale floored at the
    tensor's RMS so that outputs that happen to cancel to ~0 are judged against the typical magnitude."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    rms = float(np.sqrt(np.mean(ref * ref))) if ref.size else 0.0
    scale = np.maximum(np.abs(ref), max(rms, 1e-30))
    return float(np.max(np.abs(got - ref) / scale)) if ref.size else 0.0


def cosine(a: np.ndarray, b: np.ndarray) -> float:
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))


def unpack_q8_k(blocks: np.ndarray, T: int, nb: int):
    """Oracle Q8_K blocks (array of structs) -> (qs [T, nb*256] natural order, d [T, nb], bsums [T, nb*16])."""
    b = blocks.reshape(T, nb, 292)
    d = b[:, :, 0:4].copy().view(np.float32).reshape(T, nb)
    qs = b[:, :, 4:260].copy().view(np.int8).reshape(T, nb * 256)
    bsums = b[:, :, 260:292].copy().view(np.int16).reshape(T, nb * 16)
    return qs, d, bsums


def unsplit_q8_k(qs_split: np.ndarray) -> np.ndarray:
    """Undo the library's in-block order (value 64g+32b+i stored at b*128+g*32+i)."""
    T, kp = qs_split.shape
    v = qs_split.reshape(T, kp // 256, 2, 4, 32)       # [T, blk, b, g, i]
    return np.ascontiguousarray(v.transpose(0, 1, 3, 2, 4)).reshape(T, kp)  # [T, blk, g, b, i]


def unpack_q8_0(blocks: np.ndarray, T: int, nb: int):
    b = blocks.reshape(T, nb, 34)
    d = b[:, :, 0:2].copy().view(np.float16).astype(np.float32).reshape(T, nb)
    qs = b[:, :, 2:34].copy().view(np.int8).reshape(T, nb * 32)
    return qs, d
