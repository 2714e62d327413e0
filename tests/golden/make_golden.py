#!/usr/bin/env python3
"""Regenerate the committed golden fixtures.  Needs the reference checkout; run once, commit the .npz files.

Two fixture files are produced next to this script:

* ``llama_goldens.npz`` - the known-answer vectors the reference's own tests
  hold for the Q4_K / Q6_K / Q8_0 path (llama.cpp-generated): the quantized
  matmul cases of tests/backend/golden_matmul_llama.h, the row-dot scalars of
  tests/backend/golden_vec_dot_llama.h and the quantizer blocks + dequantised
  values of tests/backend/golden_quant_llama.h.  They are read by compiling a
  small dumper against those headers (the arrays are C initialisers).
* ``decoder_cases.npz`` - RMSNorm / RoPE / SwiGLU / paged attention of the reference CPU backend on seeded inputs
* ``ref_cases.npz`` - seeded inputs pushed through the reference CPU backend
  itself (oracle/_ref/libmarmot_ref.so): quantized weights, dequantised values,
  matmul and MoE outputs at small ragged shapes.

Usage: python tests/golden/make_golden.py [reference_root]
"""
from __future__ import annotations

import os
import struct
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(REPO))

DUMPER = r"""
#include <stdio.h>
#include <stdint.h>
#include "marmot/quant_block.h"
#include "backend/golden_matmul_llama.h"
#include "backend/golden_vec_dot_llama.h"
#include "backend/golden_quant_llama.h"
static void put(FILE *f, const char *name, const void *p, size_t n) {
    uint32_t len = (uint32_t)strlen(name);
    uint64_t bytes = n;
    fwrite(&len, 4, 1, f); fwrite(name, 1, len, f); fwrite(&bytes, 8, 1, f); fwrite(p, 1, n, f);
}
#define PUT(x) put(f, #x, &(x), sizeof(x))
#define MATMUL(l, U) do { \
    uint64_t dims[3] = {MATMUL_##U##_N, MATMUL_##U##_K, MATMUL_##U##_M}; \
    put(f, "matmul_" #l "_dims", dims, sizeof(dims)); \
    PUT(g_matmul_##l##_input_f32); PUT(g_matmul_##l##_weight); PUT(g_matmul_##l##_output_from_f32); \
    PUT(g_matmul_##l##_input_f16); PUT(g_matmul_##l##_output_from_f16); } while (0)
int main(int argc, char **argv) {
    FILE *f = fopen(argv[1], "wb");
    MATMUL(q4_k, Q4_K); MATMUL(q6_k, Q6_K); MATMUL(q8_0, Q8_0);
    PUT(g_vec_dot_q8_0_activations); PUT(g_vec_dot_q8_k_activations);
    PUT(g_vec_dot_q4_k_weights); PUT(g_vec_dot_q6_k_weights); PUT(g_vec_dot_q8_0_weights);
    PUT(g_vec_dot_q4_k_q8_k_expected); PUT(g_vec_dot_q6_k_q8_k_expected); PUT(g_vec_dot_q8_0_q8_0_expected);
    PUT(g_llama_test_input);
    PUT(g_llama_q4_k); PUT(g_llama_q4_k_dequant);
    PUT(g_llama_q6_k); PUT(g_llama_q6_k_dequant);
    PUT(g_llama_q8_0); PUT(g_llama_q8_0_dequant);
    fclose(f);
    return 0;
}
"""

F32_KEYS = ("input_f32", "output_from_f32", "output_from_f16", "expected", "dequant", "test_input")  # input_f16 stays raw bytes


def dump_reference_goldens(ref_root: Path) -> dict[str, np.ndarray]:
    with tempfile.TemporaryDirectory() as td:
        src = Path(td) / "dump.c"
        src.write_text("#include <string.h>\n" + DUMPER)
        exe = Path(td) / "dump"
        subprocess.run(
            ["gcc", "-std=c2x", "-w", f"-I{ref_root / 'include'}", f"-I{ref_root / 'tests'}", str(src), "-o", str(exe)],
            check=True,
        )
        blob = Path(td) / "out.bin"
        subprocess.run([str(exe), str(blob)], check=True)
        data = blob.read_bytes()
    out, pos = {}, 0
    while pos < len(data):
        (ln,) = struct.unpack_from("<I", data, pos); pos += 4
        name = data[pos:pos + ln].decode(); pos += ln
        (nb,) = struct.unpack_from("<Q", data, pos); pos += 8
        raw = data[pos:pos + nb]; pos += nb
        key = name.removeprefix("g_")
        if key.endswith("_dims"):
            out[key] = np.frombuffer(raw, dtype=np.uint64).astype(np.int64)
        elif any(key.endswith(s) for s in F32_KEYS):
            out[key] = np.frombuffer(raw, dtype=np.float32).copy()
        else:
            out[key] = np.frombuffer(raw, dtype=np.uint8).copy()
    return out


def make_ref_cases() -> dict[str, np.ndarray]:
    from oracle.bindings import (KIND_Q4_K, KIND_Q6_K, KIND_Q8_0, POLICY_RENORMALIZE_SELECTED,
                                 POLICY_SOFTMAX_SELECTED, Oracle, Reference)
    ref = Reference(threads=os.cpu_count())
    orc = Oracle()
    out: dict[str, np.ndarray] = {}
    rng = np.random.default_rng(0xB200)
    shapes = {"q4_k": (KIND_Q4_K, [(1, 256, 5), (3, 768, 17), (17, 512, 33)]),
              "q6_k": (KIND_Q6_K, [(1, 256, 5), (5, 512, 9), (16, 1024, 31)]),
              "q8_0": (KIND_Q8_0, [(1, 64, 3), (2, 96, 7), (33, 2144, 12)])}
    for name, (kind, cases) in shapes.items():
        for i, (T, K, F) in enumerate(cases):
            w = rng.normal(0, 0.05, (F, K)).astype(np.float32)
            x = rng.normal(0, 1, (T, K)).astype(np.float32)
            if i == 1:
                x[0, : K // 2] = 0.0  # an all-zero activation block
            W = ref.quantize(kind, w)
            out[f"{name}_{i}_w"] = W
            out[f"{name}_{i}_x"] = x
            out[f"{name}_{i}_deq"] = ref.dequantize(kind, W, F * K)
            out[f"{name}_{i}_y"] = ref.linear(kind, x, W, F)
    # MoE: Q4_K gate/up + Q6_K down (the Q4_K_M mix), grouped and small-batch routes
    T, H, FF, E, k = 21, 256, 512, 4, 2
    hid = rng.normal(0, 1, (T, H)).astype(np.float32)
    gate = np.concatenate([ref.quantize(KIND_Q4_K, rng.normal(0, 0.05, (FF, H)).astype(np.float32)) for _ in range(E)])
    up = np.concatenate([ref.quantize(KIND_Q4_K, rng.normal(0, 0.05, (FF, H)).astype(np.float32)) for _ in range(E)])
    down = np.concatenate([ref.quantize(KIND_Q6_K, rng.normal(0, 0.05, (H, FF)).astype(np.float32)) for _ in range(E)])
    logits = rng.normal(0, 1, (T, E)).astype(np.float32)
    p = np.exp(logits - logits.max(1, keepdims=True))
    p = (p / p.sum(1, keepdims=True)).astype(np.float32)
    vals, ids = orc.topk(p, k)
    kinds = (KIND_Q4_K, KIND_Q4_K, KIND_Q6_K)
    out.update(moe_hidden=hid, moe_gate=gate, moe_up=up, moe_down=down, moe_probs=p, moe_ids=ids, moe_weights=vals,
               moe_dims=np.array([T, H, FF, E, k], dtype=np.int64))
    out["moe_out_renorm"] = ref.moe_experts(kinds, hid, gate, up, down, ids, vals, FF, E,
                                            policy=POLICY_RENORMALIZE_SELECTED)
    out["moe_out_softmax"] = ref.moe_experts(kinds, hid, gate, up, down, ids, vals, FF, E,
                                             policy=POLICY_SOFTMAX_SELECTED, weights_scale=0.5)
    out["moe_out_decode"] = ref.moe_experts(kinds, hid[:3], gate, up, down, ids[:3], vals[:3], FF, E)
    ref.close()
    return out


def make_decoder_cases() -> dict[str, np.ndarray]:
    """RMSNorm / RoPE / SwiGLU / paged-attention outputs of the reference CPU backend (one thread: see
    tests/test_oracle_decoder.py) on seeded inputs; the attention cases are the ones the tests rebuild."""
    from oracle.bindings import Reference
    from tests.test_oracle_decoder import ATTENTION_CASES, attention_case

    ref = Reference(threads=1)
    rng = np.random.default_rng(99)
    out: dict[str, np.ndarray] = {}
    x = rng.normal(0, 2, (5, 256)).astype(np.float32)
    w = rng.normal(1, 0.1, 256).astype(np.float32)
    res = rng.normal(0, 1, (5, 256)).astype(np.float32)
    out.update(rms_x=x, rms_w=w, rms_res=res, rms_out=ref.rmsnorm(x, w, 1e-5, residual=res))
    xr = rng.normal(0, 1, (6, 128)).astype(np.float32)
    pos = np.array([0, 1, 31, 255, 1000, 4095], dtype=np.int32)
    out.update(rope_x=xr, rope_pos=pos, rope_out=ref.rope(xr, pos, 500000.0))
    a, b = rng.normal(0, 3, 512).astype(np.float32), rng.normal(0, 1, 512).astype(np.float32)
    out.update(glu_a=a, glu_b=b, glu_out=ref.swiglu(a, b))
    for name in sorted(ATTENTION_CASES):
        case = attention_case(np.random.default_rng(sum(map(ord, name))), **ATTENTION_CASES[name])
        o, kk, vv = ref.paged_attention(case["meta"], case["q"], case["k_new"], case["v_new"], case["kv_k"].copy(),
                                        case["kv_v"].copy(), case["table"], case["layer"], case["block_size"],
                                        case["scale"])
        for k, v in case.items():
            out[f"{name}.{k}"] = np.asarray(v)
        out[f"{name}.out"] = o
        out[f"{name}.kv_k_after"] = kk
    ref.close()
    return out


def make_kv_pool_traces() -> dict:
    """Everything observable of the reference's KV-cache pool (status codes, sequence and kv slots, free counts, block
    tables) on the seeded random schedules of tests/kv_pool_ref.py:drive."""
    import json

    from oracle.bindings import Reference
    from tests.kv_pool_ref import RefKvPool
    from tests.test_kv_pool_cpu import CONFIGS, run

    ref = Reference()
    out = {}
    for name in sorted(CONFIGS):
        for seed in (1, 2):
            pool = RefKvPool(ref, **CONFIGS[name])
            out[f"{name}/{seed}"] = json.loads(json.dumps(run(pool, name, seed)))
            pool.close()
    ref.close()
    return out


def main() -> None:
    from oracle.build_ref import find_reference_root

    ref_root = Path(sys.argv[1]) if len(sys.argv) > 1 else find_reference_root()
    if ref_root is None:
        sys.exit("no marmot checkout: pass its path or set MARMOT_REFERENCE_ROOT")
    np.savez_compressed(HERE / "llama_goldens.npz", **dump_reference_goldens(ref_root))
    np.savez_compressed(HERE / "ref_cases.npz", **make_ref_cases())
    np.savez_compressed(HERE / "decoder_cases.npz", **make_decoder_cases())
    import json

    (HERE / "kv_pool_traces.json").write_text(json.dumps(make_kv_pool_traces(), separators=(",", ":")))
    for f in ("llama_goldens.npz", "ref_cases.npz", "decoder_cases.npz", "kv_pool_traces.json"):
        print(f, (HERE / f).stat().st_size, "bytes")


if __name__ == "__main__":
    main()
