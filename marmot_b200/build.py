"""Build libmarmot_cuda.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "libmarmot_cuda.so"
OBJ_DIR = PKG / "build"

SOURCES = ["abi.cu", "act_quant.cu", "dequant.cu", "gemv.cu", "gemv_stream.cu", "gemv_stream_addnorm.cu", "gemv_stream_swiglu.cu", "gemm_tc.cu", "gemm_tma.cu", "gemm_warp.cu", "gemm_i8.cu", "linear_f16.cu", "moe.cu", "static_scratch.cu", "peer.cu", "decoder.cu", "decode_step.cu", "kv_pool.cu", "gguf.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else "nvcc"


def _newest_input() -> float:
    files = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    files.append(PKG.parent / "include" / "marmot_cuda.h")
    return max(f.stat().st_mtime for f in files)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and OUT.exists() and OUT.stat().st_mtime >= _newest_input():
        return OUT
    OBJ_DIR.mkdir(exist_ok=True)
    nvcc = _nvcc()
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: str):
        obj = OBJ_DIR / (src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", str(CSRC / src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, obj, r

    objs = []
    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 4)) as ex:
        for src, obj, r in ex.map(compile_one, SOURCES):
            if verbose or r.returncode != 0:
                sys.stderr.write(f"--- {src}\n{r.stdout}{r.stderr}\n")
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}")
            objs.append(str(obj))
    subprocess.run([nvcc, "-shared", "-o", str(OUT), *objs, "-lcudart"], check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
