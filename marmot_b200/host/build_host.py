"""Build libmarmot_cuda_backend.so: the C23 host layer (cuda_backend.c) compiled against marmot's own
headers and linked to libmarmot_cuda.so.

The marmot headers are not part of this package, so the build needs a marmot source checkout
(`MARMOT_SOURCE_DIR`, or the path given to build()).  The marmot_* helper symbols the layer calls
(marmot_set_error, marmot_matmul_validate_quantized, ...) stay undefined in the library and resolve at load
time against libmarmot, exactly as a backend object inside the marmot build would.
"""
from __future__ import annotations

import os
import subprocess
from pathlib import Path

HOST = Path(__file__).resolve().parent
PKG = HOST.parent
OUT = PKG / "libmarmot_cuda_backend.so"
SRC = HOST / "cuda_backend.c"


def build(marmot_root: Path | None = None, force: bool = False) -> Path:
    root = Path(marmot_root or os.environ.get("MARMOT_SOURCE_DIR", ""))
    if not (root / "include" / "marmot" / "device.h").exists():
        raise FileNotFoundError(f"no marmot checkout at {root!s} (set MARMOT_SOURCE_DIR)")
    cuda_lib = PKG / "libmarmot_cuda.so"
    if not cuda_lib.exists():
        raise FileNotFoundError("build libmarmot_cuda.so first (marmot_b200/build.py)")
    newest = max(SRC.stat().st_mtime, (PKG.parent / "include" / "marmot_cuda.h").stat().st_mtime)
    if not force and OUT.exists() and OUT.stat().st_mtime >= newest:
        return OUT
    cmd = [
        os.environ.get("CC", "gcc"), "-std=c2x", "-O2", "-fPIC", "-shared", "-Wall", "-Wextra", "-D_GNU_SOURCE",
        f"-I{root / 'include'}", f"-I{root / 'src'}", f"-I{PKG.parent / 'include'}",
        str(SRC), "-o", str(OUT), f"-L{PKG}", "-lmarmot_cuda", "-Wl,-rpath,$ORIGIN", "-lpthread",
    ]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    import sys

    print(build(Path(sys.argv[1]) if len(sys.argv) > 1 else None, force=True))
