#!/usr/bin/env python3
"""Build the reference's own CPU backend into oracle/_ref/libmarmot_ref.so.

Test infrastructure only: the product (marmot_b200/) never loads this library.

The reference (darekhta/marmot) builds with meson + clang on macOS; neither is available here and its Linux/x86 gcc
build is broken as shipped.  This recipe compiles the C core and the CPU backend (scalar flavour, no libdispatch)
with gcc directly from the reference checkout.  Nothing from the reference is copied into this repository: sources
are staged in a temporary directory outside the repo, five build fixes (no arithmetic changes; listed in
marmot_b200/host/marmot_tree.py, which does the staging) are applied to the staged copy, objects are compiled
there, and only the linked shared library lands in oracle/_ref/ (git-ignored).

Flags: -std=c2x -O2 -march=x86-64-v3 -ffp-contract=off, MARMOT_ENABLE_AVX2=0 (scalar kernels: the reference's x86
"AVX2" K-quant dots are the scalar C code under another name, and the scalar flavour fixes the activation rounding
mode).
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
if str(HERE.parent) not in sys.path:
    sys.path.insert(0, str(HERE.parent))

from marmot_b200.host import marmot_tree  # noqa: E402
from marmot_b200.host.marmot_tree import CFLAGS, DEFINES  # noqa: E402

OUT_DIR = HERE / "_ref"
OUT_LIB = OUT_DIR / "libmarmot_ref.so"


def build(ref_root: Path, jobs: int | None = None, verbose: bool = True) -> Path:
    ref_root = ref_root.resolve()
    if not (ref_root / "meson.build").exists():
        raise FileNotFoundError(f"reference checkout not found at {ref_root}")
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    sources = marmot_tree.c_sources(ref_root)

    stage = Path(tempfile.mkdtemp(prefix="marmot_ref_stage_"))
    try:
        marmot_tree.stage(ref_root, stage)
        incs = [f"-I{stage / p}" for p in marmot_tree.INCLUDE_DIRS]
        objdir = stage / "obj"
        objdir.mkdir()

        def compile_one(idx_src):
            idx, src = idx_src
            obj = objdir / f"{idx:03d}_{Path(src).stem}.o"
            cmd = ["gcc", *CFLAGS, *DEFINES, *incs, "-c", str(stage / src), "-o", str(obj)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            return src, obj, r.returncode, r.stderr

        objs, failed = [], []
        with cf.ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as ex:
            for src, obj, rc, err in ex.map(compile_one, enumerate(sources)):
                if rc == 0:
                    objs.append(str(obj))
                else:
                    failed.append((src, err.strip().splitlines()[:3]))
        if verbose:
            print(f"[build_ref] compiled {len(objs)}/{len(sources)} translation units", file=sys.stderr)
            for src, err in failed:
                print(f"[build_ref]   failed: {src}: {err}", file=sys.stderr)
        if failed:
            raise RuntimeError(f"{len(failed)} reference translation units failed to compile")
        tmp_lib = stage / "libmarmot_ref.so"
        link = ["gcc", "-shared", "-o", str(tmp_lib), *objs, "-lm", "-pthread", "-Wl,--allow-shlib-undefined"]
        subprocess.run(link, check=True)
        shutil.copyfile(tmp_lib, OUT_LIB)
    finally:
        shutil.rmtree(stage, ignore_errors=True)
    return OUT_LIB


KV_POOL_LIB = OUT_DIR / "libmarmot_ref_kvpool.so"
KV_POOL_SOURCES = ("src/inference/kv_pool/kv_pool.cpp", "src/inference/common/storage.cpp", "src/api/kv_pool_api.cpp")


def build_kv_pool(ref_root: Path) -> Path:
    """The reference's paged KV-cache pool (C++23, three translation units compiled where they lie) as a second
    library beside libmarmot_ref.so, which supplies the tensor API it uses.  The checker of the CUDA pool's books."""
    ref_root = ref_root.resolve()
    if not OUT_LIB.exists():
        raise FileNotFoundError("build libmarmot_ref.so first")
    newest = max((ref_root / s).stat().st_mtime for s in KV_POOL_SOURCES)
    if KV_POOL_LIB.exists() and KV_POOL_LIB.stat().st_mtime >= max(newest, OUT_LIB.stat().st_mtime):
        return KV_POOL_LIB
    stage = Path(tempfile.mkdtemp(prefix="marmot_ref_kvpool_"))
    try:
        objs = []
        for i, src in enumerate(KV_POOL_SOURCES):
            obj = stage / f"{i}.o"
            subprocess.run(["g++", "-std=c++23", "-O1", "-fPIC", "-w", "-include", "utility", "-include", "cmath", *DEFINES,
                            f"-I{ref_root / 'include'}", f"-I{ref_root / 'src'}", f"-I{ref_root}", "-c", str(ref_root / src),
                            "-o", str(obj)], check=True)
            objs.append(str(obj))
        tmp = stage / KV_POOL_LIB.name
        subprocess.run(["g++", "-shared", "-o", str(tmp), *objs, f"-L{OUT_DIR}", f"-l:{OUT_LIB.name}", "-Wl,-rpath,$ORIGIN"],
                       check=True)
        shutil.copyfile(tmp, KV_POOL_LIB)
    finally:
        shutil.rmtree(stage, ignore_errors=True)
    return KV_POOL_LIB


def find_reference_root() -> Path | None:
    """The marmot checkout to build from: $MARMOT_REFERENCE_ROOT, else a directory `reference` beside this
    repository; None when neither holds a marmot source tree."""
    cands = []
    if os.environ.get("MARMOT_REFERENCE_ROOT"):
        cands.append(Path(os.environ["MARMOT_REFERENCE_ROOT"]))
    cands.append(Path(__file__).resolve().parent.parent.parent / "reference")
    for c in cands:
        if (c / "meson.build").exists() and (c / "include" / "marmot").is_dir():
            return c
    return None


if __name__ == "__main__":
    root = Path(sys.argv[1]) if len(sys.argv) > 1 else find_reference_root()
    if root is None:
        sys.exit("no marmot checkout: pass its path or set MARMOT_REFERENCE_ROOT")
    print(build(root))
    print(build_kv_pool(root))
