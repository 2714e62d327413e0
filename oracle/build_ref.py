#!/usr/bin/env python3
"""Build the reference's own CPU backend into oracle/_ref/libmarmot_ref.so.

Test infrastructure only: the product (marmot_b200/) never loads this library.

The reference (darekhta/marmot) builds with meson + clang on macOS; neither is
available here and its Linux/x86 gcc build is broken as shipped.  This recipe
compiles the C core and the CPU backend (scalar flavour, no libdispatch) with
gcc directly from the reference checkout.  Nothing from the reference is copied
into this repository: sources are staged in a temporary directory outside the
repo, five build fixes (no arithmetic changes) are applied to the staged copy,
objects are compiled there, and only the linked shared library lands in
oracle/_ref/ (git-ignored).

Build fixes applied to the staged copy:
  1. src/backends/cpu/cpu_backend_internal.h: cpu_sincosf/cpu_sincos have a
     second `#if defined(__GNUC__) && !defined(__clang__)` body that redefines
     the locals of the `__has_builtin` body under gcc -> second body dropped.
  2. same header: `__STDC_VERSION__ >= 202311L` guard around the _Float16 bit
     helpers -> `>= 202000L` (gcc 13 -std=c2x reports 202000).
  3. src/backends/cpu/ops/matmul/quantized/matmul_quant_compute.c: the
     `#if NEON && aarch64 && DOTPROD` block opened before the NEON row kernels
     swallows the portable tile dispatchers (no matching #endif) -> close it
     before the portable section and re-open it before the row-panel section.
  4. src/backends/cpu/cpu_caps.c: MARMOT_PROFILE_AVX512 is not an enumerator ->
     -DMARMOT_PROFILE_AVX512=MARMOT_PROFILE_AVX2.
  5. src/backends/cpu/memory/allocator.c: `huge_alignment` declared twice in one
     scope on Linux -> second declaration renamed.

Flags: -std=c2x -O2 -march=x86-64-v3 -ffp-contract=off, MARMOT_ENABLE_AVX2=0
(scalar kernels: the reference's x86 "AVX2" K-quant dots are the scalar C code
under another name, and the scalar flavour fixes the activation rounding mode).
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import re
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
OUT_LIB = OUT_DIR / "libmarmot_ref.so"

DEFINES = [
    "-D_GNU_SOURCE",
    "-DMARMOT_ENABLE_NEON=0", "-DMARMOT_ENABLE_AVX2=0", "-DMARMOT_ENABLE_AVX512=0",
    "-DMARMOT_ENABLE_SCALAR=1", "-DMARMOT_ENABLE_FP8=1", "-DMARMOT_ENABLE_ACCELERATE=0",
    "-DMARMOT_ENABLE_LIBDISPATCH=0", "-DMARMOT_ENABLE_METAL=0",
    "-DMARMOT_PROFILE_AVX512=MARMOT_PROFILE_AVX2",
]
CFLAGS = ["-std=c2x", "-O2", "-march=x86-64-v3", "-ffp-contract=off", "-fPIC", "-w", "-pthread"]

# C++ translation units (graph / inference / tokenizer / api) are not on the
# quantized-matmul path and are left out; the C core references a few of their
# symbols lazily, so the library links with --allow-shlib-undefined semantics.
SKIP_SUBSTR = (
    "/neon/matmul_neon.c",  # unconditional <arm_neon.h>
)


def _meson_sources(meson_text: str, var: str) -> list[str]:
    m = re.search(rf"{var}\s*=\s*files\((.*?)\n\)", meson_text, re.S)
    assert m, var
    return re.findall(r"'([^']+)'", m.group(1))


def _patch(path: Path, fn) -> None:
    text = path.read_text()
    new = fn(text)
    if new == text:
        raise RuntimeError(f"build fix did not apply: {path}")
    path.write_text(new)


def _fix_internal_header(text: str) -> str:
    # (1) drop the second, gcc-only body of cpu_sincosf / cpu_sincos
    pat = re.compile(
        r"#if defined\(__GNUC__\) && !defined\(__clang__\)\n"
        r"\s+(?:float|double) sin_val = 0\.0f?;\n.*?\n\s+return;\n#endif\n",
        re.S,
    )
    text, n = pat.subn("", text)
    if n != 2:
        raise RuntimeError(f"expected 2 duplicate sincos bodies, found {n}")
    # (2) C23 version guard
    return text.replace(
        "#if defined(__STDC_VERSION__) && __STDC_VERSION__ >= 202311L\nstatic inline _Float16 marmot_f16_from_bits",
        "#if defined(__STDC_VERSION__) && __STDC_VERSION__ >= 202000L\nstatic inline _Float16 marmot_f16_from_bits",
    )


NEON_IF = "#if MARMOT_ENABLE_NEON && defined(__aarch64__) && defined(__ARM_FEATURE_DOTPROD)\n"


def _fix_compute(text: str) -> str:
    # (3) close the NEON block before the portable fp16-tile context struct and
    # re-open it before the NEON row-panel dispatcher.
    anchor_close = (
        "typedef struct {\n    const cpu_matmul_quant_kernel_t *kernel;\n    const uint8_t *weight_bytes;\n"
        "    size_t row_bytes;\n    size_t blocks_per_row;\n    const marmot_float16_t *const *activation_rows;\n"
    )
    prev = "cpu_quant_matmul_q6_k_decoded_row_panel_dispatch_range_dual(void *ctx"
    if text.count(prev) != 1 or anchor_close not in text:
        raise RuntimeError("portable-section anchor not found")
    close_at = text.index(anchor_close, text.index(prev))
    text = text[:close_at] + "#endif\n" + text[close_at:]
    anchor_open = "void cpu_quant_matmul_dispatch_quant_tile_row_panel(\n"
    first = text.index(anchor_open)
    return text[:first] + NEON_IF + text[first:]


def _fix_allocator(text: str) -> str:
    # (5) second declaration in the same scope
    needle = (
        "#endif\n            const size_t huge_alignment = (size_t)2 * 1024 * 1024;\n"
        "            request_alignment = normalize_alignment(alignment == 0 ? huge_alignment : alignment);"
    )
    repl = (
        "#endif\n            const size_t huge_alignment_fallback = (size_t)2 * 1024 * 1024;\n"
        "            request_alignment = normalize_alignment(alignment == 0 ? huge_alignment_fallback : alignment);"
    )
    return text.replace(needle, repl)


def build(ref_root: Path, jobs: int | None = None, verbose: bool = True) -> Path:
    ref_root = ref_root.resolve()
    if not (ref_root / "meson.build").exists():
        raise FileNotFoundError(f"reference checkout not found at {ref_root}")
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    meson = (ref_root / "meson.build").read_text()
    sources = [s for s in _meson_sources(meson, "core_sources") if s.endswith(".c")]
    sources += _meson_sources(meson, "utils_sources")
    sources += [s for s in _meson_sources(meson, "cpu_backend_sources") if s.endswith(".c")]
    sources = [s for s in sources if not any(k in "/" + s for k in SKIP_SUBSTR)]

    stage = Path(tempfile.mkdtemp(prefix="marmot_ref_stage_"))
    try:
        shutil.copytree(ref_root / "include", stage / "include")
        shutil.copytree(
            ref_root / "src", stage / "src",
            ignore=shutil.ignore_patterns("metal", "*.metal", "*.mm"),
        )
        (stage / "third_party").mkdir()
        shutil.copytree(ref_root / "third_party" / "yyjson", stage / "third_party" / "yyjson")
        _patch(stage / "src/backends/cpu/cpu_backend_internal.h", _fix_internal_header)
        _patch(stage / "src/backends/cpu/ops/matmul/quantized/matmul_quant_compute.c", _fix_compute)
        _patch(stage / "src/backends/cpu/memory/allocator.c", _fix_allocator)

        incs = [f"-I{stage / p}" for p in (
            "include", "src", "src/graph", "src/backends/cpu", "src/backends/metal", "third_party/yyjson", ".")]
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
