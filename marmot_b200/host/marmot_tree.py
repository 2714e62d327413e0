"""Staging a marmot source checkout for a gcc / Linux build.

marmot (darekhta/marmot) builds with meson + clang on macOS; its Linux / x86 gcc build is broken as shipped.  The
recipes that compile it here - the CPU checker library the tests compare against and the full library with the
CUDA backend linked in (marmot_b200/host/build_marmot.py) - first copy the checkout to a temporary directory and
apply five build fixes there, none of which changes arithmetic:

  1. src/backends/cpu/cpu_backend_internal.h: cpu_sincosf / cpu_sincos have a second
     `#if defined(__GNUC__) && !defined(__clang__)` body that redefines the locals of the `__has_builtin` body
     under gcc -> second body dropped.
  2. same header: `__STDC_VERSION__ >= 202311L` guard around the _Float16 bit helpers -> `>= 202000L` (gcc 13
     -std=c2x reports 202000).
  3. src/backends/cpu/ops/matmul/quantized/matmul_quant_compute.c: the `#if NEON && aarch64 && DOTPROD` block opened
     before the NEON row kernels swallows the portable tile dispatchers (no matching #endif) -> closed before the
     portable section and re-opened before the row-panel section.
  4. src/backends/cpu/cpu_caps.c: MARMOT_PROFILE_AVX512 is not an enumerator ->
     -DMARMOT_PROFILE_AVX512=MARMOT_PROFILE_AVX2 (in DEFINES).
  5. src/backends/cpu/memory/allocator.c: `huge_alignment` declared twice in one scope on Linux -> second
     declaration renamed.

Nothing of the checkout is copied into this repository: the staged copy lives in a temporary directory and only
linked libraries leave it.
"""
from __future__ import annotations

import re
import shutil
from pathlib import Path

DEFINES = [
    "-D_GNU_SOURCE",
    "-DMARMOT_ENABLE_NEON=0", "-DMARMOT_ENABLE_AVX2=0", "-DMARMOT_ENABLE_AVX512=0",
    "-DMARMOT_ENABLE_SCALAR=1", "-DMARMOT_ENABLE_FP8=1", "-DMARMOT_ENABLE_ACCELERATE=0",
    "-DMARMOT_ENABLE_LIBDISPATCH=0", "-DMARMOT_ENABLE_METAL=0",
    "-DMARMOT_PROFILE_AVX512=MARMOT_PROFILE_AVX2",
]
CFLAGS = ["-std=c2x", "-O2", "-march=x86-64-v3", "-ffp-contract=off", "-fPIC", "-w", "-pthread"]
INCLUDE_DIRS = ("include", "src", "src/graph", "src/backends/cpu", "src/backends/metal", "third_party/yyjson", ".")

# C++ translation units (graph / inference / tokenizer / api) are not on the quantized-matmul path and are left out;
# the C core references a few of their symbols lazily, so the libraries link with --allow-shlib-undefined.
SKIP_SUBSTR = (
    "/neon/matmul_neon.c",  # unconditional <arm_neon.h>
)


def meson_sources(meson_text: str, var: str) -> list[str]:
    m = re.search(rf"{var}\s*=\s*files\((.*?)\n\)", meson_text, re.S)
    assert m, var
    return re.findall(r"'([^']+)'", m.group(1))


def c_sources(ref_root: Path) -> list[str]:
    """The C translation units of marmot's core, utilities and CPU backend, from its meson source lists."""
    meson = (ref_root / "meson.build").read_text()
    sources = [s for s in meson_sources(meson, "core_sources") if s.endswith(".c")]
    sources += meson_sources(meson, "utils_sources")
    sources += [s for s in meson_sources(meson, "cpu_backend_sources") if s.endswith(".c")]
    return [s for s in sources if not any(k in "/" + s for k in SKIP_SUBSTR)]


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


def stage(ref_root: Path, stage_dir: Path, with_codegen: bool = False) -> None:
    """Copy what a build needs from the checkout into `stage_dir` and apply the build fixes."""
    shutil.copytree(ref_root / "include", stage_dir / "include")
    shutil.copytree(ref_root / "src", stage_dir / "src", ignore=shutil.ignore_patterns("*.metal", "*.mm"))
    (stage_dir / "third_party").mkdir()
    shutil.copytree(ref_root / "third_party" / "yyjson", stage_dir / "third_party" / "yyjson")
    if with_codegen:
        shutil.copytree(ref_root / "scripts" / "codegen", stage_dir / "scripts" / "codegen",
                        ignore=shutil.ignore_patterns("__pycache__"))
    _patch(stage_dir / "src/backends/cpu/cpu_backend_internal.h", _fix_internal_header)
    _patch(stage_dir / "src/backends/cpu/ops/matmul/quantized/matmul_quant_compute.c", _fix_compute)
    _patch(stage_dir / "src/backends/cpu/memory/allocator.c", _fix_allocator)
