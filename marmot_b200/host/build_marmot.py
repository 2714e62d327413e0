"""Build libmarmot with the CUDA backend in it: marmot_b200/libmarmot_b200.so.

What a marmot maintainer would get from adding this backend to the tree, done here on a temporary copy of a marmot
checkout (nothing of marmot is copied into this repository; only the linked library leaves the copy):

  1. stage the checkout with the gcc / Linux build fixes (marmot_tree.py);
  2. add the backend where marmot expects one: `src/backends/cuda/kernels/*.def` (this package's host/kernels/, plus
     the metadata sets the CPU backend's `.def` files share), `src/backends/cuda/cuda_backend.{c,h}`;
  3. register it with the kernel-DSL code generator: a `CUDA_CONFIG` entry in scripts/codegen/backend_config.py
     (which handler each operator family calls), then run scripts/codegen/gen_kernels.py for `cpu metal cuda`
     together - the kernel ids in include/marmot/traits_ids.gen.h are shared by all backends - which emits
     `marmot_cuda_query_kernel`, the `marmot_cuda_*_exec` dispatch wrappers and the bytecode tables
     `marmot_cuda_bc_{imm_size,schema_id,exec_table}`;
  4. give the three switch statements of the core their CUDA case: `marmot_init` (src/core/context/context.c),
     kernel query / default caps / default preferences (src/core/dispatch/kernel_query.c) and the bytecode tables
     (src/core/bytecode/bytecode_compile.c);
  5. compile the C core, the CPU backend (the reference arithmetic stays available beside the CUDA one: tests compare
     the two through the same public API) and the CUDA backend, and link against libmarmot_cuda.so.

After that `marmot_init(MARMOT_BACKEND_CUDA)` works and `marmot_linear`, `marmot_moe_experts`, `marmot_topk`,
`marmot_dequantize_*`, `marmot_vec_dot`, ... reach the sm_100a kernels through marmot's own dispatch: signature ->
generated query -> one-instruction bytecode program -> generated exec wrapper -> cuda_backend.c -> C ABI.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HOST = Path(__file__).resolve().parent
PKG = HOST.parent
if str(PKG.parent) not in sys.path:
    sys.path.insert(0, str(PKG.parent))

from marmot_b200.host import marmot_tree  # noqa: E402

OUT = PKG / "libmarmot_b200.so"

CUDA_CONFIG = '''

# ---- CUDA (sm_100a) backend: host layer in src/backends/cuda/cuda_backend.c over the C ABI of libmarmot_cuda ----
CUDA_CONFIG = BackendConfig(
    name="cuda",
    file_extension=".c",
    internal_header="backends/cuda/cuda_backend.h",
    extra_includes=[
        "marmot/ops/matmul.h",
        "marmot/ops/neural.h",
        "marmot/ops_types.h",
        "marmot/quant_traits.h",
        "marmot/tensor.h",
        "marmot/traits_ids.gen.h",
        "graph/kernel_dispatch_args.gen.h",
    ],
    needs_extern_c=False,
    handlers={
        "matmul_quantized": "cuda_matmul_quantized_any",
        "vec_dot": "cuda_vec_dot",
        "dequantize": "cuda_dequantize_dispatch",
        "rms_norm": "cuda_rmsnorm_impl",
        "rope": "cuda_rope",
        "paged_attention": "cuda_paged_attention_impl",
        "embedding": "cuda_embedding_gather",
        "binary": "cuda_elementwise_binary_impl",
    },
    supports_fusion=False,
    matmul_needs_dimension_extraction=False,
    matmul_needs_epilogue_apply=False,
    quantize_uses_unified_dispatcher=True,
    reduction_uses_generic_handler=False,
    split_and_slice_unified=False,
    allows_kernel_func_override=True,
    uses_platform_guards=False,
    context_type="void",
)
BACKENDS["cuda"] = CUDA_CONFIG
'''


def _replace_once(path: Path, old: str, new: str) -> None:
    text = path.read_text()
    if text.count(old) != 1:
        raise RuntimeError(f"{path}: expected exactly one occurrence of the patch anchor {old[:60]!r}")
    path.write_text(text.replace(old, new))


def _patch_core(stage: Path) -> None:
    """The CUDA cases of the core's three per-backend switch statements."""
    _replace_once(
        stage / "src/core/context/context.c",
        '''    case MARMOT_BACKEND_CUDA:
        marmot_set_error(MARMOT_ERROR_NOT_IMPLEMENTED, "CUDA backend not yet implemented");
        return nullptr;
''',
        '''    case MARMOT_BACKEND_CUDA:
        ops = marmot_get_cuda_ops();
        break;
''')
    ctx_c = stage / "src/core/context/context.c"
    ctx_c.write_text('#include "backends/cuda/cuda_backend.h"\n' + ctx_c.read_text())

    kq = stage / "src/core/dispatch/kernel_query.c"
    _replace_once(kq, "static marmot_kernel_selection_t marmot_kernel_selection_unsupported(const char *reason) {",
                  '''extern marmot_kernel_selection_t
marmot_cuda_query_kernel(const marmot_op_signature_t *sig, const marmot_device_caps_t *caps);
extern marmot_device_caps_t marmot_cuda_detect_default_caps(void);
extern bool marmot_cuda_default_preferences(const marmot_device_caps_t *caps, marmot_backend_preferences_t *out);

static marmot_kernel_selection_t marmot_kernel_selection_unsupported(const char *reason) {''')
    text = kq.read_text()
    anchors = [
        ("    default:\n        return marmot_kernel_selection_unsupported(\"Backend query not available\");",
         "    case MARMOT_BACKEND_CUDA:\n        return marmot_cuda_query_kernel(sig, caps);\n"),
        ("    default:\n        return false;\n    }\n}\n\nbool marmot_backend_get_default_preferences(",
         "    case MARMOT_BACKEND_CUDA:\n        *caps_out = marmot_cuda_detect_default_caps();\n        return true;\n"),
    ]
    for anchor, case in anchors:
        if text.count(anchor) != 1:
            raise RuntimeError(f"kernel_query.c: patch anchor not found: {anchor[:50]!r}")
        text = text.replace(anchor, case + anchor)
    # the last switch of the file: default preferences
    tail_anchor = "    default:\n        return false;\n    }\n}\n"
    at = text.rfind(tail_anchor)
    if at < 0:
        raise RuntimeError("kernel_query.c: preferences switch not found")
    text = text[:at] + "    case MARMOT_BACKEND_CUDA:\n        return marmot_cuda_default_preferences(caps, prefs_out);\n" + text[at:]
    kq.write_text(text)

    bc = stage / "src/core/bytecode/bytecode_compile.c"
    _replace_once(
        bc, "    default:\n        return false;\n    }\n}\n\nbool marmot_bc_exec_supported(",
        '''    case MARMOT_BACKEND_CUDA:
        *out = (marmot_bc_tables_t){
            .imm_size = marmot_cuda_bc_imm_size,
            .exec_table = marmot_cuda_bc_exec_table,
            .schema_id = marmot_cuda_bc_schema_id,
            .op_count = MARMOT_CUDA_BC_OP_COUNT,
        };
        return true;
    default:
        return false;
    }
}

bool marmot_bc_exec_supported(''')
    bc.write_text('#include "backends/cuda/dispatch/bytecode_exec_cuda.gen.h"\n' + bc.read_text())


def _run_codegen(stage: Path) -> list[Path]:
    """Run marmot's generator for the three backends; returns the generated CUDA translation units."""
    cg = stage / "scripts" / "codegen"
    with open(cg / "backend_config.py", "a") as f:
        f.write(CUDA_CONFIG)
    cuda = stage / "src/backends/cuda"
    disp = cuda / "dispatch"
    disp.mkdir(parents=True, exist_ok=True)
    scratch = stage / "metal_scratch"  # Metal outputs are Objective-C++ and are not compiled here
    scratch.mkdir()
    cpu_d = stage / "src/backends/cpu/dispatch"
    cmd = [
        sys.executable, str(cg / "gen_kernels.py"),
        "--backends", "cpu", "metal", "cuda",
        "--backend-dirs", str(stage / "src/backends/cpu/kernels"), str(stage / "src/backends/metal/kernels"),
        str(cuda / "kernels"),
        "--traits-header", str(stage / "include/marmot/traits_ids.gen.h"),
        "--query-sources", str(cpu_d / "cpu_kernel_query.gen.c"), str(scratch / "metal_kernel_query.gen.mm"),
        str(disp / "cuda_kernel_query.gen.c"),
        "--dispatch-sources", str(scratch / "metal_kernel_dispatch.gen.mm"), str(disp / "cuda_kernel_dispatch.gen.c"),
        "--dispatch-dirs", f"cpu:{cpu_d}",
        "--op-signature-hash-header", str(stage / "include/marmot/op_signature_hash.gen.h"),
        "--bytecode-table-headers", str(cpu_d / "bytecode_tables_cpu.gen.h"), str(scratch / "bytecode_tables_metal.gen.h"),
        str(disp / "bytecode_tables_cuda.gen.h"),
        "--bytecode-table-sources", str(cpu_d / "bytecode_tables_cpu.gen.c"), str(scratch / "bytecode_tables_metal.gen.mm"),
        str(disp / "bytecode_tables_cuda.gen.c"),
        "--bytecode-exec-headers", str(cpu_d / "bytecode_exec_cpu.gen.h"), str(scratch / "bytecode_exec_metal.gen.h"),
        str(disp / "bytecode_exec_cuda.gen.h"),
        "--bytecode-exec-sources", str(cpu_d / "bytecode_exec_cpu.gen.c"), str(scratch / "bytecode_exec_metal.gen.mm"),
        str(disp / "bytecode_exec_cuda.gen.c"),
        "--metal-unary-tables-header", str(scratch / "metal_unary_tables.gen.h"),
        "--template-dir", str(cg / "templates"),
    ]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"gen_kernels.py failed:\n{r.stdout}\n{r.stderr}")
    return [disp / n for n in ("cuda_kernel_query.gen.c", "cuda_kernel_dispatch.gen.c", "bytecode_tables_cuda.gen.c",
                               "bytecode_exec_cuda.gen.c")]


def build(marmot_root: Path | None = None, jobs: int | None = None, keep_generated: Path | None = None) -> Path:
    """`keep_generated`: a directory that receives a copy of the generated CUDA sources (for inspection)."""
    root = Path(marmot_root) if marmot_root else None
    if root is None and os.environ.get("MARMOT_SOURCE_DIR"):
        root = Path(os.environ["MARMOT_SOURCE_DIR"])
    if root is None or not (root / "meson.build").exists():
        raise FileNotFoundError("no marmot checkout: pass its path or set MARMOT_SOURCE_DIR")
    root = root.resolve()
    cuda_lib = PKG / "libmarmot_cuda.so"
    if not cuda_lib.exists():
        raise FileNotFoundError("build libmarmot_cuda.so first (marmot_b200/build.py)")
    sources = marmot_tree.c_sources(root)
    stage = Path(tempfile.mkdtemp(prefix="marmot_cuda_stage_"))
    try:
        marmot_tree.stage(root, stage, with_codegen=True)
        cuda = stage / "src/backends/cuda"
        (cuda / "kernels").mkdir(parents=True)
        for f in sorted((HOST / "kernels").glob("*.def")):
            shutil.copyfile(f, cuda / "kernels" / f.name)
        # the dtype / scheme sets and QUANT_SCHEME blocks every backend's .def files refer to
        shutil.copytree(stage / "src/backends/cpu/kernels/metadata", cuda / "kernels" / "metadata")
        shutil.copyfile(HOST / "cuda_backend.c", cuda / "cuda_backend.c")
        shutil.copyfile(HOST / "cuda_backend.h", cuda / "cuda_backend.h")
        generated = _run_codegen(stage)
        if keep_generated is not None:
            keep_generated.mkdir(parents=True, exist_ok=True)
            for g in generated + [g.with_suffix(".h") for g in generated if g.with_suffix(".h").exists()]:
                shutil.copyfile(g, keep_generated / g.name)
        _patch_core(stage)

        incs = [f"-I{stage / p}" for p in marmot_tree.INCLUDE_DIRS] + [f"-I{PKG.parent / 'include'}"]
        objdir = stage / "obj"
        objdir.mkdir()
        units = [(stage / s, []) for s in sources]
        units += [(g, []) for g in generated]
        # the generated query replaces the hand-written one of the stand-alone host layer
        units.append((cuda / "cuda_backend.c", ["-DMARMOT_CUDA_GENERATED_QUERY=1", "-Wall", "-Wextra"]))

        def compile_one(item):
            idx, (src, extra) = item
            obj = objdir / f"{idx:03d}_{src.stem}.o"
            cmd = ["gcc", *marmot_tree.CFLAGS, *marmot_tree.DEFINES, *incs, *extra, "-c", str(src), "-o", str(obj)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            return src, obj, r.returncode, r.stderr

        objs, failed = [], []
        with cf.ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as ex:
            for src, obj, rc, err in ex.map(compile_one, enumerate(units)):
                if rc == 0:
                    objs.append(str(obj))
                else:
                    failed.append((src, err.strip().splitlines()[:6]))
        if failed:
            msg = "\n".join(f"{src}: {err}" for src, err in failed)
            raise RuntimeError(f"{len(failed)} translation units failed to compile:\n{msg}")
        tmp = stage / OUT.name
        # -Bsymbolic: the library's own marmot_* calls bind to its own definitions, also in a process where another
        # marmot build was loaded with global symbols first (a CPU-only one would otherwise answer the dispatch)
        subprocess.run(["gcc", "-shared", "-o", str(tmp), *objs, f"-L{PKG}", "-lmarmot_cuda", "-Wl,-rpath,$ORIGIN", "-lm",
                        "-pthread", "-Wl,--allow-shlib-undefined", "-Wl,-Bsymbolic"], check=True)
        shutil.copyfile(tmp, OUT)
    finally:
        shutil.rmtree(stage, ignore_errors=True)
    return OUT


if __name__ == "__main__":
    print(build(Path(sys.argv[1]) if len(sys.argv) > 1 else None,
                keep_generated=Path(sys.argv[2]) if len(sys.argv) > 2 else None))
