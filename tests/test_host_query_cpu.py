"""Kernel query, default preferences and capability detection of the C23 host layer: the entry points marmot's
dispatcher binds per backend (src/core/dispatch/kernel_query.c:10-17).  The checks themselves are C
(tests/host_query_check.c), compiled here against marmot's headers, so they run where a marmot checkout is present."""
from __future__ import annotations

import os
import subprocess
import tempfile
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]


def _marmot_checkout() -> Path:
    """$MARMOT_SOURCE_DIR, else the checkout the oracle recipes find; a path that does not exist when there is none."""
    if os.environ.get("MARMOT_SOURCE_DIR"):
        return Path(os.environ["MARMOT_SOURCE_DIR"])
    from oracle.build_ref import find_reference_root

    return find_reference_root() or REPO / "no-marmot-checkout"


MARMOT = _marmot_checkout()
PKG = REPO / "marmot_b200"


def _build_and_run(arg: str | None):
    from oracle.bindings import REF_LIB

    if not (MARMOT / "include" / "marmot" / "device.h").exists():
        pytest.skip("no marmot checkout: the check program needs marmot's headers")
    if not (PKG / "libmarmot_cuda_backend.so").exists() or not Path(REF_LIB).exists():
        pytest.skip("host layer or reference library not built")
    with tempfile.TemporaryDirectory() as d:
        exe = Path(d) / "host_query_check"
        ref_dir = Path(REF_LIB).parent
        subprocess.run(["gcc", "-std=c2x", "-O1", "-Wall", "-Wextra", f"-I{MARMOT / 'include'}", f"-I{MARMOT / 'src'}",
                        str(REPO / "tests" / "host_query_check.c"), "-o", str(exe), f"-L{PKG}", "-lmarmot_cuda_backend",
                        "-lmarmot_cuda", f"-L{ref_dir}", f"-l:{Path(REF_LIB).name}",
                        f"-Wl,-rpath,{PKG}", f"-Wl,-rpath,{ref_dir}"], check=True)
        r = subprocess.run([str(exe)] + ([arg] if arg else []), capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr


def test_query_preferences_and_caps_without_a_device():
    _build_and_run(None)


@pytest.mark.gpu
def test_query_with_detected_caps():
    _build_and_run("device")
