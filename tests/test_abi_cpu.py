"""CPU-side checks of the C-ABI library: it builds for sm_100a, loads, exports every symbol the
header declares, and refuses to run without a GPU instead of falling back."""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from marmot_b200 import build, runtime

    build.build()
    return runtime.load_library()


def test_header_symbols_are_exported(lib):
    header = (REPO / "include" / "marmot_cuda.h").read_text()
    declared = set(re.findall(r"\b(mcu_[a-z0-9_]+)\s*\(", header))
    from marmot_b200.runtime import EXPORTS

    assert declared == set(EXPORTS), declared ^ set(EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_row_bytes(lib):
    assert lib.mcu_row_bytes(9, 4096) == 16 * 144
    assert lib.mcu_row_bytes(11, 4096) == 16 * 210
    assert lib.mcu_row_bytes(5, 4096) == 128 * 34
    assert lib.mcu_row_bytes(9, 257) == 2 * 144
    assert lib.mcu_row_bytes(4, 4096) == 0  # Q5_1: not a kind this backend implements


def test_no_cpu_fallback_without_device(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    rc = lib.mcu_context_create(0, C.byref(h))
    assert rc == -3 and not h.value  # MARMOT_ERROR_DEVICE_NOT_AVAILABLE
    assert b"CUDA" in lib.mcu_last_error_message()
    # operations on a null context fail the same way
    assert lib.mcu_linear(None, 9, None, 0, None, 1, 256, 1, None, None, 1) == -3
    assert lib.mcu_synchronize(None) == -3


class DeviceCaps(C.Structure):
    """struct mcu_device_caps, include/marmot_cuda.h."""
    _fields_ = [("sm_count", C.c_int), ("compute_capability", C.c_int), ("shared_mem_kb", C.c_int),
                ("l2_cache_kb", C.c_int), ("sm_clock_mhz", C.c_int), ("mem_bw_gbps", C.c_float),
                ("total_mem_bytes", C.c_size_t), ("copy_engines", C.c_int)]


def test_device_caps_without_device(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    caps = DeviceCaps(sm_count=7)
    lib.mcu_device_caps.argtypes = [C.c_int, C.POINTER(DeviceCaps)]
    assert lib.mcu_device_caps(0, C.byref(caps)) == -3  # MCU_ERROR_DEVICE_NOT_AVAILABLE
    assert caps.sm_count == 0  # cleared, not left as it was
    assert lib.mcu_device_caps(0, None) != 0


@pytest.mark.gpu
def test_device_caps_of_a_b200(lib):
    caps = DeviceCaps()
    lib.mcu_device_caps.argtypes = [C.c_int, C.POINTER(DeviceCaps)]
    assert lib.mcu_device_caps(0, C.byref(caps)) == 0
    assert caps.compute_capability == 100 and caps.sm_count >= 100
    assert caps.mem_bw_gbps > 4000 and caps.total_mem_bytes > 100 << 30 and caps.shared_mem_kb >= 200
    assert lib.mcu_device_caps(99, C.byref(caps)) == -3


def test_missing_library_is_loud(monkeypatch, tmp_path):
    from marmot_b200 import runtime

    monkeypatch.setattr(runtime, "_lib", None)
    monkeypatch.setattr(runtime, "LIB_PATH", tmp_path / "libmarmot_cuda.so")
    with pytest.raises(FileNotFoundError):
        runtime.load_library()


def test_product_does_not_import_the_oracle():
    for f in (REPO / "marmot_b200").rglob("*"):
        if f.suffix in {".py", ".cu", ".cuh", ".h", ".c"}:
            text = f.read_text()
            assert "oracle" not in text.lower(), f
