"""Tensor-/expert-parallel layers on real GPUs: one process per GPU (NCCL + the library's peer all-reduce).
Needs at least two GPUs; the worker (tests/tp_worker.py) does the comparisons."""
from __future__ import annotations

import json
import socket
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
REPO = Path(__file__).resolve().parents[1]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_ranks(world):
    import torch

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(REPO / "tests" / "tp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=REPO,
                       env={**__import__("os").environ, "NCCL_NVLS_ENABLE": "0"})
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    assert len(lines) == world and all(l["ok"] for l in lines), lines
