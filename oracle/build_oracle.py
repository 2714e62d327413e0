#!/usr/bin/env python3
"""Compile the plain-C oracle (oracle/marmot_oracle.c) into oracle/libmarmot_oracle.so.

Test infrastructure only.  -ffp-contract=off keeps every multiply and add a
separately rounded binary32 operation, which is what the reference's scalar
build does; OpenMP only spreads independent output rows over host threads.
"""
from __future__ import annotations

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "marmot_oracle.c"
SRC_DECODER = HERE / "marmot_oracle_decoder.c"
OUT = HERE / "libmarmot_oracle.so"


def build(force: bool = False) -> Path:
    if not force and OUT.exists() and OUT.stat().st_mtime >= max(
        SRC.stat().st_mtime, SRC_DECODER.stat().st_mtime, (HERE / "marmot_oracle.h").stat().st_mtime
    ):
        return OUT
    cmd = [
        "gcc", "-std=c11", "-O2", "-march=x86-64-v3", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared",
        "-Wall", "-Wextra", "-o", str(OUT), str(SRC), str(SRC_DECODER), "-lm",
    ]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
