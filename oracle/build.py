"""Builds the CPU oracle (test infrastructure) into ``oracle/liboracle.so``.

    python -m oracle.build [--force]

``-march=x86-64-v3`` (AVX2 + FMA) rather than ``native`` so the library built on one machine runs on
another. When the reference checkout is present, also compiles the reference's own CUDA kernels for
sm_100a into ``oracle/_ref/*.cubin`` (see ``oracle/ref_kernels.py``); sources are compiled where they
lie and never copied.
"""
from __future__ import annotations

import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "talker_oracle.cpp"
LIB = HERE / "liboracle.so"


def build(force: bool = False) -> Path:
    if force or not LIB.exists() or LIB.stat().st_mtime < SRC.stat().st_mtime:
        cmd = ["g++", "-O3", "-march=x86-64-v3", "-fopenmp", "-shared", "-fPIC", "-std=c++17", "-o", str(LIB), str(SRC)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"g++ failed:\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
