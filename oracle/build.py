"""Compile the C part of the CPU oracle into ``oracle/_build/liboracle.so`` (test infrastructure)."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_build", "liboracle.so")
SOURCES = ["qmm_cpu.c"]


def build_oracle(force: bool = False) -> str:
    srcs = [os.path.join(HERE, s) for s in SOURCES]
    if not force and os.path.exists(LIB) and all(
            os.path.getmtime(LIB) >= os.path.getmtime(s) for s in srcs):
        return LIB
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    cmd = ["gcc", "-O3", "-fPIC", "-fopenmp", "-ffp-contract=off", "-Wall", "-shared",
           "-o", LIB] + srcs + ["-lm"]
    subprocess.run(cmd, check=True, cwd=HERE)
    return LIB


if __name__ == "__main__":
    print(build_oracle(force=True))
