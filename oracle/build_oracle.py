"""TEST INFRASTRUCTURE. Compile the C oracles into oracle/_build/ (gcc, -O2, OpenMP)."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build")

TARGETS = {
    "libdot_oracle.so": ["dot_oracle.c"],
    "libloop_split_oracle.so": ["loop_split_oracle.c"],
}


def build(force: bool = False) -> dict:
    os.makedirs(OUT, exist_ok=True)
    paths = {}
    for lib, srcs in TARGETS.items():
        out = os.path.join(OUT, lib)
        src_paths = [os.path.join(HERE, s) for s in srcs]
        if force or not os.path.exists(out) or any(os.path.getmtime(s) > os.path.getmtime(out) for s in src_paths):
            subprocess.run(["gcc", "-O2", "-fopenmp", "-shared", "-fPIC", "-fvisibility=hidden", "-o", out, *src_paths, "-lm"],
                           check=True)
        paths[lib] = out
    return paths


if __name__ == "__main__":
    for k, v in build(force=True).items():
        print(v)
