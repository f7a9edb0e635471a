"""Builds the CPU oracle (test infrastructure) into oracle/_build/.

The reference is OCaml and cannot be compiled on this toolchain (no ocaml,
dune or opam), so there is no oracle/_ref: the C restatement is the only
checker.  Run as ``python oracle/build.py``.
"""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libnative_oracle.so")
SRC = os.path.join(HERE, "native_oracle.c")


def build_oracle(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-fvisibility=hidden",
           "-Wall", "-Wextra", "-o", LIB, SRC, "-lm", "-lpthread"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("gcc failed building the oracle:\n" + res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    print(build_oracle(force=True))
