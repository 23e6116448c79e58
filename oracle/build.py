"""Compile the oracle's C restatement into ``oracle/libkquants_oracle.so``.

Test infrastructure: building the checker is not using it. Tries OpenMP first (the timed CPU
baseline wants every host core) and falls back to a single-threaded build when the compiler has no
OpenMP runtime.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "kquants_oracle.c")
LIB = os.path.join(HERE, "libkquants_oracle.so")

_BASE = ["-O2", "-ffp-contract=off", "-fPIC", "-std=c11", "-shared"]


def _compilers() -> list[str]:
    out = []
    for cand in (os.environ.get("ORACLE_CC"), "/usr/bin/gcc", shutil.which("gcc"), shutil.which("cc")):
        if cand and cand not in out and os.path.exists(cand):
            out.append(cand)
    return out


def build(force: bool = False) -> str:
    """Build the library if it is missing or older than its source; return its path."""
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    errors = []
    for openmp in (True, False):
        for cc in _compilers():
            cmd = [cc, *_BASE, *(["-fopenmp"] if openmp else []), "-o", LIB + ".tmp", SRC, "-lm"]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode == 0:
                os.replace(LIB + ".tmp", LIB)
                return LIB
            errors.append(f"{' '.join(cmd)}\n{res.stderr.strip()}")
    raise RuntimeError("could not compile the oracle:\n" + "\n".join(errors))


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
