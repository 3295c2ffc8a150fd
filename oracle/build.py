"""Build the C restatement of the reference's eager path (test infrastructure).

    python oracle/build.py        ->  oracle/_build/libck_oracle.so

Plain gcc: OpenMP for the row loops, no fast-math and no FMA contraction so that every float
operation stays one IEEE binary32 operation.
"""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "ck_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libck_oracle.so")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    flags = ["-O2", "-fPIC", "-shared", "-std=c11", "-fno-fast-math", "-ffp-contract=off", "-fno-unsafe-math-optimizations"]
    compilers = [c for c in (os.environ.get("CC"), "/usr/bin/gcc", shutil.which("gcc"), shutil.which("cc")) if c]
    last = None
    # OpenMP where the compiler has its runtime; a single-threaded build otherwise
    for extra in (["-fopenmp"], []):
        for cc in compilers:
            r = subprocess.run([cc, *flags, *extra, "-o", LIB, SRC, "-lm"], capture_output=True, text=True)
            if r.returncode == 0:
                return LIB
            last = r.stderr
    raise RuntimeError(f"could not compile {SRC}: {last}")


if __name__ == "__main__":
    print(build(force=True))
