"""Compiles oracle/rai_ref.c (the plain-C restatement, test infrastructure) into oracle/librai_ref.so with gcc.

    python oracle/build_ref.py
"""
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC, LIB = HERE / "rai_ref.c", HERE / "librai_ref.so"


def build(force: bool = False) -> Path:
    if force or not LIB.exists() or LIB.stat().st_mtime < SRC.stat().st_mtime:
        cmd = ["gcc", "-O2", "-fopenmp", "-shared", "-fPIC", "-Wall", "-o", str(LIB), str(SRC), "-lm"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            raise RuntimeError("gcc failed on oracle/rai_ref.c")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
