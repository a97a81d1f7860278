"""Builds librai_b200.so in-tree with nvcc for sm_100a (no GPU needed: nvcc cross-compiles).

    python -m rai_b200.build               # incremental
    python -m rai_b200.build --force       # rebuild everything
    python -m rai_b200.build --debug-aids  # a second library, librai_b200_dbg.so, compiled with -DRB_DEBUG_AIDS
                                           # (developer switches such as running one tensor-parallel shard alone);
                                           # loaded instead of the product library when RAI_B200_DEBUG_AIDS=1
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "csrc" / "build"
LIB = PKG / "librai_b200.so"
HEADER = PKG.parent / "include" / "rai_b200.h"

SOURCES = ["api.cu", "decoder_kernels.cu", "plain_kernels.cu", "primitives.cu", "primitives_more.cu", "gemm_tc.cu", "attention.cu", "attention_tc.cu", "model.cu", "safetensors.cu", "selftest.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, debug_aids: bool = False) -> Path:
    global OBJ, LIB
    flags = list(NVCC_FLAGS)
    if debug_aids:
        OBJ, LIB, flags = CSRC / "build_dbg", PKG / "librai_b200_dbg.so", flags + ["-DRB_DEBUG_AIDS"]
    else:
        OBJ, LIB = CSRC / "build", PKG / "librai_b200.so"
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [HEADER]
    nvcc = _nvcc()
    jobs = []
    for src in SOURCES:
        s, o = CSRC / src, OBJ / (src + ".o")
        if force or _stale(o, [s] + headers):
            cmd = [nvcc, *flags, "-c", str(s), "-o", str(o)]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {cmd[-3]}")
    objs = [str(OBJ / (s + ".o")) for s in SOURCES]
    if force or jobs or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", str(LIB), *objs, "-lcudart", "-ldl",
               "-Xlinker", "--no-undefined"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            raise RuntimeError("link of librai_b200.so failed")
    return LIB


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="-v" in sys.argv, debug_aids="--debug-aids" in sys.argv)
    print(p)
