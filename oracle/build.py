"""Builds the parity checkers (TEST INFRASTRUCTURE ONLY, never part of the product path).

Two artefacts:

* ``oracle/libs2v_oracle.so``  -- the plain-C restatement ``s2v_oracle.c``.
* ``oracle/_ref/libs2v_ref.so`` -- the reference's own CPU sources (every
  ``src/**/*.cpp`` of a Hanjun-Dai/graphnn checkout, compiled where they lie,
  nothing copied) + ``ref_harness.cpp`` + the MKL/TBB stand-ins in ``shim/``.
  Only built when a checkout is found: ``$GRAPHNN_REFERENCE_DIR`` or a
  ``reference`` directory next to this repository.  Machines without the checkout
  use the prebuilt file.

The reference's Makefile is not used: it needs Intel MKL and TBB.  The recipe is
the g++ line below; the forced ``-include`` headers supply standard headers the
2017 sources use without including (std::function, std::sort, ...).

Run ``python oracle/build.py`` (add ``--force`` to rebuild).
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)
ORACLE_SO = os.path.join(HERE, "libs2v_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libs2v_ref.so")

# x86-64-v3 (AVX2+FMA) rather than -march=native: the files are built on one
# machine and executed on another.
CPU_FLAGS = ["-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC"]


def reference_dir() -> str | None:
    cand = os.environ.get("GRAPHNN_REFERENCE_DIR") or os.path.join(os.path.dirname(REPO), "reference")
    return cand if os.path.isdir(os.path.join(cand, "src", "tensor")) else None


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "s2v_oracle.c")
    if force or not _newer(ORACLE_SO, [src]):
        _run(["gcc", "-std=c11", *CPU_FLAGS, "-shared", "-o", ORACLE_SO, src, "-lm"])
    return ORACLE_SO


def build_ref(force: bool = False) -> str | None:
    ref = reference_dir()
    if ref is None:
        return REF_SO if os.path.exists(REF_SO) else None
    shim = os.path.join(HERE, "shim")
    harness = os.path.join(HERE, "ref_harness.cpp")
    shim_cpp = os.path.join(shim, "mkl_shim.cpp")
    own = [harness, shim_cpp, os.path.join(shim, "mkl.h"), os.path.join(shim, "tbb", "tbb.h")]
    if not force and _newer(REF_SO, own):
        return REF_SO
    obj_dir = os.path.join(REF_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    base = ["g++", "-std=c++11", *CPU_FLAGS, "-w",
            "-include", "functional", "-include", "random", "-include", "stdexcept",
            "-include", "string", "-include", "algorithm", "-include", "cstring",
            "-I", shim, "-I", os.path.join(ref, "include")]
    sources = sorted(glob.glob(os.path.join(ref, "src", "**", "*.cpp"), recursive=True)) + [harness, shim_cpp]
    jobs = []
    for s in sources:
        tag = os.path.relpath(s, ref if s.startswith(ref) else HERE).replace(os.sep, "_")
        o = os.path.join(obj_dir, tag + ".o")
        jobs.append((s, o))

    def compile_one(job):
        s, o = job
        if force or not _newer(o, [s] + own[2:]):
            _run(base + ["-c", s, "-o", o])
        return o

    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        objs = list(ex.map(compile_one, jobs))
    _run(["g++", "-shared", "-fopenmp", "-o", REF_SO, *objs])
    return REF_SO


def main() -> None:
    force = "--force" in sys.argv
    print("oracle:", build_oracle(force))
    print("reference build:", build_ref(force) or "skipped (no reference checkout, no prebuilt file)")


if __name__ == "__main__":
    main()
