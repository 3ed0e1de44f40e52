"""Compiles the CUDA library in-tree: graphnn_b200/csrc/*.cu -> graphnn_b200/libs2v_b200.so.

sm_100a only (`-gencode arch=compute_100a,code=sm_100a`); nvcc cross-compiles without
a GPU.  Run `python -m graphnn_b200.build` (add `--force` to rebuild, `--verbose` for
ptxas register/shared-memory reports).
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libs2v_b200.so")
OBJ_DIR = os.path.join(PKG, "build")

NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC,-fopenmp", "-I", os.path.join(REPO, "include"), "-I", CSRC]


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = sorted(glob.glob(os.path.join(CSRC, "*.cuh"))) + [os.path.join(REPO, "include", "s2v_b200.h")]
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    flags = NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        if force or _stale(obj, [src] + headers):
            r = subprocess.run([nvcc, *flags, "-c", src, "-o", obj], capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
            if verbose:
                print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        objs = list(ex.map(compile_one, sources))
    if force or _stale(LIB, objs):
        r = subprocess.run([nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-lgomp"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


CXX_DIR = os.path.join(PKG, "cxx")
CXX_BIN = os.path.join(CXX_DIR, "bin")


def build_cxx(force: bool = False) -> dict:
    """Compiles the host-side C++ programs that use the graphnn operator interface this
    package provides (cxx/include): the inference driver and the host-only interface test."""
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    os.makedirs(CXX_BIN, exist_ok=True)
    headers = [h for h in glob.glob(os.path.join(CXX_DIR, "include", "**", "*.h"), recursive=True)]
    headers.append(os.path.join(REPO, "include", "s2v_b200.h"))
    headers.append(os.path.join(CXX_DIR, "examples", "dataset.h"))
    out = {}
    for name, src in (("s2v_mean_field", os.path.join(CXX_DIR, "examples", "s2v_mean_field.cpp")),
                      ("s2v_classify", os.path.join(CXX_DIR, "examples", "s2v_classify.cpp")),
                      ("s2v_multi_gpu", os.path.join(CXX_DIR, "examples", "s2v_multi_gpu.cpp")),
                      ("host_interface_test", os.path.join(CXX_DIR, "tests", "host_interface_test.cpp"))):
        exe = os.path.join(CXX_BIN, name)
        if force or _stale(exe, [src, LIB] + headers):
            cmd = ["g++", "-std=c++14", "-O2", "-Wall", "-I", os.path.join(REPO, "include"), "-I",
                   os.path.join(CXX_DIR, "include"), "-I", os.path.join(cuda, "include"), src, "-o", exe,
                   "-L", PKG, "-ls2v_b200", "-L", os.path.join(cuda, "lib64"), "-lcudart", "-pthread",
                   "-Wl,-rpath,$ORIGIN/../..", "-Wl,-rpath," + PKG, "-Wl,-rpath," + os.path.join(cuda, "lib64")]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"g++ failed on {src}:\n{r.stdout}\n{r.stderr}")
        out[name] = exe
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_cxx(force="--force" in sys.argv))
