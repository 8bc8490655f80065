"""Builds libtilespmm_b200.so (hand-written CUDA for sm_100a behind a C ABI) in-tree with nvcc."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libtilespmm_b200.so")
LIB_DEBUG = os.path.join(HERE, "libtilespmm_b200_debug.so")   # the checked build: kernels verify every index they use (-DTSP_DEBUG)
SOURCES = ["api.cu", "convert.cu", "sched.cu", "spmm_small.cu", "spmm_small_t.cu", "spmm64.cu", "model.cu", "tile_cache.cu", "selftest.cu", "multi.cu", "mtx_reader.cpp"]
BIN = os.path.join(HERE, "bin")
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v", "-w"]


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _compile_and_link(lib: str, objdir: str, extra_flags: list[str], force: bool):
    nvcc = os.environ.get("NVCC", "nvcc")
    headers = [os.path.join(CSRC, "tsp_internal.cuh"), os.path.join(HERE, "..", "include", "tilespmm_b200.h"),
               os.path.join(CSRC, "model_table.inc"), os.path.join(CSRC, "atom_table.inc")]
    objs = []
    os.makedirs(objdir, exist_ok=True)
    procs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(objdir, os.path.splitext(src)[0] + ".o")
        objs.append(o)
        if not force and _newer(o, [s] + headers):
            continue
        cmd = [nvcc, *NVCC_FLAGS, *extra_flags, "-c", s, "-o", o]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    logs = []
    for src, p in procs:
        out, _ = p.communicate()
        logs.append(f"== {src}\n{out}")
        if p.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError(f"nvcc failed on {src}")
    if procs or not os.path.exists(lib) or force:
        tmp = lib + ".tmp"
        subprocess.run([nvcc, "-shared", "-o", tmp, *objs, "-lcusparse", "-lcudart", "-ldl", "-lpthread"], check=True)
        os.replace(tmp, lib)   # the finished library appears in one step
    return logs


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles every translation unit to an object and links the shared library (and its checked twin).  Returns the
    path of the release library."""
    nvcc = os.environ.get("NVCC", "nvcc")
    headers = [os.path.join(CSRC, "tsp_internal.cuh"), os.path.join(HERE, "..", "include", "tilespmm_b200.h"),
               os.path.join(CSRC, "model_table.inc"), os.path.join(CSRC, "atom_table.inc")]
    logs = _compile_and_link(LIB, os.path.join(HERE, "build"), [], force)
    _compile_and_link(LIB_DEBUG, os.path.join(HERE, "build", "debug"), ["-DTSP_DEBUG=1"], force)
    # the two drop-in executables (upstream bin/tilespmm_fp16, bin/tilespmm_tf32)
    os.makedirs(BIN, exist_ok=True)
    cli = os.path.join(CSRC, "cli_main.cpp")
    for prec, name in ((0, "tilespmm_fp16"), (1, "tilespmm_tf32")):
        exe = os.path.join(BIN, name)
        if force or not _newer(exe, [cli, LIB] + headers):
            subprocess.run([nvcc, "-std=c++17", "-O2", "-w", f"-DTSP_PRECISION={prec}", cli, "-o", exe, f"-L{HERE}", "-ltilespmm_b200",
                            "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/..", "-lcudart"], check=True)
    if logs:
        with open(os.path.join(HERE, "build", "ptxas.log"), "w") as fh:
            fh.write("\n".join(logs))
        if verbose:
            print("\n".join(logs))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
