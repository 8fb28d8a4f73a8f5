#!/usr/bin/env python3
"""Build librwkvq.so (hand-written CUDA for sm_100a, C ABI declared in include/rwkvq.h) in-tree with nvcc.

    python build_ext.py [--force] [--verbose] [--trace]

Each csrc/*.cu is compiled to an object file (in parallel) and linked into librwkvq.so next to this file.
Nothing is cross-compiled for any other architecture: the kernels use sm_100a-only instructions.
"""
import concurrent.futures
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "librwkvq.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
         "-Xcompiler", "-fPIC,-O3", "--expt-relaxed-constexpr"]


def _newer(src, dst, deps):
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(p) > t for p in [src] + deps)


def build(force=False, verbose=False, trace=False):
    """trace=True compiles the kernels' milestone stamps in (-DRWKVQ_TRACE, see rwkvq_gemv_set_trace); rebuild with --force
    when switching."""
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    deps = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    jobs = []
    for s in srcs:
        o = os.path.join(OBJ, os.path.basename(s)[:-3] + ".o")
        if force or _newer(s, o, deps):
            cmd = [NVCC] + FLAGS + (["-DRWKVQ_TRACE"] if trace else []) + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            jobs.append((s, cmd))

    def run(job):
        s, cmd = job
        p = subprocess.run(cmd, capture_output=True, text=True)
        return s, p.returncode, p.stdout + p.stderr

    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        for s, rc, out in ex.map(run, jobs):
            if verbose or rc:
                sys.stderr.write(out)
            if rc:
                raise RuntimeError(f"nvcc failed on {s}")
    objs = [os.path.join(OBJ, os.path.basename(s)[:-3] + ".o") for s in srcs]
    if force or jobs or not os.path.exists(LIB):
        cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode:
            sys.stderr.write(p.stdout + p.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, trace="--trace" in sys.argv))
