"""Builds libb200moe.so (the C-ABI product library) in-tree with nvcc for sm_100a.

    python -m cudapp_b200.build [--force]

Sources: cudapp_b200/csrc/*.cu; output: cudapp_b200/lib/libb200moe.so. Objects are rebuilt when a source or
header is newer than them. No torch, no JIT cache: the shared object travels with the tree.
"""
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "libb200moe.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-extended-lambda",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-Wno-format-truncation"]


def _newest(paths):
    return max(os.path.getmtime(p) for p in paths)


def build(force=False, verbose=False):
    os.makedirs(os.path.join(LIBDIR, "obj"), exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdrs = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(os.path.dirname(HERE), "include", "*.h"))
    hdr_time = _newest(hdrs)
    jobs = []
    objs = []
    for s in srcs:
        o = os.path.join(LIBDIR, "obj", os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_time):
            jobs.append([NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: %s\n%s%s" % (" ".join(cmd), r.stdout, r.stderr))
        return r.stderr

    with ThreadPoolExecutor(max(1, min(8, len(jobs) or 1))) as ex:
        logs = list(ex.map(run, jobs))
    if verbose:
        for lg in logs:
            sys.stderr.write(lg)
    if jobs or not os.path.exists(LIB) or force:
        run([NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcuda"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
