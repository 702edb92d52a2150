"""Builds the CUDA library (csrc/*.cu -> libaig_b200.so) in-tree with nvcc for sm_100a.

nvcc cross-compiles without a GPU.  Objects are cached under build/ and rebuilt when a source or a
header is newer.  Run as a script or call build().
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
HOST = os.path.join(HERE, "host")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libaig_b200.so")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-I" + os.path.join(ROOT, "include"), "-I" + CSRC, "-I" + HOST, "-I" + os.path.join(HOST, "layers"),
]


def _newest_header():
    t = 0.0
    for d in (CSRC, HOST, os.path.join(HOST, "layers"), os.path.join(ROOT, "include")):
        if not os.path.isdir(d):
            continue
        for f in os.listdir(d):
            if f.endswith((".h", ".cuh", ".hpp")):
                t = max(t, os.path.getmtime(os.path.join(d, f)))
    return t


def sources():
    out = []
    for d in (CSRC, HOST, os.path.join(HOST, "layers")):
        if os.path.isdir(d):
            out += [os.path.join(d, f) for f in sorted(os.listdir(d)) if f.endswith((".cu", ".cpp"))]
    return out


def build(force=False, verbose=False, defines=()):
    """defines: extra -D macros (AIG_TUNING compiles the kernels' timeline stamps and tile-search switches in)."""
    os.makedirs(OBJ, exist_ok=True)
    extra = ["-D" + d for d in defines]
    stamp = os.path.join(OBJ, ".defines")  # objects built with other macros are stale
    if not os.path.exists(stamp) or open(stamp).read() != " ".join(extra):
        force = True
    hdr_t = _newest_header()
    jobs = []
    objs = []
    for src in sources():
        obj = os.path.join(OBJ, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_t):
            cmd = ["nvcc"] + NVCC_FLAGS + extra + (["-x", "cu"] if src.endswith(".cpp") else []) + ["-c", src, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
        return r

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(run, jobs))
    if jobs or not os.path.exists(LIB):
        run(["nvcc", "-shared", "-o", LIB] + objs + ["-lcudart"])
    with open(stamp, "w") as f:
        f.write(" ".join(extra))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, defines=[a[2:] for a in sys.argv[1:] if a.startswith("-D")]))
