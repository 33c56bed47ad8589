"""Builds ``libtessel_b200.so`` in-tree with nvcc for sm_100a.

``python -m tessel_b200.build`` (or :func:`build`) compiles every ``csrc/*.cu``
to an object file (in parallel) and links them into
``tessel_b200/libtessel_b200.so``. A file is recompiled only when it, or a
header, is newer than its object. No GPU is needed: nvcc cross-compiles.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
SO = os.path.join(HERE, "libtessel_b200.so")
SO_TRACE = os.path.join(HERE, "libtessel_b200_trace.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _newest_header() -> float:
    hs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return max(os.path.getmtime(h) for h in hs)


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False, trace: bool = False) -> str:
    """``trace``: a second library, ``libtessel_b200_trace.so``, whose exchange kernel stamps
    %globaltimer at its phase boundaries (``-DTB200_TRACE``); select it with TESSEL_B200_LIB."""
    obj_dir, so = (OBJ + "_trace", SO_TRACE) if trace else (OBJ, SO)
    os.makedirs(obj_dir, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdr = _newest_header()
    jobs = []
    objs = []
    for s in srcs:
        o = os.path.join(obj_dir, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr):
            cmd = [nvcc(), *NVCC_FLAGS, *(["-DTB200_TRACE"] if trace else []), "-c", s, "-o", o]
            if ptxas_info:
                cmd += ["-Xptxas", "-v"]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for cmd, r in ex.map(run, jobs):
                if verbose or r.returncode != 0 or ptxas_info:
                    sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
                if r.returncode != 0:
                    raise RuntimeError("nvcc failed on " + cmd[-3])
    if jobs or not os.path.exists(so):
        link = [nvcc(), "-shared", "-o", so, *objs, "-ldl", "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(link, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return so


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv, ptxas_info="--ptxas" in sys.argv,
                trace="--trace" in sys.argv))
