"""Ahead-of-time build of libringrnn.so (nvcc, sm_100a only) next to this file.

    python -m rnn_train_ring_attractor_b200.build [--force]

The reference JIT-compiles two pybind modules for whatever GPU it finds at import time
(cpp/rnn_cuda.py:34-91).  Here one C-ABI shared library is built in-tree, without a GPU present.
"""
import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libringrnn.so")
OBJ = os.path.join(PKG, "build")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I" + os.path.join(ROOT, "include"), "-I" + CSRC]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps_mtime():
    files = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    return max(os.path.getmtime(f) for f in files)


TIMELINE_LIB = os.path.join(PKG, "libringrnn_timeline.so")


def build_timeline():
    """The same library with the in-kernel timeline compiled in (-DRINGRNN_TIMELINE: cycle stamps of one CTA of each
    recurrent kernel, read with ringrnn_debug_timeline_read*; see `bench.py --timeline`).  A diagnostic build: the
    stamps cost a few percent, so it is never the library the operator loads."""
    nvcc = os.environ.get("NVCC") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    objdir = os.path.join(OBJ, "timeline")
    os.makedirs(objdir, exist_ok=True)
    procs, objs = [], []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        procs.append((src, subprocess.Popen([nvcc] + NVCC_FLAGS + ["-DRINGRNN_TIMELINE", "-c", src, "-o", obj],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError(f"nvcc failed on {src}")
    subprocess.run([nvcc, "-shared", "-o", TIMELINE_LIB] + objs, check=True)
    return TIMELINE_LIB


def build(force=False, verbose=False):
    """Compile every .cu under csrc/ into libringrnn.so; skipped when the library is newer than all sources."""
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _deps_mtime():
        return LIB
    nvcc = os.environ.get("NVCC") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    os.makedirs(OBJ, exist_ok=True)
    procs = []
    objs = []
    hdr_mtime = max(os.path.getmtime(f) for f in
                    glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h")))
    for src in sources():
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_mtime):
            continue
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, pr in procs:
        out, _ = pr.communicate()
        if verbose or pr.returncode != 0:
            sys.stderr.write(out)
        if pr.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    cmd = [nvcc, "-shared", "-o", LIB] + objs
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    if "--timeline" in sys.argv:
        print(build_timeline())
    else:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
