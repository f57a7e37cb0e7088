"""Builds ``libscn_b200.so`` (the C-ABI library declared in ``include/scn_b200.h``) in-tree.

Every ``csrc/*.cu`` is compiled for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``) and linked into one shared library next to
this file.  nvcc cross-compiles without a GPU.

Usage:  python sparseconvnet_b200/build.py [--force] [--verbose]
(run as a script: importing the package needs the library this builds)
"""
import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libscn_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps():
    return _sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(HERE, "..", "include", "*.h"))


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(f) > t for f in _deps())


def _compile(src, verbose):
    obj = os.path.join(HERE, "build", os.path.basename(src)[:-3] + ".o")
    hdr_t = max(os.path.getmtime(f) for f in _deps() if not f.endswith(".cu"))
    if os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(src), hdr_t):
        return obj
    cmd = [NVCC, "-c", src, "-o", obj] + FLAGS + (["-Xptxas", "-v"] if verbose else [])
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed on %s:\n%s" % (src, r.stderr[-6000:]))
    if verbose:
        sys.stderr.write(r.stderr)
    return obj


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    if force:
        for f in glob.glob(os.path.join(HERE, "build", "*.o")):
            os.remove(f)
    with cf.ThreadPoolExecutor(max(1, min(8, os.cpu_count() or 1))) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), _sources()))
    cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                   "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n%s" % r.stderr[-4000:])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
