"""Build recipe for ``oracle/_ref`` -- TEST INFRASTRUCTURE ONLY.

Compiles the reference's *own* CPU sources, where they lie in a read-only
reference checkout, into two Python extension modules:

``oracle/_ref/SCN.so``
    the reference's pybind module (sparseconvnet/SCN/pybind.cpp +
    sparseconvnet/SCN/sparseconvnet_cpu.cpp, flags from the reference's
    setup.py:17: ``-std=c++17 -fopenmp -O3``), unmodified.
``oracle/_ref/SCN_shim.so``
    ``oracle/ref_shim.cpp`` compiled against the reference's
    ``Metadata/Metadata.cpp`` so rulebooks can be read back.

No reference source is copied: the compiler reads the files through ``-I``.
Outputs go only into ``oracle/_ref`` (git-ignored).  The reference's own build
system (setup.py / build.sh) is not run; the link line is written by hand
because passing ``-fopenmp`` to this image's g++ wrapper at link time fails to
find libgomp.spec, so libgomp is named explicitly.

Usage:  python oracle/build_ref.py [--reference /path/to/SparseConvNet] [--force]
"""
import argparse
import concurrent.futures as cf
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def _flags():
    import torch
    from torch.utils import cpp_extension as ce

    inc = ce.include_paths() + [sysconfig.get_paths()["include"]]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cflags = ["-std=c++17", "-fopenmp", "-O3", "-fPIC", "-w",
              f"-D_GLIBCXX_USE_CXX11_ABI={abi}"] + [f"-I{i}" for i in inc]
    gomp_dirs = [d for d in ("/usr/lib/gcc/x86_64-linux-gnu/13", "/usr/lib/x86_64-linux-gnu")
                 if os.path.isdir(d)]
    ldflags = ["-shared"] + [f"-L{d}" for d in gomp_dirs] + [
        "-lgomp", f"-L{tlib}", f"-Wl,-rpath,{tlib}",
        "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python"]
    return cflags, ldflags


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), r.stderr[-4000:]))


def build(reference="/root/reference", force=False, verbose=True):
    """Returns True when both modules exist afterwards, False when there is no
    reference checkout to build from (prebuilt files, if any, are left alone)."""
    scn = os.path.join(reference, "sparseconvnet", "SCN")
    targets = [os.path.join(OUT, "SCN.so"), os.path.join(OUT, "SCN_shim.so")]
    if all(os.path.exists(t) for t in targets) and not force:
        return True
    if not os.path.isdir(scn):
        return all(os.path.exists(t) for t in targets)
    os.makedirs(OUT, exist_ok=True)
    cflags, ldflags = _flags()
    cxx = os.environ.get("CXX", "g++")
    jobs = [
        (os.path.join(scn, "pybind.cpp"), os.path.join(OUT, "pybind.o"), "SCN"),
        (os.path.join(scn, "sparseconvnet_cpu.cpp"), os.path.join(OUT, "cpu.o"), "SCN"),
        (os.path.join(HERE, "ref_shim.cpp"), os.path.join(OUT, "shim.o"), "SCN_shim"),
    ]
    cmds = [[cxx, "-c", src, "-o", obj, f"-I{scn}", f"-DTORCH_EXTENSION_NAME={name}"] + cflags
            for src, obj, name in jobs]
    if verbose:
        print("[oracle/_ref] compiling the reference CPU extension (about a minute)", file=sys.stderr)
    with cf.ThreadPoolExecutor(3) as ex:
        list(ex.map(_run, cmds))
    _run([cxx, jobs[0][1], jobs[1][1], "-o", targets[0]] + ldflags)
    _run([cxx, jobs[2][1], "-o", targets[1]] + ldflags)
    for _, obj, _ in jobs:
        os.remove(obj)
    return True


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    ok = build(a.reference, a.force)
    print("oracle/_ref:", "ready" if ok else "no reference checkout; nothing built")
