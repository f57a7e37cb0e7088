"""Loads the reference's own Python package from ``oracle/_ref`` -- TEST INFRASTRUCTURE ONLY.

``oracle/build_ref.py`` stages the reference's unmodified ``sparseconvnet/*.py`` twice:

``load("cpu")``   the package beside the reference's own CPU extension: the reference's stock
                  path (sparseconvnet/ioLayers.py, networkArchitectures.py ... calling
                  sparseconvnet/SCN/pybind.cpp).  This is the oracle and the timed CPU baseline.
``load("b200")``  the same files with ``sparseconvnet.SCN`` bound to this repository's library
                  (``sparseconvnet_b200.SCN``): what "existing scn.Sequential models run
                  unchanged" means, used by the boundary tests.

Both packages are called ``sparseconvnet`` (their modules import that name), so each is imported
with ``sys.modules`` swapped around the import; afterwards the modules of a package keep working
because each holds its own package object in its globals.  The product never imports this file.
"""
import importlib
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF = os.path.join(_HERE, "_ref")
_loaded = {}


def available(binding="cpu"):
    pkg = os.path.join(_REF, "pkg_" + binding, "sparseconvnet")
    return os.path.exists(os.path.join(pkg, "__init__.py")) and \
        os.path.exists(os.path.join(pkg, "SCN.py")) and \
        (binding != "cpu" or os.path.exists(os.path.join(_REF, "SCN.so")))


def load(binding="cpu"):
    """Returns the reference's ``sparseconvnet`` package object bound to `binding`."""
    if binding in _loaded:
        return _loaded[binding]
    if not available(binding):
        raise RuntimeError("oracle/_ref/pkg_%s is not staged (python oracle/build_ref.py)" % binding)
    root = os.path.join(_REF, "pkg_" + binding)
    saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "sparseconvnet" or k.startswith("sparseconvnet.")}
    sys.path.insert(0, root)
    try:
        pkg = importlib.import_module("sparseconvnet")
    finally:
        sys.path.remove(root)
        mine = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "sparseconvnet" or k.startswith("sparseconvnet.")}
        sys.modules.update(saved)
    assert os.path.dirname(os.path.abspath(pkg.__file__)) == os.path.join(root, "sparseconvnet")
    pkg._oracle_modules = mine  # keeps the submodules alive
    _loaded[binding] = pkg
    return pkg
