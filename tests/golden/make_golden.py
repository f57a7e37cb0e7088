"""Generates the golden fixtures in this directory by running the cases of ``cases.py`` on the
REFERENCE's own CPU implementation (compiled from the reference checkout by
``oracle/build_ref.py`` into ``oracle/_ref``).  Run from the repository root in a container
that has the reference checkout:

    python oracle/build_ref.py && python tests/golden/make_golden.py

Each ``<case>.npz`` stores the inputs, every parameter and buffer of the modules, and what
the reference produced: active-site locations and features at every stage, the canonical
form of the rulebooks (``oracle.scn_oracle.canonical_rules``), the dense output and the
multiply-add count.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import runner, scn_oracle as port  # noqa: E402
from tests.golden import cases  # noqa: E402


def _state(prefix, module, out):
    for k, v in module.state_dict().items():
        out["%s/%s" % (prefix, k)] = v.detach().cpu().numpy()


def ops_case(name, be):
    net = cases.ops_modules(name)
    coords, feats, bs = cases.ops_inputs(name)
    st = cases.run_ops(net, (coords, feats, bs), lambda m, x: runner.run_module(m, x, be), be.locations)
    c = cases.OPS_CASES[name]
    out = {"coords": coords, "feats": feats, "batch_size_arg": np.int64(bs)}
    _state("state", net, out)
    for k in ("x0", "x1", "x2", "x3", "x4", "x5", "x6", "x7"):
        out["loc/" + k] = be.locations(st[k])
        out["feat/" + k] = st[k].features
    out["dense"] = st["dense"]
    out["batch_size"] = np.int64(be.batch_size(st["x0"]))
    d = c["dim"]
    sub = port.canonical_rules(be.submanifold_rulebook(st["x0"], [3] * d), out["loc/x0"], out["loc/x0"])
    strided = port.canonical_rules(be.strided_rulebook(st["x1"], st["x2"].spatial_size, [c["f"]] * d, [c["s"]] * d),
                                   out["loc/x1"], out["loc/x2"])
    for k, r in enumerate(sub):
        out["rules_sub/%03d" % k] = r
    for k, r in enumerate(strided):
        out["rules_strided/%03d" % k] = r
    return out


def io_case(name, be):
    mods = cases.io_modules(name)
    coords, feats = cases.io_inputs(name)
    st = cases.run_io(mods, (coords, feats), lambda m, x: runner.run_module(m, x, be))
    out = {"coords": coords, "feats": feats}
    _state("state", mods[1], out)
    for k in ("x0", "x1"):
        out["loc/" + k] = be.locations(st[k])
        out["feat/" + k] = st[k].features
    out["back0"], out["back1"] = st["back0"], st["back1"]
    return out


def net_case(name, be):
    inp, net, head = cases.net_modules(name)
    coords, feats = cases.net_inputs(name)
    stats = {}
    x0 = runner.run_module(inp, [coords, feats], be)
    y = runner.run_module(net, x0, be, stats)
    out = {"coords": coords, "feats": feats, "macs": np.float64(stats.get("macs", 0.0)),
           "loc/x0": be.locations(x0), "feat/x0": x0.features}
    _state("state", net, out)
    if isinstance(y, np.ndarray):
        out["dense"] = y
    else:
        out["loc/y"] = be.locations(y)
        out["feat/y"] = y.features
        if head is not None:
            _state("head", head, out)
            out["head_out"] = runner.run_module(head, y, be)
    return out


def main():
    be = runner.RefBackend()
    for name in cases.OPS_CASES:
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **ops_case(name, be))
    for name in cases.IO_CASES:
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **io_case(name, be))
    for name in cases.NET_CASES:
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **net_case(name, be))
    total = sum(os.path.getsize(os.path.join(HERE, f)) for f in os.listdir(HERE) if f.endswith(".npz"))
    print("wrote %d cases, %.1f KiB" % (len(cases.OPS_CASES) + len(cases.IO_CASES) + len(cases.NET_CASES), total / 1024.0))


if __name__ == "__main__":
    main()
