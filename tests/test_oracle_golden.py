"""The numpy restatement (oracle/scn_oracle.py) against the golden fixtures that were produced
by the reference's own CPU build (tests/golden/make_golden.py).  CPU only."""
import numpy as np
import pytest

from oracle import runner, scn_oracle as port
from tests import helpers
from tests.golden import cases


@pytest.mark.parametrize("name", sorted(cases.OPS_CASES))
def test_port_ops_match_reference_golden(name):
    g = helpers.load_golden(name)
    net = cases.ops_modules(name)
    helpers.load_state(net, g, "state")
    be = runner.PortBackend()
    st = cases.run_ops(net, (g["coords"], g["feats"], int(g["batch_size_arg"])), helpers.oracle_run(be),
                       be.locations)
    c = cases.OPS_CASES[name]
    d = c["dim"]
    assert be.batch_size(st["x0"]) == int(g["batch_size"])
    # input-level stages share the reference's row numbering exactly
    for k in ("x0", "x1", "x4", "x7"):
        helpers.assert_features_match(be.locations(st[k]), st[k].features, g["loc/" + k], g["feat/" + k],
                                      1e-5, same_rows=True, what=name + ":" + k)
    assert np.array_equal(st["x0"].features, g["feat/x0"]), "input layer features must be bit exact"
    for k in ("x2", "x3", "x5", "x6"):
        helpers.assert_features_match(be.locations(st[k]), st[k].features, g["loc/" + k], g["feat/" + k],
                                      1e-5, what=name + ":" + k)
    assert helpers.rel_err(st["dense"], g["dense"]) <= 1e-5
    sub = port.canonical_rules(be.submanifold_rulebook(st["x0"], [3] * d), be.locations(st["x0"]),
                               be.locations(st["x0"]))
    helpers.assert_rules_equal(sub, helpers.golden_rules(g, "rules_sub"), name + " submanifold")
    strided = port.canonical_rules(
        be.strided_rulebook(st["x1"], st["x2"].spatial_size, [c["f"]] * d, [c["s"]] * d),
        be.locations(st["x1"]), be.locations(st["x2"]))
    helpers.assert_rules_equal(strided, helpers.golden_rules(g, "rules_strided"), name + " strided")


@pytest.mark.parametrize("name", sorted(cases.NET_CASES))
def test_port_networks_match_reference_golden(name):
    g = helpers.load_golden(name)
    inp, net, head = cases.net_modules(name)
    helpers.load_state(net, g, "state")
    be = runner.PortBackend()
    stats = {}
    x0 = runner.run_module(inp, [g["coords"], g["feats"]], be)
    assert np.array_equal(be.locations(x0), g["loc/x0"])
    assert np.array_equal(x0.features, g["feat/x0"])
    y = runner.run_module(net, x0, be, stats)
    assert stats.get("macs", 0.0) == float(g["macs"])
    if "dense" in g:
        assert helpers.rel_err(y, g["dense"]) <= 1e-4
    else:
        helpers.assert_features_match(be.locations(y), y.features, g["loc/y"], g["feat/y"], 1e-4, what=name)
        if head is not None:
            helpers.load_state(head, g, "head")
            p = port.align_rows(be.locations(y), g["loc/y"])
            assert helpers.rel_err(runner.run_module(head, y, be), g["head_out"][p]) <= 1e-4


@pytest.mark.parametrize("name", sorted(cases.IO_CASES))
def test_port_io_layers_match_reference_golden(name):
    """InputLayer / BLInputLayer -> SubmanifoldConvolution -> OutputLayer / BLOutputLayer: the input
    side is numbered exactly like the reference, so everything is compared row for row, and the
    copies back to the points are bit exact."""
    g = helpers.load_golden(name)
    mods = cases.io_modules(name)
    helpers.load_state(mods[1], g, "state")
    be = runner.PortBackend()
    st = cases.run_io(mods, (g["coords"], g["feats"]), helpers.oracle_run(be))
    assert np.array_equal(be.locations(st["x0"]), g["loc/x0"])
    assert np.array_equal(st["x0"].features, g["feat/x0"]) or cases.IO_CASES[name]["mode"] == 4
    assert helpers.rel_err(st["x0"].features, g["feat/x0"]) <= 1e-6
    assert helpers.rel_err(st["x1"].features, g["feat/x1"]) <= 1e-5
    assert st["back0"].shape == g["back0"].shape
    assert helpers.rel_err(st["back0"], g["back0"]) <= 1e-6
    assert helpers.rel_err(st["back1"], g["back1"]) <= 1e-5
