"""The numpy restatement against the LIVE reference CPU build (oracle/_ref) on fresh random
cases -- complements the stored fixtures.  Skipped where oracle/_ref has not been built."""
import numpy as np
import pytest
import torch

from oracle import runner, scn_oracle as port
from tests import helpers

pytestmark = pytest.mark.skipif(not runner.reference_available(), reason="oracle/_ref not built")


@pytest.mark.parametrize("dim,size,n,batch", [(2, [21, 21], 300, 3), (3, [15, 15, 15], 900, 2), (4, [9, 9, 9, 5], 700, 2)])
@pytest.mark.parametrize("mode", [0, 1, 2, 3, 4])
def test_port_matches_live_reference(dim, size, n, batch, mode):
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200 import workloads
    rng = np.random.default_rng(1000 * dim + mode)
    coords = np.stack([rng.integers(0, s, n) for s in size] + [rng.integers(0, batch, n)], axis=1)
    if mode == 0:
        coords = np.unique(coords, axis=0)
        rng.shuffle(coords)
    feats = rng.standard_normal((coords.shape[0], 5)).astype(np.float32)
    torch.manual_seed(dim * 10 + mode)
    mods = [scn.InputLayer(dim, size, mode), scn.SubmanifoldConvolution(dim, 5, 7, 3, True),
            scn.Convolution(dim, 7, 6, 3, 2, False), scn.BatchNormLeakyReLU(6, leakiness=0.1),
            scn.Deconvolution(dim, 6, 4, 3, 2, True)]
    mods[1].bias.data.normal_()
    mods[4].bias.data.normal_()
    net = torch.nn.ModuleList(mods)
    workloads.randomize(net, 5)
    net.eval()
    outs = []
    for be in (runner.RefBackend(), runner.PortBackend()):
        x = [coords, feats]
        stages = []
        for m in mods:
            x = runner.run_module(m, x, be)
            stages.append((be.locations(x), x.features))
        rules = port.canonical_rules(be.strided_rulebook(runner.run_module(mods[1], runner.run_module(mods[0], [coords, feats], be), be),
                                                         [(s - 3) // 2 + 1 for s in size], [3] * dim, [2] * dim),
                                     stages[1][0], stages[2][0])
        outs.append((stages, rules))
    (sa, ra), (sb, rb) = outs
    assert np.array_equal(sa[0][1], sb[0][1])                      # input layer: bit exact
    for i in (0, 1, 4):
        helpers.assert_features_match(sa[i][0], sa[i][1], sb[i][0], sb[i][1], 1e-5, same_rows=True, what="stage %d" % i)
    for i in (2, 3):
        helpers.assert_features_match(sb[i][0], sb[i][1], sa[i][0], sa[i][1], 1e-5, what="stage %d" % i)
    helpers.assert_rules_equal(rb, ra, "strided rulebook")


def test_batchnorm_training_statistics_match_reference():
    import sparseconvnet_b200 as scn
    rng = np.random.default_rng(3)
    x = rng.standard_normal((500, 6)).astype(np.float32) * 3 + 1
    outs = []
    for be in (runner.RefBackend(), runner.PortBackend()):
        bn = scn.BatchNormReLU(6)
        bn.train()
        t = runner.OTensor(x.copy(), None, [1])
        if be.name == "reference":
            y = be.batchnorm(t, bn)
            outs.append(y.features)
        else:
            y, rm, rv = port.batchnorm(x, bn.running_mean.numpy(), bn.running_var.numpy(), bn.weight.detach().numpy(),
                                       bn.bias.detach().numpy(), bn.eps, bn.momentum, True, bn.leakiness)
            outs.append(y)
    assert helpers.rel_err(outs[1], outs[0]) <= 1e-5
