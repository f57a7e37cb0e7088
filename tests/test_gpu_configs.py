"""The five benchmark configurations on the GPU against the CPU oracles: the compiled
reference (oracle/_ref) where it travelled with the tree, the numpy restatement otherwise,
plus size-independent properties at the full benchmark sizes."""
import numpy as np
import pytest
import torch

from oracle import runner, scn_oracle as port
from sparseconvnet_b200 import workloads
from tests import helpers

pytestmark = pytest.mark.gpu


def _oracle():
    return runner.RefBackend() if runner.reference_available() else runner.PortBackend()


def _run_both(config, coords, feats, precision="fp32", be=None):
    import sparseconvnet_b200 as scn
    inp, net, head = workloads.build_config(config)
    be = be or _oracle()
    yo = runner.run_module(net, runner.run_module(inp, [coords, feats], be), be)
    gpu = helpers.GpuBackend()
    scn.set_precision(precision)
    try:
        x = gpu.run(inp, [coords, feats])
        yg = gpu.run(net, x)
        if isinstance(yg, helpers.GpuTensor):
            yg.t.metadata.poll_errors()
    finally:
        scn.set_precision("fp32")
    return be, yo, gpu, yg


@pytest.fixture
def restore_precision():
    import sparseconvnet_b200 as scn
    yield
    scn.set_precision("fp32")


def test_config1_full_size(cuda):
    """One 3-D submanifold convolution 32->32 on the full 256^3 cloud: rulebook bit for bit
    against the restatement, features within the fp32 bar, and rulebook invariants."""
    coords, feats = workloads.make_batch(1, [0])
    pb = runner.PortBackend()
    be, yo, gpu, yg = _run_both(1, coords, feats, be=pb)
    assert np.array_equal(gpu.locations(yg), coords_with_batch(coords))
    helpers.assert_features_match(gpu.locations(yg), yg.features, pb.locations(yo), yo.features, helpers.FP32_TOL,
                                  same_rows=True, what="config 1")
    rg = gpu.submanifold_rulebook(yg, [3, 3, 3])
    rp = pb.submanifold_rulebook(yo, [3, 3, 3])
    n = coords.shape[0]
    assert len(rg) == 27 and rg[13].shape[0] == n, "centre offset must hold one rule per site"
    for k in range(27):
        assert np.array_equal(rg[k], rp[k]), "offset %d" % k
        # (i -> o) through offset k  <=>  (o -> i) through offset 26 - k
        mirrored = rg[26 - k][:, ::-1]
        assert np.array_equal(rg[k][np.lexsort(rg[k].T[::-1])], mirrored[np.lexsort(mirrored.T[::-1])])


def coords_with_batch(coords):
    return np.concatenate([coords, np.zeros((coords.shape[0], 1), dtype=np.int64)], axis=1)


@pytest.mark.parametrize("precision,tol", [("fp32", helpers.FP32_TOL), ("tf32x3", helpers.FP32_TOL)])
def test_config2_full_batch(precision, tol, cuda):
    coords, feats = workloads.make_batch(2, range(100))
    be, yo, gpu, yg = _run_both(2, coords, feats, precision)
    assert yg.shape == (100, 32, 10, 10)
    assert helpers.rel_err(yg, yo) <= tol


@pytest.mark.parametrize("precision,tol", [("fp32", helpers.FP32_TOL), ("tf32x3", helpers.FP32_TOL),
                                           ("tf32", helpers.TC_TOL), ("bf16", helpers.TC_TOL)])
def test_config3_one_room(precision, tol, cuda):
    """The U-Net of configuration 3 on one full room (~200 k voxels) against the reference's
    CPU build; against the restatement on a 20 k-voxel room where that is absent."""
    ref = runner.reference_available()
    coords, feats = workloads.batch_config3([0], target_voxels=200000 if ref else 20000)
    be, yo, gpu, yg = _run_both(3, coords, feats, precision)
    e = helpers.assert_features_match(gpu.locations(yg), yg.features, be.locations(yo), yo.features, tol,
                                      what="config 3 " + precision)
    print("config3 %s rel err %.3g" % (precision, e))


def test_config4_shapes(cuda):
    coords, feats = workloads.make_batch(4, range(4))
    be, yo, gpu, yg = _run_both(4, coords, feats)
    assert yg.spatial_size == [7, 7, 7] and yg.features.shape[1] == 128
    helpers.assert_features_match(gpu.locations(yg), yg.features, be.locations(yo), yo.features, helpers.FP32_TOL,
                                  what="config 4")


@pytest.mark.parametrize("precision,tol", [("fp32", helpers.FP32_TOL), ("bf16", helpers.TC_TOL),
                                           ("tf32x3", helpers.FP32_TOL)])
def test_config5_reduced(precision, tol, cuda):
    """4-D stack (81 offsets): one sequence of three frames.  In the fp32-accuracy tensor mode the 64-plane
    layers are too wide in offsets for the warp-level kernels (32 at most) and go on to tcgen05."""
    c = workloads.sequence_config5(0, frames=3)
    coords = np.concatenate([c, np.zeros((c.shape[0], 1), np.int64)], axis=1)
    feats = np.random.default_rng(5).standard_normal((coords.shape[0], 64)).astype(np.float32)
    be, yo, gpu, yg = _run_both(5, coords, feats, precision)
    helpers.assert_features_match(gpu.locations(yg), yg.features, be.locations(yo), yo.features, tol,
                                  same_rows=True, what="config 5 " + precision)


def test_config3_full_batch_properties(cuda, restore_precision):
    """Full benchmark size (8 rooms, ~1.6 M voxels), properties that need no oracle: active
    sites reported in input order, one centre rule per site, mirrored offsets hold mirrored
    rules, strided rulebook covers every fine site exactly once, the convolution is linear,
    and two runs give identical bits."""
    import sparseconvnet_b200 as scn
    coords, feats = workloads.make_batch(3, range(8))
    dev = cuda
    inp = scn.InputLayer(3, 4096, mode=4)
    f = torch.from_numpy(feats).to(dev)
    x = inp([torch.from_numpy(coords), f])
    n = coords.shape[0]
    assert x.features.shape == (n, 3)
    assert torch.equal(x.get_spatial_locations(), torch.from_numpy(coords))
    torch.manual_seed(0)
    sc = scn.SubmanifoldConvolution(3, 3, 32, 3, False).to(dev)
    down = scn.Convolution(3, 32, 64, 2, 2, False).to(dev)
    up = scn.Deconvolution(3, 64, 32, 2, 2, False).to(dev)
    with torch.no_grad():
        y = sc(x)
        z = down(y)
        w = up(z)
        x.metadata.poll_errors()
        rules = x.metadata.rulebook(0, [4096] * 3, [3] * 3)
        assert rules[13].shape[0] == n
        counts = [r.shape[0] for r in rules]
        assert counts == counts[::-1]
        strided = x.metadata.rulebook(1, [4096] * 3, [2] * 3, [2] * 3)
        fine = torch.cat([r[:, 0] for r in strided]).long()
        assert fine.numel() == n and torch.equal(torch.sort(fine).values, torch.arange(n, device=dev))
        assert w.features.shape == (n, 32)
        # linearity of the convolution on the full cloud
        a = torch.randn(n, 3, device=dev)
        xa = scn.SparseConvNetTensor(a, x.metadata, x.spatial_size)
        xb = scn.SparseConvNetTensor(f, x.metadata, x.spatial_size)
        xab = scn.SparseConvNetTensor(a + f, x.metadata, x.spatial_size)
        lhs = sc(xab).features
        rhs = sc(xa).features + sc(xb).features
        assert float((lhs - rhs).abs().max() / rhs.abs().max()) < 1e-5
        # determinism
        assert torch.equal(sc(x).features, y.features)
        x2 = inp([torch.from_numpy(coords), f])
        assert torch.equal(down(sc(x2)).features, z.features)
