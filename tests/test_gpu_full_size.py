"""Full benchmark sizes on the GPU against the reference's own stock path: the reference's
unmodified Python package (its scn.UNet / SparseResNet / SparseVggNet builders, InputLayer ...)
on its own CPU extension, both staged under oracle/_ref by oracle/build_ref.py.

Every convolution kernel of the library is also compared here, one layer at a time, with the
reference's CPU operator directly (not with another CUDA kernel): the row-stationary
warp-level kernel, the persistent tcgen05 kernel in every arithmetic mode, and the per-tile
tcgen05 kernel with and without the split of the filter offsets.

Tolerances relative to the tensor's largest magnitude: 1e-4 for fp32 and the fp32-class split
mode, 1e-2 for single-pass tf32 / bf16."""
import numpy as np
import pytest
import torch

from oracle import refpkg, runner
from sparseconvnet_b200 import workloads
from tests import helpers

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not (refpkg.available("cpu") and runner.reference_available()),
                                 reason="oracle/_ref (the compiled reference) is not present")]

_cache = {}


def _reference_forward(config, samples, key):
    """(locations, features | None, dense | None) of the configuration's network on the reference."""
    if key in _cache:
        return _cache[key]
    ref = refpkg.load("cpu")
    torch.set_num_threads(max(1, torch.get_num_threads()))
    inp, net, _ = workloads.build_config(config, scn=ref)
    coords, feats = workloads.make_batch(config, samples)
    with torch.no_grad():
        y = net(inp([torch.from_numpy(coords), torch.from_numpy(feats)]))
    if isinstance(y, torch.Tensor):
        out = (None, None, y.numpy())
    else:
        out = (y.get_spatial_locations().numpy(), y.features.numpy(), None)
    _cache[key] = out
    return out


def _gpu_forward(config, samples, precision, profile=False):
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200 import SCN
    dev = torch.device("cuda:0")
    inp, net, _ = workloads.build_config(config)
    net.to(dev)
    coords, feats = workloads.make_batch(config, samples)
    scn.set_precision(precision)
    kernels = None
    try:
        with torch.no_grad():
            if profile:
                with SCN.Profile() as prof:
                    x = inp([torch.from_numpy(coords), torch.from_numpy(feats).to(dev)])
                    y = net(x)
                kernels = [r["kernel"] for r in prof.rows() if r["kind"] == "conv"]
            else:
                x = inp([torch.from_numpy(coords), torch.from_numpy(feats).to(dev)])
                y = net(x)
        torch.cuda.synchronize()
        x.metadata.poll_errors()
    finally:
        scn.set_precision("fp32")
    if isinstance(y, torch.Tensor):
        return None, None, y.cpu().numpy(), kernels
    return y.get_spatial_locations().numpy(), y.features.cpu().numpy(), None, kernels


@pytest.mark.parametrize("precision,tol", [("tf32x3", helpers.FP32_TOL), ("fp32", helpers.FP32_TOL)])
def test_config3_full_batch_vs_reference(precision, tol, cuda):
    """The benchmark's own shape: the U-Net on all 8 rooms (~1.6 M voxels).  In the fp32-class mode
    every convolution kernel class of the step must have run: warp-level rows kernel (32 / 64
    output planes), persistent tcgen05 (96 / 128 planes on the large levels), per-tile tcgen05
    (the small deep levels)."""
    loc_r, feat_r, _ = _reference_forward(3, list(range(8)), "c3x8")
    loc_g, feat_g, _, kernels = _gpu_forward(3, list(range(8)), precision, profile=True)
    e = helpers.assert_features_match(loc_g, feat_g, loc_r, feat_r, tol, what="config 3 x 8 rooms " + precision)
    print("config3 x8 %s rel err %.3g kernels %s" % (precision, e, sorted(set(kernels))))
    assert len(kernels) == 39
    if precision == "tf32x3":
        assert {"k_conv_rows", "k_conv_wide", "k_conv_tc"} <= set(kernels), sorted(set(kernels))
    else:
        assert set(kernels) == {"k_conv_simt"}, sorted(set(kernels))


@pytest.mark.parametrize("precision,tol", [("fp32", helpers.FP32_TOL), ("tf32x3", helpers.FP32_TOL)])
def test_config4_all_shapes_vs_reference(precision, tol, cuda):
    loc_r, feat_r, _ = _reference_forward(4, list(range(16)), "c4x16")
    loc_g, feat_g, _, _ = _gpu_forward(4, list(range(16)), precision)
    assert feat_g.shape[1] == 128
    helpers.assert_features_match(loc_g, feat_g, loc_r, feat_r, tol, what="config 4 x 16 shapes " + precision)


@pytest.mark.parametrize("precision,tol", [("bf16", helpers.TC_TOL), ("tf32x3", helpers.FP32_TOL)])
def test_config5_full_vs_reference(precision, tol, cuda):
    """4 sequences x 8 frames (~1.6 M sites, 81 filter offsets, 64 -> 64 planes, four layers)."""
    loc_r, feat_r, _ = _reference_forward(5, list(range(4)), "c5x4")
    loc_g, feat_g, _, kernels = _gpu_forward(5, list(range(4)), precision, profile=True)
    e = helpers.assert_features_match(loc_g, feat_g, loc_r, feat_r, tol, same_rows=True, what="config 5 " + precision)
    print("config5 full %s rel err %.3g kernels %s" % (precision, e, sorted(set(kernels))))


def test_config2_full_batch_vs_reference(cuda):
    _, _, dense_r = _reference_forward(2, list(range(100)), "c2x100")
    _, _, dense_g, _ = _gpu_forward(2, list(range(100)), "fp32")
    assert dense_g.shape == (100, 32, 10, 10)
    assert helpers.rel_err(dense_g, dense_r) <= helpers.FP32_TOL


def test_config1_vs_reference(cuda):
    """Config 1 (one 32 -> 32 submanifold convolution on the 256^3 cloud) against the reference's CPU
    operator, rulebook included (canonical comparison: rules as coordinate pairs per offset)."""
    from oracle import scn_oracle as port
    coords, feats = workloads.make_batch(1, [0])
    inp, net, _ = workloads.build_config(1)
    be = runner.RefBackend()
    xo = runner.run_module(inp, [coords, feats], be)
    yo = runner.run_module(net, xo, be)
    gpu = helpers.GpuBackend()
    xg = gpu.run(inp, [coords, feats])
    yg = gpu.run(net, xg)
    yg.t.metadata.poll_errors()
    helpers.assert_features_match(gpu.locations(yg), yg.features, be.locations(yo), yo.features, helpers.FP32_TOL,
                                  what="config 1 vs reference")
    rg = port.canonical_rules(gpu.submanifold_rulebook(yg, [3, 3, 3]), gpu.locations(yg), gpu.locations(yg))
    rr = port.canonical_rules(be.submanifold_rulebook(yo, [3, 3, 3]), be.locations(yo), be.locations(yo))
    helpers.assert_rules_equal(rg, rr, "config 1 rulebook vs reference")


# ---- one layer at a time: every tensor kernel against the reference's CPU operator -------------------

def _surface(n, size, batch, seed):
    rng = np.random.default_rng(seed)
    pts = rng.integers(0, size, (n, 2))
    z = (size / 2 + size / 5 * np.sin(pts[:, 0] / 6.0) + size / 8 * np.cos(pts[:, 1] / 4.0)).astype(np.int64)
    return np.concatenate([pts, z[:, None], rng.integers(0, batch, (n, 1))], axis=1)


def _layer_vs_reference(cin, cout, precision, tol, expect_kernel, n=60000, size=160, env=None, monkeypatch=None,
                        bias=True):
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200._lib import lib
    for k, v in (env or {}).items():
        monkeypatch.setenv(k, v)
    coords = _surface(n, size, 2, 7 + cin)
    rng = np.random.default_rng(cin * 31 + cout)
    feats = rng.standard_normal((coords.shape[0], cin)).astype(np.float32)
    torch.manual_seed(cin * 1000 + cout)
    inp = scn.InputLayer(3, size, mode=3)
    sc = scn.SubmanifoldConvolution(3, cin, cout, 3, bias)
    if bias:
        sc.bias.data.normal_()
    be = runner.RefBackend()
    yo = runner.run_module(sc, runner.run_module(inp, [coords, feats], be), be)
    gpu = helpers.GpuBackend()
    scn.set_precision(precision)
    try:
        xg = gpu.run(inp, [coords, feats])
        yg = gpu.run(sc, xg)
        kernel = lib.scn_last_conv_kernel()
        yg.t.metadata.poll_errors()
    finally:
        scn.set_precision("fp32")
    assert kernel == expect_kernel, "kernel %d ran, expected %d" % (kernel, expect_kernel)
    e = helpers.assert_features_match(gpu.locations(yg), yg.features, be.locations(yo), yo.features, tol,
                                      what="%d->%d %s" % (cin, cout, precision))
    return e, yg.features.shape[0]


@pytest.mark.parametrize("precision,form,tol,kernel", [
    ("tf32x3", "bf16", helpers.FP32_TOL, 5),   # k_conv_wide, three bf16 products
    ("bf16", "bf16", helpers.TC_TOL, 5),       # k_conv_wide, one product
    ("tf32x3", "tf32", helpers.FP32_TOL, 2),   # k_conv_tma, three-pass tf32 split
    ("tf32", "bf16", helpers.TC_TOL, 2)])      # k_conv_tma, single tf32 pass
@pytest.mark.parametrize("cin,cout", [(96, 96), (128, 128), (192, 96), (64, 64), (96, 160), (256, 224)])
def test_persistent_tcgen05_vs_reference(cin, cout, precision, form, tol, kernel, cuda, monkeypatch):
    """The two persistent tcgen05 kernels forced on (SCN_TC_PERSISTENT=1; 64 output planes sent to them by
    SCN_X3_MIN_COUT) in every arithmetic mode, for one and two 128-plane accumulator tiles."""
    if precision == "tf32x3" and form == "tf32" and cout > 160:
        pytest.skip("two fp32 weight slabs of this width leave k_conv_tma a single stage: k_conv_tc takes the shape")
    e, rows = _layer_vs_reference(cin, cout, precision, tol, kernel, monkeypatch=monkeypatch,
                                  env={"SCN_TC_PERSISTENT": "1", "SCN_X3_FORM": form, "SCN_X3_MIN_COUT": "64",
                                       "SCN_X3_ROWS": "0" if cout == 64 and precision != "tf32x3" else "1"})
    print("persistent tcgen05 %d->%d %s/%s: %d rows, rel err %.3g" % (cin, cout, precision, form, rows, e))


@pytest.mark.parametrize("split", ["1", "4"])
@pytest.mark.parametrize("precision,form,tol", [("tf32x3", "bf16", helpers.FP32_TOL), ("tf32x3", "tf32", helpers.FP32_TOL),
                                                ("bf16", "bf16", helpers.TC_TOL)])
@pytest.mark.parametrize("cin,cout", [(96, 96), (160, 160), (224, 224)])
def test_per_tile_tcgen05_vs_reference(cin, cout, precision, form, tol, split, cuda, monkeypatch):
    """k_conv_tc (the default below 148 tiles) without and with the split of the filter offsets over CTAs,
    in both forms of the fp32-class mode."""
    e, rows = _layer_vs_reference(cin, cout, precision, tol, 1, n=20000, size=96,
                                  env={"SCN_TC_SPLIT": split, "SCN_X3_FORM": form}, monkeypatch=monkeypatch)
    print("k_conv_tc %d->%d %s/%s split %s: %d rows, rel err %.3g" % (cin, cout, precision, form, split, rows, e))


@pytest.mark.parametrize("precision,form,tol", [("tf32x3", "bf16", helpers.FP32_TOL), ("tf32x3", "tf32", helpers.FP32_TOL),
                                                ("tf32", "bf16", helpers.TC_TOL), ("bf16", "bf16", helpers.TC_TOL)])
@pytest.mark.parametrize("cin,cout", [(32, 32), (64, 32), (64, 64), (128, 64)])
def test_rows_kernel_vs_reference(cin, cout, precision, form, tol, cuda, monkeypatch):
    """k_conv_rows (32 / 64 output planes) in its arithmetic modes, both forms of the fp32-class one."""
    e, rows = _layer_vs_reference(cin, cout, precision, tol, 4, monkeypatch=monkeypatch, bias=(cin == 64),
                                  env={"SCN_X3_FORM": form})
    print("k_conv_rows %d->%d %s/%s: %d rows, rel err %.3g" % (cin, cout, precision, form, rows, e))
