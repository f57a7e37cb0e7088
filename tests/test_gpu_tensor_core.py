"""The tcgen05 / TMEM convolution path against the fp32 kernel (itself checked against the
reference in test_gpu_parity.py) and against the numpy restatement.

Tolerances (relative to the largest output magnitude): 1e-2 for single-pass tf32 and bf16
tensor-core arithmetic, 1e-4 -- the fp32 bar -- for the three-pass tf32 split."""
import numpy as np
import pytest
import torch

from tests import helpers

pytestmark = pytest.mark.gpu

MODES = [("tf32", helpers.TC_TOL), ("bf16", helpers.TC_TOL), ("tf32x3", helpers.FP32_TOL)]


def _surface(n, size, batch, seed):
    rng = np.random.default_rng(seed)
    pts = rng.integers(0, size, (n, 2))
    z = (size / 2 + size / 5 * np.sin(pts[:, 0] / 6.0) + size / 8 * np.cos(pts[:, 1] / 4.0)).astype(np.int64)
    return np.concatenate([pts, z[:, None], rng.integers(0, batch, (n, 1))], axis=1)


@pytest.fixture
def restore_precision():
    import sparseconvnet_b200 as scn
    yield
    scn.set_precision("fp32")


@pytest.mark.parametrize("mode,tol", MODES)
@pytest.mark.parametrize("cin,cout", [(32, 32), (64, 64), (32, 16), (96, 160), (224, 224), (256, 128)])
def test_submanifold_conv_tensor_core(mode, tol, cin, cout, cuda, restore_precision):
    import sparseconvnet_b200 as scn
    coords = _surface(5000, 40, 2, 1)
    rng = np.random.default_rng(2)
    torch.manual_seed(cin * 1000 + cout)
    inp = scn.InputLayer(3, 40, mode=3)
    sc = scn.SubmanifoldConvolution(3, cin, cout, 3, True).to(cuda)
    sc.bias.data.normal_()
    feats = torch.from_numpy(rng.standard_normal((coords.shape[0], cin)).astype(np.float32)).to(cuda)
    with torch.no_grad():
        x = inp([torch.from_numpy(coords), feats])
        scn.set_precision("fp32")
        want = sc(x).features
        scn.set_precision(mode)
        got = sc(x).features
        x.metadata.poll_errors()
    err = helpers.rel_err(got.cpu().numpy(), want.cpu().numpy())
    assert err <= tol, "%s %d->%d: relative error %.3g" % (mode, cin, cout, err)
    assert err > 0 or mode == "tf32x3", "tensor-core result identical to fp32: the path did not run"


@pytest.mark.parametrize("rows", ["1", "0"])
@pytest.mark.parametrize("cin,cout", [(32, 32), (64, 32), (64, 64), (128, 64)])
def test_narrow_three_pass_kernels(cin, cout, rows, cuda, restore_precision, monkeypatch):
    """Layers with 32 or 64 output planes in the fp32-accuracy mode: the row-stationary kernel
    (default) and the compacting pipelined kernel (SCN_X3_ROWS=0), on a row count that is not a
    multiple of the 32-row warp tile, for a submanifold, a strided and a transposed rulebook."""
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200._lib import lib
    monkeypatch.setenv("SCN_X3_ROWS", rows)
    coords = _surface(7001, 56, 2, 31)
    rng = np.random.default_rng(32)
    torch.manual_seed(cin + 7 * cout)
    inp = scn.InputLayer(3, 56, mode=3)
    layers = [scn.SubmanifoldConvolution(3, cin, cout, 3, True).to(cuda),
              scn.Convolution(3, cin, cout, 2, 2, False).to(cuda)]
    feats = torch.from_numpy(rng.standard_normal((coords.shape[0], cin)).astype(np.float32)).to(cuda)
    with torch.no_grad():
        x = inp([torch.from_numpy(coords), feats])
        assert x.features.size(0) % 32 != 0
        for layer in layers + [None]:
            if layer is None:  # transposed rulebook: back from the coarse grid
                layer = scn.Deconvolution(3, cout, cout, 2, 2, False).to(cuda)
                scn.set_precision("fp32")
                x = layers[1](x)
            scn.set_precision("fp32")
            want = layer(x).features
            scn.set_precision("tf32x3")
            got = layer(x).features
            kernel = lib.scn_last_conv_kernel()
            x.metadata.poll_errors()
            assert kernel == (4 if rows == "1" else 3), "kernel %d ran" % kernel
            err = helpers.rel_err(got.cpu().numpy(), want.cpu().numpy())
            assert err <= helpers.FP32_TOL, "%d->%d rows=%s: relative error %.3g" % (cin, cout, rows, err)


@pytest.mark.parametrize("cin,cout", [(3, 32), (1, 16), (4, 64), (2, 32)])
def test_first_layer_three_pass_kernel(cin, cout, cuda, restore_precision):
    """First layers (at most four input planes) in the fp32-accuracy mode run on the warp-level
    tensor path too; other plane counts keep the fp32 kernel."""
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200._lib import lib
    coords = _surface(6007, 48, 3, 41)
    rng = np.random.default_rng(42)
    torch.manual_seed(cin + 11 * cout)
    inp = scn.InputLayer(3, 48, mode=3)
    sc = scn.SubmanifoldConvolution(3, cin, cout, 3, True).to(cuda)
    sc.bias.data.normal_()
    down = scn.Convolution(3, cin, cout, 2, 2, False).to(cuda)
    feats = torch.from_numpy(rng.standard_normal((coords.shape[0], cin)).astype(np.float32)).to(cuda)
    with torch.no_grad():
        x = inp([torch.from_numpy(coords), feats])
        for layer in (sc, down):
            scn.set_precision("fp32")
            want = layer(x).features
            assert lib.scn_last_conv_kernel() == 0
            scn.set_precision("tf32x3")
            got = layer(x).features
            assert lib.scn_last_conv_kernel() == 4
            x.metadata.poll_errors()
            err = helpers.rel_err(got.cpu().numpy(), want.cpu().numpy())
            assert err <= helpers.FP32_TOL, "%d->%d: relative error %.3g" % (cin, cout, err)


@pytest.mark.parametrize("gather", ["cp.async", "tma"])
@pytest.mark.parametrize("mode,tol", MODES)
def test_persistent_kernel_both_gathers(mode, tol, gather, cuda, restore_precision, monkeypatch):
    """The persistent kernel (double-buffered TMEM accumulators, one CTA per SM) forced on for
    every arithmetic mode, with its cp.async gather and with the TMA tile::gather4 gather
    (rows without a rule are out-of-bounds coordinates that the TMA unit zero-fills)."""
    import sparseconvnet_b200 as scn
    monkeypatch.setenv("SCN_TC_PERSISTENT", "1")
    monkeypatch.setenv("SCN_TC_TMA_GATHER", "1" if gather == "tma" else "0")
    coords = _surface(9000, 64, 3, 21)
    rng = np.random.default_rng(22)
    for cin, cout in ((32, 32), (64, 96), (128, 64)):
        torch.manual_seed(cin + cout)
        inp = scn.InputLayer(3, 64, mode=3)
        sc = scn.SubmanifoldConvolution(3, cin, cout, 3, True).to(cuda)
        sc.bias.data.normal_()
        feats = torch.from_numpy(rng.standard_normal((coords.shape[0], cin)).astype(np.float32)).to(cuda)
        with torch.no_grad():
            x = inp([torch.from_numpy(coords), feats])
            scn.set_precision("fp32")
            want = sc(x).features
            scn.set_precision(mode)
            got = sc(x).features
            x.metadata.poll_errors()
        err = helpers.rel_err(got.cpu().numpy(), want.cpu().numpy())
        assert err <= tol, "%s %s %d->%d: relative error %.3g" % (gather, mode, cin, cout, err)


@pytest.mark.parametrize("mode,tol", MODES)
def test_strided_and_transposed_tensor_core(mode, tol, cuda, restore_precision):
    import sparseconvnet_b200 as scn
    coords = _surface(6000, 48, 3, 3)
    rng = np.random.default_rng(4)
    torch.manual_seed(7)
    inp = scn.InputLayer(3, 48, mode=4)
    down = scn.Convolution(3, 32, 64, 2, 2, False).to(cuda)
    up = scn.Deconvolution(3, 64, 32, 2, 2, False).to(cuda)
    down3 = scn.Convolution(3, 32, 48, 3, 2, False).to(cuda)
    feats = torch.from_numpy(rng.standard_normal((coords.shape[0], 32)).astype(np.float32)).to(cuda)
    outs = {}
    with torch.no_grad():
        for m in ("fp32", mode):
            scn.set_precision(m)
            x = inp([torch.from_numpy(coords), feats])
            y = down(x)
            z = up(y)
            x47 = scn.InputLayer(3, 47, mode=4)([torch.from_numpy(np.minimum(coords, [46, 46, 46, 9])), feats])
            w = down3(x47)
            x.metadata.poll_errors()
            x47.metadata.poll_errors()
            outs[m] = [t.features.cpu().numpy() for t in (y, z, w)]
    for a, b, name in zip(outs[mode], outs["fp32"], ("conv 2/2", "deconv 2/2", "conv 3/2")):
        err = helpers.rel_err(a, b)
        assert err <= tol, "%s %s: relative error %.3g" % (mode, name, err)


@pytest.mark.parametrize("mode,tol", MODES)
def test_unet_tensor_core_against_golden(mode, tol, cuda, restore_precision):
    """Whole small U-Net (planes 8..32: only the 32-plane layers take the tensor path, the
    rest fall back to the fp32 kernel) against the reference's stored output."""
    import sparseconvnet_b200 as scn
    from tests.golden import cases
    g = helpers.load_golden("net_unet3d")
    inp, net, head = cases.net_modules("net_unet3d")
    helpers.load_state(net, g, "state")
    gpu = helpers.GpuBackend()
    scn.set_precision(mode)
    y = gpu.run(net, gpu.run(inp, [g["coords"], g["feats"]]))
    helpers.assert_features_match(gpu.locations(y), y.features, g["loc/y"], g["feat/y"], tol, what=mode)


def test_bounded_wait_runs_out_and_the_library_recovers(cuda, restore_precision):
    """Failure path of the tensor-core kernels, made on the host: one barrier arrival of one CTA is left
    out (a flag that nothing sets), so the MMA thread's bounded wait runs out.  The kernel must return on
    its own, the status must reach the host through poll_errors, and the next call must work."""
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200._lib import ScnError, lib
    coords = _surface(20000, 96, 2, 5)
    rng = np.random.default_rng(6)
    torch.manual_seed(7)
    inp = scn.InputLayer(3, 96, mode=3)
    sc = scn.SubmanifoldConvolution(3, 96, 96, 3, False).to(cuda)
    feats = torch.from_numpy(rng.standard_normal((coords.shape[0], 96)).astype(np.float32)).to(cuda)
    with torch.no_grad():
        x = inp([torch.from_numpy(coords), feats])
        scn.set_precision("fp32")
        want = sc(x).features
        scn.set_precision("bf16")
        good = sc(x).features.clone()
        assert lib.scn_last_conv_kernel() == 1      # the per-tile kernel: the one the hook reaches
        x.metadata.poll_errors()
        assert lib.scn_test_drop_barrier_arrival() == 0
        sc(x)                                        # returns: the launch is asynchronous
        torch.cuda.synchronize()                     # ... and the kernel ends by itself
        with pytest.raises(ScnError) as failure:
            x.metadata.poll_errors()
        assert "bounded wait" in str(failure.value)
        again = sc(x).features                       # the flag was cleared by the poll; the library works on
        x.metadata.poll_errors()
    assert torch.equal(again, good)
    assert helpers.rel_err(again.cpu().numpy(), want.cpu().numpy()) <= helpers.TC_TOL
