"""Backward passes through the C ABI (autograd wiring of sparseconvnet_b200) against the backward
functions of the reference's own CPU build (oracle/_ref), operator by operator, and a training
step of a small U-Net.  Rows of strided levels are numbered differently by the two (see
helpers / oracle.align_rows), so gradients are compared after matching rows by coordinates.

Tolerance: 1e-4 of the largest magnitude (fp32; sums are formed in different orders)."""
import numpy as np
import pytest
import torch

from oracle import runner, scn_oracle as port
from tests import helpers

pytestmark = pytest.mark.gpu

TOL = helpers.FP32_TOL


def _lt(v):
    return torch.LongTensor([int(i) for i in v])


def _rel(a, b):
    a, b = torch.as_tensor(a).float().cpu(), torch.as_tensor(b).float().cpu()
    assert a.shape == b.shape, (a.shape, b.shape)
    return (a - b).abs().max().item() / max(b.abs().max().item(), 1e-12) if a.numel() else 0.0


@pytest.fixture(scope="module")
def ref():
    if not runner.reference_available():
        pytest.skip("reference build (oracle/_ref) not available")
    return runner.RefBackend().SCN


def _cloud(rng, size, n, batch):
    return np.concatenate([np.stack([rng.integers(0, v, n) for v in size], 1), rng.integers(0, batch, (n, 1))], 1)


def _ref_input(ref, dim, size, coords, feats, mode=3):
    md = getattr(ref, "Metadata_%d" % dim)()
    out = torch.empty(0)
    ref.InputLayer_updateOutput(md, _lt(size), torch.from_numpy(coords).long(), torch.from_numpy(feats), out, 0, mode)
    return md, out


@pytest.mark.parametrize("dim,size,cin,cout,groups,bias", [(2, [17, 17], 6, 8, 2, True), (3, [15, 15, 15], 5, 7, 1, True),
                                                            (3, [16, 16, 16], 32, 32, 1, False),
                                                            (3, [16, 16, 16], 64, 48, 1, True),
                                                            (3, [16, 16, 16], 64, 96, 1, True)])
@pytest.mark.parametrize("kind", ["sub", "conv", "deconv"])
@pytest.mark.parametrize("bwd", ["fp32", "tf32x3"])
def test_convolution_gradients(ref, cuda, dim, size, cin, cout, groups, bias, kind, bwd):
    """`bwd`: arithmetic of the input-gradient pass (fp32 FMA, or the fp32-class tensor kernels)."""
    import sparseconvnet_b200 as scn
    scn.set_backward_precision(bwd)
    try:
        _convolution_gradients(ref, cuda, dim, size, cin, cout, groups, bias, kind)
    finally:
        scn.set_backward_precision("fp32")


def _convolution_gradients(ref, cuda, dim, size, cin, cout, groups, bias, kind):
    import sparseconvnet_b200 as scn
    rng = np.random.default_rng(dim * 100 + cin)
    coords = _cloud(rng, size, 500, 2)
    feats = rng.standard_normal((500, cin)).astype(np.float32)
    f = 3 if size[0] % 2 else 2
    torch.manual_seed(1)
    if kind == "sub":
        m = scn.SubmanifoldConvolution(dim, cin, cout, 3, bias, groups)
    elif kind == "conv":
        m = scn.Convolution(dim, cin, cout, f, 2, bias, groups)
    else:
        m = scn.Deconvolution(dim, cout, cin, f, 2, bias, groups)
    if bias:
        m.bias.data.normal_()
    m = m.to(cuda)
    x = scn.InputLayer(dim, size, 3)([torch.from_numpy(coords), torch.from_numpy(feats).to(cuda)])
    down = scn.Convolution(dim, cin, cout, f, 2, False, groups).to(cuda)
    if kind == "deconv":
        with torch.no_grad():
            x = down(x)
    x.features = x.features.detach().clone().requires_grad_(True)
    y = m(x)
    go = torch.randn_like(y.features)
    y.features.backward(go)

    md, o = _ref_input(ref, dim, size, coords, feats)
    w = m.weight.detach().cpu()
    b = m.bias.detach().cpu() if bias else torch.empty(0)
    fin = x.features.detach().cpu()
    gi, gw, gb = torch.empty(0), torch.zeros_like(w), torch.zeros_like(b)
    insz, outsz = _lt(size), _lt([(s - f) // 2 + 1 for s in size])
    fs, st = _lt([f] * dim), _lt([2] * dim)
    if kind == "sub":
        ref.SubmanifoldConvolution_backward(insz, _lt([3] * dim), md, fin, gi, go.cpu(), w, gw, gb)
    else:
        wd = (down.weight if kind == "deconv" else m.weight).detach().cpu()
        tmp = torch.empty(0)
        ref.Convolution_updateOutput(insz, outsz, fs, st, md, o, tmp, wd, torch.empty(0))  # makes the coarse grid
        loc_gpu = (y if kind == "conv" else x).get_spatial_locations().numpy()
        p = torch.from_numpy(port.align_rows(loc_gpu, md.getSpatialLocations(outsz).numpy()))
        if kind == "conv":
            go_ref = torch.zeros_like(go.cpu())
            go_ref[p] = go.cpu()
            ref.Convolution_backward(insz, outsz, fs, st, md, fin, gi, go_ref, w, gw, gb)
        else:
            fin_ref = torch.zeros_like(fin)
            fin_ref[p] = fin
            ref.Deconvolution_backward(outsz, insz, fs, st, md, fin_ref, gi, go.cpu(), w, gw, gb)
            gi = gi[p]
    assert _rel(x.features.grad, gi) <= TOL
    assert _rel(m.weight.grad, gw) <= TOL
    if bias:
        assert _rel(m.bias.grad, gb) <= TOL


@pytest.mark.parametrize("leak,affine,train", [(0.0, True, True), (0.333, True, True), (1.0, False, True),
                                               (0.0, True, False)])
def test_batchnorm_gradients(ref, cuda, leak, affine, train):
    import sparseconvnet_b200 as scn
    rng = np.random.default_rng(5)
    n, c = 700, 12
    feats = (rng.standard_normal((n, c)) * 2 + 0.5).astype(np.float32)
    m = scn.BatchNormalization(c, 1e-4, 0.9, affine, leak).to(cuda)
    if affine:
        m.weight.data.uniform_(0.5, 1.5)
        m.bias.data.normal_()
    m.running_mean.normal_()
    m.running_var.uniform_(0.5, 2.0)
    m.train(train)
    rm, rv = m.running_mean.clone().cpu(), m.running_var.clone().cpu()
    x = scn.SparseConvNetTensor(torch.from_numpy(feats).to(cuda).requires_grad_(True), None, None)
    y = m(x)
    go = torch.randn_like(y.features)
    y.features.backward(go)

    fin = torch.from_numpy(feats)
    out, sm, si = torch.empty(0), torch.empty(c), torch.empty(c)
    w = m.weight.detach().cpu() if affine else torch.empty(0)
    b = m.bias.detach().cpu() if affine else torch.empty(0)
    ref.BatchNormalization_updateOutput(fin, out, sm, si, rm, rv, w, b, 1e-4, 0.9, train, leak)
    gi, gw, gb = torch.empty(0), torch.zeros_like(w), torch.zeros_like(b)
    ref.BatchNormalization_backward(fin, gi, out, go.cpu().clone(), sm, si, rm, rv, w, b, gw, gb, leak)
    assert _rel(y.features, out) <= TOL
    assert _rel(x.features.grad, gi) <= TOL
    if affine:
        assert _rel(m.weight.grad, gw) <= TOL and _rel(m.bias.grad, gb) <= TOL


@pytest.mark.parametrize("leak,affine", [(0.0, True), (0.333, True), (1.0, False)])
def test_batchnorm_statistics_over_several_ranks(ref, cuda, leak, affine):
    """Training-mode BatchNorm with its rows spread over three ranks (one of them without rows): the two-phase
    entry points with the ranks' sums added in between give what the reference gives for the whole matrix on one
    device (CPU/BatchNormalization.cpp:12-107) -- outputs, running statistics, d_input, and parameter gradients
    once the ranks' shares are added.  The ranks run one after the other here; the all-reduce is stood in for by
    a function that returns the sum of what every rank contributed."""
    from sparseconvnet_b200 import SCN
    rng = np.random.default_rng(15)
    n, c = 1900, 12
    feats = (rng.standard_normal((n, c)) * 2 + 0.5).astype(np.float32)
    go = rng.standard_normal((n, c)).astype(np.float32)
    cuts = [(0, 1200), (1200, 1900), (1900, 1900)]
    w = torch.from_numpy(rng.uniform(0.5, 1.5, c).astype(np.float32)) if affine else torch.empty(0)
    b = torch.from_numpy(rng.standard_normal(c).astype(np.float32)) if affine else torch.empty(0)
    rm0 = torch.from_numpy(rng.standard_normal(c).astype(np.float32))
    rv0 = torch.from_numpy(rng.uniform(0.5, 2.0, c).astype(np.float32))

    def forward(reduce):
        res = []
        for lo, hi in cuts:
            f = torch.from_numpy(feats[lo:hi]).to(cuda)
            out, sm, si = f.new_empty(0), f.new_empty(c), f.new_empty(c)
            rm, rv = rm0.clone().to(cuda), rv0.clone().to(cuda)
            sums = SCN.BatchNormalization_updateOutput_acrossRanks(f, out, sm, si, rm, rv, w.to(cuda), b.to(cuda), 1e-4,
                                                                   0.9, leak, reduce=reduce)
            res.append((f, out, sm, si, rm, rv, sums))
        return res

    def backward(fwd, reduce):
        res = []
        for (lo, hi), (f, out, sm, si, rm, rv, sums) in zip(cuts, fwd):
            g = torch.from_numpy(go[lo:hi]).to(cuda)
            d_in = f.new_empty(0)
            dw = torch.zeros(c, device=cuda) if affine else None
            db = torch.zeros(c, device=cuda) if affine else None
            SCN.BatchNormalization_backward_acrossRanks(f, d_in, out, g, sm, si, w.to(cuda), dw, db, leak, sums,
                                                        reduce=reduce)
            res.append((d_in, dw, db))
        return res

    parts = []
    forward(lambda t, g: parts.append(t.clone()))
    assert len(parts) == 3 and parts[2][:2 * c].abs().max().item() == 0 and parts[0][2 * c].item() == 1200
    total = sum(parts)
    fwd = forward(lambda t, g: t.copy_(total))
    parts_b = []
    backward(fwd, lambda t, g: parts_b.append(t.clone()))
    total_b = sum(parts_b)
    bwd = backward(fwd, lambda t, g: t.copy_(total_b))

    fin = torch.from_numpy(feats)
    out, sm, si = torch.empty(0), torch.empty(c), torch.empty(c)
    rm, rv = rm0.clone(), rv0.clone()
    ref.BatchNormalization_updateOutput(fin, out, sm, si, rm, rv, w, b, 1e-4, 0.9, True, leak)
    gi, gw, gb = torch.empty(0), torch.zeros_like(w), torch.zeros_like(b)
    ref.BatchNormalization_backward(fin, gi, out, torch.from_numpy(go).clone(), sm, si, rm, rv, w, b, gw, gb, leak)
    assert fwd[2][1].shape == (0, c) and bwd[2][0].shape == (0, c)
    assert _rel(torch.cat([r[1] for r in fwd]), out) <= TOL
    assert _rel(torch.cat([r[0] for r in bwd]), gi) <= TOL
    for r in fwd:   # every rank, the one without rows too, keeps the same running statistics
        assert _rel(r[4], rm) <= TOL and _rel(r[5], rv) <= TOL and _rel(r[2], sm) <= TOL and _rel(r[3], si) <= TOL
    if affine:
        assert _rel(sum(r[1] for r in bwd), gw) <= TOL and _rel(sum(r[2] for r in bwd), gb) <= TOL
    # one rank holding everything: the two phases are the one-call operator
    f = torch.from_numpy(feats).to(cuda)
    one, sm1, si1 = f.new_empty(0), f.new_empty(c), f.new_empty(c)
    SCN.BatchNormalization_updateOutput(f, one, sm1, si1, rm0.clone().to(cuda), rv0.clone().to(cuda), w.to(cuda),
                                        b.to(cuda), 1e-4, 0.9, True, leak)
    two, sm2, si2 = f.new_empty(0), f.new_empty(c), f.new_empty(c)
    SCN.BatchNormalization_updateOutput_acrossRanks(f, two, sm2, si2, rm0.clone().to(cuda), rv0.clone().to(cuda),
                                                    w.to(cuda), b.to(cuda), 1e-4, 0.9, leak, reduce=lambda t, g: None)
    assert _rel(two, one) <= 1e-6 and _rel(sm2, sm1) <= 1e-6 and _rel(si2, si1) <= 1e-6


@pytest.mark.parametrize("kind", ["max", "avg", "unpool"])
@pytest.mark.parametrize("dim,size,f,s", [(2, [17, 17], 3, 2), (3, [16, 16, 16], 2, 2)])
def test_pooling_gradients(ref, cuda, kind, dim, size, f, s):
    import sparseconvnet_b200 as scn
    rng = np.random.default_rng(9)
    # The reference's MaxPooling backward ignores nFeaturesToDrop when it indexes the input
    # (CPU/MaxPooling.cpp:74-77 against :52-55), so it is only comparable with nothing dropped.
    n, c, drop = 400, 5, 1 if kind == "avg" else 0
    coords = _cloud(rng, size, n, 2)
    feats = rng.standard_normal((n, c)).astype(np.float32)
    x0 = scn.InputLayer(dim, size, 3)([torch.from_numpy(coords), torch.from_numpy(feats).to(cuda)])
    md, o = _ref_input(ref, dim, size, coords, feats)
    insz, outsz = _lt(size), _lt([(v - f) // s + 1 for v in size])
    ps, st = _lt([f] * dim), _lt([s] * dim)
    if kind == "unpool":
        # coarse features come from an average pooling; un-pool them back onto the input's sites
        with torch.no_grad():
            xc = scn.AveragePooling(dim, f, s)(x0)
        xc.features = xc.features.detach().clone().requires_grad_(True)
        y = scn.UnPooling(dim, f, s)(xc)
        go = torch.randn_like(y.features)
        y.features.backward(go)
        tmp = torch.empty(0)
        ref.AveragePooling_updateOutput(insz, outsz, ps, st, md, o, tmp, 0)
        p = torch.from_numpy(port.align_rows(xc.get_spatial_locations().numpy(), md.getSpatialLocations(outsz).numpy()))
        gi = torch.zeros(tmp.shape)
        ref.UnPooling_updateGradInput(outsz, insz, ps, st, md, gi, go.cpu(), 0)
        assert _rel(xc.features.grad, gi[p]) <= TOL
        return
    x0.features = x0.features.detach().clone().requires_grad_(True)
    mod = scn.MaxPooling(dim, f, s, drop) if kind == "max" else scn.AveragePooling(dim, f, s, drop)
    y = mod(x0)
    go = torch.randn_like(y.features)
    y.features.backward(go)
    out = torch.empty(0)
    fwd = ref.MaxPooling_updateOutput if kind == "max" else ref.AveragePooling_updateOutput
    fwd(insz, outsz, ps, st, md, o, out, drop)
    p = torch.from_numpy(port.align_rows(y.get_spatial_locations().numpy(), md.getSpatialLocations(outsz).numpy()))
    go_ref = torch.zeros_like(go.cpu())
    go_ref[p] = go.cpu()
    gi = torch.empty(0)
    if kind == "max":
        ref.MaxPooling_updateGradInput(insz, outsz, ps, st, md, o, gi, out, go_ref, drop)
    else:
        ref.AveragePooling_updateGradInput(insz, outsz, ps, st, md, o, gi, go_ref, drop)
    assert _rel(x0.features.grad, gi) <= TOL


@pytest.mark.parametrize("mode", [0, 1, 2, 3, 4])
def test_io_layer_and_dense_gradients(ref, cuda, mode):
    import sparseconvnet_b200 as scn
    rng = np.random.default_rng(20 + mode)
    dim, size, n, c = 2, [9, 9], 150, 4
    coords = _cloud(rng, size, n, 2)
    if mode == 0:
        coords = np.unique(coords, axis=0)
        n = coords.shape[0]
    feats = rng.standard_normal((n, c)).astype(np.float32)
    pts = torch.from_numpy(feats).to(cuda).requires_grad_(True)
    x = scn.InputLayer(dim, size, mode)([torch.from_numpy(coords), pts])
    dense = scn.SparseToDense(dim, c)(x)
    back = scn.OutputLayer(dim)(x)
    g_dense, g_back = torch.randn_like(dense), torch.randn_like(back)
    (dense * g_dense).sum().backward(retain_graph=True)
    grad_from_dense = pts.grad.clone()
    pts.grad = None
    (back * g_back).sum().backward()
    grad_from_back = pts.grad.clone()

    md, o = _ref_input(ref, dim, size, coords, feats, mode)
    # SparseToDense -> sites -> points
    d_sites = torch.empty(0)
    ref.SparseToDense_updateGradInput(_lt(size), md, o, d_sites, g_dense.cpu())
    d_pts = torch.empty(0)
    ref.InputLayer_updateGradInput(md, d_pts, d_sites)
    assert _rel(grad_from_dense, d_pts) <= 1e-6
    # OutputLayer -> sites -> points
    d_sites2 = torch.empty(0)
    ref.OutputLayer_updateGradInput(md, d_sites2, g_back.cpu())
    d_pts2 = torch.empty(0)
    ref.InputLayer_updateGradInput(md, d_pts2, d_sites2)
    assert _rel(grad_from_back, d_pts2) <= 1e-6


def test_unet_training_step_reduces_the_loss(cuda):
    """Three SGD steps on a small U-Net with per-voxel labels: gradients reach every parameter, are
    finite and reproducible bit for bit, and the loss goes down."""
    import sparseconvnet_b200 as scn
    from tests.golden import cases
    coords, feats = cases.net_inputs("net_unet3d")
    torch.manual_seed(3)
    net = scn.Sequential().add(scn.SubmanifoldConvolution(3, 3, 8, 3, False)).add(
        scn.UNet(3, 1, [8, 16, 24], residual_blocks=True)).add(scn.BatchNormReLU(8)).to(cuda)
    head = torch.nn.Linear(8, 5).to(cuda)
    params = list(net.parameters()) + list(head.parameters())
    opt = torch.optim.SGD(params, lr=0.05)
    inp = scn.InputLayer(3, 64, mode=4)
    labels = None
    losses, first_grads = [], None
    for step in range(3):
        x = inp([torch.from_numpy(coords), torch.from_numpy(feats).to(cuda)])
        logits = head(net(x).features)
        if labels is None:
            labels = torch.randint(0, 5, (logits.size(0),), device=cuda, generator=torch.Generator(cuda).manual_seed(1))
        loss = torch.nn.functional.cross_entropy(logits, labels)
        opt.zero_grad()
        loss.backward()
        assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in params)
        if step == 0:
            first_grads = [p.grad.clone() for p in params]
            # the same step again: bit-identical gradients
            opt.zero_grad()
            x2 = inp([torch.from_numpy(coords), torch.from_numpy(feats).to(cuda)])
            torch.nn.functional.cross_entropy(head(net(x2).features), labels).backward()
            assert all(torch.equal(a, p.grad) for a, p in zip(first_grads, params))
        losses.append(loss.item())
        opt.step()
    assert losses[-1] < losses[0], losses
