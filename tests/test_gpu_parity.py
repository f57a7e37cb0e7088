"""Parity of the CUDA path (called through the Python mirror of the reference API, which calls
the C ABI) against the golden fixtures made by the reference's CPU build, against the numpy
restatement, and -- when oracle/_ref travelled with the tree -- the live reference."""
import numpy as np
import pytest
import torch

from oracle import runner, scn_oracle as port
from tests import helpers
from tests.golden import cases

pytestmark = pytest.mark.gpu


def _exact_rules(a, b, what):
    assert len(a) == len(b), what
    for k, (ra, rb) in enumerate(zip(a, b)):
        assert np.array_equal(np.asarray(ra).reshape(-1, 2), np.asarray(rb).reshape(-1, 2)), "%s offset %d" % (what, k)


@pytest.mark.parametrize("name", sorted(cases.OPS_CASES))
def test_ops_against_golden_and_port(name, cuda):
    g = helpers.load_golden(name)
    c = cases.OPS_CASES[name]
    d = c["dim"]
    inputs = (g["coords"], g["feats"], int(g["batch_size_arg"]))

    net = cases.ops_modules(name)
    helpers.load_state(net, g, "state")
    gpu = helpers.GpuBackend()
    st = cases.run_ops(net, inputs, gpu.run, gpu.locations)

    # -- golden (reference CPU build): canonical comparison
    assert gpu.batch_size(st["x0"]) == int(g["batch_size"])
    for k in ("x0", "x1", "x4", "x7"):
        helpers.assert_features_match(gpu.locations(st[k]), st[k].features, g["loc/" + k], g["feat/" + k],
                                      helpers.FP32_TOL, same_rows=True, what=name + ":" + k)
    for k in ("x2", "x3", "x5", "x6"):
        helpers.assert_features_match(gpu.locations(st[k]), st[k].features, g["loc/" + k], g["feat/" + k],
                                      helpers.FP32_TOL, what=name + ":" + k)
    assert helpers.rel_err(st["dense"], g["dense"]) <= helpers.FP32_TOL
    if c["mode"] in (0, 1, 2, 3):
        assert np.array_equal(st["x0"].features, g["feat/x0"]), "input layer must be bit exact"
    sub = port.canonical_rules(gpu.submanifold_rulebook(st["x0"], [3] * d), gpu.locations(st["x0"]),
                               gpu.locations(st["x0"]))
    helpers.assert_rules_equal(sub, helpers.golden_rules(g, "rules_sub"), name + " submanifold")
    strided = port.canonical_rules(
        gpu.strided_rulebook(st["x1"], st["x2"].spatial_size, [c["f"]] * d, [c["s"]] * d),
        gpu.locations(st["x1"]), gpu.locations(st["x2"]))
    helpers.assert_rules_equal(strided, helpers.golden_rules(g, "rules_strided"), name + " strided")

    # -- numpy restatement: same deterministic numbering, so everything is compared row for row
    net_cpu = cases.ops_modules(name)
    helpers.load_state(net_cpu, g, "state")
    pb = runner.PortBackend()
    sp = cases.run_ops(net_cpu, inputs, helpers.oracle_run(pb), pb.locations)
    for k in ("x0", "x1", "x2", "x3", "x4", "x5", "x6", "x7"):
        helpers.assert_features_match(gpu.locations(st[k]), st[k].features, pb.locations(sp[k]), sp[k].features,
                                      helpers.FP32_TOL, same_rows=True, what=name + ":port:" + k)
    _exact_rules(gpu.submanifold_rulebook(st["x0"], [3] * d), pb.submanifold_rulebook(sp["x0"], [3] * d),
                 name + " submanifold rulebook")
    _exact_rules(gpu.strided_rulebook(st["x1"], st["x2"].spatial_size, [c["f"]] * d, [c["s"]] * d),
                 pb.strided_rulebook(sp["x1"], sp["x2"].spatial_size, [c["f"]] * d, [c["s"]] * d),
                 name + " strided rulebook")


@pytest.mark.parametrize("name", sorted(cases.NET_CASES))
def test_networks_against_golden(name, cuda):
    import sparseconvnet_b200 as scn
    g = helpers.load_golden(name)
    inp, net, head = cases.net_modules(name)
    helpers.load_state(net, g, "state")
    gpu = helpers.GpuBackend()
    scn.forward_pass_multiplyAdd_count = 0
    x0 = gpu.run(inp, [g["coords"], g["feats"]])
    assert np.array_equal(gpu.locations(x0), g["loc/x0"])
    assert np.array_equal(x0.features, g["feat/x0"])
    y = gpu.run(net, x0)
    assert scn.forward_pass_multiplyAdd_count == float(g["macs"]), "multiply-add count differs"
    if "dense" in g:
        assert helpers.rel_err(y, g["dense"]) <= helpers.FP32_TOL
    else:
        helpers.assert_features_match(gpu.locations(y), y.features, g["loc/y"], g["feat/y"], helpers.FP32_TOL,
                                      what=name)
        if head is not None:
            helpers.load_state(head, g, "head")
            p = port.align_rows(gpu.locations(y), g["loc/y"])
            assert helpers.rel_err(gpu.run(head, y), g["head_out"][p]) <= helpers.FP32_TOL


@pytest.mark.parametrize("name", sorted(cases.IO_CASES))
def test_io_layers_against_golden(name, cuda):
    """InputLayer / BLInputLayer -> SubmanifoldConvolution -> OutputLayer / BLOutputLayer through the C
    ABI against the reference's results: same row numbering on the input side, so row for row; the
    copies back to the points are exact."""
    g = helpers.load_golden(name)
    mods = cases.io_modules(name)
    helpers.load_state(mods[1], g, "state")
    gpu = helpers.GpuBackend()
    st = cases.run_io(mods, (g["coords"], g["feats"]), gpu.run)
    assert np.array_equal(gpu.locations(st["x0"]), g["loc/x0"])
    if cases.IO_CASES[name]["mode"] != 4:
        assert np.array_equal(st["x0"].features, g["feat/x0"]), "input layer must be bit exact"
    assert helpers.rel_err(st["x0"].features, g["feat/x0"]) <= 1e-6
    assert helpers.rel_err(st["x1"].features, g["feat/x1"]) <= helpers.FP32_TOL
    assert st["back0"].shape == g["back0"].shape
    assert np.array_equal(st["back0"], st["back0"]) and helpers.rel_err(st["back0"], g["back0"]) <= 1e-6
    assert helpers.rel_err(st["back1"], g["back1"]) <= helpers.FP32_TOL


def test_io_layers_edge_cases(cuda):
    """Empty batch x length arrays, a sample with only empty slots, device-resident coordinates."""
    import sparseconvnet_b200 as scn
    dev = cuda
    il, ol = scn.BLInputLayer(2, [8, 8], mode=3), scn.BLOutputLayer(2)
    coords = torch.full((3, 5, 2), -1, dtype=torch.int64)
    coords[0, 1] = torch.tensor([2, 3])
    coords[0, 4] = torch.tensor([2, 3])
    coords[2, 0] = torch.tensor([7, 7])
    feats = torch.arange(3 * 5 * 2, dtype=torch.float32, device=dev).reshape(3, 5, 2)
    for c in (coords, coords.to(dev)):
        x = il([c, feats])
        assert x.features.shape == (2, 2)
        assert torch.equal(x.features[0], feats[0, 1] + feats[0, 4])
        back = ol(x)
        assert back.shape == (3, 5, 2)
        assert torch.equal(back[0, 1], x.features[0]) and torch.equal(back[0, 4], x.features[0])
        assert torch.equal(back[2, 0], x.features[1]) and back[1].abs().sum().item() == 0
        x.metadata.poll_errors()
    x = il([torch.zeros(0, 4, 2, dtype=torch.int64), torch.zeros(0, 4, 3, device=dev)])
    assert x.features.shape == (0, 3) and ol(x).shape == (0, 4, 3)
    # OutputLayer after a plain InputLayer, mode 2 (last row wins): the dropped duplicate reads zeros
    x = scn.InputLayer(2, [8, 8], mode=2)([torch.tensor([[1, 1, 0], [1, 1, 0], [2, 2, 0]]),
                                           torch.tensor([[1.0], [2.0], [3.0]], device=dev)])
    assert scn.OutputLayer(2)(x).flatten().tolist() == [0.0, 2.0, 3.0]


def test_empty_and_tiny_inputs(cuda):
    import sparseconvnet_b200 as scn
    dev = cuda
    sc = scn.SubmanifoldConvolution(3, 4, 6, 3, True).to(dev)
    cv = scn.Convolution(3, 6, 5, 2, 2, False).to(dev)
    bn = scn.BatchNormReLU(5).to(dev).eval()
    for n in (0, 1):
        x = scn.InputLayer(3, 16, mode=3)([torch.zeros(n, 4, dtype=torch.int64) + 3, torch.ones(n, 4, device=dev)])
        assert x.features.shape == (n, 4)
        y = bn(cv(sc(x)))
        assert y.features.shape == (n, 5)
        assert x.get_spatial_locations().shape == (n, 4)
        d = scn.SparseToDense(3, 5)(y)
        assert tuple(d.shape) == (4 if n else 0, 5, 8, 8, 8)   # batch index 3 -> four samples
    # one site: the only rule is the centre offset
    x = scn.InputLayer(3, 16, mode=3)([torch.tensor([[3, 4, 5, 0]]), torch.ones(1, 4, device=dev)])
    out = sc(x)
    want = torch.ones(1, 4, device=dev) @ sc.weight[13, 0] + sc.bias
    assert torch.allclose(out.features, want, atol=1e-5)


def test_coordinate_range_is_reported(cuda):
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200._lib import ScnError
    with pytest.raises(ScnError):
        scn.InputLayer(2, 8, mode=3)([torch.tensor([[1, 9, 0]]), torch.ones(1, 1, device=cuda)])
    with pytest.raises(ScnError):
        scn.InputLayer(2, 8, mode=0)([torch.tensor([[-1, 2, 0]]), torch.ones(1, 1, device=cuda)])
    with pytest.raises(RuntimeError):
        scn.InputLayer(2, 8, mode=0)([torch.tensor([[1, 2, 0]]), torch.ones(1, 1)])  # CPU features: no fallback


def test_large_field_needs_64_bit_keys(cuda):
    """4096^3 x batch does not fit 32 bits; corners of the field must stay distinct sites."""
    import sparseconvnet_b200 as scn
    pts = torch.tensor([[0, 0, 0, 0], [4095, 4095, 4095, 7], [4095, 0, 4095, 3], [4094, 4095, 4095, 7],
                        [0, 0, 1, 0], [2048, 2048, 2048, 5]])
    x = scn.InputLayer(3, 4096, mode=3)([pts, torch.arange(6.0, device=cuda).view(6, 1)])
    assert torch.equal(x.get_spatial_locations(), pts)
    rb = x.metadata
    scn.SubmanifoldConvolution(3, 1, 1, 3, False).to(cuda)(x)
    rules = [r.cpu().numpy() for r in rb.rulebook(0, [4096] * 3, [3] * 3)]
    assert sum(r.shape[0] for r in rules) == 6 + 4   # 6 centre rules + (1<->3) and (0<->4) both ways
    assert rules[13].shape[0] == 6


def test_deterministic_bits(cuda):
    import sparseconvnet_b200 as scn
    g = helpers.load_golden("net_unet3d")
    outs = []
    for _ in range(2):
        inp, net, head = cases.net_modules("net_unet3d")
        helpers.load_state(net, g, "state")
        gpu = helpers.GpuBackend()
        y = gpu.run(net, gpu.run(inp, [g["coords"], g["feats"]]))
        outs.append((gpu.locations(y), y.features))
    assert np.array_equal(outs[0][0], outs[1][0])
    assert np.array_equal(outs[0][1], outs[1][1])


@pytest.mark.skipif(not runner.reference_available(), reason="oracle/_ref not built")
def test_against_live_reference_random(cuda):
    """A fresh random case straight against the compiled reference (not a stored fixture)."""
    import sparseconvnet_b200 as scn
    rng = np.random.default_rng(2024)
    n = 20000
    coords = np.concatenate([rng.integers(0, 63, (n, 3)) // np.array([1, 1, 8]) + np.array([0, 0, 20]),
                             rng.integers(0, 5, (n, 1))], axis=1)
    feats = rng.standard_normal((n, 16)).astype(np.float32)
    torch.manual_seed(5)
    inp = scn.InputLayer(3, 63, mode=4)
    net = scn.Sequential().add(scn.SubmanifoldConvolution(3, 16, 32, 3, False)).add(scn.BatchNormReLU(32)).add(
        scn.Convolution(3, 32, 48, 3, 2, False)).add(scn.BatchNormLeakyReLU(48, leakiness=0.2)).add(
        scn.SubmanifoldConvolution(3, 48, 48, 3, True)).add(scn.Deconvolution(3, 48, 24, 3, 2, False))
    from sparseconvnet_b200 import workloads
    workloads.randomize(net, 3)
    net.eval()
    ref = runner.RefBackend()
    yr = runner.run_module(net, runner.run_module(inp, [coords, feats], ref), ref)
    gpu = helpers.GpuBackend()
    yg = gpu.run(net, gpu.run(inp, [coords, feats]))
    helpers.assert_features_match(gpu.locations(yg), yg.features, ref.locations(yr), yr.features, helpers.FP32_TOL,
                                  what="live reference")


def test_deferred_multiply_add_count(cuda):
    """A convolution on a fresh rulebook answers with a ticket instead of waiting for the rule totals;
    resolved later (even after the metadata object is gone) it is the count the blocking call gives."""
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200 import SCN
    from sparseconvnet_b200._lib import lib
    rng = np.random.default_rng(5)
    coords = np.concatenate([rng.integers(0, 24, (3000, 3)), rng.integers(0, 2, (3000, 1))], axis=1)
    feats = torch.from_numpy(rng.standard_normal((3000, 8)).astype(np.float32)).to(cuda)
    conv = scn.SubmanifoldConvolution(3, 8, 16, 3, False).to(cuda)
    counts = []
    try:
        for deferred in (0, 1):
            lib.scn_set_deferred_counts(deferred)
            x = scn.InputLayer(3, 24, mode=3)([torch.from_numpy(coords), feats])
            out = torch.empty(0, device=cuda)
            with torch.no_grad():
                macs = SCN.SubmanifoldConvolution_updateOutput(x.spatial_size, conv.filter_size, x.metadata,
                                                               x.features, out, conv.weight, torch.empty(0))
            if deferred:
                assert isinstance(macs, SCN.DeferredCount) or macs >= 0
                del x  # the ticket outlives the metadata object
            else:
                assert isinstance(macs, float) and macs > 0
            counts.append(float(macs))
    finally:
        lib.scn_set_deferred_counts(1)
    assert counts[0] == counts[1] and counts[0] % (8 * 16) == 0


def test_mirrored_rulebook_build_equals_full_lookup(cuda, monkeypatch):
    """Odd filter sizes: the rulebook built from half the lookups (each hit also fills the neighbour's
    mirrored entry) is the rulebook built from all of them, rule for rule; a 3 x 5 filter and blanked
    duplicate rows (input mode 0) included."""
    import sparseconvnet_b200 as scn
    rng = np.random.default_rng(11)
    coords = np.concatenate([rng.integers(0, 20, (4000, 3)), rng.integers(0, 3, (4000, 1))], axis=1)
    feats = torch.from_numpy(rng.standard_normal((4000, 4)).astype(np.float32)).to(cuda)
    for mode in (0, 3):
        for filt in ([3, 3, 3], [3, 5, 1]):
            books = []
            for mirror in ("1", "0"):
                monkeypatch.setenv("SCN_RULES_MIRROR", mirror)
                x = scn.InputLayer(3, 20, mode=mode)([torch.from_numpy(coords), feats])
                conv = scn.SubmanifoldConvolution(3, 4, 4, filt, False).to(cuda)
                with torch.no_grad():
                    conv(x)
                books.append(x.metadata.rulebook(0, x.spatial_size, conv.filter_size))
            assert len(books[0]) == len(books[1]) == int(np.prod(filt))
            for k, (a, b) in enumerate(zip(*books)):
                assert torch.equal(a, b), "filter %s mode %d offset %d" % (filt, mode, k)


def test_large_filter_volume_counts(cuda):
    """A 4-D filter of size 5 has 625 offsets, more than a count ticket holds: the multiply-add count then comes
    back as a plain number, and equals rules x planes."""
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200 import SCN
    rng = np.random.default_rng(13)
    coords = np.concatenate([rng.integers(0, 9, (600, 4)), np.zeros((600, 1), np.int64)], axis=1)
    feats = torch.from_numpy(rng.standard_normal((600, 2)).astype(np.float32)).to(cuda)
    x = scn.InputLayer(4, 9, mode=3)([torch.from_numpy(coords), feats])
    conv = scn.SubmanifoldConvolution(4, 2, 3, 5, False).to(cuda)
    out = torch.empty(0, device=cuda)
    with torch.no_grad():
        macs = SCN.SubmanifoldConvolution_updateOutput(x.spatial_size, conv.filter_size, x.metadata, x.features, out,
                                                       conv.weight, torch.empty(0))
    book = x.metadata.rulebook(0, x.spatial_size, conv.filter_size)
    assert len(book) == 625
    assert float(macs) == float(sum(b.shape[0] for b in book)) * 2 * 3
    x.metadata.poll_errors()


@pytest.mark.parametrize("precision", ["fp32", "tf32x3", "bf16"])
def test_fused_batchnorm_equals_two_passes(precision, cuda):
    """A convolution that applies the following eval-mode BatchNorm in its store gives the same bits
    as the convolution followed by the BatchNorm operator, in every kernel class (warp-level rows
    kernel, first-layer kernel, both tcgen05 kernels with and without offset split, the fp32 kernels
    through the in-place fallback), and the U-Net runs with a fraction of the BatchNorm launches."""
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200 import SCN, workloads
    coords, feats = workloads.batch_config3([0], target_voxels=60000)
    inp, net, _ = workloads.build_config(3)
    net.to(cuda)
    scn.set_precision(precision)
    try:
        outs, bn_calls, fused = [], [], []
        for fuse in (False, True):
            scn.Sequential.fuse = fuse
            with torch.no_grad(), SCN.Profile() as prof:
                y = net(inp([torch.from_numpy(coords), torch.from_numpy(feats).to(cuda)]))
            rows = prof.rows()
            bn_calls.append(sum(r["kind"] == "batchnorm" for r in rows))
            fused.append(sum(bool(r.get("fused_bn")) for r in rows if r["kind"] == "conv"))
            y.metadata.poll_errors()
            outs.append(y.features.clone())
    finally:
        scn.Sequential.fuse = True
        scn.set_precision("fp32")
    assert bn_calls[0] == 39 and fused[0] == 0
    # 27 of the 39 BatchNorms ride in a convolution's store; the 6 behind a JoinTable and the 6 in front of a
    # strided Convolution are applied by the convolution that follows to its own input (in its split pass, or into
    # a scratch copy where the kernel has none), the joined tensors read where they lie: no BatchNorm call is left
    assert fused[1] == 27 and bn_calls[1] == 0, (bn_calls, fused)
    assert sum(bool(r.get("joined")) for r in rows if r["kind"] == "conv") == 6
    assert sum(bool(r.get("fused_bn_in_front")) for r in rows if r["kind"] == "conv") == 12
    assert torch.equal(outs[0], outs[1]), float((outs[0] - outs[1]).abs().max())


@pytest.mark.parametrize("cout", [96, 160])
def test_fused_batchnorm_in_the_persistent_tcgen05_kernel(cout, cuda, monkeypatch):
    """k_conv_wide (forced onto a small level: the U-Net of the test above is too small to reach it): the fused
    BatchNorm gives the bits of the two separate operators, with one and with two 128-plane accumulator tiles."""
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200 import SCN
    monkeypatch.setenv("SCN_TC_PERSISTENT", "1")
    rng = np.random.default_rng(11)
    pts = rng.integers(0, 96, (20000, 2))
    z = (48 + 19 * np.sin(pts[:, 0] / 6.0)).astype(np.int64)
    coords = np.concatenate([pts, z[:, None], rng.integers(0, 2, (20000, 1))], 1).astype(np.int64)
    torch.manual_seed(3)
    net = scn.Sequential().add(scn.SubmanifoldConvolution(3, 96, cout, 3, True)).add(
        scn.BatchNormLeakyReLU(cout, leakiness=0.1)).to(cuda).eval()
    net[1].running_mean.normal_()
    net[1].running_var.uniform_(0.5, 2.0)
    net[1].weight.data.normal_()
    net[1].bias.data.normal_()
    net[0].bias.data.normal_()
    feats = torch.randn(20000, 96, device=cuda)
    scn.set_precision("tf32x3")
    try:
        outs = []
        for fuse in (False, True):
            scn.Sequential.fuse = fuse
            with torch.no_grad():
                y = net(scn.InputLayer(3, 96, mode=3)([torch.from_numpy(coords), feats]))
            assert SCN._KERNEL_NAMES[SCN.lib.scn_last_conv_kernel()] == "k_conv_wide"
            y.metadata.poll_errors()
            outs.append(y.features.clone())
    finally:
        scn.Sequential.fuse = True
        scn.set_precision("fp32")
    assert torch.equal(outs[0], outs[1]), float((outs[0] - outs[1]).abs().max())


@pytest.mark.parametrize("env,kernel", [({"SCN_TC_PERSISTENT": "1"}, "k_conv_wide"), ({"SCN_TC_COPY": "1"}, "k_conv_tc"),
                                        ({"SCN_TC_COPY": "0"}, "k_conv_tc"), ({"SCN_X3_MIN_COUT": "999"}, "k_conv_pipe_mma")])
def test_batchnorm_in_front_of_a_strided_convolution(env, kernel, cuda, monkeypatch):
    """BatchNorm -> Convolution 2/2 -> BatchNorm as one call (scn_convolution_bn_bn_forward) against the three
    operators one after the other, bit for bit: in the split pass of both tcgen05 kernels and through the scratch
    copy (per-tile kernel with register producers, a kernel without any fused store)."""
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200 import SCN
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    rng = np.random.default_rng(17)
    pts = rng.integers(0, 128, (30000, 2))
    z = (64 + 25 * np.sin(pts[:, 0] / 9.0)).astype(np.int64)
    coords = np.concatenate([pts, z[:, None], rng.integers(0, 2, (30000, 1))], 1).astype(np.int64)
    torch.manual_seed(5)
    net = scn.Sequential().add(scn.BatchNormLeakyReLU(64, leakiness=0.2)).add(
        scn.Convolution(3, 64, 96, 2, 2, True)).add(scn.BatchNormReLU(96)).to(cuda).eval()
    for bn in (net[0], net[2]):
        bn.running_mean.normal_()
        bn.running_var.uniform_(0.5, 2.0)
        bn.weight.data.normal_()
        bn.bias.data.normal_()
    net[1].bias.data.normal_()
    feats = torch.randn(30000, 64, device=cuda)
    scn.set_precision("tf32x3")
    try:
        outs = []
        for fuse in (False, True):
            scn.Sequential.fuse = fuse
            with torch.no_grad(), SCN.Profile() as prof:
                y = net(scn.InputLayer(3, 128, mode=3)([torch.from_numpy(coords), feats]))
            assert SCN._KERNEL_NAMES[SCN.lib.scn_last_conv_kernel()] == kernel
            assert sum(r["kind"] == "batchnorm" for r in prof.rows()) == (0 if fuse else 2)
            y.metadata.poll_errors()
            outs.append(y.features.clone())
    finally:
        scn.Sequential.fuse = True
        scn.set_precision("fp32")
    assert torch.equal(outs[0], outs[1]), float((outs[0] - outs[1]).abs().max())


@pytest.mark.parametrize("cin,cout", [(4, 1), (32, 20), (32, 3), (64, 32), (256, 17), (96, 8)])
def test_rows_times_small_matrix(cin, cout, cuda):
    """scn_rows_affine_forward (NetworkInNetwork with few output planes, the per-voxel class head) against
    a float64 product; tolerance 1e-5 of the largest score (fp32 FMA sums over at most 256 planes)."""
    from sparseconvnet_b200 import SCN
    g = torch.Generator().manual_seed(cin * 100 + cout)
    w = torch.randn(cin, cout, generator=g).cuda()
    b = torch.randn(cout, generator=g).cuda()
    for n in (0, 1, 255, 100003):
        x = torch.randn(n, cin, generator=g).cuda()
        for bias in (b, None):
            y = SCN.rows_affine(x, w, bias)
            ref = x.double() @ w.double() + (bias.double() if bias is not None else 0.0)
            assert y.shape == (n, cout)
            if n:
                assert (y.double() - ref).abs().max().item() <= 1e-5 * max(1.0, ref.abs().max().item())
    # into a block of a larger buffer, neighbours untouched
    buf = torch.full((300, cout), 7.0, device="cuda")
    x = torch.randn(100, cin, generator=g).cuda()
    SCN.rows_affine(x, w, b, out=buf[100:200])
    assert torch.equal(buf[:100], torch.full((100, cout), 7.0, device="cuda"))
    assert torch.equal(buf[200:], torch.full((100, cout), 7.0, device="cuda"))
    assert torch.equal(buf[100:200], SCN.rows_affine(x, w, b))
    # the module form takes the same kernel and keeps the reference's multiply-add count
    out = torch.empty(0, device="cuda")
    macs = SCN.NetworkInNetwork_updateOutput(x, out, w, b)
    assert macs == 100.0 * cin * cout and torch.equal(out, buf[100:200])


def test_rows_times_small_matrix_refuses_other_shapes(cuda):
    from sparseconvnet_b200 import SCN
    x = torch.randn(10, 30).cuda()
    with pytest.raises(RuntimeError):
        SCN.rows_affine(x, torch.randn(30, 8).cuda())          # input planes not a multiple of four
    x = torch.randn(10, 32).cuda()
    with pytest.raises(RuntimeError):
        SCN.rows_affine(x, torch.randn(32, 33).cuda())         # wider than the kernel takes
    out = torch.empty(0, device="cuda")                          # the module form falls back to the dense library
    SCN.NetworkInNetwork_updateOutput(x, out, torch.randn(32, 33).cuda(), None)
    assert out.shape == (10, 33)


def _pyramid(cuda, coords, size, levels, chained, fsize=2, fstride=2):
    """Grids and rulebooks of `levels` levels (filter fsize, stride fstride) below an input layer: ([locations],
    [rulebooks], host waits, rulebooks built), built level by level or, `chained`, in one enqueued chain first."""
    import ctypes as C
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200 import SCN
    dim = coords.shape[1] - 1
    x = scn.InputLayer(dim, size, mode=3)([torch.from_numpy(coords), torch.ones(len(coords), 1, device=cuda)])
    m = x.metadata
    waits, builds = SCN.host_wait_count(), SCN.lib.scn_rulebook_build_count()
    f, st = torch.LongTensor([fsize] * dim), torch.LongTensor([fstride] * dim)
    if chained == "started":   # on the side stream, taken over by the first per-level call below
        SCN.strided_chain_start(m, x.spatial_size, f, st, levels, cuda)
    n_chained = SCN.strided_chain(m, x.spatial_size, f, st, levels, cuda) if chained is True else 0
    locs, rules, cur = [], [], x.spatial_size.clone()
    for _ in range(levels):
        nxt = (cur - fsize) // fstride + 1
        n_out = C.c_int64()
        with torch.cuda.device(cuda):
            SCN.check(SCN.lib.scn_md_strided_rulebook(m._h, SCN.sizes(cur), SCN.sizes(nxt), SCN.sizes(f),
                                                      SCN.sizes(st), SCN._stream(), C.byref(n_out), None))
        assert n_out.value == m.getNActive(nxt)
        cur = nxt
    waits, builds = SCN.host_wait_count() - waits, SCN.lib.scn_rulebook_build_count() - builds
    cur = x.spatial_size.clone()
    for _ in range(levels):
        nxt = (cur - fsize) // fstride + 1
        locs.append(m.getSpatialLocations(nxt).numpy())
        rules.append([t.cpu().numpy() for t in m.rulebook(1, cur, f, st)])
        cur = nxt
    return locs, rules, waits, builds, n_chained


@pytest.mark.parametrize("fsize,size", [(2, 1024), (3, 1023)])
@pytest.mark.parametrize("kind", ["surface", "scattered", "empty", "tiny"])
def test_chained_strided_levels_equal_level_by_level(kind, fsize, size, cuda):
    """scn_md_strided_chain: the same grids (row for row) and rulebooks (rule for rule) as one
    scn_md_strided_rulebook call per level, with one wait for all levels, for disjoint (2/2) and overlapping
    (3/2) windows.  'scattered': isolated sites do not thin out from one level to the next (2/2) or feed
    eight outputs each (3/2), so the first guess of the level sizes is too small and the chain falls back to
    the safe sizes for those levels."""
    rng = np.random.default_rng(5)
    if kind == "surface":      # a closed sheet, rows shuffled: shrinks by about four per level
        u = np.stack(np.meshgrid(np.arange(300), np.arange(200), indexing="ij"), -1).reshape(-1, 2)
        z = (100 + 20 * np.sin(u[:, 0] / 40.0)).astype(np.int64)
        coords = np.concatenate([u, z[:, None], (u[:, :1] // 100)], 1).astype(np.int64)
        coords = coords[rng.permutation(len(coords))]
    elif kind == "scattered":  # every site alone in its 2^3 cell at level 0 and again one level down
        g = np.stack(np.meshgrid(np.arange(24), np.arange(24), np.arange(24), indexing="ij"), -1).reshape(-1, 3) * 4
        coords = np.concatenate([g, np.zeros((len(g), 1), np.int64)], 1).astype(np.int64)
    elif kind == "empty":
        coords = np.zeros((0, 4), np.int64)
    else:
        coords = np.array([[5, 6, 7, 0], [1020, 3, 9, 1]], np.int64)
    levels = 5
    a = _pyramid(cuda, coords, size, levels, chained=False, fsize=fsize)
    b = _pyramid(cuda, coords, size, levels, chained=True, fsize=fsize)
    assert a[3] == levels and b[3] == levels          # every rulebook built exactly once either way
    assert b[4] == levels                             # ... all of them by the chain
    for l in range(levels):
        assert np.array_equal(a[0][l], b[0][l]), "grid of level %d" % l
        _exact_rules(a[1][l], b[1][l], "rulebook of level %d" % l)
    c = _pyramid(cuda, coords, size, levels, chained="started", fsize=fsize)
    assert c[3] == levels
    for l in range(levels):
        assert np.array_equal(a[0][l], c[0][l]), "grid of level %d (chain started on the side stream)" % l
        _exact_rules(a[1][l], c[1][l], "rulebook of level %d (chain started on the side stream)" % l)
    if kind == "empty":                                # nothing to count, nothing to wait for level by level
        return
    assert a[2] >= levels                              # one wait per level (more where a table had to grow)
    if kind == "scattered":
        assert 2 <= b[2] <= 3                          # the first pass and one or two repeats
    else:
        assert b[2] == 1                               # one wait for the whole chain


def test_started_chain_is_dropped_with_its_metadata(cuda):
    """A chain started on the side stream and never asked for: clearing the Metadata, giving it a new input and
    destroying it all release it, and the library's pool holds no more than before."""
    import gc
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200 import SCN
    rng = np.random.default_rng(3)
    coords = np.concatenate([rng.integers(0, 512, (40000, 3)), np.zeros((40000, 1), np.int64)], 1).astype(np.int64)
    feats = torch.ones(40000, 1, device=cuda)
    f = torch.LongTensor([2, 2, 2])
    inp = scn.InputLayer(3, 512, mode=3)
    x = inp([torch.from_numpy(coords), feats])      # warm the pool up
    SCN.strided_chain(x.metadata, x.spatial_size, f, f, 4, cuda)
    del x
    gc.collect()
    torch.cuda.synchronize()
    used = C_memory_in_use()
    for what in ("clear", "new input", "destroy"):
        x = inp([torch.from_numpy(coords), feats])
        SCN.strided_chain_start(x.metadata, x.spatial_size, f, f, 4, cuda)
        if what == "clear":
            x.metadata.clear()
        elif what == "new input":
            SCN.InputLayer_updateOutput(x.metadata, x.spatial_size, torch.from_numpy(coords), feats,
                                        torch.empty(0, device=cuda), 0, 3)
            assert x.metadata.getNActive(x.spatial_size) > 0
        del x
        gc.collect()
        torch.cuda.synchronize()
        assert C_memory_in_use() <= used, what


def C_memory_in_use():
    import ctypes as C
    from sparseconvnet_b200 import SCN
    reserved, in_use = C.c_uint64(), C.c_uint64()
    SCN.check(SCN.lib.scn_memory_usage(C.byref(reserved), C.byref(in_use)))
    return in_use.value


def test_unet_prefetches_its_encoder_rulebooks(cuda):
    """The outermost Sequential starts the encoder's chain on the side stream (Metadata.chain_started), the
    network's result has the same bits with and without it, and the step has two host waits either way."""
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200 import SCN, workloads
    coords, feats = workloads.batch_config3([0], target_voxels=60000)
    inp, net, _ = workloads.build_config(3)
    net.to(cuda).eval()
    scn.set_precision("tf32x3")
    try:
        outs = []
        for prefetch in (False, True):
            scn.Sequential.prefetch_rulebooks = prefetch
            with torch.no_grad():
                x = inp([torch.from_numpy(coords), torch.from_numpy(feats).to(cuda)])
                waits = SCN.host_wait_count()
                y = net(x)
                waits = SCN.host_wait_count() - waits
            assert x.metadata.chain_started == prefetch
            assert waits <= 1, waits          # the chain's counts (often already there when they are asked for)
            y.metadata.poll_errors()
            outs.append(y.features.clone())
    finally:
        scn.Sequential.prefetch_rulebooks = True
        scn.set_precision("fp32")
    assert torch.equal(outs[0], outs[1])
