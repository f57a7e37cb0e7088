"""Definitions of the golden cases: seeded inputs and the module chains / small networks they
run through.  Shared by ``make_golden.py`` (which runs them on the compiled reference and
stores the results) and by the tests (which run the numpy restatement and the CUDA library
on the same inputs and compare with the stored results)."""
import numpy as np
import torch

import sparseconvnet_b200 as scn
from sparseconvnet_b200 import workloads

# ---- operator chains ---------------------------------------------------------------------------
# x0 = InputLayer(mode); x1 = SC(x0) (+bias); x2 = Conv f/s (x1); x3 = BNReLU(x2); x4 = Deconv(x3) (+bias);
# x5 = MaxPool f/s (x1); dense = SparseToDense(x5); x6 = AveragePool f/s (x1); x7 = UnPool f/s (x6)
OPS_CASES = {
    "ops1d_m3": dict(dim=1, size=[33], n=40, batch=2, mode=3, planes=3, f=3, s=2, groups=1),
    "ops2d_m0": dict(dim=2, size=[17, 17], n=150, batch=3, mode=0, planes=5, f=3, s=2, groups=1),
    "ops2d_m0_dup": dict(dim=2, size=[9, 9], n=120, batch=2, mode=0, planes=4, f=3, s=2, groups=1, keep_dups=True),
    "ops2d_m1": dict(dim=2, size=[17, 17], n=300, batch=3, mode=1, planes=5, f=3, s=2, groups=1),
    "ops2d_m2": dict(dim=2, size=[17, 17], n=300, batch=3, mode=2, planes=5, f=3, s=2, groups=1),
    "ops2d_m4_f2": dict(dim=2, size=[16, 16], n=300, batch=3, mode=4, planes=6, f=2, s=2, groups=2),
    "ops3d_m3": dict(dim=3, size=[15, 15, 15], n=600, batch=2, mode=3, planes=5, f=3, s=2, groups=1),
    "ops3d_m4_f2": dict(dim=3, size=[16, 16, 16], n=700, batch=3, mode=4, planes=8, f=2, s=2, groups=1),
    "ops3d_nobatchcol": dict(dim=3, size=[15, 15, 15], n=300, batch=0, mode=3, planes=4, f=3, s=2, groups=1),
    "ops3d_emptysample": dict(dim=3, size=[15, 15, 15], n=200, batch=4, mode=3, planes=4, f=3, s=2, groups=1,
                              skip_sample=2, batch_size_arg=6),
    "ops4d_m0": dict(dim=4, size=[9, 9, 9, 5], n=500, batch=2, mode=0, planes=5, f=3, s=2, groups=1),
}


# ---- input / output layer pairs (per-point networks) ----------------------------------------------
# x0 = InputLayer or BLInputLayer (mode); x1 = SC(x0) (+bias); points = OutputLayer / BLOutputLayer (x1)
IO_CASES = {
    "io_il2d_m0": dict(dim=2, size=[11, 11], bl=False, n=90, batch=2, mode=0, planes=3),
    "io_il2d_m1": dict(dim=2, size=[9, 9], bl=False, n=200, batch=3, mode=1, planes=3),
    "io_il2d_m2": dict(dim=2, size=[9, 9], bl=False, n=200, batch=3, mode=2, planes=3),
    "io_il3d_m4": dict(dim=3, size=[7, 7, 7], bl=False, n=500, batch=2, mode=4, planes=4),
    "io_bl2d_m0": dict(dim=2, size=[11, 11], bl=True, batch=3, length=40, mode=0, planes=3),
    "io_bl2d_m1": dict(dim=2, size=[7, 7], bl=True, batch=3, length=60, mode=1, planes=3, empty=0.2),
    "io_bl2d_m2": dict(dim=2, size=[7, 7], bl=True, batch=3, length=60, mode=2, planes=3, empty=0.2),
    "io_bl3d_m3": dict(dim=3, size=[5, 5, 5], bl=True, batch=4, length=90, mode=3, planes=4, empty=0.3),
    "io_bl1d_m4": dict(dim=1, size=[9], bl=True, batch=2, length=30, mode=4, planes=2, empty=0.5),
}


def io_inputs(case):
    c = IO_CASES[case]
    rng = np.random.default_rng(sum(map(ord, case)))
    d = c["dim"]
    if not c["bl"]:
        cols = [rng.integers(0, s, c["n"]) for s in c["size"]] + [rng.integers(0, c["batch"], c["n"])]
        coords = np.stack(cols, axis=1).astype(np.int64)
        if c["mode"] == 0:
            coords = np.unique(coords, axis=0)
            rng.shuffle(coords)
        feats = rng.standard_normal((coords.shape[0], c["planes"])).astype(np.float32)
        return coords, feats
    B, L = c["batch"], c["length"]
    if c["mode"] == 0:  # all present, unique within a sample
        coords = np.zeros((B, L, d), dtype=np.int64)
        for b in range(B):
            cells = rng.permutation(int(np.prod(c["size"])))[:L]
            coords[b] = np.stack(np.unravel_index(cells, c["size"]), axis=1)
    else:
        coords = np.stack([rng.integers(0, s, (B, L)) for s in c["size"]], axis=2).astype(np.int64)
        coords[rng.random((B, L)) < c["empty"]] = -1
    feats = rng.standard_normal((B, L, c["planes"])).astype(np.float32)
    return coords, feats


def io_modules(case):
    c = IO_CASES[case]
    torch.manual_seed(sum(map(ord, case)))
    d, p = c["dim"], c["planes"]
    mods = dict(sc=scn.SubmanifoldConvolution(d, p, p + 2, 3, True))
    mods["sc"].bias.data.normal_()
    net = torch.nn.ModuleDict(mods)
    workloads.randomize(net, 11)
    net.eval()
    il = scn.BLInputLayer(d, c["size"], c["mode"]) if c["bl"] else scn.InputLayer(d, c["size"], c["mode"])
    ol = scn.BLOutputLayer(d) if c["bl"] else scn.OutputLayer(d)
    return il, net, ol


def run_io(mods, inputs, run):
    il, net, ol = mods
    x0 = run(il, list(inputs))
    x1 = run(net["sc"], x0)
    return dict(x0=x0, x1=x1, back0=run(ol, x0), back1=run(ol, x1))


def ops_inputs(case):
    c = OPS_CASES[case]
    rng = np.random.default_rng(sum(map(ord, case)))
    cols = [rng.integers(0, s, c["n"]) for s in c["size"]]
    if c["batch"]:
        b = rng.integers(0, c["batch"], c["n"])
        if "skip_sample" in c:
            b[b == c["skip_sample"]] = 0
        cols.append(b)
    coords = np.stack(cols, axis=1).astype(np.int64)
    if c["mode"] == 0 and not c.get("keep_dups"):
        coords = np.unique(coords, axis=0)
        rng.shuffle(coords)
    feats = rng.standard_normal((coords.shape[0], c["planes"])).astype(np.float32)
    return coords, feats, c.get("batch_size_arg", 0)


def ops_modules(case):
    c = OPS_CASES[case]
    torch.manual_seed(sum(map(ord, case)))
    d, p, g = c["dim"], c["planes"], c["groups"]
    mods = dict(
        il=scn.InputLayer(d, c["size"], c["mode"]),
        sc=scn.SubmanifoldConvolution(d, p, 2 * p, 3, True, g),
        cv=scn.Convolution(d, 2 * p, 6 * g, c["f"], c["s"], False, g),
        bn=scn.BatchNormReLU(6 * g),
        dc=scn.Deconvolution(d, 6 * g, 4 * g, c["f"], c["s"], True, g),
        mp=scn.MaxPooling(d, c["f"], c["s"], 1),
        sd=scn.SparseToDense(d, 2 * p - 1),
        ap=scn.AveragePooling(d, c["f"], c["s"], 1),
        up=scn.UnPooling(d, c["f"], c["s"]),
    )
    mods["sc"].bias.data.normal_()
    mods["dc"].bias.data.normal_()
    net = torch.nn.ModuleDict(mods)
    workloads.randomize(net, 7)
    net.eval()
    return net


def run_ops(net, inputs, run, locations):
    """`run(module, x)` applies a module; `locations(x)` gives [N, D+1] of a sparse tensor.
    Returns {stage: (locations or None, features)}."""
    coords, feats, bs = inputs
    x0 = run(net["il"], [coords, feats, bs])
    x1 = run(net["sc"], x0)
    x2 = run(net["cv"], x1)
    x3 = run(net["bn"], x2)
    x4 = run(net["dc"], x3)
    x5 = run(net["mp"], x1)
    dense = run(net["sd"], x5)
    x6 = run(net["ap"], x1)
    x7 = run(net["up"], x6)
    return dict(x0=x0, x1=x1, x2=x2, x3=x3, x4=x4, x5=x5, dense=dense, x6=x6, x7=x7)


# ---- small networks ------------------------------------------------------------------------------

def _mini_vgg():
    net = scn.Sequential().add(
        scn.SparseVggNet(2, 1, [["C", 8], ["C", 8], ["MP", 3, 2], ["C", 16], ["C", 16], ["MP", 3, 2],
                                ["C", 24], ["C", 24], ["MP", 3, 2]])).add(
        scn.SubmanifoldConvolution(2, 24, 32, 3, False)).add(scn.BatchNormReLU(32)).add(scn.SparseToDense(2, 32))
    inp = scn.InputLayer(2, net.input_spatial_size(torch.LongTensor([10, 10])), mode=3)
    return inp, net, None


def _mini_unet():
    inp = scn.InputLayer(3, 64, mode=4)
    net = scn.Sequential().add(scn.SubmanifoldConvolution(3, 3, 8, 3, False)).add(
        scn.UNet(3, 2, [8, 16, 24, 32], False)).add(scn.BatchNormReLU(8))
    return inp, net, torch.nn.Linear(8, 5)


def _mini_fcn():
    # per-point network: residual FullyConvolutionalNet (UnPooling back to the input sites), then
    # OutputLayer hands every input point its site's features
    inp = scn.InputLayer(3, 64, mode=3)
    net = scn.Sequential().add(scn.SubmanifoldConvolution(3, 3, 8, 3, False)).add(
        scn.FullyConvolutionalNet(3, 1, [8, 12, 16], residual_blocks=True)).add(scn.BatchNormReLU(36)).add(
        scn.OutputLayer(3))
    return inp, net, None


def _mini_resnet():
    inp = scn.InputLayer(3, 31, mode=3)
    net = scn.Sequential().add(scn.SubmanifoldConvolution(3, 1, 8, 3, False)).add(scn.MaxPooling(3, 3, 2)).add(
        scn.SparseResNet(3, 8, [["b", 8, 2, 1], ["b", 16, 2, 2], ["b", 24, 1, 1]]))
    return inp, net, torch.nn.Linear(24, 7)


def _mini_vgg_plus():
    inp = scn.InputLayer(2, 47, mode=3)
    net = scn.Sequential().add(scn.SparseVggNet(2, 2, [["C", 8, 4], ["C", 8, 4, 4], "MP", ["C3/2", 12]]))
    return inp, net, None


def _mini_4d():
    inp = scn.InputLayer(4, [12, 12, 12, 6], mode=0)
    net = scn.Sequential()
    for _ in range(2):
        net.add(scn.SubmanifoldConvolution(4, 8, 8, 3, False)).add(scn.BatchNormReLU(8))
    return inp, net, None


NET_CASES = {"net_vgg2d": _mini_vgg, "net_unet3d": _mini_unet, "net_resnet3d": _mini_resnet,
             "net_vggplus2d": _mini_vgg_plus, "net_stack4d": _mini_4d, "net_fcn3d": _mini_fcn}


def net_inputs(case):
    rng = np.random.default_rng(sum(map(ord, case)))
    if case == "net_vgg2d":
        return workloads.batch_config2([0, 1, 2, 3])
    if case in ("net_unet3d", "net_fcn3d"):
        n = 3000
        pts = rng.integers(0, 64, (n, 2))
        z = (20 + 10 * np.sin(pts[:, 0] / 9.0) + 6 * np.cos(pts[:, 1] / 7.0)).astype(np.int64)
        coords = np.concatenate([pts, z[:, None], rng.integers(0, 2, (n, 1))], axis=1)
        return coords, rng.uniform(-1, 1, (n, 3)).astype(np.float32)
    if case == "net_resnet3d":
        n = 1500
        v = rng.standard_normal((n, 3))
        v = (15 + 11 * v / np.linalg.norm(v, axis=1, keepdims=True)).round().astype(np.int64)
        coords = np.concatenate([v, rng.integers(0, 3, (n, 1))], axis=1)
        return coords, np.ones((n, 1), dtype=np.float32)
    if case == "net_vggplus2d":
        n = 900
        coords = np.concatenate([rng.integers(0, 47, (n, 2)), rng.integers(0, 2, (n, 1))], axis=1)
        return coords, rng.standard_normal((n, 2)).astype(np.float32)
    if case == "net_stack4d":
        n = 2500
        coords = np.unique(np.concatenate([rng.integers(0, 12, (n, 3)), rng.integers(0, 6, (n, 1)),
                                           rng.integers(0, 2, (n, 1))], axis=1), axis=0)
        return coords, rng.standard_normal((coords.shape[0], 8)).astype(np.float32)
    raise KeyError(case)


def net_modules(case):
    torch.manual_seed(sum(map(ord, case)))
    inp, net, head = NET_CASES[case]()
    workloads.randomize(net, 11)
    net.eval()
    if head is not None:
        head.eval()
    return inp, net, head
