"""CPU-only checks of the boundary: the shared library loads, exports exactly the symbols that
include/scn_b200.h declares, and the host-side mirror of the reference API behaves (sizes,
parameter names and shapes, failure modes) without touching a GPU."""
import ctypes
import os
import re
import subprocess

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "scn_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"SCN_API\s+[\w\s\*]+?\b(scn_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from sparseconvnet_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), "libscn_b200.so does not export %s" % n
    # and the ctypes table binds exactly the declared set
    assert sorted(_lib.SIGNATURES) == names


def test_no_undeclared_exports():
    from sparseconvnet_b200 import _lib
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True).stdout
    exported = sorted(l.split()[-1] for l in out.splitlines() if " T " in l)
    assert exported == declared_symbols()


def test_status_strings_and_version():
    from sparseconvnet_b200._lib import lib
    assert lib.scn_abi_version() == 1
    assert lib.scn_status_string(0) == b"ok"
    assert b"coordinate" in lib.scn_status_string(3)
    assert lib.scn_launch_count() >= 0


def test_metadata_create_bad_dimension():
    from sparseconvnet_b200._lib import lib
    h = ctypes.c_void_p()
    assert lib.scn_md_create(0, ctypes.byref(h)) == 1
    assert lib.scn_md_create(7, ctypes.byref(h)) == 1
    assert b"dimension" in lib.scn_last_error()
    assert lib.scn_md_create(3, ctypes.byref(h)) == 0
    n = ctypes.c_int64(-1)
    size = (ctypes.c_int64 * 3)(8, 8, 8)
    assert lib.scn_md_n_active(h, size, ctypes.byref(n)) == 0 and n.value == 0   # unknown scale: 0, as the reference
    assert lib.scn_md_destroy(h) == 0


def test_cpu_features_are_refused():
    import sparseconvnet_b200 as scn
    with pytest.raises(RuntimeError, match="no CPU path"):
        scn.InputLayer(2, 8)([torch.zeros(1, 3, dtype=torch.int64), torch.ones(1, 1)])
    x = scn.SparseConvNetTensor(torch.ones(2, 4), scn.Metadata(2), torch.LongTensor([8, 8]))
    with pytest.raises(RuntimeError, match="CUDA"):
        scn.SubmanifoldConvolution(2, 4, 4, 3, False)(x)


def test_spatial_size_protocol_and_parameter_shapes():
    import sparseconvnet_b200 as scn
    net = scn.Sequential().add(scn.SparseVggNet(2, 1, [["C", 8], ["C", 8], ["MP", 3, 2], ["C", 16], ["C", 16],
                                                       ["MP", 3, 2], ["C", 24], ["C", 24], ["MP", 3, 2]])).add(
        scn.SubmanifoldConvolution(2, 24, 32, 3, False)).add(scn.BatchNormReLU(32)).add(scn.SparseToDense(2, 32))
    assert net.input_spatial_size(torch.LongTensor([10, 10])).tolist() == [87, 87]
    sc = scn.SubmanifoldConvolution(3, 6, 8, 3, True, groups=2)
    assert tuple(sc.weight.shape) == (27, 2, 3, 4) and tuple(sc.bias.shape) == (8,)
    cv = scn.Convolution(3, 4, 6, [2, 3, 2], 2, False)
    assert tuple(cv.weight.shape) == (12, 1, 4, 6)
    assert cv.input_spatial_size(torch.LongTensor([4, 4, 4])).tolist() == [8, 9, 8]
    bn = scn.BatchNormReLU(5)
    assert sorted(bn.state_dict()) == ["bias", "running_mean", "running_var", "weight"]
    assert bn.eps == 1e-4 and bn.momentum == 0.99 and bn.leakiness == 0
    u = scn.UNet(3, 2, [32, 64, 96], False)
    keys = list(u.state_dict())
    assert keys[0] == "0.0.weight" and "2.1.2.0.1.weight" in keys   # nested like the reference's builder
    d = scn.Deconvolution(2, 4, 4, 3, 2, False)
    assert d.input_spatial_size(torch.LongTensor([9, 9])).tolist() == [4, 4]


def test_precision_switch():
    import sparseconvnet_b200 as scn
    assert scn.get_precision() == "fp32"
    for p in ("tf32", "bf16", "tf32x3", "fp32"):
        scn.set_precision(p)
        assert scn.get_precision() == p
    with pytest.raises(ValueError):
        scn.set_precision("fp8")


def test_batchnorm_layers_are_switched_to_shared_statistics():
    """shard.share_batchnorm_statistics marks every BatchNorm layer of a network; without a process group (one
    process) the layers keep the one-device operator, in training mode too."""
    import sparseconvnet_b200 as scn
    from sparseconvnet_b200 import shard
    net = scn.Sequential().add(scn.SubmanifoldConvolution(3, 3, 8, 3, False)).add(
        scn.UNet(3, 1, [8, 16], residual_blocks=False)).add(scn.BatchNormReLU(8))
    layers = [m for m in net.modules() if isinstance(m, scn.BatchNormalization)]
    assert len(layers) >= 3 and not any(m.across_ranks for m in layers)
    assert shard.share_batchnorm_statistics(net) is net
    assert all(m.across_ranks and m.ranks_group is None for m in layers)
    net.train()
    assert not any(m._shares_statistics() for m in layers)   # no process group: nothing to share with
    net.eval()
    assert not any(m._shares_statistics() for m in layers)
    # a single process sums nothing and leaves the gradients alone (scaled if asked)
    p = [m.weight for m in layers]
    for t in p:
        t.grad = t.detach().clone() * 0 + 2.0
    assert shard.sum_gradients(p) == 0 and all(float(t.grad[0]) == 2.0 for t in p)
    shard.sum_gradients(p, scale=0.5)
    assert all(float(t.grad[0]) == 1.0 for t in p)
