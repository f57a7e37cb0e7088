"""The drop-in boundary, proven with the reference's own code: the reference's unmodified Python
package (sparseconvnet/*.py, staged under oracle/_ref by oracle/build_ref.py) with
``sparseconvnet.SCN`` bound to this library (sparseconvnet/SCN/pybind.cpp:201-237 is the
module it stands in for) runs the reference's example networks on the GPU, and the results
match the same package on the reference's own CPU extension.

CPU part: both bindings import, and this repository's network builders produce the same module
tree as the reference's (equal state_dict keys, shapes and -- same seed -- values)."""
import numpy as np
import pytest
import torch

from oracle import refpkg, runner
from sparseconvnet_b200 import workloads
from tests import helpers

needs_ref = pytest.mark.skipif(not (refpkg.available("cpu") and refpkg.available("b200") and
                                    runner.reference_available()),
                               reason="oracle/_ref (the staged reference) is not present")


@needs_ref
def test_both_bindings_import():
    cpu, b200 = refpkg.load("cpu"), refpkg.load("b200")
    import sparseconvnet_b200.SCN as ours
    assert b200.SCN is ours and cpu.SCN is not ours
    assert cpu.SCN.n_rulebook_bits() == 32 and b200.SCN.n_rulebook_bits() == 32
    assert not cpu.SCN.is_cuda_build() and b200.SCN.is_cuda_build()
    # every binding function the reference's modules of the path call exists in the mirror
    for name in ("InputLayer_updateOutput", "OutputLayer_updateOutput", "BLInputLayer_updateOutput",
                 "BLOutputLayer_updateOutput", "SubmanifoldConvolution_updateOutput", "Convolution_updateOutput",
                 "Deconvolution_updateOutput", "BatchNormalization_updateOutput", "MaxPooling_updateOutput",
                 "AveragePooling_updateOutput", "UnPooling_updateOutput", "SparseToDense_updateOutput",
                 "NetworkInNetwork_updateOutput", "Metadata_2", "Metadata_3", "Metadata_4"):
        assert hasattr(cpu.SCN, name) and hasattr(b200.SCN, name), name


@needs_ref
@pytest.mark.parametrize("config", [1, 2, 3, 4, 5])
def test_builders_equal_reference_builders(config):
    """architectures.py against networkArchitectures.py (SparseVggNet :12-72, SparseResNet :132-200,
    UNet :203-257): same parameter and buffer names in the same order, same shapes, and with the same
    seed the same initial values, so checkpoints move both ways."""
    ref = refpkg.load("cpu")
    inp_a, net_a, _ = workloads.build_config(config)
    inp_b, net_b, _ = workloads.build_config(config, scn=ref)
    sa, sb = net_a.state_dict(), net_b.state_dict()
    assert list(sa.keys()) == list(sb.keys())
    for k in sa:
        assert sa[k].shape == sb[k].shape and torch.equal(sa[k], sb[k]), k
    assert inp_a.spatial_size.tolist() == inp_b.spatial_size.tolist()
    assert [type(m).__name__ for m in net_a.modules()] == [type(m).__name__ for m in net_b.modules()]


def _run_reference_package(binding, build, coords, feats, device):
    scn = refpkg.load(binding)
    torch.manual_seed(77)
    model, head = build(scn)
    workloads.randomize(model, 5)
    model.eval()
    if device != "cpu":
        model = model.to(device)
        head = head.to(device) if head is not None else None
    with torch.no_grad():
        y = model([torch.from_numpy(coords), torch.from_numpy(feats).to(device)])
        if head is not None:
            y = head(y)
    return model, y


def _hello_world(scn):
    # the network of examples/hello-world.py:19-30
    model = scn.Sequential().add(
        scn.SparseVggNet(2, 1, [["C", 8], ["C", 8], ["MP", 3, 2], ["C", 16], ["C", 16], ["MP", 3, 2],
                                ["C", 24], ["C", 24], ["MP", 3, 2]])).add(
        scn.SubmanifoldConvolution(2, 24, 32, 3, False)).add(scn.BatchNormReLU(32)).add(scn.SparseToDense(2, 32))
    size = model.input_spatial_size(torch.LongTensor([10, 10]))
    full = scn.Sequential().add(scn.InputLayer(2, size)).add(model)
    return full, None


def _scannet_unet(m, reps):
    def build(scn):
        # the model of examples/ScanNet/unet.py:25-38 (InputLayer mode 4 ... OutputLayer, then Linear)
        sparse = scn.Sequential().add(scn.InputLayer(3, 4096, mode=4)).add(
            scn.SubmanifoldConvolution(3, 3, m, 3, False)).add(
            scn.UNet(3, reps, [m, 2 * m, 3 * m, 4 * m, 5 * m, 6 * m, 7 * m], False)).add(
            scn.BatchNormReLU(m)).add(scn.OutputLayer(3))
        return sparse, torch.nn.Linear(m, 20)
    return build


@needs_ref
@pytest.mark.gpu
def test_hello_world_network_on_this_library(cuda):
    coords, feats = workloads.make_batch(2, range(20))
    _, want = _run_reference_package("cpu", _hello_world, coords, feats, "cpu")
    model, got = _run_reference_package("b200", _hello_world, coords, feats, "cuda:0")
    assert got.is_cuda and tuple(got.shape) == (20, 32, 10, 10)
    assert helpers.rel_err(got.cpu().numpy(), want.numpy()) <= helpers.FP32_TOL


@needs_ref
@pytest.mark.gpu
@pytest.mark.parametrize("m,reps,precision", [(16, 1, "fp32"), (32, 2, "fp32"), (32, 2, "tf32x3")])
def test_scannet_unet_on_this_library(m, reps, precision, cuda):
    """Per-point scores through InputLayer(mode 4) ... OutputLayer: rows are the input points, so the two
    sides compare row for row.  Input with duplicate points (mode 4 averages them)."""
    import sparseconvnet_b200 as ours
    coords, feats = workloads.batch_config3([0, 1], target_voxels=30000)
    rng = np.random.default_rng(3)
    dup = rng.integers(0, coords.shape[0], 5000)
    coords = np.concatenate([coords, coords[dup]])
    feats = np.concatenate([feats, rng.uniform(-1, 1, (dup.size, 3)).astype(np.float32)])
    _, want = _run_reference_package("cpu", _scannet_unet(m, reps), coords, feats, "cpu")
    ours.set_precision(precision)
    try:
        _, got = _run_reference_package("b200", _scannet_unet(m, reps), coords, feats, "cuda:0")
        torch.cuda.synchronize()
    finally:
        ours.set_precision("fp32")
    assert tuple(got.shape) == (coords.shape[0], 20)
    e = helpers.rel_err(got.cpu().numpy(), want.numpy())
    assert e <= helpers.FP32_TOL, "relative error %.3g" % e
