"""Shared comparison code of the test-suite."""
import os

import numpy as np
import torch

from oracle import runner, scn_oracle as port

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FP32_TOL = 1e-4   # relative to the tensor's largest magnitude: the bar for fp32 features
TC_TOL = 1e-2     # bf16 / tf32 tensor-core arithmetic


def load_golden(name):
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


def load_state(module, golden, prefix):
    sd = {k[len(prefix) + 1:]: torch.from_numpy(v) for k, v in golden.items() if k.startswith(prefix + "/")}
    module.load_state_dict(sd, strict=True)


def rel_err(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape, (a.shape, b.shape)
    if a.size == 0:
        return 0.0
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def assert_features_match(loc_a, feat_a, loc_b, feat_b, tol, same_rows=False, what=""):
    """Rows matched by (coords, batch) unless the two sides share the row numbering."""
    if same_rows:
        assert np.array_equal(loc_a, loc_b), "%s: locations differ" % what
        e = rel_err(feat_a, feat_b)
    else:
        p = port.align_rows(loc_a, loc_b)
        e = rel_err(feat_a, np.asarray(feat_b)[p])
    assert e <= tol, "%s: relative error %.3g > %.1g" % (what, e, tol)
    return e


def golden_rules(golden, prefix):
    keys = sorted(k for k in golden if k.startswith(prefix + "/"))
    return [golden[k] for k in keys]


def assert_rules_equal(canon_a, canon_b, what=""):
    assert len(canon_a) == len(canon_b), "%s: offset counts differ" % what
    for k, (a, b) in enumerate(zip(canon_a, canon_b)):
        a = np.asarray(a).reshape(-1, b.shape[1]) if np.asarray(a).size == 0 and b.ndim == 2 else np.asarray(a)
        assert a.shape[0] == b.shape[0], "%s offset %d: %d vs %d rules" % (what, k, a.shape[0], b.shape[0])
        if a.shape[0]:
            assert np.array_equal(a, b), "%s offset %d: rules differ" % (what, k)


# ---- the CUDA path as a back end with the oracle runner's vocabulary --------------------------

class GpuTensor(object):
    def __init__(self, t):
        self.t = t

    @property
    def features(self):
        return self.t.features.detach().cpu().numpy()

    @property
    def spatial_size(self):
        return self.t.spatial_size.tolist()


class GpuBackend(object):
    """Runs sparseconvnet_b200 modules on cuda:0 and hands results back as numpy."""
    name = "cuda"

    def __init__(self, device="cuda:0"):
        self.device = torch.device(device)

    def run(self, m, x):
        import sparseconvnet_b200 as scn
        m = m.to(self.device) if not isinstance(m, (scn.InputLayer, scn.BLInputLayer)) else m
        with torch.no_grad():
            if isinstance(m, scn.BLInputLayer):
                coords = torch.as_tensor(np.asarray(x[0])).long()
                feats = torch.as_tensor(np.asarray(x[1], dtype=np.float32)).to(self.device)
                y = m([coords, feats])
            elif isinstance(m, scn.InputLayer):
                coords = torch.as_tensor(np.asarray(x[0])).long()
                feats = torch.as_tensor(np.asarray(x[1], dtype=np.float32)).to(self.device)
                y = m([coords, feats] + list(x[2:]))
            elif isinstance(m, torch.nn.Linear):
                y = m(x.t.features if isinstance(x, GpuTensor) else x)
            else:
                y = m(x.t if isinstance(x, GpuTensor) else [i.t for i in x])
        if isinstance(y, torch.Tensor):
            return y.detach().cpu().numpy()
        return GpuTensor(y)

    def locations(self, x, spatial_size=None):
        return x.t.get_spatial_locations(spatial_size).numpy()

    def batch_size(self, x):
        return x.t.batch_size()

    def submanifold_rulebook(self, x, filter_size):
        from sparseconvnet_b200 import _lib
        r = x.t.metadata.rulebook(0, x.spatial_size, filter_size)
        return [t.cpu().numpy() for t in r]

    def strided_rulebook(self, x, out_size, filter_size, stride):
        r = x.t.metadata.rulebook(1, x.spatial_size, filter_size, stride)
        return [t.cpu().numpy() for t in r]


def oracle_run(be):
    return lambda m, x: runner.run_module(m, x, be)
