"""Runs a ``sparseconvnet_b200`` module tree on the CPU oracles -- TEST INFRASTRUCTURE ONLY.

Two back ends execute the same walk over the model's modules (found by class name, weights
read from the modules' parameters):

``RefBackend``   the reference's own CPU extension, compiled by ``oracle/build_ref.py`` into
                 ``oracle/_ref/SCN.so`` (+ ``SCN_shim.so`` for rulebook read-back).  Calls the
                 functions bound in the reference's sparseconvnet/SCN/pybind.cpp directly.
``PortBackend``  the numpy restatement in ``oracle/scn_oracle.py``.

The product never imports this file; only tests, ``__graft_entry__.smoke()`` and the
CPU-baseline leg of ``bench.py`` do.
"""
import importlib.util
import os

import numpy as np
import torch

from . import scn_oracle as port

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF = os.path.join(_HERE, "_ref")


_EXTENSION_KEY = "_scn_reference_cpu_extension"  # shared with the staged package (oracle/build_ref.py)


def _load(name):
    import sys
    if name == "SCN" and _EXTENSION_KEY in sys.modules:
        return sys.modules[_EXTENSION_KEY]
    spec = importlib.util.spec_from_file_location(name, os.path.join(_REF, name + ".so"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    if name == "SCN":
        sys.modules[_EXTENSION_KEY] = mod
    return mod


_ref_modules = None


def reference_available():
    return os.path.exists(os.path.join(_REF, "SCN.so")) and os.path.exists(os.path.join(_REF, "SCN_shim.so"))


def reference_modules():
    """(SCN, SCN_shim) of the compiled reference; raises if oracle/_ref has not been built."""
    global _ref_modules
    if _ref_modules is None:
        if not reference_available():
            raise RuntimeError("oracle/_ref is not built (python oracle/build_ref.py)")
        _ref_modules = (_load("SCN"), _load("SCN_shim"))
    return _ref_modules


class OTensor(object):
    """Sparse activation on the oracle side: features [N, C] float32 (numpy), the back end's
    metadata handle and the spatial size."""

    def __init__(self, features, metadata, spatial_size):
        self.features = features
        self.metadata = metadata
        self.spatial_size = [int(v) for v in spatial_size]


def _lt(v):
    return torch.tensor([int(i) for i in v], dtype=torch.int64)


def _np(t):
    return None if t is None else t.detach().cpu().numpy().astype(np.float32)


class RefBackend(object):
    name = "reference"

    def __init__(self):
        self.SCN, self.shim = reference_modules()

    @staticmethod
    def _t(a):
        return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32))

    @staticmethod
    def _opt(p):
        return torch.empty(0) if p is None else p.detach().cpu().float().contiguous()

    def input_layer(self, dim, spatial_size, mode, coords, features, batch_size):
        md = getattr(self.SCN, "Metadata_%d" % dim)()
        out = torch.empty(0)
        self.SCN.InputLayer_updateOutput(md, _lt(spatial_size), torch.as_tensor(np.asarray(coords)).long().contiguous(),
                                         self._t(features), out, int(batch_size), int(mode))
        return OTensor(out.numpy(), md, spatial_size)

    def bl_input_layer(self, dim, spatial_size, mode, coords, features):
        md = getattr(self.SCN, "Metadata_%d" % dim)()
        out = torch.empty(0)
        f = np.ascontiguousarray(features, dtype=np.float32)
        self.SCN.BLInputLayer_updateOutput(md, _lt(spatial_size), torch.as_tensor(np.asarray(coords)).long().contiguous(),
                                           torch.from_numpy(f), out, int(mode))
        return OTensor(out.numpy(), md, spatial_size)

    def output_layer(self, x):
        out = torch.empty(0)
        self.SCN.OutputLayer_updateOutput(x.metadata, self._t(x.features), out)
        return out.numpy()

    def bl_output_layer(self, x):
        out = torch.empty(0)
        self.SCN.BLOutputLayer_updateOutput(x.metadata, self._t(x.features), out)
        return out.numpy()

    def locations(self, x, spatial_size=None):
        return x.metadata.getSpatialLocations(_lt(spatial_size or x.spatial_size)).numpy()

    def batch_size(self, x):
        return x.metadata.getBatchSize(_lt(x.spatial_size))

    def submanifold_rulebook(self, x, filter_size):
        return [r.numpy().reshape(-1, 2) for r in self.shim.submanifold_rulebook(x.metadata, _lt(x.spatial_size), _lt(filter_size))]

    def strided_rulebook(self, x, out_size, filter_size, stride):
        return [r.numpy().reshape(-1, 2) for r in
                self.shim.strided_rulebook(x.metadata, _lt(x.spatial_size), _lt(out_size), _lt(filter_size), _lt(stride))]

    def subconv(self, x, filter_size, weight, bias):
        out = torch.empty(0)
        macs = self.SCN.SubmanifoldConvolution_updateOutput(_lt(x.spatial_size), _lt(filter_size), x.metadata,
                                                            self._t(x.features), out, self._opt(weight), self._opt(bias))
        return OTensor(out.numpy(), x.metadata, x.spatial_size), macs

    def conv(self, x, out_size, filter_size, stride, weight, bias):
        out = torch.empty(0)
        macs = self.SCN.Convolution_updateOutput(_lt(x.spatial_size), _lt(out_size), _lt(filter_size), _lt(stride),
                                                 x.metadata, self._t(x.features), out, self._opt(weight), self._opt(bias))
        return OTensor(out.numpy(), x.metadata, out_size), macs

    def deconv(self, x, out_size, filter_size, stride, weight, bias):
        out = torch.empty(0)
        macs = self.SCN.Deconvolution_updateOutput(_lt(x.spatial_size), _lt(out_size), _lt(filter_size), _lt(stride),
                                                   x.metadata, self._t(x.features), out, self._opt(weight), self._opt(bias))
        return OTensor(out.numpy(), x.metadata, out_size), macs

    def batchnorm(self, x, m):
        if x.features.size == 0:
            return x
        out = torch.empty(0)
        c = x.features.shape[1]
        self.SCN.BatchNormalization_updateOutput(
            self._t(x.features), out, torch.empty(c), torch.empty(c), m.running_mean.detach().cpu().float(),
            m.running_var.detach().cpu().float(), self._opt(getattr(m, "weight", None)),
            self._opt(getattr(m, "bias", None)), m.eps, m.momentum, bool(m.training), m.leakiness)
        return OTensor(out.numpy(), x.metadata, x.spatial_size)

    def maxpool(self, x, out_size, pool_size, stride, drop):
        out = torch.empty(0)
        self.SCN.MaxPooling_updateOutput(_lt(x.spatial_size), _lt(out_size), _lt(pool_size), _lt(stride), x.metadata,
                                         self._t(x.features), out, int(drop))
        return OTensor(out.numpy(), x.metadata, out_size)

    def avgpool(self, x, out_size, pool_size, stride, drop):
        out = torch.empty(0)
        self.SCN.AveragePooling_updateOutput(_lt(x.spatial_size), _lt(out_size), _lt(pool_size), _lt(stride),
                                             x.metadata, self._t(x.features), out, int(drop))
        return OTensor(out.numpy(), x.metadata, out_size)

    def unpool(self, x, out_size, pool_size, stride, drop):
        out = torch.empty(0)
        self.SCN.UnPooling_updateOutput(_lt(x.spatial_size), _lt(out_size), _lt(pool_size), _lt(stride),
                                        x.metadata, self._t(x.features), out, int(drop))
        return OTensor(out.numpy(), x.metadata, out_size)

    def sparse_to_dense(self, x, n_planes):
        out = torch.empty(0)
        self.SCN.SparseToDense_updateOutput(_lt(x.spatial_size), x.metadata, self._t(x.features), out, int(n_planes))
        return out.numpy()

    def nin(self, x, weight, bias):
        out = torch.empty(0)
        macs = self.SCN.NetworkInNetwork_updateOutput(self._t(x.features), out, self._opt(weight), self._opt(bias))
        return OTensor(out.numpy(), x.metadata, x.spatial_size), macs


class _PortMetadata(object):
    def __init__(self):
        self.grids = {}
        self.sub = {}
        self.strided = {}


class PortBackend(object):
    name = "port"

    def input_layer(self, dim, spatial_size, mode, coords, features, batch_size):
        md = _PortMetadata()
        grid, rules = port.input_layer([int(v) for v in spatial_size], np.asarray(coords), batch_size, mode)
        md.grids[tuple(int(v) for v in spatial_size)] = grid
        md.input_rules, md.point_mode, md.point_shape = rules, mode, (np.asarray(coords).shape[0],)
        out = port.input_layer_features(features, grid.n_active, rules, mode)
        return OTensor(out, md, spatial_size)

    def bl_input_layer(self, dim, spatial_size, mode, coords, features):
        md = _PortMetadata()
        coords = np.asarray(coords)
        grid, rules, point_mode = port.bl_input_layer([int(v) for v in spatial_size], coords, mode)
        md.grids[tuple(int(v) for v in spatial_size)] = grid
        md.input_rules, md.point_mode, md.point_shape = rules, point_mode, coords.shape[:2]
        f = np.asarray(features, dtype=np.float32).reshape(coords.shape[0] * coords.shape[1], -1)
        out = port.input_layer_features(f, grid.n_active, rules, point_mode)
        return OTensor(out, md, spatial_size)

    def output_layer(self, x):
        md = x.metadata
        n = int(np.prod(md.point_shape))
        return port.output_layer_features(x.features, n, md.input_rules, md.point_mode)

    def bl_output_layer(self, x):
        out = self.output_layer(x)
        return out.reshape(tuple(x.metadata.point_shape) + (out.shape[1],))

    def _grid(self, x, size=None):
        return x.metadata.grids[tuple(size or x.spatial_size)]

    def locations(self, x, spatial_size=None):
        return port.spatial_locations(self._grid(x, spatial_size and [int(v) for v in spatial_size]))

    def batch_size(self, x):
        return self._grid(x).batch_size

    def submanifold_rulebook(self, x, filter_size):
        key = (tuple(x.spatial_size), tuple(int(v) for v in filter_size))
        if key not in x.metadata.sub:
            x.metadata.sub[key] = port.submanifold_rules(self._grid(x), filter_size)
        return x.metadata.sub[key]

    def strided_rulebook(self, x, out_size, filter_size, stride):
        key = (tuple(x.spatial_size), tuple(int(v) for v in filter_size), tuple(int(v) for v in stride))
        if key not in x.metadata.strided:
            g, rules = port.strided_rules(self._grid(x), out_size, filter_size, stride)
            x.metadata.grids[tuple(int(v) for v in out_size)] = g
            x.metadata.strided[key] = rules
        return x.metadata.strided[key]

    def subconv(self, x, filter_size, weight, bias):
        rules = self.submanifold_rulebook(x, filter_size)
        out, macs = port.convolution(x.features, self._grid(x).n_active, rules, _np(weight), _np(bias))
        return OTensor(out, x.metadata, x.spatial_size), macs

    def conv(self, x, out_size, filter_size, stride, weight, bias):
        rules = self.strided_rulebook(x, out_size, filter_size, stride)
        n_out = x.metadata.grids[tuple(int(v) for v in out_size)].n_active
        out, macs = port.convolution(x.features, n_out, rules, _np(weight), _np(bias))
        return OTensor(out, x.metadata, out_size), macs

    def deconv(self, x, out_size, filter_size, stride, weight, bias):
        fine = OTensor(None, x.metadata, out_size)
        rules = self.strided_rulebook(fine, x.spatial_size, filter_size, stride)
        n_out = x.metadata.grids[tuple(int(v) for v in out_size)].n_active
        out, macs = port.deconvolution(x.features, n_out, rules, _np(weight), _np(bias))
        return OTensor(out, x.metadata, out_size), macs

    def batchnorm(self, x, m):
        if x.features.size == 0:
            return x
        y, rm, rv = port.batchnorm(x.features, _np(m.running_mean), _np(m.running_var),
                                   _np(getattr(m, "weight", None)), _np(getattr(m, "bias", None)), m.eps,
                                   m.momentum, bool(m.training), m.leakiness)
        return OTensor(y, x.metadata, x.spatial_size)

    def maxpool(self, x, out_size, pool_size, stride, drop):
        rules = self.strided_rulebook(x, out_size, pool_size, stride)
        n_out = x.metadata.grids[tuple(int(v) for v in out_size)].n_active
        return OTensor(port.max_pooling(x.features, n_out, rules, drop), x.metadata, out_size)

    def avgpool(self, x, out_size, pool_size, stride, drop):
        rules = self.strided_rulebook(x, out_size, pool_size, stride)
        n_out = x.metadata.grids[tuple(int(v) for v in out_size)].n_active
        return OTensor(port.average_pooling(x.features, n_out, rules, drop), x.metadata, out_size)

    def unpool(self, x, out_size, pool_size, stride, drop):
        fine = OTensor(None, x.metadata, out_size)   # the fine grid must exist already
        rules = self.strided_rulebook(fine, [int(v) for v in x.spatial_size], pool_size, stride)
        n_fine = x.metadata.grids[tuple(int(v) for v in out_size)].n_active
        return OTensor(port.unpooling(x.features, n_fine, rules, drop), x.metadata, out_size)

    def sparse_to_dense(self, x, n_planes):
        return port.sparse_to_dense(self._grid(x), x.features, n_planes)

    def nin(self, x, weight, bias):
        out = x.features @ _np(weight)
        if bias is not None:
            out = out + _np(bias)
        macs = float(x.features.shape[0]) * weight.shape[0] * weight.shape[1]  # CPU/NetworkInNetwork.cpp:22
        return OTensor(out.astype(np.float32), x.metadata, x.spatial_size), macs


def run_module(m, x, be, stats=None):
    """Applies module `m` (a sparseconvnet_b200 module tree) to `x` on back end `be`.
    `x` is [coords, features(, batch_size)] for an InputLayer, an OTensor, or a list of
    OTensors for Join/AddTable.  `stats` (dict) accumulates the multiply-add count."""
    name = type(m).__name__

    def count(macs):
        if stats is not None:
            stats["macs"] = stats.get("macs", 0.0) + macs

    if name in ("Sequential",):
        for child in m.children():
            x = run_module(child, x, be, stats)
        return x
    if name == "ConcatTable":
        return [run_module(child, x, be, stats) for child in m.children()]
    if name == "JoinTable":
        return OTensor(np.concatenate([i.features for i in x], axis=1), x[0].metadata, x[0].spatial_size)
    if name == "AddTable":
        acc = x[0].features
        for i in x[1:]:
            acc = acc + i.features
        return OTensor(acc, x[0].metadata, x[0].spatial_size)
    if name == "Identity":
        return x
    if name == "InputLayer":
        coords, feats = np.asarray(x[0]), np.asarray(x[1], dtype=np.float32)
        return be.input_layer(m.dimension, m.spatial_size.tolist(), m.mode, coords, feats, 0 if len(x) == 2 else x[2])
    if name == "BLInputLayer":
        return be.bl_input_layer(m.dimension, m.spatial_size.tolist(), m.mode, np.asarray(x[0]),
                                 np.asarray(x[1], dtype=np.float32))
    if name == "OutputLayer":
        return be.output_layer(x)
    if name == "BLOutputLayer":
        return be.bl_output_layer(x)
    if name in ("SubmanifoldConvolution", "ValidConvolution"):
        y, macs = be.subconv(x, m.filter_size.tolist(), m.weight, getattr(m, "bias", None))
        count(macs)
        return y
    if name == "Convolution":
        out_size = [(i - f) // s + 1 for i, f, s in zip(x.spatial_size, m.filter_size.tolist(), m.filter_stride.tolist())]
        y, macs = be.conv(x, out_size, m.filter_size.tolist(), m.filter_stride.tolist(), m.weight, getattr(m, "bias", None))
        count(macs)
        return y
    if name == "Deconvolution":
        out_size = [(i - 1) * s + f for i, f, s in zip(x.spatial_size, m.filter_size.tolist(), m.filter_stride.tolist())]
        y, macs = be.deconv(x, out_size, m.filter_size.tolist(), m.filter_stride.tolist(), m.weight, getattr(m, "bias", None))
        count(macs)
        return y
    if name in ("BatchNormalization", "BatchNormReLU", "BatchNormLeakyReLU"):
        return be.batchnorm(x, m)
    if name == "MaxPooling":
        out_size = [(i - f) // s + 1 for i, f, s in zip(x.spatial_size, m.pool_size.tolist(), m.pool_stride.tolist())]
        return be.maxpool(x, out_size, m.pool_size.tolist(), m.pool_stride.tolist(), m.nFeaturesToDrop)
    if name == "AveragePooling":
        out_size = [(i - f) // s + 1 for i, f, s in zip(x.spatial_size, m.pool_size.tolist(), m.pool_stride.tolist())]
        return be.avgpool(x, out_size, m.pool_size.tolist(), m.pool_stride.tolist(), m.nFeaturesToDrop)
    if name == "UnPooling":
        out_size = [(i - 1) * s + f for i, f, s in zip(x.spatial_size, m.pool_size.tolist(), m.pool_stride.tolist())]
        return be.unpool(x, out_size, m.pool_size.tolist(), m.pool_stride.tolist(), m.nFeaturesToDrop)
    if name == "SparseToDense":
        return be.sparse_to_dense(x, m.nPlanes)
    if name == "NetworkInNetwork":
        y, macs = be.nin(x, m.weight, getattr(m, "bias", None))
        count(macs)
        return y
    if name == "Linear":
        f = x.features if isinstance(x, OTensor) else x
        y = f @ _np(m.weight).T
        if m.bias is not None:
            y = y + _np(m.bias)
        return y.astype(np.float32)
    raise NotImplementedError("oracle runner: module %s" % name)
