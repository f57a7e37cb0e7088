"""The inference-path modules, API-compatible with the reference's ``sparseconvnet`` package:
same class names, constructor arguments, parameter names and shapes (so reference
``state_dict``s load), same ``input_spatial_size`` protocol.  Forward only: every module
runs under ``torch.no_grad`` semantics and calls the ``SCN`` mirror module, which calls the
C-ABI library.

Reference counterparts: sparseconvnet/ioLayers.py:15-65, submanifoldConvolution.py:14-60,
convolution.py:13-66, deconvolution.py:13-64, batchNormalization.py:13-91,
maxPooling.py:71-104, sparseToDense.py:59-75, networkInNetwork.py, identity.py.
"""
import weakref

import torch
from torch.nn import Module, Parameter

import sparseconvnet_b200 as _pkg
from . import SCN, autograd
from .sparse_tensor import SparseConvNetTensor, optional_tensor, to_long_tensor


def _size_str(t):
    v = t.tolist()
    return str(v[0]) if min(v) == max(v) else "(" + ",".join(str(i) for i in v) + ")"


class InputLayer(Module):
    """Takes ``[coords, features]`` or ``[coords, features, batch_size]``.

    coords: LongTensor [N, dimension] (one sample) or [N, dimension+1] (last column = batch
    index), on the CPU as in the reference or already on the GPU.  features: CUDA float
    tensor [N, planes].  mode: how repeated coordinates are merged -- 0 none expected,
    1 keep the first row, 2 keep the last row, 3 sum, 4 mean (what the reference's code does,
    sparseconvnet/SCN/Metadata/IOLayersRules.h:96-120).
    """

    def __init__(self, dimension, spatial_size, mode=3):
        Module.__init__(self)
        self.dimension = dimension
        self.spatial_size = to_long_tensor(dimension, spatial_size)
        self.mode = mode
        self.device = None

    def to(self, device):
        self.device = device
        return self

    def forward(self, input):
        coords, features = input[0], input[1]
        if self.device is not None:
            features = features.to(self.device)
        elif not features.is_cuda:
            raise RuntimeError("InputLayer: features must be on a CUDA device (or call .to(device) on "
                               "the layer): sparseconvnet_b200 has no CPU path")
        output = SparseConvNetTensor(metadata=_pkg.Metadata(self.dimension), spatial_size=self.spatial_size)
        batch_size = 0 if len(input) == 2 else input[2]

        def run(f):
            out = f.new_empty(0)
            SCN.InputLayer_updateOutput(output.metadata, self.spatial_size, coords.long(),
                                        f.detach().float().contiguous(), out, batch_size, self.mode)
            return out

        if autograd.needs_grad(features):
            output.features = autograd.input_features(features, output.metadata, run)
        else:
            output.features = run(features)
        return output

    def input_spatial_size(self, out_size):
        return out_size

    def __repr__(self):
        return "InputLayer(mode=%d)" % self.mode


class OutputLayer(Module):
    """The inverse of InputLayer for 'autoencoder' / per-point networks (ioLayers.py:68-91): takes a
    SparseConvNetTensor whose metadata was made by an InputLayer and returns a float tensor
    [n_points, planes]: every input point gets the row of its site (points that the InputLayer's
    mode dropped get zeros)."""

    def __init__(self, dimension):
        Module.__init__(self)
        self.dimension = dimension

    def forward(self, input):
        if autograd.needs_grad(input.features):
            return autograd.output_features(input.features, input.metadata, False)
        output = input.features.new_empty(0)
        SCN.OutputLayer_updateOutput(input.metadata, input.features.detach().contiguous(), output)
        return output

    def input_spatial_size(self, out_size):
        return out_size

    def __repr__(self):
        return "OutputLayer()"


class BLInputLayer(Module):
    """Takes ``[coords, features]`` with coords a LongTensor [batch, length, dimension] (-1 = empty
    slot) and features [batch, length, planes] (ioLayers.py:94-138).  mode: 0 all points present
    and unique, 1 use the last point of a site, 2 keep the first, 3 sum, 4 mean."""

    def __init__(self, dimension, spatial_size, mode=3):
        Module.__init__(self)
        self.dimension = dimension
        self.spatial_size = to_long_tensor(dimension, spatial_size)
        self.mode = mode
        self.device = None

    def to(self, device):
        self.device = device
        return self

    def forward(self, input):
        coords, features = input[0], input[1]
        if self.device is not None:
            features = features.to(self.device)
        elif not features.is_cuda:
            raise RuntimeError("BLInputLayer: features must be on a CUDA device (or call .to(device) on "
                               "the layer): sparseconvnet_b200 has no CPU path")
        output = SparseConvNetTensor(metadata=_pkg.Metadata(self.dimension), spatial_size=self.spatial_size)
        def run(f):
            out = f.new_empty(0)
            SCN.BLInputLayer_updateOutput(output.metadata, self.spatial_size, coords.long(),
                                          f.detach().float().contiguous(), out, self.mode)
            return out

        if autograd.needs_grad(features):
            output.features = autograd.input_features(features, output.metadata, run)
        else:
            output.features = run(features)
        return output

    def input_spatial_size(self, out_size):
        return out_size

    def __repr__(self):
        return "BLInputLayer(mode=%d)" % self.mode


class BLOutputLayer(Module):
    """The inverse of BLInputLayer (ioLayers.py:141-164): returns [batch, length, planes]."""

    def __init__(self, dimension):
        Module.__init__(self)
        self.dimension = dimension

    def forward(self, input):
        if autograd.needs_grad(input.features):
            return autograd.output_features(input.features, input.metadata, True)
        output = input.features.new_empty(0)
        SCN.BLOutputLayer_updateOutput(input.metadata, input.features.detach().contiguous(), output)
        return output

    def input_spatial_size(self, out_size):
        return out_size

    def __repr__(self):
        return "BLOutputLayer()"


class _ConvBase(Module):
    def _init_weight(self, dimension, nIn, nOut, filter_size, bias, groups):
        self.dimension = dimension
        self.groups = groups
        self.nIn = nIn
        self.nOut = nOut
        self.filter_size = to_long_tensor(dimension, filter_size)
        self.filter_volume = int(self.filter_size.prod().item())
        std = (2.0 * groups / nIn / self.filter_volume) ** 0.5
        self.weight = Parameter(torch.empty(self.filter_volume, groups, nIn // groups,
                                            nOut // groups).normal_(0, std))
        if bias:
            self.bias = Parameter(torch.zeros(nOut))

    cache_weight_images = True   # class-wide switch (tests turn it off to compare)

    def _weight_token(self):
        """Token under which this layer's prepared weight images are kept by the library: renewed
        whenever the weight tensor is written (version counter) or moved (data pointer)."""
        if not _ConvBase.cache_weight_images:
            return 0
        w = self.weight
        key = (w.data_ptr(), w._version)
        if getattr(self, "_wkey", None) != key:
            old = getattr(self, "_wtoken", 0)
            if old:
                SCN.release_weight_token(old)
                self._wfinal.detach()
            self._wtoken = SCN.new_weight_token()
            self._wkey = key
            self._wfinal = weakref.finalize(self, SCN.release_weight_token, self._wtoken)
        return self._wtoken

    def _count(self, macs, output_features):
        SCN.flop_counter.add(macs)
        _pkg.forward_pass_hidden_states += output_features.nelement()


class SubmanifoldConvolution(_ConvBase):
    def __init__(self, dimension, nIn, nOut, filter_size, bias, groups=1):
        Module.__init__(self)
        self._init_weight(dimension, nIn, nOut, filter_size, bias, groups)

    def forward(self, input, bn=None):
        """`bn` (used by Sequential): an eval-mode BatchNormalization that follows this layer and is
        applied in the convolution's store instead of as a pass of its own."""
        assert input.features.nelement() == 0 or input.features.size(1) == self.nIn, (self.nIn, self.nOut, input)
        output = SparseConvNetTensor(metadata=input.metadata, spatial_size=input.spatial_size)
        bias = optional_tensor(self, "bias")
        if autograd.needs_grad(input.features, self.weight, bias):
            assert bn is None
            output.features, macs = autograd.convolution(
                autograd.SUBMANIFOLD, input.features, self.weight, bias.to(self.weight.device), input.metadata,
                input.spatial_size, None, self.filter_size, None)
        else:
            output.features = input.features.new_empty(0)
            with SCN.weight_token(self._weight_token()):
                macs = SCN.SubmanifoldConvolution_updateOutput(
                    input.spatial_size, self.filter_size, input.metadata, input.features.detach().contiguous(),
                    output.features, self.weight, bias, epilogue=bn.folded() if bn is not None else None)
        self._count(macs, output.features)
        return output

    def forward_joined(self, inputs, pre_bn=None, bn=None):
        """This layer applied to the concatenation of `inputs` (what a JoinTable in front of it would produce),
        through the eval-mode BatchNormalization `pre_bn` between the two if given, without the concatenation and
        the normalised copy being built as tensors of their own.  None when the shapes do not allow it."""
        output = SparseConvNetTensor(metadata=inputs[0].metadata, spatial_size=inputs[0].spatial_size)
        output.features = inputs[0].features.new_empty(0)
        with SCN.weight_token(self._weight_token()):
            macs = SCN.SubmanifoldConvolution_joined(
                inputs[0].spatial_size, self.filter_size, inputs[0].metadata,
                [i.features.detach().contiguous() for i in inputs], output.features, self.weight,
                optional_tensor(self, "bias"), prologue=pre_bn.folded() if pre_bn is not None else None,
                epilogue=bn.folded() if bn is not None else None)
        if macs is None:
            return None
        self._count(macs, output.features)
        return output

    def input_spatial_size(self, out_size):
        return out_size

    def __repr__(self):
        return "SubmanifoldConvolution %d->%d C%s" % (self.nIn, self.nOut, _size_str(self.filter_size))


class ValidConvolution(SubmanifoldConvolution):
    pass


class Convolution(_ConvBase):
    # Not in the reference: how many consecutive levels of this same downsampling the network goes down
    # from here (this layer included), set by the network builders that know (UNet, FullyConvolutionalNet).
    # More than one: the grids and rulebooks of all those levels are built together on first use
    # (SCN.strided_chain), with one wait for their site counts instead of one per level.
    levels_below = 1

    def __init__(self, dimension, nIn, nOut, filter_size, filter_stride, bias, groups=1):
        Module.__init__(self)
        self._init_weight(dimension, nIn, nOut, filter_size, bias, groups)
        self.filter_stride = to_long_tensor(dimension, filter_stride)

    def forward(self, input, bn=None, pre_bn=None):
        """`bn` / `pre_bn` (used by Sequential): eval-mode BatchNormalizations behind / in front of this layer that
        are applied inside the convolution call instead of as passes of their own."""
        assert input.features.nelement() == 0 or input.features.size(1) == self.nIn
        out_size = torch.div(input.spatial_size - self.filter_size, self.filter_stride, rounding_mode="trunc") + 1
        assert ((out_size - 1) * self.filter_stride + self.filter_size == input.spatial_size).all(), \
            (input.spatial_size, out_size, self.filter_size, self.filter_stride)
        output = SparseConvNetTensor(metadata=input.metadata, spatial_size=out_size)
        bias = optional_tensor(self, "bias")
        if self.levels_below > 1 and input.features.is_cuda:
            SCN.strided_chain(input.metadata, input.spatial_size, self.filter_size, self.filter_stride,
                              self.levels_below, input.features.device)
        if autograd.needs_grad(input.features, self.weight, bias):
            assert bn is None and pre_bn is None  # (the fused forms are inference-only; Sequential checks the same)
            output.features, macs = autograd.convolution(
                autograd.STRIDED, input.features, self.weight, bias.to(self.weight.device), input.metadata,
                input.spatial_size, out_size, self.filter_size, self.filter_stride)
        else:
            output.features = input.features.new_empty(0)
            with SCN.weight_token(self._weight_token()):
                macs = SCN.Convolution_updateOutput(
                    input.spatial_size, out_size, self.filter_size, self.filter_stride, input.metadata,
                    input.features.detach().contiguous(), output.features, self.weight, bias,
                    epilogue=bn.folded() if bn is not None else None,
                    prologue=pre_bn.folded() if pre_bn is not None else None)
        self._count(macs, output.features)
        return output

    def input_spatial_size(self, out_size):
        return (out_size - 1) * self.filter_stride + self.filter_size

    def __repr__(self):
        return "Convolution %d->%d C%s/%s" % (self.nIn, self.nOut, _size_str(self.filter_size),
                                              _size_str(self.filter_stride))


class Deconvolution(_ConvBase):
    def __init__(self, dimension, nIn, nOut, filter_size, filter_stride, bias, groups=1):
        Module.__init__(self)
        self._init_weight(dimension, nIn, nOut, filter_size, bias, groups)
        self.filter_stride = to_long_tensor(dimension, filter_stride)

    def forward(self, input, bn=None):
        assert input.features.nelement() == 0 or input.features.size(1) == self.nIn
        out_size = (input.spatial_size - 1) * self.filter_stride + self.filter_size
        output = SparseConvNetTensor(metadata=input.metadata, spatial_size=out_size)
        bias = optional_tensor(self, "bias")
        if autograd.needs_grad(input.features, self.weight, bias):
            output.features, macs = autograd.convolution(
                autograd.TRANSPOSED, input.features, self.weight, bias.to(self.weight.device), input.metadata,
                input.spatial_size, out_size, self.filter_size, self.filter_stride)
        else:
            output.features = input.features.new_empty(0)
            with SCN.weight_token(self._weight_token()):
                macs = SCN.Deconvolution_updateOutput(
                    input.spatial_size, out_size, self.filter_size, self.filter_stride, input.metadata,
                    input.features.detach().contiguous(), output.features, self.weight, bias,
                    epilogue=bn.folded() if bn is not None else None)
        self._count(macs, output.features)
        return output

    def input_spatial_size(self, out_size):
        return torch.div(out_size - self.filter_size, self.filter_stride, rounding_mode="trunc") + 1

    def __repr__(self):
        return "Deconvolution %d->%d C%s/%s" % (self.nIn, self.nOut, _size_str(self.filter_size),
                                                _size_str(self.filter_stride))


class BatchNormalization(Module):
    """Batch normalisation fused with a leaky ReLU: leakiness 1 = no activation, 0 = ReLU.
    eps 1e-4 and momentum 0.99 (weight of the OLD running value) are the reference's defaults
    (sparseconvnet/batchNormalization.py:24-30)."""

    def __init__(self, nPlanes, eps=1e-4, momentum=0.99, affine=True, leakiness=1):
        Module.__init__(self)
        self.nPlanes = nPlanes
        self.eps = eps
        self.momentum = momentum
        self.affine = affine
        self.leakiness = leakiness
        self.register_buffer("running_mean", torch.zeros(nPlanes))
        self.register_buffer("running_var", torch.ones(nPlanes))
        if affine:
            self.weight = Parameter(torch.ones(nPlanes))
            self.bias = Parameter(torch.zeros(nPlanes))

    def folded(self):
        """(scale, shift, leakiness) of this layer in eval mode, for a convolution that applies it in its
        store.  Kept until a parameter or running statistic changes (tensor version counters)."""
        tensors = (self.running_mean, self.running_var, getattr(self, "weight", None), getattr(self, "bias", None))
        key = tuple((t.data_ptr(), t._version) if t is not None else None for t in tensors) + (self.eps,)
        cached = getattr(self, "_folded", None)
        if cached is None or cached[0] != key:
            scale, shift = SCN.batchnorm_fold(self.running_mean, self.running_var, optional_tensor(self, "weight"),
                                              optional_tensor(self, "bias"), self.eps)
            cached = (key, scale, shift)
            self._folded = cached
        return cached[1], cached[2], self.leakiness

    def fusable(self, features):
        """True when a preceding convolution may apply this layer in its store: eval mode, no gradients
        wanted, statistics on the features' device."""
        return (not self.training and not autograd.needs_grad(features, optional_tensor(self, "weight"),
                                                              optional_tensor(self, "bias"))
                and self.running_mean.is_cuda and self.running_mean.device == features.device
                and not self._forward_hooks and not self._forward_pre_hooks)

    def forward_joined(self, inputs):
        """This layer (eval mode) applied to the concatenation of `inputs` (what a JoinTable in front of
        it would produce) without building the concatenation first."""
        assert sum(i.features.size(1) for i in inputs) == self.nPlanes
        features = SCN.batchnorm_concat([i.features.detach().contiguous() for i in inputs], self.running_mean,
                                        self.running_var, optional_tensor(self, "weight"),
                                        optional_tensor(self, "bias"), self.eps, self.leakiness)
        if features is None:  # shapes the fused kernel does not take
            return None
        output = SparseConvNetTensor(metadata=inputs[0].metadata, spatial_size=inputs[0].spatial_size)
        output.features = features
        return output

    # Data-parallel training: with `across_ranks` the training-mode statistics cover the rows of every rank of
    # `ranks_group` (shard.share_batchnorm_statistics sets both on all layers of a network).
    across_ranks = False
    ranks_group = None

    def _shares_statistics(self):
        if not (self.training and self.across_ranks):
            return False
        import torch.distributed as dist
        return dist.is_available() and dist.is_initialized() and dist.get_world_size(self.ranks_group) > 1

    def forward(self, input):
        if self._shares_statistics():  # a rank without rows still takes part in the exchange
            features = input.features
            if features.dim() != 2:
                features = features.new_zeros(0, self.nPlanes)
            assert features.size(1) == self.nPlanes, (self.nPlanes, features.shape)
            output = SparseConvNetTensor(metadata=input.metadata, spatial_size=input.spatial_size)
            dev = features.device
            output.features = autograd.batchnorm_across_ranks(
                features, optional_tensor(self, "weight").to(dev), optional_tensor(self, "bias").to(dev),
                self.running_mean, self.running_var, self.eps, self.momentum, self.leakiness, self.ranks_group)
            return output
        if input.features.nelement() == 0:
            return input
        assert input.features.size(1) == self.nPlanes, (self.nPlanes, input.features.shape)
        output = SparseConvNetTensor(metadata=input.metadata, spatial_size=input.spatial_size)
        weight, bias = optional_tensor(self, "weight"), optional_tensor(self, "bias")
        if autograd.needs_grad(input.features, weight, bias):
            dev = input.features.device
            output.features = autograd.batchnorm(input.features, weight.to(dev), bias.to(dev), self.running_mean,
                                                 self.running_var, self.eps, self.momentum, self.training,
                                                 self.leakiness)
            return output
        output.features = input.features.new_empty(0)
        save_mean = input.features.new_empty(self.nPlanes)
        save_invstd = input.features.new_empty(self.nPlanes)
        SCN.BatchNormalization_updateOutput(
            input.features.detach(), output.features, save_mean, save_invstd, self.running_mean,
            self.running_var, optional_tensor(self, "weight"), optional_tensor(self, "bias"), self.eps,
            self.momentum, self.training, self.leakiness)
        return output

    def input_spatial_size(self, out_size):
        return out_size

    def __repr__(self):
        s = "BatchNorm(%d,eps=%g,momentum=%g,affine=%s" % (self.nPlanes, self.eps, self.momentum, self.affine)
        if self.leakiness > 0:
            s += ",leakiness=%g" % self.leakiness
        return s + ")"


class BatchNormReLU(BatchNormalization):
    def __init__(self, nPlanes, eps=1e-4, momentum=0.99):
        BatchNormalization.__init__(self, nPlanes, eps, momentum, True, 0)

    def __repr__(self):
        return "BatchNormReLU(%d,eps=%g,momentum=%g,affine=%s)" % (self.nPlanes, self.eps, self.momentum,
                                                                   self.affine)


class BatchNormLeakyReLU(BatchNormalization):
    def __init__(self, nPlanes, eps=1e-4, momentum=0.99, leakiness=0.333):
        BatchNormalization.__init__(self, nPlanes, eps, momentum, True, leakiness)

    def __repr__(self):
        return "BatchNormLeakyReLU(%d,eps=%g,momentum=%g,affine=%s,leakiness=%g)" % (
            self.nPlanes, self.eps, self.momentum, self.affine, self.leakiness)


class MaxPooling(Module):
    def __init__(self, dimension, pool_size, pool_stride, nFeaturesToDrop=0):
        Module.__init__(self)
        self.dimension = dimension
        self.pool_size = to_long_tensor(dimension, pool_size)
        self.pool_stride = to_long_tensor(dimension, pool_stride)
        self.nFeaturesToDrop = nFeaturesToDrop

    def forward(self, input):
        out_size = torch.div(input.spatial_size - self.pool_size, self.pool_stride, rounding_mode="trunc") + 1
        assert ((out_size - 1) * self.pool_stride + self.pool_size == input.spatial_size).all()
        output = SparseConvNetTensor(metadata=input.metadata, spatial_size=out_size)
        if autograd.needs_grad(input.features):
            output.features = autograd.pooling("max", input.features, input.metadata, input.spatial_size, out_size,
                                               self.pool_size, self.pool_stride, self.nFeaturesToDrop)
            return output
        output.features = input.features.new_empty(0)
        SCN.MaxPooling_updateOutput(input.spatial_size, out_size, self.pool_size, self.pool_stride,
                                    input.metadata, input.features.detach().contiguous(), output.features,
                                    self.nFeaturesToDrop)
        return output

    def input_spatial_size(self, out_size):
        return (out_size - 1) * self.pool_stride + self.pool_size

    def __repr__(self):
        return "MaxPooling%s/%s" % (_size_str(self.pool_size), _size_str(self.pool_stride))


class AveragePooling(Module):
    """averagePooling.py: like MaxPooling, but every output site gets the sum of its inputs divided
    by the pool volume (not by the number of active inputs)."""

    def __init__(self, dimension, pool_size, pool_stride, nFeaturesToDrop=0):
        Module.__init__(self)
        self.dimension = dimension
        self.pool_size = to_long_tensor(dimension, pool_size)
        self.pool_stride = to_long_tensor(dimension, pool_stride)
        self.nFeaturesToDrop = nFeaturesToDrop

    def forward(self, input):
        out_size = torch.div(input.spatial_size - self.pool_size, self.pool_stride, rounding_mode="trunc") + 1
        assert ((out_size - 1) * self.pool_stride + self.pool_size == input.spatial_size).all()
        output = SparseConvNetTensor(metadata=input.metadata, spatial_size=out_size)
        if autograd.needs_grad(input.features):
            output.features = autograd.pooling("avg", input.features, input.metadata, input.spatial_size, out_size,
                                               self.pool_size, self.pool_stride, self.nFeaturesToDrop)
            return output
        output.features = input.features.new_empty(0)
        SCN.AveragePooling_updateOutput(input.spatial_size, out_size, self.pool_size, self.pool_stride,
                                        input.metadata, input.features.detach().contiguous(), output.features,
                                        self.nFeaturesToDrop)
        return output

    def input_spatial_size(self, out_size):
        return (out_size - 1) * self.pool_stride + self.pool_size

    def __repr__(self):
        return "AveragePooling%s/%s" % (_size_str(self.pool_size), _size_str(self.pool_stride))


class UnPooling(Module):
    """unPooling.py: the inverse geometry of a pooling layer -- every site of the fine scale (which
    must already exist in the metadata) gets the sum of the coarse sites whose window holds it."""

    def __init__(self, dimension, pool_size, pool_stride, nFeaturesToDrop=0):
        Module.__init__(self)
        self.dimension = dimension
        self.pool_size = to_long_tensor(dimension, pool_size)
        self.pool_stride = to_long_tensor(dimension, pool_stride)
        self.nFeaturesToDrop = nFeaturesToDrop

    def forward(self, input):
        out_size = (input.spatial_size - 1) * self.pool_stride + self.pool_size
        output = SparseConvNetTensor(metadata=input.metadata, spatial_size=out_size)
        if autograd.needs_grad(input.features):
            output.features = autograd.pooling("unpool", input.features, input.metadata, input.spatial_size, out_size,
                                               self.pool_size, self.pool_stride, self.nFeaturesToDrop)
            return output
        output.features = input.features.new_empty(0)
        SCN.UnPooling_updateOutput(input.spatial_size, out_size, self.pool_size, self.pool_stride,
                                   input.metadata, input.features.detach().contiguous(), output.features,
                                   self.nFeaturesToDrop)
        return output

    def input_spatial_size(self, out_size):
        return torch.div(out_size - self.pool_size, self.pool_stride, rounding_mode="trunc") + 1

    def __repr__(self):
        return "UnPooling%s/%s" % (_size_str(self.pool_size), _size_str(self.pool_stride))


class SparseToDense(Module):
    """SparseConvNetTensor -> dense tensor [batch, nPlanes, *spatial_size]."""

    def __init__(self, dimension, nPlanes):
        Module.__init__(self)
        self.dimension = dimension
        self.nPlanes = nPlanes

    def forward(self, input):
        if autograd.needs_grad(input.features):
            return autograd.sparse_to_dense(input.features, input.metadata, input.spatial_size, self.nPlanes)
        output = input.features.new_empty(0)
        SCN.SparseToDense_updateOutput(input.spatial_size, input.metadata,
                                       input.features.detach().contiguous(), output, self.nPlanes)
        return output

    def input_spatial_size(self, out_size):
        return out_size

    def __repr__(self):
        return "SparseToDense(%d,%d)" % (self.dimension, self.nPlanes)


class NetworkInNetwork(Module):
    """1x1 convolution; weight [nIn, nOut] (reference: sparseconvnet/networkInNetwork.py)."""

    def __init__(self, nIn, nOut, bias):
        Module.__init__(self)
        self.nIn = nIn
        self.nOut = nOut
        std = (2.0 / nIn) ** 0.5
        self.weight = Parameter(torch.empty(nIn, nOut).normal_(0, std))
        if bias:
            self.bias = Parameter(torch.zeros(nOut))

    def forward(self, input):
        assert input.features.nelement() == 0 or input.features.size(1) == self.nIn
        output = SparseConvNetTensor(metadata=input.metadata, spatial_size=input.spatial_size)
        if autograd.needs_grad(input.features, self.weight):
            # a dense matrix product: torch's own autograd covers it (the reference calls addmm as well)
            output.features = input.features @ self.weight
            if hasattr(self, "bias"):
                output.features = output.features + self.bias
            macs = float(input.features.size(0) * self.nIn * self.nOut)
            SCN.flop_counter.add(macs)
            _pkg.forward_pass_hidden_states += output.features.nelement()
            return output
        output.features = input.features.new_empty(0)
        macs = SCN.NetworkInNetwork_updateOutput(input.features.detach().contiguous(), output.features,
                                                 self.weight, optional_tensor(self, "bias"))
        SCN.flop_counter.add(macs)
        _pkg.forward_pass_hidden_states += output.features.nelement()
        return output

    def input_spatial_size(self, out_size):
        return out_size

    def __repr__(self):
        return "NetworkInNetwork%d->%d" % (self.nIn, self.nOut)


class Identity(Module):
    def forward(self, input):
        return input

    def input_spatial_size(self, out_size):
        return out_size
