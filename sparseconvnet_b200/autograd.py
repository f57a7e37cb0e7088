"""torch.autograd wiring of the operators that have a backward pass in the library (training).

The modules in ``layers.py`` call the C ABI directly when no gradient is wanted (inference, the
measured path); when gradients are enabled and an input or a parameter requires them, they go
through the Functions here, which save what the backward entry points need.  The reference does the
same with one Function per operator (e.g. submanifoldConvolution.py:62-113)."""
import torch

from . import SCN

SUBMANIFOLD, STRIDED, TRANSPOSED = 0, 1, 2


def needs_grad(*tensors):
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)


class _Convolution(torch.autograd.Function):
    """features, weight, bias (0-element tensor = none) -> output features; `info` is a dict that
    receives the multiply-add count of the forward pass."""

    @staticmethod
    def forward(ctx, features, weight, bias, kind, metadata, in_size, out_size, filter_size, filter_stride, info):
        features = features.contiguous()
        out = features.new_empty(0)
        if kind == SUBMANIFOLD:
            macs = SCN.SubmanifoldConvolution_updateOutput(in_size, filter_size, metadata, features, out, weight, bias)
        elif kind == STRIDED:
            macs = SCN.Convolution_updateOutput(in_size, out_size, filter_size, filter_stride, metadata, features, out,
                                                weight, bias)
        else:
            macs = SCN.Deconvolution_updateOutput(in_size, out_size, filter_size, filter_stride, metadata, features,
                                                  out, weight, bias)
        info["macs"] = macs
        ctx.save_for_backward(features, weight, bias)
        ctx.args = (kind, metadata, in_size, out_size, filter_size, filter_stride)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        features, weight, bias = ctx.saved_tensors
        kind, metadata, in_size, out_size, filter_size, filter_stride = ctx.args
        grad_out = grad_out.contiguous()
        d_in = grad_out.new_empty(0)
        d_w = torch.empty_like(weight)
        d_b = torch.empty_like(bias) if bias.numel() else None
        w = weight.detach()
        if kind == SUBMANIFOLD:
            SCN.SubmanifoldConvolution_backward(in_size, filter_size, metadata, features, d_in, grad_out, w, d_w, d_b)
        elif kind == STRIDED:
            SCN.Convolution_backward(in_size, out_size, filter_size, filter_stride, metadata, features, d_in, grad_out,
                                     w, d_w, d_b)
        else:
            SCN.Deconvolution_backward(in_size, out_size, filter_size, filter_stride, metadata, features, d_in,
                                       grad_out, w, d_w, d_b)
        return d_in, d_w, d_b, None, None, None, None, None, None, None


def convolution(kind, features, weight, bias, metadata, in_size, out_size, filter_size, filter_stride):
    """Returns (output features, multiply-add count)."""
    info = {}
    out = _Convolution.apply(features, weight, bias, kind, metadata, in_size, out_size, filter_size, filter_stride,
                             info)
    return out, info["macs"]


class _BatchNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, features, weight, bias, running_mean, running_var, eps, momentum, train, leakiness):
        features = features.contiguous()
        out = features.new_empty(0)
        save_mean = features.new_empty(features.size(1))
        save_invstd = features.new_empty(features.size(1))
        SCN.BatchNormalization_updateOutput(features, out, save_mean, save_invstd, running_mean, running_var, weight,
                                            bias, eps, momentum, train, leakiness)
        ctx.save_for_backward(features, out, weight, bias, save_mean, save_invstd)
        ctx.leakiness = leakiness
        return out

    @staticmethod
    def backward(ctx, grad_out):
        features, out, weight, bias, save_mean, save_invstd = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        d_in = grad_out.new_empty(0)
        affine = weight.numel() > 0
        d_w = torch.empty_like(weight) if affine else None
        d_b = torch.empty_like(bias) if affine else None
        SCN.BatchNormalization_backward(features, d_in, out, grad_out, save_mean, save_invstd, None, None,
                                        weight.detach(), bias.detach(), d_w, d_b, ctx.leakiness)
        return d_in, d_w, d_b, None, None, None, None, None, None


def batchnorm(features, weight, bias, running_mean, running_var, eps, momentum, train, leakiness):
    return _BatchNorm.apply(features, weight, bias, running_mean, running_var, eps, momentum, train, leakiness)


class _BatchNormAcrossRanks(torch.autograd.Function):
    """Training-mode BatchNorm whose statistics cover the rows of every rank of a process group (data-parallel
    training): one small all-reduce in the forward pass, one in the backward pass."""

    @staticmethod
    def forward(ctx, features, weight, bias, running_mean, running_var, eps, momentum, leakiness, group):
        features = features.contiguous()
        out = features.new_empty(0)
        save_mean = features.new_empty(features.size(1))
        save_invstd = features.new_empty(features.size(1))
        sums = SCN.BatchNormalization_updateOutput_acrossRanks(features, out, save_mean, save_invstd, running_mean,
                                                               running_var, weight, bias, eps, momentum, leakiness,
                                                               group)
        ctx.save_for_backward(features, out, weight, bias, save_mean, save_invstd, sums)
        ctx.leakiness, ctx.group = leakiness, group
        return out

    @staticmethod
    def backward(ctx, grad_out):
        features, out, weight, bias, save_mean, save_invstd, sums = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        d_in = grad_out.new_empty(0)
        affine = weight.numel() > 0
        d_w = torch.empty_like(weight) if affine else None
        d_b = torch.empty_like(bias) if affine else None
        SCN.BatchNormalization_backward_acrossRanks(features, d_in, out, grad_out, save_mean, save_invstd,
                                                    weight.detach(), d_w, d_b, ctx.leakiness, sums, ctx.group)
        return d_in, d_w, d_b, None, None, None, None, None, None


def batchnorm_across_ranks(features, weight, bias, running_mean, running_var, eps, momentum, leakiness, group):
    return _BatchNormAcrossRanks.apply(features, weight, bias, running_mean, running_var, eps, momentum, leakiness,
                                       group)


class _Pooling(torch.autograd.Function):
    """kind: 'max' | 'avg' | 'unpool'."""

    @staticmethod
    def forward(ctx, features, kind, metadata, in_size, out_size, pool_size, pool_stride, drop):
        features = features.contiguous()
        out = features.new_empty(0)
        fn = {"max": SCN.MaxPooling_updateOutput, "avg": SCN.AveragePooling_updateOutput,
              "unpool": SCN.UnPooling_updateOutput}[kind]
        fn(in_size, out_size, pool_size, pool_stride, metadata, features, out, drop)
        ctx.save_for_backward(features, out)
        ctx.args = (kind, metadata, in_size, out_size, pool_size, pool_stride, drop)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        features, out = ctx.saved_tensors
        kind, metadata, in_size, out_size, pool_size, pool_stride, drop = ctx.args
        grad_out = grad_out.contiguous()
        d_in = torch.empty_like(features)
        if kind == "max":
            SCN.MaxPooling_updateGradInput(in_size, out_size, pool_size, pool_stride, metadata, features, d_in, out,
                                           grad_out, drop)
        elif kind == "avg":
            SCN.AveragePooling_updateGradInput(in_size, out_size, pool_size, pool_stride, metadata, features, d_in,
                                               grad_out, drop)
        else:
            SCN.UnPooling_updateGradInput(in_size, out_size, pool_size, pool_stride, metadata, d_in, grad_out, drop)
        return d_in, None, None, None, None, None, None, None


def pooling(kind, features, metadata, in_size, out_size, pool_size, pool_stride, drop):
    return _Pooling.apply(features, kind, metadata, in_size, out_size, pool_size, pool_stride, drop)


class _SparseToDense(torch.autograd.Function):
    @staticmethod
    def forward(ctx, features, metadata, spatial_size, n_planes):
        features = features.contiguous()
        out = features.new_empty(0)
        SCN.SparseToDense_updateOutput(spatial_size, metadata, features, out, n_planes)
        ctx.save_for_backward(features)
        ctx.args = (metadata, spatial_size)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (features,) = ctx.saved_tensors
        metadata, spatial_size = ctx.args
        d_in = torch.empty_like(features)
        SCN.SparseToDense_updateGradInput(spatial_size, metadata, features, d_in, grad_out.contiguous())
        return d_in, None, None, None


def sparse_to_dense(features, metadata, spatial_size, n_planes):
    return _SparseToDense.apply(features, metadata, spatial_size, n_planes)


class _InputFeatures(torch.autograd.Function):
    """The feature pass of InputLayer / BLInputLayer (the metadata is built before, outside autograd)."""

    @staticmethod
    def forward(ctx, features, metadata, run):
        out = run(features.contiguous())
        ctx.md, ctx.in_shape = metadata, features.shape
        return out

    @staticmethod
    def backward(ctx, grad_out):
        d_in = grad_out.new_empty(0)
        SCN.InputLayer_updateGradInput(ctx.md, d_in, grad_out.contiguous())
        return d_in.view(ctx.in_shape), None, None


def input_features(features, metadata, run):
    return _InputFeatures.apply(features, metadata, run)


class _OutputFeatures(torch.autograd.Function):
    @staticmethod
    def forward(ctx, features, metadata, bl):
        features = features.contiguous()
        out = features.new_empty(0)
        (SCN.BLOutputLayer_updateOutput if bl else SCN.OutputLayer_updateOutput)(metadata, features, out)
        ctx.md, ctx.in_shape = metadata, features.shape
        return out

    @staticmethod
    def backward(ctx, grad_out):
        d_in = grad_out.new_empty(ctx.in_shape)
        SCN.OutputLayer_updateGradInput(ctx.md, d_in, grad_out.contiguous())
        return d_in, None, None


def output_features(features, metadata, bl):
    return _OutputFeatures.apply(features, metadata, bl)
