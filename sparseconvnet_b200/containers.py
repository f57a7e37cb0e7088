"""Containers (reference: sparseconvnet/sequential.py:10-33, sparseconvnet/tables.py:13-55)."""
import torch

from .sparse_tensor import SparseConvNetTensor


def _flatten(seq, out):
    """The leaf steps of a Sequential in execution order: nested Sequentials without hooks are expanded."""
    for m in seq._modules.values():
        if type(m) is Sequential and not m._forward_hooks and not m._forward_pre_hooks:
            _flatten(m, out)
        else:
            out.append(m)
    return out


class Sequential(torch.nn.Sequential):
    """Runs its children in order, like the reference's container.  One peephole: a convolution whose
    output goes straight into an eval-mode BatchNormalization (possibly across the boundary of a
    nested Sequential, as in the U-Net's blocks) applies that layer's scale, shift and leaky ReLU in
    its own store -- same arithmetic, one pass over the activation less.  `Sequential.fuse = False`
    turns it off."""
    fuse = True

    def forward(self, input):
        from . import layers
        steps = _flatten(self, [])
        i, n = 0, len(steps)
        while i < n:
            m = steps[i]
            nxt = steps[i + 1] if i + 1 < n else None
            if (Sequential.fuse and isinstance(m, layers._ConvBase) and isinstance(nxt, layers.BatchNormalization)
                    and not m._forward_hooks and not m._forward_pre_hooks
                    and input.features.nelement() > 0 and nxt.fusable(input.features)
                    and not layers.autograd.needs_grad(input.features, m.weight)):
                input = m.forward(input, bn=nxt)  # (no output rows: nothing to apply, as the BatchNorm itself)
                i += 2
                continue
            # a JoinTable whose result goes straight into an eval-mode BatchNormalization: every joined tensor is
            # normalised into its columns of the result, the concatenation itself is never written
            if (Sequential.fuse and type(m) is JoinTable and isinstance(nxt, layers.BatchNormalization)
                    and not m._forward_hooks and not m._forward_pre_hooks and isinstance(input, (list, tuple))
                    and len(input) > 0 and all(t.features.nelement() > 0 and t.features.dim() == 2 for t in input)
                    and nxt.fusable(input[0].features)
                    and not any(layers.autograd.needs_grad(t.features) for t in input)):
                joined = nxt.forward_joined(input)
                if joined is not None:
                    input = joined
                    i += 2
                    continue
            input = m(input)
            i += 1
        return input

    def input_spatial_size(self, out_size):
        for name in reversed(list(self._modules)):
            out_size = self._modules[name].input_spatial_size(out_size)
        return out_size

    def add(self, module):
        self._modules[str(len(self._modules))] = module
        return self

    def append(self, module):
        return self.add(module)

    def insert(self, index, module):
        for i in range(len(self._modules), index, -1):
            self._modules[str(i)] = self._modules[str(i - 1)]
        self._modules[str(index)] = module

    def __add__(self, other):
        r = Sequential()
        for m in self:
            r.add(m)
        for m in other:
            r.add(m)
        return r


class ConcatTable(torch.nn.Sequential):
    """Feeds one input to every child; returns the list of outputs."""

    def forward(self, input):
        return [module(input) for module in self._modules.values()]

    def add(self, module):
        self._modules[str(len(self._modules))] = module
        return self

    def input_spatial_size(self, out_size):
        return self._modules["0"].input_spatial_size(out_size)


class JoinTable(torch.nn.Sequential):
    """Concatenates the feature planes of a list of tensors that share one set of sites."""

    def forward(self, input):
        output = SparseConvNetTensor(metadata=input[0].metadata, spatial_size=input[0].spatial_size)
        if input[0].features.numel():
            output.features = torch.cat([i.features for i in input], 1)
        else:
            output.features = input[0].features
        return output

    def input_spatial_size(self, out_size):
        return out_size


class AddTable(torch.nn.Sequential):
    """Sums the features of a list of tensors that share one set of sites."""

    def forward(self, input):
        output = SparseConvNetTensor(metadata=input[0].metadata, spatial_size=input[0].spatial_size)
        output.features = sum([i.features for i in input])
        return output

    def input_spatial_size(self, out_size):
        return out_size
