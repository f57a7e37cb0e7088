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


def _keeps_sites(m):
    """True for a module whose output has the sites and the spatial size of its input."""
    from . import layers
    if isinstance(m, (layers.SubmanifoldConvolution, layers.BatchNormalization, layers.Identity, layers.NetworkInNetwork,
                      AddTable, JoinTable)):
        return True
    if type(m) is Sequential:
        return all(_keeps_sites(c) for c in m._modules.values())
    if type(m) is ConcatTable:
        return all(_keeps_sites(c) for c in m._modules.values())
    return False


def _chain_ahead(steps):
    """The first downsampling Convolution that announces further levels (``levels_below > 1``) and is reached
    from the start of `steps` through modules that keep the sites and the spatial size -- so that its input grid
    is the grid of the tensor that enters `steps` -- looking into the branches of a ConcatTable.  None if there
    is none."""
    from . import layers
    for m in steps:
        if isinstance(m, layers.Convolution):
            return m if m.levels_below > 1 else None
        if type(m) is ConcatTable:
            for branch in m._modules.values():
                found = _chain_ahead(_flatten(branch, []) if type(branch) is Sequential else [branch])
                if found is not None:
                    return found
        if not _keeps_sites(m):
            return None
    return None


class Sequential(torch.nn.Sequential):
    """Runs its children in order, like the reference's container.  Peepholes (inference only, same
    arithmetic and the same bits as the separate layers; `Sequential.fuse = False` turns them off):
    a convolution whose output goes straight into an eval-mode BatchNormalization (possibly across
    the boundary of a nested Sequential, as in the U-Net's blocks) applies that layer's scale, shift
    and leaky ReLU in its own store; an eval-mode BatchNormalization in front of a strided Convolution
    is applied by that convolution to its input; JoinTable -> BatchNormalization ->
    SubmanifoldConvolution is one call on the tensors that would have been joined; a JoinTable
    followed by a BatchNormalization alone is one pass without the concatenation.

    And one look ahead (`Sequential.prefetch_rulebooks = False` turns it off): the first Sequential that sees a
    tensor of a new Metadata looks for the encoder's first downsampling Convolution behind the layers that keep
    the sites (the builders mark it with the number of levels below it) and has the grids and rulebooks of all
    those levels started on the library's side stream (SCN.strided_chain_start).  They are built while the
    layers of the finest level run, and the Convolution, when its turn comes, finds them finished instead of
    building them and waiting with an empty stream."""
    fuse = True
    prefetch_rulebooks = True

    def forward(self, input):
        from . import layers
        steps = _flatten(self, [])
        if (Sequential.prefetch_rulebooks and isinstance(input, SparseConvNetTensor) and input.features.is_cuda
                and not getattr(input.metadata, "chain_looked_for", True)):
            input.metadata.chain_looked_for = True  # one look per Metadata, by the outermost container
            conv = _chain_ahead(steps)
            if conv is not None:
                layers.SCN.strided_chain_start(input.metadata, input.spatial_size, conv.filter_size, conv.filter_stride,
                                               conv.levels_below, input.features.device)
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
            # an eval-mode BatchNormalization whose result goes straight into a strided Convolution (the way down of a
            # U-Net): the convolution normalises its input itself (in the pass that splits the rows for the tensor
            # core, where there is one) -- and the BatchNormalization behind it rides in its store as above
            nxt2 = steps[i + 2] if i + 2 < n else None
            if (Sequential.fuse and isinstance(m, layers.BatchNormalization) and type(nxt) is layers.Convolution
                    and not m._forward_hooks and not m._forward_pre_hooks and not nxt._forward_hooks
                    and not nxt._forward_pre_hooks and isinstance(input, SparseConvNetTensor)
                    and input.features.nelement() > 0 and m.fusable(input.features)
                    and not layers.autograd.needs_grad(input.features, nxt.weight, getattr(nxt, "bias", None))):
                post = nxt2 if (isinstance(nxt2, layers.BatchNormalization) and nxt2.fusable(input.features)) else None
                input = nxt.forward(input, bn=post, pre_bn=m)
                i += 3 if post is not None else 2
                continue
            # JoinTable -> eval-mode BatchNormalization -> SubmanifoldConvolution (-> BatchNormalization): the layers
            # behind the skip connection of a U-Net as one call; the convolution reads the joined tensors where they
            # lie (in the pass that splits its rows for the tensor core, where the kernel has one)
            if (Sequential.fuse and type(m) is JoinTable and isinstance(nxt, layers.BatchNormalization)
                    and type(nxt2) is layers.SubmanifoldConvolution and not m._forward_hooks and not m._forward_pre_hooks
                    and not nxt2._forward_hooks and not nxt2._forward_pre_hooks and isinstance(input, (list, tuple))
                    and len(input) == 2 and all(t.features.nelement() > 0 and t.features.dim() == 2 for t in input)
                    and nxt.fusable(input[0].features) and nxt2.groups == 1
                    and not any(layers.autograd.needs_grad(t.features) for t in input)
                    and not layers.autograd.needs_grad(input[0].features, nxt2.weight, getattr(nxt2, "bias", None))):
                nxt3 = steps[i + 3] if i + 3 < n else None
                post = nxt3 if (isinstance(nxt3, layers.BatchNormalization) and nxt3.fusable(input[0].features)) else None
                joined = nxt2.forward_joined(input, pre_bn=nxt, bn=post)
                if joined is not None:
                    input = joined
                    i += 4 if post is not None else 3
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
