"""sparseconvnet_b200: the inference path of SparseConvNet (InputLayer, SubmanifoldConvolution,
Convolution, Deconvolution, BatchNormReLU, MaxPooling, SparseToDense and the Metadata object)
on sm_100a, with the reference package's module API:

    import sparseconvnet_b200 as scn
    model = scn.Sequential().add(scn.SubmanifoldConvolution(3, 3, 32, 3, False)).add(...)

All compute runs in ``libscn_b200.so`` (C ABI in ``include/scn_b200.h``); there is no CPU path.
"""
import sys as _sys
import types as _types

forward_pass_hidden_states = 0

from . import SCN  # noqa: E402  (loads libscn_b200.so; fails loudly if it is missing)
from .SCN import set_precision, get_precision, set_backward_precision, get_backward_precision  # noqa: E402
from .sparse_tensor import SparseConvNetTensor, to_long_tensor as toLongTensor  # noqa: E402


class _Package(_types.ModuleType):
    """``forward_pass_multiplyAdd_count`` (reference: sparseconvnet/__init__.py) is read and reset
    like the reference's module attribute; reading it folds in the counts of convolutions whose
    rule totals were still travelling to the host when they returned (SCN.DeferredCount)."""

    @property
    def forward_pass_multiplyAdd_count(self):
        return SCN.flop_counter.value()

    @forward_pass_multiplyAdd_count.setter
    def forward_pass_multiplyAdd_count(self, value):
        SCN.flop_counter.reset(value)


_sys.modules[__name__].__class__ = _Package


def Metadata(dim):
    """A fresh Metadata object for `dim` spatial dimensions (reference: sparseconvnet/metadata.py:16-17)."""
    return getattr(SCN, "Metadata_%d" % dim)()


from .layers import (InputLayer, OutputLayer, BLInputLayer, BLOutputLayer, SubmanifoldConvolution, ValidConvolution, Convolution,  # noqa: E402
                     Deconvolution, BatchNormalization, BatchNormReLU, BatchNormLeakyReLU, MaxPooling, AveragePooling, UnPooling,
                     SparseToDense, NetworkInNetwork, Identity)
from .containers import Sequential, ConcatTable, JoinTable, AddTable  # noqa: E402
from .architectures import SparseVggNet, SparseResNet, UNet, FullyConvolutionalNet  # noqa: E402
