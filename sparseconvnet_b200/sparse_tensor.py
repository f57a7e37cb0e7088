"""``SparseConvNetTensor``: features + shared Metadata + spatial size
(reference: sparseconvnet/sparseConvNetTensor.py:12-16)."""
import torch


def to_long_tensor(dimension, x):
    """Spatial sizes / filter sizes / strides travel as CPU LongTensors of length `dimension`
    (reference: sparseconvnet/utils.py:12-19)."""
    if isinstance(x, torch.Tensor):
        if x.dtype == torch.int64 and not x.is_cuda:
            return x
        return x.to("cpu", torch.int64)
    if isinstance(x, (list, tuple)):
        assert len(x) == dimension, (dimension, x)
        return torch.tensor([int(v) for v in x], dtype=torch.int64)
    return torch.full((dimension,), int(x), dtype=torch.int64)


def optional_tensor(module, name):
    """Absent parameters are passed as 0-element tensors (reference: utils.py:21-22)."""
    t = getattr(module, name, None)
    return t if t is not None else torch.empty(0)


class SparseConvNetTensor(object):
    def __init__(self, features=None, metadata=None, spatial_size=None):
        self.features = features
        self.metadata = metadata
        self.spatial_size = spatial_size

    def get_spatial_locations(self, spatial_size=None):
        """LongTensor [nActive, dimension+1]: coordinates and batch index of every feature row."""
        if spatial_size is None:
            spatial_size = self.spatial_size
        return self.metadata.getSpatialLocations(spatial_size)

    def batch_size(self):
        return self.metadata.getBatchSize(self.spatial_size)

    def to(self, device):
        self.features = self.features.to(device)
        return self

    def type(self, t=None):
        if t:
            self.features = self.features.type(t)
            return self
        return self.features.type()

    def cuda(self):
        self.features = self.features.cuda()
        return self

    def cpu(self):
        self.features = self.features.cpu()
        return self

    def detach(self):
        return SparseConvNetTensor(self.features.detach(), self.metadata, self.spatial_size)

    @property
    def requires_grad(self):
        return self.features.requires_grad

    def __repr__(self):
        shape = tuple(self.features.shape) if self.features is not None else None
        size = self.spatial_size.tolist() if self.spatial_size is not None else None
        return "SparseConvNetTensor<<features.shape=%r, spatial size=%r>>" % (shape, size)
