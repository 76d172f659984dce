"""Pooling / upsampling modules (reference: nn/modules/spatial.py:23-217): same constructor arguments,
attributes and error text; forward delegates to the functional forms."""
from torch import nn

from sparsetriton_b200.nn.functional.spatial import sparse_pooling, sparse_upsample
from sparsetriton_b200.tensor import SparseTensor

__all__ = ["SparsePooling", "SparseUpsample", "SparseDownsample"]


class SparsePooling(nn.Module):
    def __init__(self, kernel_size, mode="avg", stride=1, padding=0):
        super().__init__()
        if mode not in ("avg", "max"):
            raise ValueError(f"mode must be 'avg' or 'max', got '{mode}'")
        self.kernel_size, self.stride, self.mode, self.padding = kernel_size, stride, mode, padding

    def forward(self, x: SparseTensor) -> SparseTensor:
        return sparse_pooling(x, self.kernel_size, self.padding, self.stride, self.mode)


class SparseUpsample(nn.Module):
    def __init__(self, scale_factor=None):
        super().__init__()
        self.scale_factor = scale_factor

    def forward(self, input: SparseTensor) -> SparseTensor:
        return sparse_upsample(input, self.scale_factor)


class SparseDownsample(SparsePooling):
    """Pooling with kernel_size = stride = scale_factor and no padding."""

    def __init__(self, scale_factor=None, mode="max"):
        super().__init__(kernel_size=scale_factor, stride=scale_factor, mode=mode, padding=0)
