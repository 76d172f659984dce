from .conv import SparseConv3D, SparseConvTransposed3D, SubMConv3D
from .norm import SparseBatchNorm
from .simple import ReLU, SparseLinear
from .spatial import SparseDownsample, SparsePooling, SparseUpsample

__all__ = ["SparseConv3D", "SubMConv3D", "SparseConvTransposed3D", "SparseBatchNorm", "SparseLinear", "ReLU",
           "SparsePooling", "SparseUpsample", "SparseDownsample"]
