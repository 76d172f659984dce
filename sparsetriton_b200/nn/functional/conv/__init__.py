from .conv import compute_neighbor_indices, sparse_conv3d
from .kmap import build_out_coords

__all__ = ["sparse_conv3d", "compute_neighbor_indices", "build_out_coords"]
