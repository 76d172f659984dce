from .conv import ConvPreparation, compute_neighbor_indices, prepare_conv3d, sparse_conv3d
from .kmap import build_out_coords

__all__ = ["sparse_conv3d", "prepare_conv3d", "ConvPreparation", "compute_neighbor_indices", "build_out_coords"]
