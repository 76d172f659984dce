"""Functional API (reference: sparsetriton/nn/functional/__init__.py)."""
from . import conv
from .conv import ConvPreparation, prepare_conv3d, sparse_conv3d
from .norm import sparse_batch_norm
from .spatial import sparse_pooling, sparse_upsample

__all__ = ["conv", "sparse_conv3d", "prepare_conv3d", "ConvPreparation", "sparse_batch_norm", "sparse_pooling", "sparse_upsample"]
