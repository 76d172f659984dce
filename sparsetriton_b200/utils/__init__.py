"""Helpers of the sparse-convolution path (reference: sparsetriton/utils/__init__.py)."""
from .hash import HashTable
from .to_dense import to_dense
from .utils import make_ntuple

__all__ = ["HashTable", "to_dense", "make_ntuple"]
