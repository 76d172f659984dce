"""B200-native sparse-convolution hot path behind the Python surface of ptj0225/SparseTriton.

    from sparsetriton_b200 import SparseTensor, randn, nn
    from sparsetriton_b200.config import set_conv_algo, ConvAlgo

Every kernel is hand-written CUDA for sm_100a in libsparsetriton_b200.so (C ABI declared in
include/sparsetriton_b200.h); there is no Triton and no CPU fallback.  To run code written
against the reference's import path, call `sparsetriton_b200.compat.install()` first.
"""
from .tensor import SparseTensor, randn
from . import nn

__all__ = ["SparseTensor", "randn", "nn"]
