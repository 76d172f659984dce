"""Convolution layers over SparseTensor (reference: nn/modules/conv.py:31-365).

Parameter names, shapes and initialisation match the reference so its state_dicts load:
weight (K, C_in, C_out) with K = kx*ky*kz ordered x-major, bias (C_out,), both drawn from
U(-1/sqrt(C_in*K), +1/sqrt(C_in*K)).
"""
import math

import torch
from torch import nn

from sparsetriton_b200.nn import functional as F
from sparsetriton_b200.tensor import SparseTensor
from sparsetriton_b200.utils.utils import make_ntuple

__all__ = ["SparseConv3D", "SubMConv3D", "SparseConvTransposed3D"]


class SparseConv3DBase(nn.Module):
    """Holds the parameters and forwards to `sparse_conv3d` (modules/conv.py:31-159)."""

    def __init__(self, in_channels, out_channels, kernel_size=3, stride=1, padding=0, dilation=1, subm=True,
                 bias=True, transposed=False):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size = make_ntuple(kernel_size, 3)
        self.stride = make_ntuple(stride, 3)
        self.padding = make_ntuple(padding, 3)
        self.dilation = make_ntuple(dilation, 3)
        self.subm, self.transposed = subm, transposed
        self.kernel_volume = self.kernel_size[0] * self.kernel_size[1] * self.kernel_size[2]
        self.weight = nn.Parameter(torch.empty(self.kernel_volume, in_channels, out_channels))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_channels))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self):
        bound = 1.0 / math.sqrt(self.in_channels * self.kernel_volume)
        with torch.no_grad():
            self.weight.uniform_(-bound, bound)
            if self.bias is not None:
                self.bias.uniform_(-bound, bound)

    def forward(self, input: SparseTensor) -> SparseTensor:
        return F.conv.sparse_conv3d(
            tensor=input, weight=self.weight, kernel_size=self.kernel_size, bias=self.bias, stride=self.stride,
            dilation=self.dilation, padding=self.padding, submanifold=self.subm, transposed=self.transposed)

    def extra_repr(self):
        return (f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, stride={self.stride}, "
                f"padding={self.padding}, dilation={self.dilation}, subm={self.subm}, transposed={self.transposed}")


class SparseConv3D(SparseConv3DBase):
    """Regular (non-submanifold) convolution; stride > 1 downsamples (modules/conv.py:162-226)."""

    def __init__(self, in_channels, out_channels, kernel_size=3, stride=1, padding=0, dilation=1, bias=True):
        super().__init__(in_channels, out_channels, kernel_size=kernel_size, stride=stride, padding=padding,
                         dilation=dilation, subm=False, bias=bias, transposed=False)


class SubMConv3D(SparseConv3DBase):
    """Submanifold convolution: output coordinates = input coordinates (modules/conv.py:229-289)."""

    def __init__(self, in_channels, out_channels, kernel_size=3, stride=1, dilation=1, bias=True):
        super().__init__(in_channels, out_channels, kernel_size=kernel_size, stride=stride, dilation=dilation,
                         subm=True, bias=bias, transposed=False)


class SparseConvTransposed3D(SparseConv3DBase):
    """Transposed convolution; stride > 1 upsamples (modules/conv.py:292-365).  `subm` and
    `transposed` are accepted for signature compatibility and ignored, as in the reference."""

    def __init__(self, in_channels, out_channels, kernel_size=3, stride=1, padding=0, dilation=1, subm=True,
                 bias=True, transposed=False):
        super().__init__(in_channels, out_channels, kernel_size=kernel_size, stride=stride, padding=padding,
                         dilation=dilation, subm=False, bias=bias, transposed=True)
