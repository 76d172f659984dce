"""Thin torch wrappers that act on SparseTensor.F (reference: nn/modules/linear.py:23-73,
nn/modules/activation.py:23-65)."""
from torch import nn

from sparsetriton_b200.tensor import SparseTensor

__all__ = ["SparseLinear", "ReLU"]


class SparseLinear(nn.Linear):
    def forward(self, input):
        if isinstance(input, SparseTensor):
            return input.replace(super().forward(input.F))
        return super().forward(input)


class ReLU(nn.ReLU):
    def forward(self, input):
        if isinstance(input, SparseTensor):
            return input.replace(super().forward(input.F))
        return super().forward(input)
