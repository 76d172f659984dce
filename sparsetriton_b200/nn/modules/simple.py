"""Thin torch wrappers that act on SparseTensor.F (reference: nn/modules/linear.py:23-73,
nn/modules/activation.py:23-65)."""
import torch
from torch import nn

from sparsetriton_b200.tensor import SparseTensor

__all__ = ["SparseLinear", "ReLU"]

_SPLIT_ROWS = 8192          # rows per partial product of the weight gradient
_TALL = 1 << 16             # from this many rows on the weight gradient is split


class _TallLinear(torch.autograd.Function):
    """y = x W^T + b for a matrix of very many rows and few columns (a per-voxel head).  Only the weight gradient
    differs from torch's: dW = dY^T X reduces over all N rows into an (out, in) result of a few hundred entries, a shape
    for which the library GEMM runs on a handful of SMs (0.65 ms for 1.7 M x 32 -> 20 in fp32).  Here the rows are cut
    into pieces of 8192, the pieces multiplied as one batched product and the partial results added in a fixed order."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        return torch.addmm(bias, x, weight.t()) if bias is not None else x @ weight.t()

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dy @ weight if ctx.needs_input_grad[0] else None
        dw = db = None
        if ctx.needs_input_grad[1]:
            n = x.shape[0]
            full = n // _SPLIT_ROWS * _SPLIT_ROWS
            dw = torch.zeros_like(weight)
            if full:
                parts = torch.bmm(dy[:full].view(-1, _SPLIT_ROWS, dy.shape[1]).transpose(1, 2),
                                  x[:full].view(-1, _SPLIT_ROWS, x.shape[1]))
                dw = parts.sum(0)
            if full < n:
                dw = dw + dy[full:].t() @ x[full:]
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.sum(0)
        return dx, dw, db


class SparseLinear(nn.Linear):
    def _apply_rows(self, feats):
        if feats.is_cuda and feats.ndim == 2 and feats.shape[0] >= _TALL and feats.is_contiguous() and \
                feats.dtype == self.weight.dtype and torch.is_grad_enabled() and self.weight.requires_grad:
            return _TallLinear.apply(feats, self.weight, self.bias)
        return super().forward(feats)

    def forward(self, input):
        if isinstance(input, SparseTensor):
            return input.replace(self._apply_rows(input.F))
        return self._apply_rows(input)


class ReLU(nn.ReLU):
    def forward(self, input):
        if isinstance(input, SparseTensor):
            return input.replace(super().forward(input.F))
        return super().forward(input)
