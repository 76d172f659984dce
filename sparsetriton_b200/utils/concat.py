"""Channel-wise concatenation of two feature matrices with contiguous gradients (no reference counterpart: the
reference's networks call torch.cat on the features of a skip connection).

torch.cat's backward hands its two inputs strided slices of one gradient, and every consumer that wants rows in one
piece (the convolution and normalisation kernels here) copies its slice first.  `concat_features` splits the gradient
into two contiguous matrices in one pass instead (st_split_cols)."""
import torch

from sparsetriton_b200 import _lib

__all__ = ["concat_features"]


class _ConcatCols(torch.autograd.Function):
    @staticmethod
    def forward(ctx, left, right):
        n = left.shape[0]
        out = torch.empty((n, left.shape[1] + right.shape[1]), dtype=left.dtype, device=left.device)
        es = left.element_size()
        with _lib.on_device(left.device):
            _lib.check(_lib.lib().st_concat_cols(_lib.ptr(left), _lib.ptr(right), n, left.shape[1] * es, right.shape[1] * es,
                                                 _lib.ptr(out), _lib.stream_ptr()), "st_concat_cols")
        ctx.widths = (left.shape[1], right.shape[1])
        return out

    @staticmethod
    def backward(ctx, grad):
        grad = grad.contiguous()
        n, (a, b) = grad.shape[0], ctx.widths
        ga = torch.empty((n, a), dtype=grad.dtype, device=grad.device)
        gb = torch.empty((n, b), dtype=grad.dtype, device=grad.device)
        es = grad.element_size()
        with _lib.on_device(grad.device):
            _lib.check(_lib.lib().st_split_cols(_lib.ptr(grad), n, a * es, b * es, _lib.ptr(ga), _lib.ptr(gb), _lib.stream_ptr()),
                       "st_split_cols")
        return ga, gb


def concat_features(left: torch.Tensor, right: torch.Tensor) -> torch.Tensor:
    """torch.cat([left, right], dim=1) for two (N, C) matrices; on the GPU, with rows that are multiples of 16 bytes, through
    the library's copy kernels so that the backward pass yields two contiguous gradients."""
    es = left.element_size()
    if (left.is_cuda and right.is_cuda and left.ndim == 2 and right.ndim == 2 and left.dtype == right.dtype
            and left.shape[0] == right.shape[0] and (left.shape[1] * es) % 16 == 0 and (right.shape[1] * es) % 16 == 0):
        return _ConcatCols.apply(left.contiguous(), right.contiguous())
    return torch.cat([left, right], dim=1)
