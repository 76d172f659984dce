"""Sparse -> dense conversion (reference: utils/to_dense.py:143-282).

`to_dense(feats, coords, spatial_range)` keeps the reference's signature and its (B, X, Y, Z, C)
result.  Forward is one scatter kernel (st_to_dense_fwd, which also clears the volume), backward one
gather kernel (st_to_dense_bwd): both move 16-byte pieces of feature rows and are bound by HBM.

`batch_size` (no reference counterpart) lets a caller that already knows the batch size skip the
device->host read of `coords[:, 0].max()`; SparseTensor.dense() passes its own.
"""
import torch

from sparsetriton_b200 import _lib, trace

__all__ = ["to_dense", "ToDenseFunction"]


class ToDenseFunction(torch.autograd.Function):
    """feats (N, C), coords (N, 4) -> dense (batch, X, Y, Z, C); backward returns grad_feats only."""

    @staticmethod
    def forward(ctx, feats, coords, spatial_range, batch_size):
        _lib.require_cuda(feats, "to_dense")
        feats = feats.contiguous()
        coords = coords.contiguous()
        n, C = feats.shape
        shape = tuple(int(v) for v in spatial_range)
        dense = torch.empty((int(batch_size), *shape, C), dtype=feats.dtype, device=feats.device)
        status = torch.zeros(1, dtype=torch.int32, device=feats.device)
        with _lib.on_device(feats.device), trace.stage("to_dense_fwd"):
            rc = _lib.lib().st_to_dense_fwd(_lib.feat_code(feats), _lib.ptr(feats), _lib.ptr(coords), _lib.coord_code(coords),
                                            n, C, int(batch_size), _lib.host_i32(shape), _lib.ptr(dense), _lib.ptr(status),
                                            _lib.stream_ptr())
        _lib.check(rc, "st_to_dense_fwd")
        ctx.save_for_backward(coords)
        ctx.geometry = (n, C, int(batch_size), shape)
        return dense

    @staticmethod
    def backward(ctx, grad_output):
        (coords,) = ctx.saved_tensors
        n, C, batch, shape = ctx.geometry
        grad_output = grad_output.contiguous()
        grad_feats = torch.empty((n, C), dtype=grad_output.dtype, device=grad_output.device)
        with _lib.on_device(grad_output.device), trace.stage("to_dense_bwd"):
            rc = _lib.lib().st_to_dense_bwd(_lib.feat_code(grad_output), _lib.ptr(grad_output), _lib.ptr(coords),
                                            _lib.coord_code(coords), n, C, batch, _lib.host_i32(shape),
                                            _lib.ptr(grad_feats), _lib.stream_ptr())
        _lib.check(rc, "st_to_dense_bwd")
        return grad_feats, None, None, None


def to_dense(feats, coords, spatial_range, batch_size=None):
    """Dense (B, X, Y, Z, C) copy of the sparse rows; B = largest batch index + 1 (1 for an empty tensor)
    unless `batch_size` is given."""
    if batch_size is None:
        batch_size = int(coords[:, 0].max().item()) + 1 if coords.shape[0] > 0 else 1
    return ToDenseFunction.apply(feats, coords, tuple(spatial_range), batch_size)
