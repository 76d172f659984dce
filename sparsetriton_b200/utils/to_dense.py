"""Sparse -> dense scatter used by SparseTensor.dense() (reference: utils/to_dense.py:143-282).

Plain torch indexing: this conversion is a test/debug convenience, not part of the hot path.
Output layout (B, X, Y, Z, C) as in the reference; autograd flows through index_put.
"""
import torch


def to_dense(feats, coords, spatial_range):
    batch = int(coords[:, 0].max().item()) + 1 if coords.shape[0] > 0 else 1
    shape = (batch, *tuple(int(v) for v in spatial_range), feats.shape[1])
    dense = torch.zeros(shape, dtype=feats.dtype, device=feats.device)
    if coords.shape[0] == 0:
        return dense
    c = coords.long()
    return dense.index_put((c[:, 0], c[:, 1], c[:, 2], c[:, 3]), feats)
