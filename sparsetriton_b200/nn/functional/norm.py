"""Per-sample batch normalisation of sparse features (reference: nn/functional/norm.py:20-112).

Plain torch: normalisation is outside the accelerated path.  Statistics are taken per
(batch index, channel), exactly as in the reference (as matrix products with a one-hot sample
indicator instead of index_add_), so sharding a batch by sample over GPUs
needs no cross-GPU statistics.  Unlike the reference, half / bfloat16 features are accepted:
statistics are computed in fp32 and the result is cast back to the feature dtype.
"""
import torch

from sparsetriton_b200.tensor import SparseTensor

__all__ = ["sparse_batch_norm"]


def _sample_indicator(tensor: SparseTensor):
    """(N, B) fp32 one-hot of the batch column, memoised with the coordinate set.  Per-sample sums are
    then GEMMs (indicator^T @ x): no atomics, so statistics are reproducible, and far faster than
    index_add_ when millions of rows fall on a handful of samples."""
    cache = tensor._cache.kmaps
    hit = cache.get("sample_indicator")
    if hit is None or hit.shape[0] != tensor.C.shape[0]:
        hit = torch.nn.functional.one_hot(tensor.C[:, 0].long(), tensor.batch_size).to(torch.float32)
        cache["sample_indicator"] = hit
    return hit


def sparse_batch_norm(tensor: SparseTensor, weight=None, bias=None, running_mean=None, running_var=None,
                      training=True, eps=1e-5, momentum=0.1) -> SparseTensor:
    feats = tensor.F
    x = feats.float()
    if training:
        ind = _sample_indicator(tensor)                                  # (N, B)
        counts = ind.sum(0).clamp(min=1).view(-1, 1)                     # (B, 1)
        mean = (ind.t() @ x) / counts                                    # (B, C)
        centred = x - ind @ mean
        var = (ind.t() @ (centred * centred)) / counts
        if running_mean is not None:
            running_mean.mul_(1 - momentum).add_(momentum * mean.mean(0).detach())
        if running_var is not None:
            running_var.mul_(1 - momentum).add_(momentum * var.mean(0).detach())
        y = centred / torch.sqrt(ind @ var + eps)
    else:
        y = (x - running_mean) / torch.sqrt(running_var + eps)
    if weight is not None:
        y = y * weight
    if bias is not None:
        y = y + bias
    return tensor.replace(y.to(feats.dtype))
