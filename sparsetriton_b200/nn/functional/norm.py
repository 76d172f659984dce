"""Per-sample batch normalisation of sparse features (reference: nn/functional/norm.py:20-112).

Plain torch: normalisation is outside the accelerated path.  Statistics are taken per
(batch index, channel), exactly as in the reference, so sharding a batch by sample over GPUs
needs no cross-GPU statistics.  Unlike the reference, half / bfloat16 features are accepted:
statistics are computed in fp32 and the result is cast back to the feature dtype.
"""
import torch

from sparsetriton_b200.tensor import SparseTensor

__all__ = ["sparse_batch_norm"]


def sparse_batch_norm(tensor: SparseTensor, weight=None, bias=None, running_mean=None, running_var=None,
                      training=True, eps=1e-5, momentum=0.1) -> SparseTensor:
    feats = tensor.F
    x = feats.float()
    if training:
        b = tensor.C[:, 0].long()
        nb, c = tensor.batch_size, x.shape[1]
        counts = torch.bincount(b, minlength=nb).to(x.dtype).clamp(min=1).view(-1, 1)
        mean = torch.zeros(nb, c, device=x.device).index_add_(0, b, x) / counts
        centred = x - mean[b]
        var = torch.zeros(nb, c, device=x.device).index_add_(0, b, centred * centred) / counts
        if running_mean is not None:
            running_mean.mul_(1 - momentum).add_(momentum * mean.mean(0).detach())
        if running_var is not None:
            running_var.mul_(1 - momentum).add_(momentum * var.mean(0).detach())
        y = centred / torch.sqrt(var[b] + eps)
    else:
        y = (x - running_mean) / torch.sqrt(running_var + eps)
    if weight is not None:
        y = y * weight
    if bias is not None:
        y = y + bias
    return tensor.replace(y.to(feats.dtype))
