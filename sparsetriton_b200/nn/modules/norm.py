"""SparseBatchNorm (reference: nn/modules/norm.py:25-123): same parameters and buffers."""
import torch
from torch import nn

from sparsetriton_b200.nn.functional.norm import sparse_batch_norm
from sparsetriton_b200.tensor import SparseTensor

__all__ = ["SparseBatchNorm"]


class SparseBatchNorm(nn.Module):
    def __init__(self, num_features, eps=1e-5, momentum=0.1, affine=True, track_running_stats=True):
        super().__init__()
        self.num_features, self.eps, self.momentum = num_features, eps, momentum
        self.affine, self.track_running_stats = affine, track_running_stats
        if affine:
            self.weight = nn.Parameter(torch.ones(num_features))
            self.bias = nn.Parameter(torch.zeros(num_features))
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)
        if track_running_stats:
            self.register_buffer("running_mean", torch.zeros(num_features))
            self.register_buffer("running_var", torch.ones(num_features))
            self.register_buffer("num_batches_tracked", torch.tensor(0, dtype=torch.long))
        else:
            self.register_buffer("running_mean", None)
            self.register_buffer("running_var", None)
            self.register_buffer("num_batches_tracked", None)

    def forward(self, input: SparseTensor, relu: bool = False) -> SparseTensor:
        """`relu=True` folds the ReLU that follows the layer into its kernels (no reference counterpart:
        there the activation is a separate module)."""
        if input.F.shape[1] != self.num_features:
            raise ValueError(f"expected {self.num_features} channels, got {input.F.shape[1]}")
        out = sparse_batch_norm(input, self.weight, self.bias, self.running_mean, self.running_var,
                                training=self.training, eps=self.eps, momentum=self.momentum, relu=relu)
        if self.training and self.track_running_stats:
            self.num_batches_tracked += 1
        return out
