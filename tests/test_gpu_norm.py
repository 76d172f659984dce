"""Per-sample batch normalisation (+ fused ReLU) on the GPU against the reference's formulation written
out with torch ops (nn/functional/norm.py:73-112: index_add_ sums per (batch index, channel), biased
variance, eps inside the square root, affine), forward and backward, training and inference mode.

Tolerances: fp32 1e-5 max-norm relative; bf16 / fp16 1e-2 (the result is stored in the feature dtype).
"""
import numpy as np
import pytest
import torch

import sparsetriton_b200 as st
from sparsetriton_b200.nn.functional import sparse_batch_norm
from sparsetriton_b200.nn.modules import SparseBatchNorm

pytestmark = pytest.mark.gpu


def _reference(feats, batch_idx, batch_size, weight, bias, running_mean, running_var, training, eps, relu):
    x = feats.double()
    if training:
        sums = torch.zeros(batch_size, x.shape[1], dtype=torch.float64, device=x.device).index_add_(0, batch_idx, x)
        counts = torch.bincount(batch_idx, minlength=batch_size).double().view(-1, 1).clamp(min=1)
        mean = sums / counts
        cen = x - mean[batch_idx]
        var = torch.zeros_like(sums).index_add_(0, batch_idx, cen * cen) / counts
        y = cen / torch.sqrt(var[batch_idx] + eps)
    else:
        mean, var = running_mean.double(), running_var.double()
        y = (x - mean) / torch.sqrt(var + eps)
    if weight is not None:
        y = y * weight.double()
    if bias is not None:
        y = y + bias.double()
    if relu:
        y = torch.relu(y)
    return y, (mean, var) if training else None


def _rel(a, b):
    a, b = a.double(), b.double()
    return float(((a - b).abs().max() / b.abs().max().clamp(min=1e-30)).detach())


def _scene(n, C, B, dtype, dev, seed, sorted_batches=True):
    g = torch.Generator().manual_seed(seed)
    b = torch.randint(0, B, (n,), generator=g)
    if sorted_batches:
        b = b.sort().values
    coords = torch.cat([b.view(-1, 1), torch.randint(0, 64, (n, 3), generator=g)], 1).int().to(dev)
    feats = (torch.randn(n, C, generator=g) * 1.7 + 0.4).to(dev, dtype)
    return st.SparseTensor(feats, coords, spatial_shape=(64, 64, 64), batch_size=B), b.to(dev)


@pytest.mark.parametrize("relu", [False, True], ids=["plain", "relu"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16], ids=["fp32", "bf16", "fp16"])
@pytest.mark.parametrize("n,C,B,sorted_batches", [(1, 16, 1, True), (777, 32, 3, True), (20000, 64, 4, True),
                                                  (5000, 48, 5, False), (3000, 256, 2, True), (900, 5, 2, True),
                                                  (1200, 20, 4, True)])
def test_training_forward_backward(cuda_device, dtype, relu, n, C, B, sorted_batches):
    dev = cuda_device
    sp, bidx = _scene(n, C, B, dtype, dev, 100 + n + C, sorted_batches)
    g = torch.Generator().manual_seed(5)
    w = (torch.rand(C, generator=g) + 0.5).to(dev).requires_grad_(True)
    b = (torch.randn(C, generator=g) * 0.3).to(dev).requires_grad_(True)
    rm, rv = torch.zeros(C, device=dev), torch.ones(C, device=dev)
    x = sp.F.detach().clone().requires_grad_(True)
    out = sparse_batch_norm(sp.replace(x), w, b, rm, rv, training=True, eps=1e-5, momentum=0.1, relu=relu)
    dy = torch.randn(n, C, generator=g).to(dev, dtype)
    (out.F.float() * dy.float()).sum().backward()

    xr = sp.F.detach().double().requires_grad_(True)
    wr, br = w.detach().double().requires_grad_(True), b.detach().double().requires_grad_(True)
    yr, (mean, var) = _reference(xr, bidx, B, wr, br, None, None, True, 1e-5, relu)
    (yr * dy.double()).sum().backward()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert out.F.dtype == dtype
    assert _rel(out.F, yr) < tol
    assert _rel(x.grad, xr.grad) < (2e-4 if dtype == torch.float32 else 2e-2)
    assert _rel(w.grad, wr.grad) < (2e-4 if dtype == torch.float32 else 2e-2)
    assert _rel(b.grad, br.grad) < (2e-4 if dtype == torch.float32 else 2e-2)
    # running statistics follow the reference's update
    assert _rel(rm, 0.1 * mean.mean(0)) < (1e-4 if dtype == torch.float32 else 1e-2)
    assert _rel(rv, 0.9 + 0.1 * var.mean(0)) < (1e-4 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("relu", [False, True], ids=["plain", "relu"])
def test_inference_mode_uses_running_statistics(cuda_device, relu):
    dev = cuda_device
    sp, bidx = _scene(4000, 32, 3, torch.float32, dev, 9)
    bn = SparseBatchNorm(32).to(dev)
    with torch.no_grad():
        bn.running_mean.copy_(torch.randn(32, device=dev) * 0.2)
        bn.running_var.copy_(torch.rand(32, device=dev) + 0.5)
        bn.weight.copy_(torch.rand(32, device=dev) + 0.5)
        bn.bias.copy_(torch.randn(32, device=dev) * 0.1)
    bn.eval()
    x = sp.F.detach().clone().requires_grad_(True)
    out = bn(sp.replace(x), relu=relu)
    out.F.sum().backward()
    xr = sp.F.detach().double().requires_grad_(True)
    yr, _ = _reference(xr, bidx, 3, bn.weight.detach(), bn.bias.detach(), bn.running_mean, bn.running_var, False, bn.eps, relu)
    yr.sum().backward()
    assert _rel(out.F, yr) < 1e-5
    assert _rel(x.grad, xr.grad) < 1e-5


def test_module_counts_batches_and_rejects_wrong_width(cuda_device):
    sp, _ = _scene(100, 16, 2, torch.float32, cuda_device, 3)
    bn = SparseBatchNorm(16).to(cuda_device)
    bn(sp)
    bn(sp)
    assert int(bn.num_batches_tracked) == 2
    with pytest.raises(ValueError):
        SparseBatchNorm(8).to(cuda_device)(sp)
