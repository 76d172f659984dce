"""Per-sample batch normalisation (+ fused ReLU) on the GPU against the oracle's float64 restatement of the
reference's formulation (oracle.batch_norm, nn/functional/norm.py:73-112: sums per (batch index, channel),
biased variance, eps inside the square root, affine), which tests/test_oracle_golden.py::test_batch_norm
holds to the reference's own output; and against that output directly (tests/golden/bn_b3_c6.npz).
Forward and backward, training and inference mode.

Tolerances (max-norm relative): fp32 2e-5 forward / 2e-4 gradients; bf16 / fp16 1e-2 / 2e-2 (the result is
stored in the feature dtype).
"""
import numpy as np
import pytest
import torch

import sparsetriton_b200 as st
from conftest import golden_files, load_golden
from sparsetriton_b200 import _lib
from sparsetriton_b200.nn.functional import sparse_batch_norm
from sparsetriton_b200.nn.functional.norm import bad_batch_index
from sparsetriton_b200.nn.modules import SparseBatchNorm

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a = a.detach().double().cpu().numpy() if isinstance(a, torch.Tensor) else np.asarray(a, np.float64)
    b = b.detach().double().cpu().numpy() if isinstance(b, torch.Tensor) else np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


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
                                                  (1200, 20, 4, True), (6000, 32, 5, False), (300_000, 32, 7, True),
                                                  (1000, 512, 2, True), (300, 2048, 2, True), (5, 8, 1, True)])
def test_training_forward_backward(cuda_device, oracle, dtype, relu, n, C, B, sorted_batches):
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

    # gradients are compared on the GPU run's own ReLU decisions, which may differ from the oracle's only where the
    # oracle's pre-activation is within rounding of zero (a flipped element would move dx by its whole magnitude)
    decisions = (out.F > 0).cpu().numpy() if relu else None
    r = oracle.batch_norm(sp.F.detach().double().cpu().numpy(), bidx.cpu().numpy(), B, w.detach().cpu().numpy(),
                          b.detach().cpu().numpy(), 1e-5, relu=relu, upstream=dy.double().cpu().numpy(),
                          running=(np.zeros(C), np.ones(C)), momentum=0.1, decisions=decisions)
    if relu:
        differ = decisions != (r["z"] > 0)
        assert not differ.any() or np.abs(r["z"][differ]).max() < (1e-4 if dtype == torch.float32 else 1e-3)
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    assert out.F.dtype == dtype
    assert _rel(out.F, r["y"]) < tol
    assert _rel(x.grad, r["dx"]) < (2e-4 if dtype == torch.float32 else 2e-2)
    assert _rel(w.grad, r["dw"]) < (2e-4 if dtype == torch.float32 else 2e-2)
    assert _rel(b.grad, r["db"]) < (2e-4 if dtype == torch.float32 else 2e-2)
    # running statistics follow the reference's update
    assert _rel(rm, r["running_mean"]) < (1e-4 if dtype == torch.float32 else 1e-2)
    assert _rel(rv, r["running_var"]) < (1e-4 if dtype == torch.float32 else 1e-2)
    assert not bad_batch_index(sp)


@pytest.mark.parametrize("relu", [False, True], ids=["plain", "relu"])
def test_inference_mode_uses_running_statistics(cuda_device, oracle, relu):
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
    wn, bn_, rmn, rvn = (t.detach().double().cpu().numpy() for t in (bn.weight, bn.bias, bn.running_mean, bn.running_var))
    z = oracle.batch_norm_eval(sp.F.double().cpu().numpy(), rmn, rvn, wn, bn_, bn.eps)
    yr = np.maximum(z, 0.0) if relu else z
    dxr = ((z > 0) if relu else 1.0) * wn / np.sqrt(rvn + bn.eps) * np.ones_like(z)      # d sum(y) / dx
    assert _rel(out.F, yr) < 1e-5
    assert _rel(x.grad, dxr) < 1e-5


def test_module_counts_batches_and_rejects_wrong_width(cuda_device):
    sp, _ = _scene(100, 16, 2, torch.float32, cuda_device, 3)
    bn = SparseBatchNorm(16).to(cuda_device)
    bn(sp)
    bn(sp)
    assert int(bn.num_batches_tracked) == 2
    with pytest.raises(ValueError):
        SparseBatchNorm(8).to(cuda_device)(sp)


def test_reference_fixture(cuda_device):
    """The reference's own sparse_batch_norm outputs (training forward + backward, the running buffers it leaves,
    and the inference form), including a batch whose middle sample is empty."""
    g = load_golden(golden_files("bn_")[0])
    dev = cuda_device
    coords = torch.as_tensor(g["coords"]).to(dev)
    x = torch.as_tensor(g["feats"]).to(dev).requires_grad_(True)
    w = torch.as_tensor(g["weight"]).to(dev).requires_grad_(True)
    b = torch.as_tensor(g["bias"]).to(dev).requires_grad_(True)
    rm, rv = torch.zeros(6, device=dev), torch.ones(6, device=dev)
    sp = st.SparseTensor(x, coords, spatial_shape=tuple(g["shape"]), batch_size=int(g["batch"]))
    out = sparse_batch_norm(sp, w, b, rm, rv, training=True, eps=float(g["eps"]), momentum=float(g["momentum"]))
    (out.F * torch.as_tensor(g["upstream"]).to(dev)).sum().backward()
    assert _rel(out.F, g["y_train"]) < 1e-5
    assert _rel(x.grad, g["grad_feats"]) < 2e-4
    assert _rel(w.grad, g["grad_weight"]) < 2e-4 and _rel(b.grad, g["grad_bias"]) < 2e-4
    assert _rel(rm, g["running_mean"]) < 1e-5 and _rel(rv, g["running_var"]) < 1e-5
    with torch.no_grad():
        ev = sparse_batch_norm(sp.replace(x.detach()), w, b, rm, rv, training=False, eps=float(g["eps"]))
    assert _rel(ev.F, g["y_eval"]) < 1e-5


@pytest.mark.parametrize("C", [32, 5], ids=["vector", "scalar"])
def test_batch_index_outside_the_batch_is_skipped_and_flagged(cuda_device, C):
    """Rows whose batch index is not in [0, B) must not reach the (B, C) arrays: they join no statistic, come
    out as zero rows, and ST_DEV_BAD_INDEX is raised.  The tensor is built through the internal constructor
    (the public one rejects such indices)."""
    dev = cuda_device
    g = torch.Generator().manual_seed(1)
    n, B = 3000, 2
    bidx = torch.randint(0, B, (n,), generator=g).sort().values
    bad = torch.zeros(n, dtype=torch.bool)
    bad[torch.randperm(n, generator=g)[:40]] = True
    bad[0] = True                                          # also the first row of a block
    stored = bidx.clone()
    stored[bad] = torch.tensor([7, -1, 2, 1 << 20] * 10 + [9])[: int(bad.sum())]
    coords = torch.cat([stored.view(-1, 1), torch.randint(0, 32, (n, 3), generator=g)], 1).int().to(dev)
    feats = torch.randn(n, C, generator=g).to(dev)
    sp = st.SparseTensor._trusted(feats.clone().requires_grad_(True), coords, (32, 32, 32), B)
    out = sparse_batch_norm(sp, None, None, None, None, training=True)
    out.F.square().sum().backward()
    assert bad_batch_index(sp)
    assert torch.equal(out.F[bad.to(dev)], torch.zeros_like(out.F[bad.to(dev)]))
    assert torch.equal(sp.F.grad[bad.to(dev)], torch.zeros_like(out.F[bad.to(dev)]))
    # the good rows are normalised with statistics taken over the good rows only
    keep = ~bad
    good = st.SparseTensor._trusted(feats[keep.to(dev)], coords[keep.to(dev)], (32, 32, 32), B)
    want = sparse_batch_norm(good, None, None, None, None, training=True)
    assert _rel(out.F[keep.to(dev)], want.F) < 1e-5
    assert not bad_batch_index(good)
    assert _lib.device_status(dev)[0] == 0
