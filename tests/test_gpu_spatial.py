"""Dense conversion, pooling and upsampling on the GPU (through the C ABI) against the reference's own
outputs (tests/golden/dense_*, pool_*, upsample_*) and against the oracle's numpy restatements, which
tests/test_oracle_golden.py holds to the same fixtures.

Bars: coordinates, row order and copied values bit-exact; reduced values (mean, summed gradients) within
1e-6 relative for fp32 and 1e-2 for fp16 / bf16 (max-norm relative; the result is stored in the feature dtype).
"""
import numpy as np
import pytest
import torch

import sparsetriton_b200 as st
from conftest import case_id, golden_files, load_golden
from gpu_util import rel_err, t2n
from sparsetriton_b200.config import set_coords_dtype
from sparsetriton_b200.nn.functional import sparse_pooling, sparse_upsample
from sparsetriton_b200.nn.modules import SparseDownsample, SparsePooling, SparseUpsample
from sparsetriton_b200.utils.to_dense import to_dense

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16, torch.bfloat16]
TOL = {torch.float32: 1e-6, torch.float16: 1e-2, torch.bfloat16: 1e-2}


# ------------------------------------------------------------------------------------ dense
def test_to_dense_reference_fixture(cuda_device):
    g = load_golden(golden_files("dense_")[0])
    set_coords_dtype(torch.int32)
    x = torch.as_tensor(g["feats"]).to(cuda_device).requires_grad_(True)
    dense = to_dense(x, torch.as_tensor(g["coords"]).to(cuda_device), tuple(g["shape"]))
    assert np.array_equal(t2n(dense), g["dense"])
    (dense * torch.as_tensor(g["upstream"]).to(cuda_device)).sum().backward()
    assert np.array_equal(t2n(x.grad), g["grad_feats"])


def test_to_dense_docstring_example(cuda_device):
    """utils/to_dense.py:263-273."""
    sp = st.SparseTensor(torch.tensor([[1.0], [2.0], [3.0]], device=cuda_device),
                         torch.tensor([[0, 0, 0, 0], [0, 0, 0, 1], [1, 0, 0, 0]], device=cuda_device))
    dense = sp.dense()
    assert dense.shape == (2, 1, 1, 2, 1) and dense[0, 0, 0, 1, 0] == 2.0 and dense[1, 0, 0, 0, 0] == 3.0


@pytest.mark.parametrize("coord_dtype", [torch.int16, torch.int32], ids=["i16", "i32"])
@pytest.mark.parametrize("dtype", DTYPES, ids=["fp32", "fp16", "bf16"])
@pytest.mark.parametrize("C", [1, 5, 8, 64, 96], ids=lambda c: f"c{c}")
def test_to_dense_vs_oracle(cuda_device, oracle, dtype, coord_dtype, C):
    set_coords_dtype(coord_dtype)
    sp = st.randn((20, 17, 9), batch_size=3, channels=C, nnz=2500, device=cuda_device, dtype=dtype)
    x = sp.F.detach().clone().requires_grad_(True)
    dense = sp.replace(x).dense()
    assert dense.dtype == dtype and dense.shape == (3, 20, 17, 9, C)
    want = oracle.to_dense(t2n(sp.F), t2n(sp.C), (20, 17, 9), batch=3)
    assert np.array_equal(t2n(dense), want)
    up = torch.randn(dense.shape, device=cuda_device).to(dtype)
    (dense.float() * up.float()).sum().backward()
    assert np.array_equal(t2n(x.grad), oracle.to_dense_bwd(t2n(up), t2n(sp.C)))


def test_to_dense_empty_and_flags(cuda_device):
    from sparsetriton_b200 import _lib
    set_coords_dtype(torch.int32)
    empty = to_dense(torch.empty(0, 4, device=cuda_device), torch.empty(0, 4, dtype=torch.int32, device=cuda_device), (2, 2, 2))
    assert empty.shape == (1, 2, 2, 2, 4) and float(empty.abs().sum()) == 0.0
    # a row outside the volume is skipped and flagged, never written
    feats = torch.ones(3, 4, device=cuda_device)
    coords = torch.tensor([[0, 0, 0, 0], [0, 5, 0, 0], [1, 1, 1, 1]], dtype=torch.int32, device=cuda_device)
    dense = torch.empty(1, 2, 2, 2, 4, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    rc = _lib.lib().st_to_dense_fwd(_lib.ST_F32, _lib.ptr(feats), _lib.ptr(coords), _lib.ST_I32, 3, 4, 1, _lib.host_i32((2, 2, 2)),
                                    _lib.ptr(dense), _lib.ptr(status), _lib.stream_ptr())
    assert rc == 0 and int(status.item()) == _lib.DEV_BAD_INDEX
    assert float(dense.sum()) == 4.0 and float(dense[0, 0, 0, 0].sum()) == 4.0
    with pytest.raises(RuntimeError, match="no CPU path"):
        to_dense(torch.ones(1, 1), torch.zeros(1, 4, dtype=torch.int32), (1, 1, 1))


# ------------------------------------------------------------------------------------ pooling
@pytest.mark.parametrize("path", golden_files("pool_"), ids=case_id)
def test_pooling_reference_fixture(cuda_device, path):
    g = load_golden(path)
    set_coords_dtype(torch.int32)
    x = torch.as_tensor(g["feats"]).to(cuda_device).requires_grad_(True)
    sp = st.SparseTensor(x, torch.as_tensor(g["coords"]).to(cuda_device), spatial_shape=tuple(g["shape"]),
                         batch_size=int(g["batch"]))
    out = sparse_pooling(sp, kernel_size=int(g["k"]), padding=int(g["p"]), stride=int(g["s"]), mode="avg")
    assert np.array_equal(t2n(out.C), g["out_coords"]) and list(out.spatial_shape) == g["new_shape"].tolist()
    assert rel_err(t2n(out.F), g["y"]) < 1e-6
    (out.F * torch.as_tensor(g["upstream"]).to(cuda_device)).sum().backward()
    assert rel_err(t2n(x.grad), g["grad_feats"]) < 1e-6


@pytest.mark.parametrize("mode", ["avg", "max"])
@pytest.mark.parametrize("dtype", DTYPES, ids=["fp32", "fp16", "bf16"])
@pytest.mark.parametrize("k,p,s,coord_dtype", [(2, 0, 2, torch.int32), (2, 1, 2, torch.int16), (3, 1, 2, torch.int32),
                                               (3, 1, 1, torch.int32), (4, 2, 4, torch.int16), (5, 0, 3, torch.int32)])
def test_pooling_vs_oracle(cuda_device, oracle, dtype, mode, k, p, s, coord_dtype):
    """Also covers negative cells (padding < kernel_size // 2), which stay exact here."""
    set_coords_dtype(coord_dtype)
    shape, B, C = (33, 20, 27), 3, 12
    sp = st.randn(shape, batch_size=B, channels=C, nnz=9000, device=cuda_device, dtype=dtype)
    x = sp.F.detach().clone().requires_grad_(True)
    out = sparse_pooling(sp.replace(x), kernel_size=k, padding=p, stride=s, mode=mode)
    oc, in_to_out = oracle.pool_map(t2n(sp.C), k, p, s)
    assert np.array_equal(t2n(out.C).astype(np.int32), oc), "pooled cells differ"
    assert out.C.dtype == coord_dtype and tuple(out.spatial_shape) == oracle.pool_new_shape(shape, k, p, s)
    want = oracle.pool_fwd(t2n(sp.F), in_to_out, oc.shape[0], mode)
    if mode == "max":
        assert np.array_equal(t2n(out.F), want.astype(np.float32))          # a maximum is one of the inputs
    else:
        assert rel_err(t2n(out.F), want) < TOL[dtype]
    up = torch.randn(out.F.shape, device=cuda_device).to(dtype)
    (out.F.float() * up.float()).sum().backward()
    want_g = oracle.pool_bwd(t2n(up), t2n(sp.F), t2n(out.F), in_to_out, mode)
    assert rel_err(t2n(x.grad), want_g) < TOL[dtype]


def test_pooling_surface(cuda_device):
    set_coords_dtype(torch.int16)
    with pytest.raises(ValueError, match="Unsupported mode"):
        sparse_pooling(st.randn((16, 16, 16), batch_size=2, nnz=10, channels=4), kernel_size=2, padding=0, stride=2, mode="invalid")
    with pytest.raises(ValueError, match="mode must be"):
        SparsePooling(kernel_size=2, mode="invalid")
    coords = torch.tensor([[0, 0, 0, 0], [0, 0, 0, 1], [0, 0, 1, 0]], dtype=torch.int16, device=cuda_device)
    feats = torch.tensor([[1.0], [2.0], [3.0]], device=cuda_device)
    sp = st.SparseTensor(feats, coords, spatial_shape=(2, 2, 2), batch_size=1)
    out = SparsePooling(kernel_size=2, mode="avg", stride=2, padding=1)(sp)
    assert isinstance(out, st.SparseTensor) and out.C.tolist() == [[0, 0, 0, 0]] and out.F.tolist() == [[2.0]]
    ds = SparseDownsample(scale_factor=2, mode="max")
    assert (ds.kernel_size, ds.stride, ds.padding, ds.mode) == (2, 2, 0, "max")
    assert ds(sp).F.max().item() == 3.0
    empty = st.SparseTensor(torch.empty(0, 3, device=cuda_device), torch.empty(0, 4, dtype=torch.int16, device=cuda_device),
                            spatial_shape=(4, 4, 4), batch_size=1)
    out = sparse_pooling(empty, 2, 0, 2, "avg")
    assert out.F.shape == (0, 3) and out.C.shape == (0, 4)


# ------------------------------------------------------------------------------------ upsample
@pytest.mark.parametrize("path", golden_files("upsample_"), ids=case_id)
def test_upsample_reference_fixture(cuda_device, path):
    g = load_golden(path)
    set_coords_dtype(torch.int32)
    x = torch.as_tensor(g["feats"]).to(cuda_device).requires_grad_(True)
    sp = st.SparseTensor(x, torch.as_tensor(g["coords"]).to(cuda_device), spatial_shape=tuple(g["shape"]), batch_size=2)
    out = sparse_upsample(sp, scale_factor=int(g["scale"]))
    assert np.array_equal(t2n(out.C), g["out_coords"]) and np.array_equal(t2n(out.F), g["y"])
    assert list(out.spatial_shape) == g["new_shape"].tolist()
    (out.F * torch.as_tensor(g["upstream"]).to(cuda_device)).sum().backward()
    assert rel_err(t2n(x.grad), g["grad_feats"]) < 1e-6


@pytest.mark.parametrize("scale", [1, 2, 3])
@pytest.mark.parametrize("dtype", DTYPES, ids=["fp32", "fp16", "bf16"])
def test_upsample_vs_oracle(cuda_device, oracle, dtype, scale):
    set_coords_dtype(torch.int16)
    sp = st.randn((10, 12, 14), batch_size=2, channels=7, nnz=1500, device=cuda_device, dtype=dtype)
    x = sp.F.detach().clone().requires_grad_(True)
    out = SparseUpsample(scale_factor=scale)(sp.replace(x))
    y, oc = oracle.upsample(t2n(sp.F), t2n(sp.C), scale)
    assert np.array_equal(t2n(out.C).astype(np.int32), oc) and np.array_equal(t2n(out.F), y)
    assert tuple(out.spatial_shape) == (10 * scale, 12 * scale, 14 * scale) and out.batch_size == 2
    up = torch.randn(out.F.shape, device=cuda_device).to(dtype)
    (out.F.float() * up.float()).sum().backward()
    assert rel_err(t2n(x.grad), oracle.upsample_bwd(t2n(up), scale)) < TOL[dtype]


def test_upsample_reference_known_answer(cuda_device):
    """tests/test_pooling.py:14-41 of the reference: one voxel at the origin."""
    set_coords_dtype(torch.int16)
    coords = torch.tensor([[0, 0, 0, 0]], dtype=torch.int16, device=cuda_device)
    feats = torch.tensor([[1.0, 2.0, 3.0]], device=cuda_device)
    for scale in (1, 2, 3):
        out = sparse_upsample(st.SparseTensor(feats, coords, spatial_shape=(10, 10, 10), batch_size=1), scale_factor=scale)
        assert out.F.shape[0] == scale ** 3 and torch.allclose(out.F, feats.repeat(scale ** 3, 1))
        want = [[0, x, y, z] for x in range(scale) for y in range(scale) for z in range(scale)]
        assert out.C.tolist() == want and tuple(out.spatial_shape) == (10 * scale,) * 3


@pytest.mark.parametrize("dtype,a,b", [(torch.bfloat16, 32, 32), (torch.float32, 4, 12), (torch.float16, 64, 8), (torch.float32, 3, 5)])
def test_concat_features_and_its_gradients(cuda_device, dtype, a, b):
    """concat_features = torch.cat along the channels, forward and backward, bit for bit (copies only); widths that are
    not whole 16-byte pieces take torch.cat itself."""
    from sparsetriton_b200.utils.concat import concat_features
    gen = torch.Generator().manual_seed(3)
    left = torch.randn(1003, a, generator=gen).to(dtype).to(cuda_device).requires_grad_(True)
    right = torch.randn(1003, b, generator=gen).to(dtype).to(cuda_device).requires_grad_(True)
    out = concat_features(left, right)
    want = torch.cat([left.detach(), right.detach()], dim=1)
    assert torch.equal(out, want)
    g = torch.randn(1003, a + b, generator=gen).to(dtype).to(cuda_device)
    out.backward(g)
    assert left.grad.is_contiguous() and right.grad.is_contiguous()
    assert torch.equal(left.grad, g[:, :a]) and torch.equal(right.grad, g[:, a:])
    empty = concat_features(left[:0].detach(), right[:0].detach())
    assert empty.shape == (0, a + b)
