"""Convolution products on the GPU, through the public API (which calls the C ABI), against the
reference's golden outputs and against the fp32 oracle.

Tolerances (max-norm relative error against the fp32 result): 2e-3 for fp32 storage (tensor-core
kernels multiply in tf32), 1e-2 for fp16 / bf16 storage.
"""
import numpy as np
import pytest
import torch
import torch.nn.functional as TF

from conftest import case_id, golden_files, load_golden
from gpu_util import ALGOS, TOL, rel_err, run_conv, t2n
import sparsetriton_b200 as st
from sparsetriton_b200 import synthetic
from sparsetriton_b200.config import ConvAlgo, set_conv_algo, set_coords_dtype
from sparsetriton_b200.nn.functional import sparse_conv3d

pytestmark = pytest.mark.gpu



@pytest.fixture(autouse=True)
def _no_device_side_errors(cuda_device):
    """No bounded wait of a tensor-core kernel may have expired during a test."""
    from sparsetriton_b200 import _lib
    yield
    status = _lib.device_status(cuda_device)
    assert status[0] == 0, f"device status after test: {status}"


@pytest.mark.parametrize("algo", ALGOS, ids=lambda a: a.name)
@pytest.mark.parametrize("path", golden_files("conv_"), ids=case_id)
def test_golden_fp32(cuda_device, path, algo):
    g = load_golden(path)
    cdt = getattr(torch, str(g["coord_dtype"]))
    oc, ns, y, dx, dw, db = run_conv(cuda_device, g["coords"], g["shape"], g["batch"], g["feats"], g["weight"],
                                     g["bias"], g["dy"], int(g["k"]), int(g["s"]), int(g["p"]), int(g["d"]),
                                     bool(g["transposed"]), bool(g["subm"]), algo, cdt, torch.float32)
    assert np.array_equal(oc, g["out_coords"])
    assert ns.tolist() == g["new_shape"].tolist()
    tol = TOL[torch.float32]
    assert rel_err(y, g["y"]) < tol
    assert rel_err(dx, g["dx"]) < tol
    assert rel_err(dw, g["dw"]) < tol
    if g["db"].size:
        assert rel_err(db, g["db"]) < tol


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("algo", ALGOS, ids=lambda a: a.name)
@pytest.mark.parametrize("name", ["conv_subm_k3_c16_32", "conv_down_k2s2_c32_64", "conv_up_k2s2_c16_8",
                                  "conv_down_k3s2_c16_16"])
def test_golden_half(cuda_device, oracle, name, algo, dtype):
    """Half-precision storage: compare with the fp32 oracle fed the SAME rounded inputs."""
    g = load_golden([p for p in golden_files("conv_") if case_id(p) == name][0])
    cdt = getattr(torch, str(g["coord_dtype"]))
    rnd = lambda a: torch.as_tensor(a).to(dtype).float().numpy()
    feats, weight, dy = rnd(g["feats"]), rnd(g["weight"]), rnd(g["dy"])
    oc, ns, y, dx, dw, db = run_conv(cuda_device, g["coords"], g["shape"], g["batch"], feats, weight, None, dy,
                                     int(g["k"]), int(g["s"]), int(g["p"]), int(g["d"]), bool(g["transposed"]),
                                     bool(g["subm"]), algo, cdt, dtype)
    assert np.array_equal(oc, g["out_coords"])
    nbr = oracle.kernel_map(g["coords"], tuple(g["shape"]), int(g["k"]), int(g["s"]), int(g["d"]), int(g["p"]),
                            bool(g["transposed"]), bool(g["subm"]))[3]
    K, cin, cout = weight.shape
    tol = TOL[dtype]
    assert rel_err(y, oracle.conv_fwd(feats, weight, nbr)) < tol
    assert rel_err(dx, oracle.conv_dgrad(dy, weight, nbr, feats.shape[0])) < tol
    assert rel_err(dw, oracle.conv_wgrad(feats, dy, nbr, K, cin, cout)) < tol


@pytest.mark.parametrize("algo", ALGOS, ids=lambda a: a.name)
def test_c1_headline_case(cuda_device, oracle, algo):
    """SubMConv3D 16->32 k3, batch 2, 64^3, 4096 voxels, loss = sum(Y).  Maps are compared with
    the exact oracle (the reference's own map has a few aliased entries on this input, see
    test_oracle_golden.py); features with the oracle's fp32 result on the exact map, and -- on the
    rows the aliasing does not touch -- with the reference's stored output."""
    g = load_golden(golden_files("c1_")[0])
    dy = np.ones((4096, 32), np.float32)
    oc, ns, y, dx, dw, _ = run_conv(cuda_device, g["coords"], (64, 64, 64), 2, g["feats"], g["weight"], None, dy,
                                    3, 1, 1, 1, False, True, algo)
    assert np.array_equal(oc, g["coords"])
    exact = oracle.kernel_map(g["coords"], (64, 64, 64), 3, 1, 1, 1, False, True)[3]
    tol = TOL[torch.float32]
    assert rel_err(y, oracle.conv_fwd(g["feats"], g["weight"], exact)) < tol
    assert rel_err(dx, oracle.conv_dgrad(dy, g["weight"], exact, 4096)) < tol
    assert rel_err(dw, oracle.conv_wgrad(g["feats"], dy, exact, 27, 16, 32)) < tol
    clean_rows = (exact == g["nbr"]).all(axis=1)
    assert clean_rows.sum() >= 4096 - 4
    assert rel_err(y[clean_rows], g["y"][clean_rows]) < tol


def test_c1_map_is_exact(cuda_device, oracle):
    from test_gpu_kmap import gpu_kernel_map
    from gpu_util import ALGOS, map_triples
    g = load_golden(golden_files("c1_")[0])
    _, _, _, nbr = gpu_kernel_map(cuda_device, g["coords"], (64, 64, 64), 3, 1, 1, 1, False, True)
    exact = oracle.kernel_map(g["coords"], (64, 64, 64), 3, 1, 1, 1, False, True)[3]
    assert np.array_equal(nbr.cpu().numpy(), exact)
    assert np.array_equal(map_triples(nbr), oracle.pairs(exact))


SHAPES = [
    # n, grid, cin, cout, k, s, p, subm, transposed
    (30_000, 48, 32, 64, 3, 1, 1, True, False),
    (30_000, 48, 64, 128, 3, 2, 1, False, False),
    (30_000, 48, 64, 32, 2, 2, 0, False, False),
    (6_000, 24, 128, 64, 2, 2, 0, False, True),
    (20_000, 40, 4, 32, 3, 1, 1, True, False),
    (20_000, 40, 32, 20, 3, 1, 1, True, False),
    (10_000, 32, 256, 256, 3, 1, 1, True, False),
    (10_000, 32, 48, 96, 3, 1, 1, True, False),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16], ids=["fp32", "fp16", "bf16"])
@pytest.mark.parametrize("algo", ALGOS, ids=lambda a: a.name)
@pytest.mark.parametrize("n,grid,cin,cout,k,s,p,subm,transposed", SHAPES)
def test_random_vs_oracle(cuda_device, oracle, n, grid, cin, cout, k, s, p, subm, transposed, algo, dtype):
    """Mid-size layers (the channel widths of the benchmark networks) against the fp32 oracle."""
    gen = torch.Generator(device="cpu").manual_seed(n + cin + cout)
    cells = synthetic.surface_scene(77, grid=grid, target=n // 2, n_spheres=2, n_boxes=3)
    coords = synthetic.batch_of([cells, cells[: cells.shape[0] // 2]]).numpy()
    n_in = coords.shape[0]
    rnd = lambda t: t.to(dtype).float().numpy()
    feats = rnd(torch.randn(n_in, cin, generator=gen))
    weight = rnd((torch.rand(k ** 3, cin, cout, generator=gen) * 2 - 1) / (cin * k ** 3) ** 0.5)
    shape = (grid,) * 3
    oc_w, ns_w, _, nbr = oracle.kernel_map(coords, shape, k, s, 1, p, transposed, subm)
    dy = rnd(torch.randn(oc_w.shape[0], cout, generator=gen))
    oc, ns, y, dx, dw, _ = run_conv(cuda_device, coords, shape, 2, feats, weight, None, dy, k, s, p, 1, transposed,
                                    subm, algo, torch.int32, dtype)
    assert np.array_equal(oc, oc_w)
    tol = TOL[dtype]
    assert rel_err(y, oracle.conv_fwd(feats, weight, nbr)) < tol
    assert rel_err(dx, oracle.conv_dgrad(dy, weight, nbr, n_in)) < tol
    assert rel_err(dw, oracle.conv_wgrad(feats, dy, nbr, k ** 3, cin, cout)) < tol


# --- the reference's own known-answer tests (tests/test_sparse_conv.py), against dense PyTorch ---

@pytest.mark.parametrize("cin,cout,k,s,p,d", [(8, 16, 3, 1, 1, 1), (4, 8, 3, 2, 1, 1), (16, 16, 5, 2, 2, 1),
                                               (16, 16, 5, 1, 2, 1)])
def test_forward_matches_dense_conv3d(cuda_device, cin, cout, k, s, p, d):
    torch.backends.cudnn.allow_tf32 = False
    torch.manual_seed(0)
    sp = st.randn((10, 10, 10), batch_size=1, channels=cin, nnz=27, device=cuda_device).half()
    w = torch.rand(k ** 3, cin, cout, device=cuda_device, dtype=torch.float16)
    out = sparse_conv3d(sp, w, kernel_size=k, stride=s, padding=p, dilation=d, submanifold=False).float()
    wt = w.view(k, k, k, cin, cout).permute(4, 3, 0, 1, 2).contiguous().float()
    dense_in = sp.dense().permute(0, 4, 1, 2, 3).contiguous().float()
    dense_out = TF.conv3d(dense_in, wt, stride=s, padding=p, dilation=d).permute(0, 2, 3, 4, 1).contiguous()
    torch.testing.assert_close(out.dense(), dense_out, atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("cin,cout,k,s,p,d", [(16, 16, 3, 1, 1, 1), (32, 32, 5, 1, 2, 1), (4, 8, 3, 2, 1, 1),
                                               (8, 16, 3, 4, 1, 1)])
def test_transposed_matches_dense_conv_transpose3d(cuda_device, cin, cout, k, s, p, d):
    torch.backends.cudnn.allow_tf32 = False
    torch.manual_seed(1)
    sp = st.randn((10, 10, 10), batch_size=1, channels=cin, nnz=27, device=cuda_device).half()
    w = torch.rand(k ** 3, cin, cout, device=cuda_device, dtype=torch.float16) / k ** 3
    out = sparse_conv3d(sp, w, kernel_size=k, stride=s, padding=p, dilation=d, submanifold=False,
                        transposed=True).float()
    wt = w.view(k, k, k, cin, cout).permute(3, 4, 0, 1, 2).contiguous().float()
    dense_in = sp.dense().permute(0, 4, 1, 2, 3).contiguous().float()
    dense_out = TF.conv_transpose3d(dense_in, wt, stride=s, padding=p, dilation=d).permute(0, 2, 3, 4, 1).contiguous()
    torch.testing.assert_close(out.dense(), dense_out, atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("cin,cout,k,s,p,d", [(16, 16, 3, 1, 2, 1), (32, 32, 3, 1, 0, 1), (16, 16, 3, 2, 1, 1),
                                               (16, 16, 3, 2, 1, 2)])
def test_gradients_vs_dense(cuda_device, cin, cout, k, s, p, d):
    torch.backends.cudnn.allow_tf32 = False
    torch.manual_seed(2)
    sp = st.randn((24, 24, 24), batch_size=1, channels=cin, nnz=12 ** 3, device=cuda_device)
    feats = sp.F.detach().half().requires_grad_(True)
    sp.F = feats
    w = (torch.randn(k ** 3, cin, cout, device=cuda_device, dtype=torch.float16) / k ** 3).requires_grad_(True)
    out = sparse_conv3d(sp, w, kernel_size=k, stride=s, padding=p, dilation=d, submanifold=False)
    out.dense().float().abs().mean().backward()
    gw, gf = w.grad.clone(), feats.grad.clone()
    w2 = w.detach().clone().requires_grad_(True)
    wt = w2.view(k, k, k, cin, cout).permute(4, 3, 0, 1, 2).contiguous()
    dense_in = sp.dense().permute(0, 4, 1, 2, 3).contiguous().detach().requires_grad_(True)
    dense_out = TF.conv3d(dense_in, wt, stride=s, padding=p, dilation=d).permute(0, 2, 3, 4, 1).contiguous()
    dense_out.float().abs().mean().backward()
    c = sp.coords.long()
    dense_gf = dense_in.grad.permute(0, 2, 3, 4, 1)[c[:, 0], c[:, 1], c[:, 2], c[:, 3]]
    torch.testing.assert_close(w2.grad, gw, atol=5e-2, rtol=5e-2)
    torch.testing.assert_close(dense_gf, gf, atol=5e-2, rtol=5e-2)


def test_submanifold_keeps_coords_and_cache(cuda_device):
    sp = st.randn((10, 10, 10), batch_size=1, channels=8, nnz=100, device=cuda_device).half()
    w = torch.rand(27, 8, 16, device=cuda_device, dtype=torch.float16)
    out = sparse_conv3d(sp, w, kernel_size=3, submanifold=True)
    assert torch.equal(out.coords, sp.coords) and out.F.shape == (100, 16)
    assert out._cache is sp._cache and sp._cache.hashtable is not None
    assert (3, 1, 1, 1, True, False) in sp._cache.neighbor_indices
    out2 = sparse_conv3d(out, torch.rand(27, 16, 8, device=cuda_device, dtype=torch.float16), kernel_size=3)
    assert len(sp._cache.neighbor_indices) == 1 and out2.F.shape == (100, 8)


@pytest.mark.parametrize("k,s,p,subm,transposed", [(3, 1, 1, True, False), (3, 2, 1, False, False), (2, 2, 0, False, False),
                                                   (2, 2, 0, False, True)])
def test_prepared_on_a_side_stream(cuda_device, k, s, p, subm, transposed):
    """prepare_conv3d under a second stream, then the layer on the first: same bits as the layer alone, and the layer
    then builds nothing of its own."""
    from sparsetriton_b200 import trace
    from sparsetriton_b200.nn.functional import ConvPreparation, prepare_conv3d
    set_conv_algo(ConvAlgo.PrecomputedNeighborGEMM)
    set_coords_dtype(torch.int32)
    n, grid, cin, cout = 40_000, 96, 32, 64
    coords = synthetic.random_cells(n, 2, grid, 77).to(cuda_device)
    gen = torch.Generator().manual_seed(78)
    feats = torch.randn(n, cin, generator=gen).to(torch.bfloat16).to(cuda_device)
    weight = (torch.randn(k ** 3, cin, cout, generator=gen) * 0.05).to(torch.bfloat16).to(cuda_device)

    def layer(cache):
        x, w = feats.clone().requires_grad_(True), weight.clone().requires_grad_(True)
        sp = st.SparseTensor(x, coords, (grid,) * 3, 2, cache=cache)
        out = sparse_conv3d(sp, w, kernel_size=k, stride=s, padding=p, submanifold=subm, transposed=transposed)
        dy = torch.ones_like(out.F) * 0.25
        dx, dw = torch.autograd.grad(out.F, [x, w], dy)
        return out.C, out.F, dx, dw

    want = layer(None)
    main, side = torch.cuda.current_stream(cuda_device), torch.cuda.Stream(cuda_device)
    side.wait_stream(main)
    with torch.cuda.stream(side):
        cache = prepare_conv3d(coords, (grid,) * 3, kernel_size=k, stride=s, padding=p, submanifold=subm,
                               transposed=transposed, consumer_stream=main)
        # two preparations in flight, begun before either is finished
        first, second = (ConvPreparation(coords, (grid,) * 3, kernel_size=k, stride=s, padding=p, submanifold=subm,
                                         transposed=transposed, consumer_stream=main) for _ in range(2))
        caches = [cache, first.finish(), second.finish()]
        ready = torch.cuda.Event()
        ready.record(side)
    main.wait_event(ready)
    for cache in caches:
        with trace.recording() as rec:
            got = layer(cache)
            torch.cuda.synchronize(cuda_device)
            stages = set(rec.summary())
        assert stages <= {"conv_fwd", "conv_dgrad", "conv_wgrad"}, stages
        for a, b in zip(got, want):
            assert torch.equal(a, b)


def test_empty_and_errors(cuda_device):
    set_coords_dtype(torch.int32)
    empty = st.SparseTensor(torch.empty(0, 4, device=cuda_device), torch.empty(0, 4, dtype=torch.int32),
                            spatial_shape=(8, 8, 8), batch_size=1)
    w = torch.rand(27, 4, 8, device=cuda_device)
    out = sparse_conv3d(empty, w, kernel_size=3, stride=2, padding=1, submanifold=False)
    assert out.F.shape == (0, 8) and out.C.shape == (0, 4)
    sp = st.randn((8, 8, 8), channels=4, nnz=20, device=cuda_device)
    with pytest.raises(AssertionError, match="Input channels"):
        sparse_conv3d(sp, torch.rand(27, 5, 8, device=cuda_device), kernel_size=3)
    with pytest.raises(AssertionError, match="Kernel size"):
        sparse_conv3d(sp, torch.rand(8, 4, 8, device=cuda_device), kernel_size=3)
    with pytest.raises(AssertionError, match="does not support transposed"):
        sparse_conv3d(sp, w, kernel_size=3, transposed=True, submanifold=True)
    with pytest.raises(AssertionError, match="Only cubic kernels"):
        sparse_conv3d(sp, w, kernel_size=(3, 3, 1))
    cpu = st.randn((8, 8, 8), channels=4, nnz=20, device="cpu")
    with pytest.raises(RuntimeError, match="no CPU path"):
        sparse_conv3d(cpu, torch.rand(27, 4, 8), kernel_size=3)


def test_modules(cuda_device):
    from sparsetriton_b200.nn import SparseConv3D, SparseConvTransposed3D, SubMConv3D
    sp = st.randn((16, 16, 16), batch_size=2, channels=4, nnz=300, device=cuda_device)
    sub = SubMConv3D(4, 8, 3).to(cuda_device)
    assert sub.weight.shape == (27, 4, 8) and sub.bias.shape == (8,) and sub.kernel_size == (3, 3, 3)
    y = sub(sp)
    assert torch.equal(y.coords, sp.coords) and y.F.shape == (300, 8)
    down = SparseConv3D(8, 16, 2, stride=2).to(cuda_device)(y)
    assert down.spatial_shape == torch.Size([8, 8, 8]) and down.F.shape[1] == 16
    up = SparseConvTransposed3D(16, 8, 2, stride=2).to(cuda_device)(down)
    assert up.spatial_shape == torch.Size([16, 16, 16]) and up.batch_size == 2
    up.F.sum().backward()
    assert sub.weight.grad is not None and torch.isfinite(sub.weight.grad).all()


def test_status_word_can_be_cleared_and_rides_with_the_output_count(cuda_device):
    """st_device_status_enqueue / _clear: the sticky word is read without a synchronisation of its own (here through
    the wait a strided layer makes for its output count) and stays 0 on a healthy run; clearing is stream-ordered."""
    import ctypes
    from sparsetriton_b200 import _lib
    _lib.clear_device_status(cuda_device)
    assert _lib.device_status(cuda_device)[0] == 0
    words = torch.full((4,), -1, dtype=torch.int32).pin_memory()
    with torch.cuda.device(cuda_device):
        _lib.check(_lib.lib().st_device_status_enqueue(ctypes.c_void_p(words.data_ptr()), _lib.stream_ptr()),
                   "st_device_status_enqueue")
    torch.cuda.synchronize(cuda_device)
    assert words.tolist()[0] == 0
    _lib.raise_on_timeout(words, cuda_device)                       # nothing expired: no exception
    with pytest.raises(RuntimeError, match="bounded wait"):
        _lib.raise_on_timeout([_lib.DEV_TIMEOUT, 33, 7, 0], cuda_device)   # host-side: what a caller would see
    sp = st.randn((24, 24, 24), batch_size=2, channels=16, nnz=3000, device=cuda_device)
    out = sparse_conv3d(sp, torch.rand(27, 16, 32, device=cuda_device), kernel_size=3, stride=2, padding=1, submanifold=False)
    assert out.F.shape[1] == 32 and out.F.shape[0] > 0
