"""Row order and tile plan of a neighbour map (st_map_row_order, st_map_plan) and the products
that walk the map through them.

The order must be the stable sort of the rows by their occupancy mask; the plan must be the map
re-laid tile by tile in that order with exact tile masks; forward and feature gradient must give
bit-identical results with and without a plan (a row's own sum never changes), the weight gradient
the same result within the storage tolerance (its row sum is reordered).
"""
import numpy as np
import pytest
import torch

from gpu_util import TOL, rel_err, t2n
from sparsetriton_b200 import _lib

pytestmark = pytest.mark.gpu


def _random_map(n_rows, n_src, K, density, seed, dev, patterns=None):
    """A map like a convolution's: within one offset no source row is used twice (so the inverse
    map exists); rows optionally draw their occupied offsets from a few masks."""
    g = torch.Generator().manual_seed(seed)
    if patterns:
        masks = torch.rand(patterns, K, generator=g) < density
        keep = masks[torch.randint(0, patterns, (n_rows,), generator=g)]
    else:
        keep = torch.rand(n_rows, K, generator=g) < density
    nbr = torch.full((n_rows, K), -1, dtype=torch.int32)
    for k in range(K):
        rows = torch.nonzero(keep[:, k]).flatten()
        rows = rows[:n_src]
        nbr[rows, k] = torch.randperm(n_src, generator=g)[:rows.numel()].to(torch.int32)
    return nbr.to(dev)


def _order(nbr):
    L = _lib.lib()
    n, K = nbr.shape
    order = torch.full((n,), -7, dtype=torch.int32, device=nbr.device)
    ws = _lib.workspace(L.st_map_row_order_workspace_bytes(n, K), nbr.device)
    with torch.cuda.device(nbr.device):
        _lib.check(L.st_map_row_order(_lib.ptr(nbr), n, K, _lib.ptr(order), _lib.ptr(ws), ws.numel(),
                                      _lib.stream_ptr()), "st_map_row_order")
    return order


@pytest.mark.parametrize("n_rows,K,density,patterns", [
    (1, 27, 0.5, None), (127, 27, 0.3, None), (5000, 27, 0.3, 40), (70001, 27, 0.2, None), (3000, 8, 0.5, None),
    (4097, 1, 0.5, None), (2500, 32, 0.4, 9), (1500, 125, 0.1, 12), (900, 343, 0.05, 5)])
def test_order_is_the_stable_sort_by_mask(cuda_device, n_rows, K, density, patterns):
    nbr = _random_map(n_rows, 1000, K, density, 11 + n_rows + K, cuda_device, patterns)
    order = _order(nbr).cpu().numpy().astype(np.int64)
    assert np.array_equal(np.sort(order), np.arange(n_rows))                  # a permutation
    occ = (nbr.cpu().numpy() >= 0)
    if K <= 32:
        key = (occ.astype(np.uint64) << np.arange(K, dtype=np.uint64)).sum(1)
        assert np.array_equal(order, np.argsort(key, kind="stable"))
    else:
        # beyond 32 offsets the key is a hash of the pattern: equal patterns stay together, in row order
        packed = np.packbits(occ, axis=1)
        sorted_patterns = packed[order]
        change = np.any(sorted_patterns[1:] != sorted_patterns[:-1], axis=1)
        n_groups = 1 + int(change.sum())
        assert n_groups == len(np.unique(packed, axis=0))
        same = ~change
        assert np.all(order[1:][same] > order[:-1][same])
    again = _order(nbr).cpu().numpy()
    assert np.array_equal(again, order)                                        # run-to-run identical


def _plan(nbr, sort_rows):
    L = _lib.lib()
    n, K = nbr.shape
    dev = nbr.device
    n_tiles, MW = (n + 127) // 128, (K + 31) // 32
    order = torch.full((n,), -7, dtype=torch.int32, device=dev) if sort_rows else None
    tmap = torch.full((n_tiles * K * 128,), -9, dtype=torch.int32, device=dev)
    tmask = torch.full((n_tiles * MW,), -9, dtype=torch.int32, device=dev)
    ws = _lib.workspace(L.st_map_plan_workspace_bytes(n, K), dev)
    with torch.cuda.device(dev):
        _lib.check(L.st_map_plan(_lib.ptr(nbr), n, K, 1 if sort_rows else 0, _lib.ptr(order), _lib.ptr(tmap),
                                 _lib.ptr(tmask), _lib.ptr(ws), ws.numel(), _lib.stream_ptr()), "st_map_plan")
    return order, tmap, tmask


@pytest.mark.parametrize("sort_rows", [False, True], ids=["natural", "sorted"])
@pytest.mark.parametrize("n_rows,K,density", [(1, 27, 0.5), (128, 27, 0.3), (129, 8, 0.4), (5000, 27, 0.2),
                                              (1000, 64, 0.1), (700, 125, 0.05), (300, 343, 0.02)])
def test_plan_is_the_relaid_map(cuda_device, n_rows, K, density, sort_rows):
    nbr = _random_map(n_rows, 3000, K, density, 7 + n_rows, cuda_device, patterns=15)
    order, tmap, tmask = _plan(nbr, sort_rows)
    m = nbr.cpu().numpy()
    n_tiles, MW = (n_rows + 127) // 128, (K + 31) // 32
    if sort_rows:
        o = order.cpu().numpy().astype(np.int64)
        assert np.array_equal(o, _order(nbr).cpu().numpy())
    else:
        o = np.arange(n_rows)
    padded = np.full((n_tiles * 128, K), -1, np.int32)
    padded[:n_rows] = m[o]
    want = padded.reshape(n_tiles, 128, K).transpose(0, 2, 1)                  # (tile, k, r)
    assert np.array_equal(tmap.cpu().numpy().reshape(n_tiles, K, 128), want)
    bits = (want >= 0).any(axis=2)                                             # (tile, k)
    want_mask = np.zeros((n_tiles, MW), np.uint32)
    for k in range(K):
        want_mask[:, k // 32] |= bits[:, k].astype(np.uint32) << np.uint32(k % 32)
    assert np.array_equal(tmask.cpu().numpy().view(np.uint32).reshape(n_tiles, MW), want_mask)


def test_empty_map(cuda_device):
    L = _lib.lib()
    assert L.st_map_row_order(None, 0, 27, None, None, 0, _lib.stream_ptr()) == 0
    assert L.st_map_row_order(None, 5, 27, None, None, 0, _lib.stream_ptr()) == -1
    assert L.st_map_plan(None, 0, 27, 1, None, None, None, None, 0, _lib.stream_ptr()) == 0
    assert L.st_map_plan(None, 5, 27, 1, None, None, None, None, 0, _lib.stream_ptr()) == -1


@pytest.mark.parametrize("form", ["order_only", "plan_natural", "plan_sorted", "plan_sorted_cp_async"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16], ids=["fp32", "bf16", "fp16"])
@pytest.mark.parametrize("n_rows,n_src,K,cin,cout,patterns", [
    (3000, 2000, 27, 32, 64, 20), (70001, 40000, 27, 64, 128, None), (5000, 5000, 8, 16, 16, None),
    (20000, 9000, 27, 128, 64, 30), (9000, 9000, 125, 32, 32, 25), (2000, 2500, 27, 256, 256, 6)])
def test_products_with_plan(cuda_device, oracle, dtype, form, n_rows, n_src, K, cin, cout, patterns):
    dev = cuda_device
    L = _lib.lib()
    nbr = _random_map(n_rows, n_src, K, 0.25, 5, dev, patterns)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(n_src, cin, generator=g).to(dev, dtype)
    w = (torch.randn(K, cin, cout, generator=g) / (cin * K * 0.25) ** 0.5).to(dev, dtype)
    dy = torch.randn(n_rows, cout, generator=g).to(dev, dtype)
    code = _lib.feat_code(x)
    inv = torch.empty((n_src, K), dtype=torch.int32, device=dev)
    y0, y1 = torch.empty(n_rows, cout, device=dev, dtype=dtype), torch.full((n_rows, cout), 7.0, device=dev, dtype=dtype)
    dx0, dx1 = torch.empty_like(x), torch.full_like(x, 7.0)
    dw0, dw1 = torch.empty_like(w), torch.full_like(w, 7.0)
    ws = _lib.workspace(L.st_conv_workspace_bytes(code, n_src, n_rows, K, cin, cout), dev)
    with torch.cuda.device(dev):
        s = _lib.stream_ptr()
        _lib.check(L.st_map_invert(_lib.ptr(nbr), n_rows, K, n_src, _lib.ptr(inv), s), "st_map_invert")
        if form == "order_only":
            fp, ip = (_order(nbr), None, None), (_order(inv), None, None)
        else:
            fp, ip = _plan(nbr, form != "plan_natural"), _plan(inv, form != "plan_natural")
        # the cp.async forms of the planned kernels (what runs when TMA cannot describe a tensor)
        L.st_set_tma(0 if form == "plan_sorted_cp_async" else 1)
        p = _lib.ptr
        fpp, ipp = [p(v) for v in fp], [p(v) for v in ip]
        _lib.check(L.st_conv_fwd(code, p(x), p(w), p(nbr), p(y0), n_src, n_rows, K, cin, cout, None, 0, s), "fwd")
        _lib.check(L.st_conv_fwd_planned(code, p(x), p(w), p(nbr), *fpp, p(y1), n_src, n_rows, K, cin, cout, None,
                                         0, s), "fwd planned")
        _lib.check(L.st_conv_dgrad(code, p(dy), p(w), p(inv), p(dx0), n_src, n_rows, K, cin, cout, None, 0, s), "dgrad")
        _lib.check(L.st_conv_dgrad_planned(code, p(dy), p(w), p(inv), *ipp, p(dx1), n_src, n_rows, K, cin, cout,
                                           None, 0, s), "dgrad planned")
        _lib.check(L.st_conv_wgrad(code, p(x), p(dy), p(nbr), p(dw0), n_src, n_rows, K, cin, cout, p(ws), ws.numel(), s),
                   "wgrad")
        _lib.check(L.st_conv_wgrad_planned(code, p(x), p(dy), p(nbr), *fpp, p(dw1), n_src, n_rows, K, cin, cout,
                                           p(ws), ws.numel(), s), "wgrad planned")
        torch.cuda.synchronize()
        L.st_set_tma(1)
    assert _lib.device_status(dev)[0] == 0
    assert torch.equal(y0, y1)
    assert torch.equal(dx0, dx1)
    tol = TOL[dtype]
    assert rel_err(t2n(dw1), t2n(dw0)) < tol
    xf, wf, dyf, m = t2n(x), t2n(w), t2n(dy), nbr.cpu().numpy()
    assert rel_err(t2n(y1), oracle.conv_fwd(xf, wf, m)) < tol
    assert rel_err(t2n(dx1), oracle.conv_dgrad(dyf, wf, m, n_src)) < tol
    assert rel_err(t2n(dw1), oracle.conv_wgrad(xf, dyf, m, K, cin, cout)) < tol


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32], ids=["bf16", "fp32"])
@pytest.mark.parametrize("n_rows,n_src,K,cin,cout,copies", [(70001, 40000, 27, 64, 128, True), (9000, 12000, 27, 128, 128, True),
                                                            (5000, 5000, 27, 32, 64, None), (3000, 3000, 8, 16, 16, False)])
def test_wgrad_in_two_calls(cuda_device, dtype, n_rows, n_src, K, cin, cout, copies):
    """st_conv_wgrad_presort on a second stream + st_conv_wgrad_planned_presorted give st_conv_wgrad_planned's dW bit
    for bit; a layer without a sorted copy answers ST_ERR_UNSUPPORTED and launches nothing."""
    dev = cuda_device
    L = _lib.lib()
    nbr = _random_map(n_rows, n_src, K, 0.25, 11, dev, 20)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(n_src, cin, generator=g).to(dev, dtype)
    dy = torch.randn(n_rows, cout, generator=g).to(dev, dtype)
    code = _lib.feat_code(x)
    dw0 = torch.full((K, cin, cout), 7.0, device=dev, dtype=dtype)
    dw1 = torch.full_like(dw0, 9.0)
    nbytes = L.st_conv_workspace_bytes(code, n_src, n_rows, K, cin, cout)
    ws0, ws1 = _lib.workspace(nbytes, dev), _lib.workspace(nbytes, dev)
    p = _lib.ptr
    with torch.cuda.device(dev):
        s = _lib.stream_ptr()
        fpp = [p(v) for v in _plan(nbr, True)]
        _lib.check(L.st_conv_wgrad_planned(code, p(x), p(dy), p(nbr), *fpp, p(dw0), n_src, n_rows, K, cin, cout, p(ws0),
                                           ws0.numel(), s), "wgrad planned")
        cur, aux = torch.cuda.current_stream(dev), torch.cuda.Stream(device=dev)
        aux.wait_stream(cur)
        with torch.cuda.stream(aux):
            rc = L.st_conv_wgrad_presort(code, p(dy), fpp[0], n_rows, K, cin, cout, p(ws1), ws1.numel(), _lib.stream_ptr())
        if copies is not None:
            assert (rc == 0) == copies
        if rc == 0:
            cur.wait_stream(aux)
            _lib.check(L.st_conv_wgrad_planned_presorted(code, p(x), p(dy), p(nbr), *fpp, p(dw1), n_src, n_rows, K, cin, cout,
                                                         p(ws1), ws1.numel(), s), "wgrad planned presorted")
        else:
            assert rc == -5
        torch.cuda.synchronize()
    assert _lib.device_status(dev)[0] == 0
    if rc == 0:
        assert torch.equal(dw0, dw1)


@pytest.mark.parametrize("n_rows,n_src,K,density,patterns", [(5000, 4000, 27, 0.25, 20), (70001, 50000, 27, 0.2, None),
                                                              (3000, 9000, 8, 0.5, None), (900, 700, 1, 0.6, None),
                                                              (40000, 30000, 32, 0.1, 50)])
def test_inverse_plan_from_the_forward_map(cuda_device, n_rows, n_src, K, density, patterns):
    """st_map_plan_inverse must give exactly the arrays of st_map_invert + st_map_plan(sorted)."""
    dev = cuda_device
    L = _lib.lib()
    nbr = _random_map(n_rows, n_src, K, density, 77 + K, dev, patterns)
    inv = torch.empty((n_src, K), dtype=torch.int32, device=dev)
    n_tiles = (n_src + 127) // 128
    order = torch.full((n_src,), -7, dtype=torch.int32, device=dev)
    tmap = torch.full((n_tiles * K * 128,), -9, dtype=torch.int32, device=dev)
    tmask = torch.full((n_tiles,), -9, dtype=torch.int32, device=dev)
    ws = _lib.workspace(L.st_map_plan_inverse_workspace_bytes(n_src, K), dev)
    with torch.cuda.device(dev):
        s = _lib.stream_ptr()
        _lib.check(L.st_map_invert(_lib.ptr(nbr), n_rows, K, n_src, _lib.ptr(inv), s), "st_map_invert")
        want = _plan(inv, True)
        _lib.check(L.st_map_plan_inverse(_lib.ptr(nbr), n_rows, K, n_src, _lib.ptr(order), _lib.ptr(tmap), _lib.ptr(tmask),
                                         _lib.ptr(ws), ws.numel(), s), "st_map_plan_inverse")
        torch.cuda.synchronize()
    assert torch.equal(order, want[0])
    assert torch.equal(tmap, want[1])
    assert torch.equal(tmask, want[2])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16], ids=["fp32", "bf16", "fp16"])
@pytest.mark.parametrize("n_rows,n_src,K,cin,cout,patterns", [(5000, 9000, 27, 64, 128, 20), (20001, 30000, 27, 32, 64, None),
                                                              (3000, 6001, 8, 128, 256, None), (900, 2000, 27, 16, 8, 5),
                                                              (129, 130, 27, 64, 64, None)])
def test_wgrad_over_the_inverse_plan(cuda_device, oracle, dtype, n_rows, n_src, K, cin, cout, patterns):
    """st_conv_wgrad_inverse_planned (tiles of input rows, dY gathered) against the oracle and against the
    forward-plan form; rows of X without any output (zero masks) and a ragged last tile included."""
    dev = cuda_device
    L = _lib.lib()
    nbr = _random_map(n_rows, n_src, K, 0.3, 5 + n_rows + K, dev, patterns)
    g = torch.Generator().manual_seed(n_rows)
    x = torch.randn(n_src, cin, generator=g).to(dtype).to(dev)
    dy = torch.randn(n_rows, cout, generator=g).to(dtype).to(dev)
    code = _lib.feat_code(x)
    if not L.st_conv_uses_tensor_cores(code, cin, cout):
        pytest.skip("shape served by the CUDA-core kernels")
    n_tiles = (n_src + 127) // 128
    order = torch.empty((n_src,), dtype=torch.int32, device=dev)
    tmap = torch.empty((n_tiles * K * 128,), dtype=torch.int32, device=dev)
    tmask = torch.empty((n_tiles,), dtype=torch.int32, device=dev)
    dw_inv = torch.empty((K, cin, cout), dtype=dtype, device=dev)
    dw_fwd = torch.empty_like(dw_inv)
    p = _lib.ptr
    with torch.cuda.device(dev):
        s = _lib.stream_ptr()
        ws = _lib.workspace(L.st_map_plan_inverse_workspace_bytes(n_src, K), dev)
        _lib.check(L.st_map_plan_inverse(p(nbr), n_rows, K, n_src, p(order), p(tmap), p(tmask), p(ws), ws.numel(), s),
                   "st_map_plan_inverse")
        ws2 = _lib.workspace(L.st_conv_wgrad_inverse_workspace_bytes(code, n_src, K, cin, cout), dev)
        _lib.check(L.st_conv_wgrad_inverse_planned(code, p(x), p(dy), p(order), p(tmap), p(tmask), p(dw_inv), n_src, n_rows, K,
                                                   cin, cout, p(ws2), ws2.numel(), s), "st_conv_wgrad_inverse_planned")
        ws3 = _lib.workspace(L.st_conv_workspace_bytes(code, n_src, n_rows, K, cin, cout), dev)
        _lib.check(L.st_conv_wgrad(code, p(x), p(dy), p(nbr), p(dw_fwd), n_src, n_rows, K, cin, cout, p(ws3), ws3.numel(), s),
                   "st_conv_wgrad")
        torch.cuda.synchronize()
    assert _lib.device_status(dev)[0] == 0
    want = oracle.conv_wgrad(t2n(x), t2n(dy), nbr.cpu().numpy(), K, cin, cout)
    tol = TOL[dtype]
    assert rel_err(t2n(dw_inv), want) < tol
    assert rel_err(t2n(dw_inv), t2n(dw_fwd)) < tol
