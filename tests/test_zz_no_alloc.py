"""The allocation-free weight gradient, st_conv_wgrad_static().

Some hosts of this library may not allocate device memory around a call: the memory pool belongs to
another runtime, or allocation is forbidden after start-up.  For them the library carries one entry
point whose scratch (the fp32 partial sums of the weight gradient) is a fixed 64 MiB array inside
the library instead of a caller-provided workspace.  This test calls it through the C ABI and checks
that it returns exactly what st_conv_wgrad() returns with a workspace, twice in a row with
different inputs (the second call finds the first call's partials still in the array), and that a
layer too large for the array is refused with a clear message.

Collected last on purpose (file name), so a failure here cannot hide another test's result.
"""
import numpy as np
import pytest
import torch

from sparsetriton_b200 import _lib

pytestmark = pytest.mark.gpu


def _inputs(dev, n_rows, n_src, K, cin, cout, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    nbr = torch.randint(0, n_src, (n_rows, K), generator=g, dtype=torch.int32)
    nbr[torch.rand(n_rows, K, generator=g) > 0.3] = -1
    x = torch.randn(n_src, cin, generator=g).to(dtype)
    dy = torch.randn(n_rows, cout, generator=g).to(dtype)
    return x.to(dev), dy.to(dev), nbr.to(dev)


def _with_workspace(x, dy, nbr, K, cin, cout):
    L = _lib.lib()
    code = _lib.feat_code(x)
    ws = _lib.workspace(L.st_conv_workspace_bytes(code, x.shape[0], nbr.shape[0], K, cin, cout), x.device)
    dw = torch.empty(K, cin, cout, dtype=x.dtype, device=x.device)
    _lib.check(L.st_conv_wgrad(code, _lib.ptr(x), _lib.ptr(dy), _lib.ptr(nbr), _lib.ptr(dw), x.shape[0], nbr.shape[0],
                               K, cin, cout, _lib.ptr(ws), ws.numel(), _lib.stream_ptr()), "st_conv_wgrad")
    return dw


def _static(x, dy, nbr, K, cin, cout):
    L = _lib.lib()
    dw = torch.empty(K, cin, cout, dtype=x.dtype, device=x.device)
    rc = L.st_conv_wgrad_static(_lib.feat_code(x), _lib.ptr(x), _lib.ptr(dy), _lib.ptr(nbr), _lib.ptr(dw),
                                x.shape[0], nbr.shape[0], K, cin, cout, _lib.stream_ptr())
    return rc, dw


@pytest.mark.parametrize("cin,cout,dtype", [(64, 128, torch.bfloat16), (32, 64, torch.float32), (4, 20, torch.float16)])
def test_matches_workspace_entry_point_twice(cuda_device, oracle, cin, cout, dtype):
    K = 27
    with torch.cuda.device(cuda_device):
        for call, (n_rows, seed) in enumerate([(20_000, 1), (9_000, 2)]):
            x, dy, nbr = _inputs(cuda_device, n_rows, n_rows // 2, K, cin, cout, dtype, seed)
            want = _with_workspace(x, dy, nbr, K, cin, cout)
            rc, got = _static(x, dy, nbr, K, cin, cout)
            _lib.check(rc, "st_conv_wgrad_static")
            torch.cuda.synchronize()
            # same kernels, same fixed summation order: the two entry points agree to the bit; the
            # suite's tolerance for this dtype is the stated bound
            tol = 2e-3 if dtype == torch.float32 else 1e-2
            w, g = want.float().cpu().numpy(), got.float().cpu().numpy()
            assert np.abs(g - w).max() <= tol * max(np.abs(w).max(), 1e-30), f"call {call}"
            assert np.array_equal(g, w), f"call {call}: not bit-identical"
            # and the entry point's own parity line: the fp32 CPU oracle on the same inputs
            ref = oracle.conv_wgrad(x.float().cpu().numpy(), dy.float().cpu().numpy(), nbr.cpu().numpy(), K, cin, cout)
            assert np.abs(g - ref).max() <= tol * max(np.abs(ref).max(), 1e-30), f"call {call}: differs from the oracle"
    assert _lib.device_status(cuda_device)[0] == 0


def test_refuses_a_layer_that_does_not_fit(cuda_device):
    L = _lib.lib()
    limit = L.st_conv_wgrad_static_max_bytes()
    assert limit == 64 << 20
    K, cin, cout = 125, 256, 512                      # one chunk of partials alone is 65.5 MB
    with torch.cuda.device(cuda_device):
        x, dy, nbr = _inputs(cuda_device, 256, 128, K, cin, cout, torch.float32, 3)
        rc, _ = _static(x, dy, nbr, K, cin, cout)
    assert rc == -3
    msg = L.st_last_error_string().decode()
    assert "built-in scratch" in msg and str(limit) in msg
