"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

import sparsetriton_b200 as st
from sparsetriton_b200 import _lib
from sparsetriton_b200.config import ConvAlgo, set_conv_algo, set_coords_dtype, set_hashfly_transient_map
from sparsetriton_b200.nn.functional import sparse_conv3d

TOL = {torch.float32: 2e-3, torch.float16: 1e-2, torch.bfloat16: 1e-2}


class Algo:
    """A convolution algorithm as the tests select it: the reference's two ConvAlgo values, the hash-on-the-fly one
    in both of its forms here (scratch map per call / probing inside the kernels)."""

    def __init__(self, algo, transient, name):
        self.algo, self.transient, self.name = algo, transient, name

    def use(self):
        set_conv_algo(self.algo)
        set_hashfly_transient_map(self.transient)


ALGOS = [Algo(ConvAlgo.PrecomputedNeighborGEMM, True, "PrecomputedNeighborGEMM"),
         Algo(ConvAlgo.ImplicitHashFlyGEMM, True, "ImplicitHashFlyGEMM"),
         Algo(ConvAlgo.ImplicitHashFlyGEMM, False, "ImplicitHashFlyGEMM_in_kernel")]


def rel_err(got, want):
    """max |got - want| / max |want|  (max-norm relative error)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    denom = max(float(np.abs(want).max()) if want.size else 0.0, 1e-30)
    return float(np.abs(got - want).max()) / denom if want.size else 0.0


def rms_err(got, want):
    """||got - want||_2 / ||want||_2 over the whole array."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    denom = max(float(np.sqrt((want * want).sum())), 1e-30)
    return float(np.sqrt(((got - want) ** 2).sum())) / denom if want.size else 0.0


def row_err(got, want, floor=0.05):
    """Largest per-row relative error, ||got_r - want_r||_2 / max(||want_r||_2, floor * median row norm): a row of
    small magnitude is measured against its own size (down to `floor` of the typical row), not against the
    largest entry of the matrix as rel_err does."""
    got = np.asarray(got, dtype=np.float64).reshape(len(got), -1)
    want = np.asarray(want, dtype=np.float64).reshape(len(want), -1)
    if want.size == 0:
        return 0.0
    norms = np.sqrt((want * want).sum(1))
    scale = np.maximum(norms, floor * max(float(np.median(norms)), 1e-30))
    return float((np.sqrt(((got - want) ** 2).sum(1)) / scale).max())


def check_close(got, want, tol, what=""):
    """The feature bar in three norms: max-norm relative (rel_err) and RMS relative below `tol`, and the worst
    row, measured against its own norm, below 4 x tol."""
    errs = (rel_err(got, want), rms_err(got, want), row_err(got, want))
    assert errs[0] < tol and errs[1] < tol and errs[2] < 4 * tol, f"{what}: max-norm {errs[0]:.2e} rms {errs[1]:.2e} " \
                                                                   f"worst row {errs[2]:.2e} (tol {tol:.0e})"
    return errs


def t2n(t):
    return t.detach().float().cpu().numpy() if t.is_floating_point() else t.detach().cpu().numpy()


def run_conv(dev, coords, shape, batch, feats, weight, bias, dy, k, s, p, d, transposed, subm, algo,
             coord_dtype=torch.int32, dtype=torch.float32):
    """sparse_conv3d forward + backward through the public API.  Returns numpy
    (out_coords, new_shape, y, dx, dw, db)."""
    set_coords_dtype(coord_dtype)
    algo.use() if isinstance(algo, Algo) else set_conv_algo(algo)
    x = torch.as_tensor(feats).to(dev, dtype).requires_grad_(True)
    w = torch.as_tensor(weight).to(dev, dtype).requires_grad_(True)
    b = None
    if bias is not None and np.size(bias):
        b = torch.as_tensor(bias).to(dev, dtype).requires_grad_(True)
    sp = st.SparseTensor(x, torch.as_tensor(coords).to(dev), spatial_shape=tuple(int(v) for v in shape),
                         batch_size=int(batch))
    out = sparse_conv3d(sp, w, kernel_size=k, bias=b, stride=s, dilation=d, padding=p, transposed=transposed,
                        submanifold=subm)
    g = torch.as_tensor(dy).to(dev, dtype)
    (out.F.float() * g.float()).sum().backward()
    return (t2n(out.C).astype(np.int32), np.array(out.spatial_shape), t2n(out.F), t2n(x.grad), t2n(w.grad),
            None if b is None else t2n(b.grad))


def map_triples(nbr):
    """(in, out, offset) triples of a device neighbour map via st_map_pairs_* (C ABI)."""
    L = _lib.lib()
    n_out, K = nbr.shape
    dev = nbr.device
    ws = _lib.workspace(L.st_map_pairs_workspace_bytes(n_out, K), dev)
    counters = torch.zeros(2, dtype=torch.int64, device=dev)
    status = counters[1:].view(torch.int32)
    with torch.cuda.device(dev):
        s = _lib.stream_ptr()
        _lib.check(L.st_map_pairs_count(_lib.ptr(nbr), n_out, K, _lib.ptr(ws), ws.numel(), _lib.ptr(counters), s),
                   "st_map_pairs_count")
        n_pairs = int(counters[0].item())
        tri = torch.empty((n_pairs, 3), dtype=torch.int32, device=dev)
        _lib.check(L.st_map_pairs_write(_lib.ptr(nbr), n_out, K, _lib.ptr(ws), ws.numel(), _lib.ptr(tri), n_pairs,
                                        _lib.ptr(status), s), "st_map_pairs_write")
    assert int(counters[1].item()) == 0
    return tri.cpu().numpy()
