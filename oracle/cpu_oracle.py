"""ctypes front end of the C oracle in ``oracle.c``.  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the benchmark's CPU-baseline / reference legs may
import this module, and only as the checker or as the timed CPU baseline.  The product
package never does; it raises if its CUDA library is missing.

All arrays are numpy, coordinates are int32 ``(N, 4)`` rows ``(batch, x, y, z)``.
Each function names the reference code it restates in ``oracle.c``.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "oracle.c")
_SO = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force=False):
    """Compile oracle.c with gcc + OpenMP into liboracle.so next to it."""
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        subprocess.check_call(["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-shared", "-fPIC", _SRC, "-o", _SO])
    return _SO


def _p(a, t):
    return a.ctypes.data_as(ctypes.POINTER(t))


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = ctypes.CDLL(_SO)
        L.orc_out_coords.restype = ctypes.c_int64
        L.orc_hash_build.restype = ctypes.c_int
        L.orc_num_threads.restype = ctypes.c_int
        _lib = L
    return _lib


def num_threads():
    return int(lib().orc_num_threads())


def set_threads(n):
    lib().orc_set_threads(ctypes.c_int(int(n)))


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def offsets(ks, dil, pad, transposed):
    """(K,3) kernel offsets: kmap.py:104-180."""
    out = np.empty((ks ** 3, 3), np.int32)
    lib().orc_offsets(int(ks), int(dil), int(pad), int(bool(transposed)), _p(out, ctypes.c_int32))
    return out


def new_shape(shape, ks, s, d, p, transposed):
    """Output spatial shape: kmap.py:254-258 / :373-377."""
    sh = _i32(shape)
    out = np.empty(3, np.int32)
    lib().orc_new_shape(_p(sh, ctypes.c_int32), int(ks), int(s), int(d), int(p), int(bool(transposed)),
                        _p(out, ctypes.c_int32))
    return out


class Table:
    """Exact-key open-addressing table: hash.py:369-580 (HashTable), with 64-bit packed keys."""

    def __init__(self, coords, capacity=None):
        coords = _i32(coords).reshape(-1, 4)
        n = coords.shape[0]
        self.cap = int(capacity) if capacity is not None else max(2 * n, 1)
        self.keys = np.empty(self.cap, np.int64)
        self.vals = np.empty(self.cap, np.int32)
        rc = lib().orc_hash_build(_p(coords, ctypes.c_int32), ctypes.c_int64(n), _p(self.keys, ctypes.c_int64),
                                  _p(self.vals, ctypes.c_int32), ctypes.c_int64(self.cap))
        if rc != 0:
            raise AssertionError("oracle table capacity too small")

    def query(self, q):
        q = _i32(q).reshape(-1, 4)
        out = np.empty(q.shape[0], np.int32)
        lib().orc_hash_query(_p(q, ctypes.c_int32), ctypes.c_int64(q.shape[0]), _p(self.keys, ctypes.c_int64),
                             _p(self.vals, ctypes.c_int32), ctypes.c_int64(self.cap), _p(out, ctypes.c_int32))
        return out


def out_coords(coords, shape, ks, s, d, p, transposed, subm):
    """build_out_coords: kmap.py:213-495.  Returns (out_coords int32, new_shape, kernel_offsets)."""
    coords = _i32(coords).reshape(-1, 4)
    off = offsets(ks, d, p, transposed)
    ns = new_shape(shape, ks, s, d, p, transposed)
    if subm and s == 1 and ((ks - 1) * d) // 2 == p:        # kmap.py:261-262 / :380-381
        return coords.copy(), _i32(shape), off
    n = coords.shape[0]
    cap = max(n * ks ** 3, 1)
    grid = int(max(coords[:, 0].max() + 1, 1)) * int(max(ns[0], 0)) * int(max(ns[1], 0)) * int(max(ns[2], 0)) if n else 0
    cap = max(min(cap, grid), 1)
    out = np.empty((cap, 4), np.int32)
    m = lib().orc_out_coords(_p(coords, ctypes.c_int32), ctypes.c_int64(n), _p(off, ctypes.c_int32), int(ks ** 3),
                             int(s), _p(ns, ctypes.c_int32), int(bool(transposed)), _p(out, ctypes.c_int32),
                             ctypes.c_int64(cap))
    assert 0 <= m <= cap
    return out[:m].copy(), ns, off


def neighbor_map(table, out_c, off, stride, lookup_shape):
    """compute_neighbor_indices: conv.py:12-75."""
    out_c = _i32(out_c).reshape(-1, 4)
    off = _i32(off)
    ls = _i32(lookup_shape)
    K = off.shape[0]
    nbr = np.empty((out_c.shape[0], K), np.int32)
    lib().orc_neighbor_map(_p(out_c, ctypes.c_int32), ctypes.c_int64(out_c.shape[0]), _p(off, ctypes.c_int32), int(K),
                           int(stride), _p(ls, ctypes.c_int32), _p(table.keys, ctypes.c_int64),
                           _p(table.vals, ctypes.c_int32), ctypes.c_int64(table.cap), _p(nbr, ctypes.c_int32))
    return nbr


def kernel_map(coords, shape, ks, s, d, p, transposed, subm):
    """The call sequence of sparse_conv3d (conv.py:120-188) up to the neighbour map.
    Returns (out_coords, new_shape, kernel_offsets, nbr)."""
    coords = _i32(coords).reshape(-1, 4)
    if subm:
        p = ((ks - 1) * d) // 2                              # conv.py:120-121
    keyc = coords.copy()
    if transposed and s > 1:
        keyc[:, 1:] *= s                                     # conv.py:138-142
    table = Table(keyc)
    oc, ns, off = out_coords(coords, shape, ks, s, d, p, transposed, subm)
    look = [v * s for v in shape] if (transposed and s > 1) else list(shape)   # conv.py:180-183
    nbr = neighbor_map(table, oc, off, 1 if transposed else s, look)
    return oc, ns, off, nbr


def conv_fwd(x, w, nbr):
    """implicit_precomputed_gemm.py:64-126."""
    x, w, nbr = _f32(x), _f32(w), _i32(nbr)
    K, cin, cout = w.shape
    y = np.empty((nbr.shape[0], cout), np.float32)
    lib().orc_conv_fwd(_p(x, ctypes.c_float), _p(w, ctypes.c_float), _p(nbr, ctypes.c_int32),
                       ctypes.c_int64(nbr.shape[0]), int(K), int(cin), int(cout), _p(y, ctypes.c_float))
    return y


def conv_dgrad(dy, w, nbr, n_in):
    """implicit_precomputed_gemm.py:129-177."""
    dy, w, nbr = _f32(dy), _f32(w), _i32(nbr)
    K, cin, cout = w.shape
    dx = np.empty((n_in, cin), np.float32)
    lib().orc_conv_dgrad(_p(dy, ctypes.c_float), _p(w, ctypes.c_float), _p(nbr, ctypes.c_int32), ctypes.c_int64(n_in),
                         ctypes.c_int64(nbr.shape[0]), int(K), int(cin), int(cout), _p(dx, ctypes.c_float))
    return dx


def conv_wgrad(x, dy, nbr, K, cin, cout):
    """implicit_precomputed_gemm.py:180-230."""
    x, dy, nbr = _f32(x), _f32(dy), _i32(nbr)
    dw = np.empty((K, cin, cout), np.float32)
    lib().orc_conv_wgrad(_p(x, ctypes.c_float), _p(dy, ctypes.c_float), _p(nbr, ctypes.c_int32),
                         ctypes.c_int64(nbr.shape[0]), int(K), int(cin), int(cout), _p(dw, ctypes.c_float))
    return dw


def pairs(nbr):
    """The (in_idx, out_idx, offset) triples of a neighbour map, in (out_idx, offset) order."""
    o, k = np.nonzero(nbr >= 0)
    return np.stack([nbr[o, k], o.astype(np.int32), k.astype(np.int32)], axis=1)


# ------------------------------------------------------------------------------------------------
# Adjacent operators (numpy restatements; same "checker only" rule as above)
# ------------------------------------------------------------------------------------------------
def to_dense(feats, coords, shape, batch=None):
    """utils/to_dense.py:143-203: dense (B, X, Y, Z, C), zeros except dense[b,x,y,z,:] = feats[i,:];
    B = largest batch index + 1 (:275-278) unless given."""
    feats = np.asarray(feats)
    coords = _i32(coords).reshape(-1, 4)
    if batch is None:
        batch = int(coords[:, 0].max()) + 1 if coords.shape[0] else 1
    dense = np.zeros((batch, *[int(v) for v in shape], feats.shape[1]), feats.dtype)
    dense[coords[:, 0], coords[:, 1], coords[:, 2], coords[:, 3]] = feats
    return dense


def to_dense_bwd(grad_dense, coords):
    """utils/to_dense.py:205-240: grad_feats[i,:] = grad_dense[b,x,y,z,:]."""
    coords = _i32(coords).reshape(-1, 4)
    return np.asarray(grad_dense)[coords[:, 0], coords[:, 1], coords[:, 2], coords[:, 3]]


def pool_map(coords, kernel_size, padding, stride):
    """nn/functional/spatial.py:121-129: cell of every input = floor((in + padding - ks//2) / stride) per
    spatial axis; output rows = distinct cells in ascending (batch, x, y, z) order.
    Returns (out_coords int32 (n_out,4), in_to_out int64 (n,))."""
    coords = _i32(coords).reshape(-1, 4)
    cells = coords.copy()
    cells[:, 1:] = np.floor_divide(coords[:, 1:] + padding - kernel_size // 2, stride)
    if coords.shape[0] == 0:
        return cells, np.zeros(0, np.int64)
    uniq, inverse = np.unique(cells, axis=0, return_inverse=True)
    return uniq.astype(np.int32), inverse.reshape(-1)


def pool_new_shape(shape, kernel_size, padding, stride):
    """nn/functional/spatial.py:116."""
    return tuple((int(s) - kernel_size + padding * 2) // stride + 1 for s in shape)


def pool_fwd(feats, in_to_out, n_out, mode):
    """nn/functional/spatial.py:37-88 + :156-157: mean ("avg") or maximum ("max") of the inputs of every cell."""
    feats = np.asarray(feats, np.float64)
    if mode == "avg":
        out = np.zeros((n_out, feats.shape[1]))
        np.add.at(out, in_to_out, feats)
        return out / np.bincount(in_to_out, minlength=n_out).reshape(-1, 1)
    out = np.full((n_out, feats.shape[1]), -np.inf)
    np.maximum.at(out, in_to_out, feats)
    return out


def pool_bwd(grad_out, feats, out, in_to_out, mode):
    """nn/functional/spatial.py:175-262: avg: grad / count; max: grad where the input equals the maximum."""
    g = np.asarray(grad_out, np.float64)[in_to_out]
    if mode == "avg":
        return g / np.bincount(in_to_out, minlength=np.asarray(grad_out).shape[0])[in_to_out].reshape(-1, 1)
    return np.where(np.asarray(feats, np.float64) == np.asarray(out, np.float64)[in_to_out], g, 0.0)


def upsample(feats, coords, scale):
    """nn/functional/spatial.py:305-396: row i -> rows i*s^3 + (dx*s + dy)*s + dz at in*s + (dx,dy,dz)."""
    coords = _i32(coords).reshape(-1, 4)
    s3 = scale ** 3
    step = np.arange(s3)
    d = np.stack([np.zeros(s3, np.int64), step // (scale * scale), (step // scale) % scale, step % scale], axis=1)
    base = coords.astype(np.int64) * np.array([1, scale, scale, scale])
    out_coords = (base[:, None, :] + d[None, :, :]).reshape(-1, 4).astype(np.int32)
    return np.repeat(np.asarray(feats), s3, axis=0), out_coords


def upsample_bwd(grad_out, scale):
    """nn/functional/spatial.py:446-480: sum of the scale^3 output rows of every input row."""
    g = np.asarray(grad_out, np.float64)
    return g.reshape(-1, scale ** 3, g.shape[1]).sum(axis=1)


def batch_norm(feats, batch_idx, n_samples, weight, bias, eps, relu=False, upstream=None, running=None, momentum=0.1,
               decisions=None):
    """nn/functional/norm.py:73-112 in float64: statistics per (sample, channel), biased variance, counts
    clamped to 1; optional ReLU on top (the reference applies it as a separate module).
    `decisions` (bool, shape of feats): the ReLU's on/off choice per element taken from another run instead of
    from this one's own sign of z -- a gradient is discontinuous where z crosses zero, so two runs are compared
    on common decisions and the caller checks `z` where they differ (it must be within rounding of zero).
    Returns dict(y, z, mean, var[, dx, dw, db][, running_mean, running_var])."""
    x = np.asarray(feats, np.float64)
    b = np.asarray(batch_idx, np.int64)
    C = x.shape[1]
    counts = np.maximum(np.bincount(b, minlength=n_samples), 1).astype(np.float64).reshape(-1, 1)
    mean = np.zeros((n_samples, C))
    np.add.at(mean, b, x)
    mean /= counts
    var = np.zeros((n_samples, C))
    np.add.at(var, b, (x - mean[b]) ** 2)
    var /= counts
    rstd = 1.0 / np.sqrt(var + eps)
    xhat = (x - mean[b]) * rstd[b]
    w = np.ones(C) if weight is None else np.asarray(weight, np.float64)
    bb = np.zeros(C) if bias is None else np.asarray(bias, np.float64)
    z = xhat * w + bb
    on = (z > 0) if decisions is None else np.asarray(decisions, bool)
    res = {"y": (z * on) if relu else z, "z": z, "mean": mean, "var": var}
    if running is not None:                                      # norm.py:91-94
        res["running_mean"] = (1 - momentum) * np.asarray(running[0], np.float64) + momentum * mean.mean(0)
        res["running_var"] = (1 - momentum) * np.asarray(running[1], np.float64) + momentum * var.mean(0)
    if upstream is not None:
        dz = np.asarray(upstream, np.float64) * (on if relu else 1.0)
        res["dw"], res["db"] = (dz * xhat).sum(0), dz.sum(0)
        dxhat = dz * w
        s0 = np.zeros((n_samples, C))
        s1 = np.zeros((n_samples, C))
        np.add.at(s0, b, dxhat)
        np.add.at(s1, b, dxhat * xhat)
        res["dx"] = rstd[b] * (dxhat - (s0[b] + xhat * s1[b]) / counts[b])
    return res


def batch_norm_eval(feats, running_mean, running_var, weight, bias, eps):
    """nn/functional/norm.py:95-110, inference form."""
    x = np.asarray(feats, np.float64)
    y = (x - np.asarray(running_mean, np.float64)) / np.sqrt(np.asarray(running_var, np.float64) + eps)
    if weight is not None:
        y = y * np.asarray(weight, np.float64)
    if bias is not None:
        y = y + np.asarray(bias, np.float64)
    return y
