"""Output coordinates of a sparse convolution (reference: nn/functional/conv/kmap.py).

`build_out_coords` keeps the reference's signature and return triple.  What differs is how the
work is done: the reference materialises all N*K candidate rows, filters them with three
boolean-mask compactions and dedupes through a scratch table of 31-bit keys; here one C-ABI call
enumerates candidates in registers, dedupes on exact 64-bit keys keeping the candidate with the
smallest flat index n*K+k, and a second call writes the survivors in that order.  The order is the
one the reference's sequential CPU path produces (first occurrence, n-major, k-minor), and it does
not depend on thread scheduling.

Two reference behaviours are intentionally not reproduced:
  * coordinates whose 31-bit keys collide are merged by the reference (kmap.py:93); here they stay
    distinct;
  * the transposed path multiplies the batch column by the stride (kmap.py:407), which breaks
    batch indices >= 1; here only the spatial columns are scaled.
"""
from typing import Tuple

import torch

from sparsetriton_b200 import _lib, trace

__all__ = ["build_out_coords", "out_coords_and_map", "kernel_offsets", "output_shape"]


def kernel_offsets(kernel_size: int, dilation: int, padding: int, transposed: bool):
    """(K,3) python list of offsets, K = kernel_size^3, k = (ix*ks + iy)*ks + iz.

    base = (i - ks//2) * dilation per axis (kmap.py:104-132);
    normal: -base + padding - ((ks-1)*dilation)//2 (:135-156); transposed: the negation (:159-180).
    """
    ks, half = kernel_size, ((kernel_size - 1) * dilation) // 2
    axis = [(i - ks // 2) * dilation for i in range(ks)]
    sign, shift = (1, half - padding) if transposed else (-1, padding - half)
    one = [sign * a + shift for a in axis]
    return [(one[ix], one[iy], one[iz]) for ix in range(ks) for iy in range(ks) for iz in range(ks)]


def output_shape(spatial_shape, kernel_size, stride, dilation, padding, transposed):
    """New spatial shape: kmap.py:254-258 (normal), :373-377 (transposed)."""
    if transposed:
        return tuple((int(s) - 1) * stride + (kernel_size - 1) * dilation - 2 * padding + 1 for s in spatial_shape)
    return tuple((int(s) - (kernel_size - 1) * dilation + 2 * padding - 1) // stride + 1 for s in spatial_shape)


def _offsets_tensor(offsets, like):
    return torch.tensor(offsets, dtype=like.dtype, device=like.device).reshape(-1, 3)


def build_out_coords(
    in_coords: torch.Tensor,
    spatial_shape: Tuple[int, int, int],
    kernel_size: int,
    stride: int = 1,
    dilation: int = 1,
    padding: int = 1,
    transposed: bool = False,
    submanifold: bool = True,
    chunk_size: int = None,
):
    """Returns (out_coords, new_spatial_shape, kernel_offsets) as kmap.py:447-495 does.

    out_coords has the dtype of in_coords; new_spatial_shape is an int64 device tensor of 3
    values, or `spatial_shape` itself on the submanifold shortcut; kernel_offsets is a (K,3)
    device tensor of the coordinate dtype.  `chunk_size` is accepted and ignored (nothing is
    materialised per chunk).
    """
    device = in_coords.device
    offsets = kernel_offsets(kernel_size, dilation, padding, transposed)
    koff = _offsets_tensor(offsets, in_coords)
    new_shape = output_shape(spatial_shape, kernel_size, stride, dilation, padding, transposed)

    # kmap.py:261-262 / :380-381
    if submanifold and stride == 1 and ((kernel_size - 1) * dilation) // 2 == padding:
        return in_coords, spatial_shape, koff

    new_shape_t = torch.tensor(new_shape, device=device)
    new_shape_t._st_host = new_shape      # spares callers in this package a device->host read
    out, _ = _run_out_coords(in_coords, offsets, new_shape, stride, transposed, with_map=False)
    return out, new_shape_t, koff


def out_coords_and_map(in_coords, spatial_shape, kernel_size, stride, dilation, padding, transposed):
    """Output coordinates AND the (N_out, K) neighbour map of a strided / transposed convolution in
    one pass over the candidates (the map is scattered from the same dedupe table instead of probing
    the input table N_out*K times).  Returns (out_coords, new_shape tuple, kernel_offsets tensor, nbr).
    Same results as build_out_coords followed by compute_neighbor_indices."""
    offsets = kernel_offsets(kernel_size, dilation, padding, transposed)
    koff = _offsets_tensor(offsets, in_coords)
    koff._st_host = [v for o in offsets for v in o]
    new_shape = output_shape(spatial_shape, kernel_size, stride, dilation, padding, transposed)
    out, nbr = _run_out_coords(in_coords, offsets, new_shape, stride, transposed, with_map=True,
                               in_shape=tuple(int(v) for v in spatial_shape))
    return out, new_shape, koff, nbr


def _run_out_coords(in_coords, offsets, new_shape, stride, transposed, with_map, in_shape=None):
    device = in_coords.device
    n, K = in_coords.shape[0], len(offsets)
    if n == 0:
        return (torch.empty((0, 4), dtype=in_coords.dtype, device=device),
                torch.empty((0, K), dtype=torch.int32, device=device) if with_map else None)
    _lib.require_cuda(in_coords, "build_out_coords")
    coords = in_coords.contiguous()
    code = _lib.coord_code(coords)
    L = _lib.lib()
    off_h = _lib.host_i32(v for o in offsets for v in o)
    shape_h = _lib.host_i32(new_shape)
    ws_bytes = L.st_outcoords_workspace_bytes(n, K, stride, int(transposed))
    ws = _lib.workspace(ws_bytes, device)
    counters = torch.zeros(2, dtype=torch.int64, device=device)      # [n_out, status]
    status = counters[1:].view(torch.int32)
    nbr = None
    with torch.cuda.device(device), trace.stage("out_coords"):
        stream = _lib.stream_ptr()
        rc = L.st_outcoords_count(_lib.ptr(coords), n, code, off_h, K, stride, int(transposed), shape_h,
                                  _lib.ptr(ws), ws.numel(), _lib.ptr(counters), _lib.ptr(status), stream)
        _lib.check(rc, "st_outcoords_count")
        n_out, flags = counters.tolist()                               # the one device->host sync
        if flags & _lib.DEV_TABLE_FULL:
            raise RuntimeError("build_out_coords: dedupe table overflow")
        out = torch.empty((n_out, 4), dtype=coords.dtype, device=device)
        if n_out > 0:
            rc = L.st_outcoords_write(_lib.ptr(coords), n, code, off_h, K, stride, int(transposed), shape_h,
                                      _lib.ptr(ws), ws.numel(), _lib.ptr(out), n_out, _lib.ptr(status), stream)
            _lib.check(rc, "st_outcoords_write")
    if with_map:
        nbr = torch.empty((n_out, K), dtype=torch.int32, device=device)
        if n_out > 0:
            with torch.cuda.device(device), trace.stage("map_scatter"):
                rc = L.st_outcoords_map(_lib.ptr(coords), n, code, off_h, K, stride, int(transposed), shape_h,
                                        _lib.host_i32(in_shape), _lib.ptr(ws), ws.numel(), _lib.ptr(nbr), n_out,
                                        _lib.stream_ptr())
                _lib.check(rc, "st_outcoords_map")
    return out, nbr
