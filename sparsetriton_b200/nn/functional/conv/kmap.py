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

import ctypes

import torch

from sparsetriton_b200 import _lib, trace

__all__ = ["build_out_coords", "out_coords_and_map", "PendingOutCoordsAndMap", "kernel_offsets", "output_shape"]


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


_CONSTANTS = {}


def _constant_tensor(values, dtype, device, shape):
    """Small constant device tensor, made once per (values, dtype, device): building one from a python list is a
    pageable host->device copy, which waits for everything its stream holds."""
    key = (tuple(values), dtype, device.type, device.index, shape)
    t = _CONSTANTS.get(key)
    if t is None:
        if len(_CONSTANTS) > 256:
            _CONSTANTS.clear()
        t = _CONSTANTS[key] = torch.tensor(list(values), dtype=dtype, device=device).reshape(shape)
    return t


def _offsets_tensor(offsets, like):
    """(K,3) device tensor of the offsets in the coordinate dtype.  Shared between calls: treat as read-only."""
    t = _constant_tensor([v for o in offsets for v in o], like.dtype, like.device, (-1, 3))
    return t.view(t.shape)            # a fresh tensor object per call (callers attach attributes), same storage


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
    koff = _offsets_tensor(offsets, in_coords).clone()          # the caller's own copy (a device-side copy: no wait)
    new_shape = output_shape(spatial_shape, kernel_size, stride, dilation, padding, transposed)

    # kmap.py:261-262 / :380-381
    if submanifold and stride == 1 and ((kernel_size - 1) * dilation) // 2 == padding:
        return in_coords, spatial_shape, koff

    new_shape_t = _constant_tensor(new_shape, torch.int64, device, (3,)).clone()
    new_shape_t._st_host = new_shape      # spares callers in this package a device->host read
    out, _ = _run_out_coords(in_coords, offsets, new_shape, stride, transposed, with_map=False)
    return out, new_shape_t, koff


def out_coords_and_map(in_coords, spatial_shape, kernel_size, stride, dilation, padding, transposed, batch_bound=0):
    """Output coordinates AND the (N_out, K) neighbour map of a strided / transposed convolution in
    one pass over the candidates (the map is scattered from the same dedupe table instead of probing
    the input table N_out*K times).  Returns (out_coords, new_shape tuple, kernel_offsets tensor, nbr).
    Same results as build_out_coords followed by compute_neighbor_indices.  `batch_bound`: the number of samples in
    the batch (every batch index below it) if the caller knows it, else 0; it lets the library dedupe by direct
    addressing instead of hashing."""
    return PendingOutCoordsAndMap(in_coords, spatial_shape, kernel_size, stride, dilation, padding, transposed,
                                  batch_bound).finish()


class _PendingOutCoords:
    """First half of the output-coordinate build: candidates counted and deduplicated on the stream current at
    construction, the count on its way to pinned host memory.  `finish()` waits for that copy alone (not for the
    stream), sizes the outputs and launches the second half on the same stream."""

    def __init__(self, in_coords, offsets, new_shape, stride, transposed, with_map, in_shape=None, batch_bound=0):
        device = in_coords.device
        self.batch_bound = int(batch_bound or 0)   # samples in the batch if known: lets the library address cells directly
        self.n, self.K = in_coords.shape[0], len(offsets)
        self.with_map, self.coord_dtype, self.device = with_map, in_coords.dtype, device
        if self.n == 0:
            return
        _lib.require_cuda(in_coords, "build_out_coords")
        self.coords = in_coords.contiguous()
        self.code = _lib.coord_code(self.coords)
        L = _lib.lib()
        self.off_h = _lib.host_i32(v for o in offsets for v in o)
        self.shape_h = _lib.host_i32(new_shape)
        self.in_shape_h = _lib.host_i32(in_shape) if in_shape is not None else None
        self.stride, self.transposed = stride, int(transposed)
        self.ws = _lib.workspace(L.st_outcoords_workspace_bytes(self.n, self.K, stride, self.transposed), device)
        self.counters = torch.zeros(2, dtype=torch.int64, device=device)      # [n_out, status]
        self.status = self.counters[1:].view(torch.int32)
        self.stream = torch.cuda.current_stream(device)
        with _lib.on_device(device), trace.stage("out_coords"):
            rc = L.st_outcoords_count(_lib.ptr(self.coords), self.n, self.code, self.off_h, self.K, stride,
                                      self.transposed, self.shape_h, self.batch_bound, _lib.ptr(self.ws), self.ws.numel(),
                                      _lib.ptr(self.counters), _lib.ptr(self.status), _lib.stream_ptr(device))
            _lib.check(rc, "st_outcoords_count")
            self.host = torch.empty(2, dtype=torch.int64, pin_memory=True)
            self.host.copy_(self.counters, non_blocking=True)
            # the tensor-core kernels' sticky status word rides along: this is the one wait a step makes anyway
            self.kernel_status = torch.empty(4, dtype=torch.int32, pin_memory=True)
            _lib.check(L.st_device_status_enqueue(ctypes.c_void_p(self.kernel_status.data_ptr()), _lib.stream_ptr(device)),
                       "st_device_status_enqueue")
            self.arrived = torch.cuda.Event()
            self.arrived.record(self.stream)

    def finish(self):
        device, K = self.device, self.K
        if self.n == 0:
            return (torch.empty((0, 4), dtype=self.coord_dtype, device=device),
                    torch.empty((0, K), dtype=torch.int32, device=device) if self.with_map else None)
        L = _lib.lib()
        self.arrived.synchronize()                                     # the one device->host wait
        n_out, flags = self.host.tolist()
        _lib.raise_on_timeout(self.kernel_status, device)
        if flags & _lib.DEV_TABLE_FULL:
            raise RuntimeError("build_out_coords: dedupe table overflow")
        if flags & _lib.DEV_BAD_INDEX:
            raise ValueError(f"build_out_coords: a batch index lies outside [0, {self.batch_bound}) (the batch size given)")
        nbr = None
        with _lib.on_device(device), torch.cuda.stream(self.stream):
            stream = _lib.stream_ptr(device)
            out = torch.empty((n_out, 4), dtype=self.coord_dtype, device=device)
            if n_out > 0:
                with trace.stage("out_coords"):
                    rc = L.st_outcoords_write(_lib.ptr(self.coords), self.n, self.code, self.off_h, K, self.stride,
                                              self.transposed, self.shape_h, self.batch_bound, _lib.ptr(self.ws), self.ws.numel(),
                                              _lib.ptr(out), n_out, _lib.ptr(self.status), stream)
                    _lib.check(rc, "st_outcoords_write")
            if self.with_map:
                nbr = torch.empty((n_out, K), dtype=torch.int32, device=device)
                if n_out > 0:
                    with trace.stage("map_scatter"):
                        rc = L.st_outcoords_map(_lib.ptr(self.coords), self.n, self.code, self.off_h, K, self.stride,
                                                self.transposed, self.shape_h, self.in_shape_h, self.batch_bound,
                                                _lib.ptr(self.ws), self.ws.numel(), _lib.ptr(nbr), n_out, stream)
                        _lib.check(rc, "st_outcoords_map")
        return out, nbr


def _run_out_coords(in_coords, offsets, new_shape, stride, transposed, with_map, in_shape=None, batch_bound=0):
    return _PendingOutCoords(in_coords, offsets, new_shape, stride, transposed, with_map, in_shape, batch_bound).finish()


class PendingOutCoordsAndMap:
    """`out_coords_and_map` in two halves: construction launches the counting half, `finish()` returns what
    `out_coords_and_map` returns.  Lets a caller put other work between the launch and the wait for the count."""

    def __init__(self, in_coords, spatial_shape, kernel_size, stride, dilation, padding, transposed, batch_bound=0):
        offsets = kernel_offsets(kernel_size, dilation, padding, transposed)
        self.koff = _offsets_tensor(offsets, in_coords)
        self.koff._st_host = [v for o in offsets for v in o]
        self.new_shape = output_shape(spatial_shape, kernel_size, stride, dilation, padding, transposed)
        self.pending = _PendingOutCoords(in_coords, offsets, self.new_shape, stride, transposed, with_map=True,
                                         in_shape=tuple(int(v) for v in spatial_shape), batch_bound=batch_bound)

    def finish(self):
        out, nbr = self.pending.finish()
        return out, self.new_shape, self.koff, nbr
