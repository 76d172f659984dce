"""Functional sparse 3-D convolution (reference: nn/functional/conv/conv.py).

`compute_neighbor_indices` and `sparse_conv3d` keep the reference's signatures, argument
normalisation, assertion messages, caching rules and return types; the work is done by the CUDA
library through the two autograd Functions.
"""
from typing import Tuple, Union

import torch

from sparsetriton_b200 import _lib, trace
from sparsetriton_b200.config import ConvAlgo, get_conv_algo, get_h_table_f
from sparsetriton_b200.tensor import SparseTensor, TensorCache
from sparsetriton_b200.utils.hash import HashTable, round_up_capacity

from .funcs import ConvHashOnTheFlyImplicitGEMM, ConvPrecomputedNeighborGEMM
from .funcs.implicit_precomputed_gemm import prepare_plans
from .kmap import PendingOutCoordsAndMap, build_out_coords, kernel_offsets, out_coords_and_map

__all__ = ["compute_neighbor_indices", "sparse_conv3d", "prepare_conv3d", "ConvPreparation"]


def compute_neighbor_indices(
    in_hash_table: HashTable,
    out_coords: torch.Tensor,
    kernel_offsets: torch.Tensor,
    spatial_shape: Tuple[int, int, int],
    stride: int,
    padding: int = 0,
    dilation: int = 1,
    queries_are_table_rows: bool = False,
) -> torch.Tensor:
    """(N_out, K) int32 map: row of (batch, out*stride - kernel_offsets[k]) in the table, or -1
    when that coordinate is outside [0, spatial_shape) or absent (conv.py:12-75).

    `padding` and `dilation` are unused: they are already folded into `kernel_offsets`.
    `queries_are_table_rows` (no reference counterpart) says that `out_coords` are the very rows the table
    was built from, as in a submanifold layer; the map is then built from half of the probes.
    One kernel launch; the (N_out*K, 4) candidate rows of the reference are never materialised.
    """
    n_out, K = out_coords.shape[0], kernel_offsets.shape[0]
    device = out_coords.device
    nbr = torch.empty((n_out, K), dtype=torch.int32, device=device)
    if n_out == 0:
        return nbr
    _lib.require_cuda(out_coords, "compute_neighbor_indices")
    keys, vals = in_hash_table.table_keys, in_hash_table.table_values
    _lib.require_cuda(keys, "compute_neighbor_indices")
    if keys.dtype != torch.int64 or vals.dtype != torch.int32:
        raise TypeError("hash table must hold int64 keys and int32 values")
    coords = out_coords.contiguous()
    host = getattr(kernel_offsets, "_st_host", None)
    if host is None:
        host = kernel_offsets.reshape(-1).tolist()
    # Submanifold layer (the queries are the rows the table was built from, stride 1, odd kernel): offsets
    # come in opposite pairs, so half of the probes give the whole map (no reference counterpart).
    if queries_are_table_rows and int(stride) == 1 and K % 2 == 1 and \
            all(host[i] == -host[3 * (K - 1) - 3 * (i // 3) + i % 3] for i in range(3 * K)):
        with _lib.on_device(device), trace.stage("map_build", 3):
            asym = torch.empty(1, dtype=torch.int32, device=device)
            rc = _lib.lib().st_map_build_symmetric(_lib.ptr(coords), n_out, _lib.coord_code(coords), _lib.host_i32(host),
                                                   K, _lib.host_i32(int(v) for v in spatial_shape), _lib.ptr(keys),
                                                   _lib.ptr(vals), keys.shape[0], _lib.ptr(nbr), _lib.ptr(asym),
                                                   _lib.stream_ptr())
        _lib.check(rc, "st_map_build_symmetric")
        # rows not returned for their own coordinate (duplicates, outside the grid); 0 = the map is its own
        # inverse up to the order of the offsets, which the feature gradient then exploits.  The count travels to
        # pinned host memory right away and an event marks its arrival, so that the backward pass, much later,
        # reads it without waiting for everything the stream holds by then.
        flag_host = torch.empty(1, dtype=torch.int32, pin_memory=True)
        flag_host.copy_(asym, non_blocking=True)
        arrived = torch.cuda.Event()
        arrived.record(torch.cuda.current_stream(device))
        nbr._st_asymmetric_rows = (flag_host, arrived)
        return nbr
    with _lib.on_device(device), trace.stage("map_build", 1):
        rc = _lib.lib().st_map_build(_lib.ptr(coords), n_out, _lib.coord_code(coords), _lib.host_i32(host), K,
                                     int(stride), _lib.host_i32(int(v) for v in spatial_shape), _lib.ptr(keys),
                                     _lib.ptr(vals), keys.shape[0], _lib.ptr(nbr), _lib.stream_ptr())
    _lib.check(rc, "st_map_build")
    return nbr


def _new_table(coords, device):
    table = HashTable(round_up_capacity(coords.shape[0], get_h_table_f()), device=device)
    table.insert(coords)
    return table


def _table_and_out_coords(cache, coords, spatial_shape, k, s, p, d, submanifold, transposed):
    """Table over the coordinates the lookup is made in (the inputs themselves, or, for an upsampling transposed
    conv, the inputs with their spatial columns scaled: conv.py:138-142) and the output coordinates."""
    device = coords.device
    if transposed and s > 1:
        scaled = coords.clone()
        scaled[:, 1:] *= s
        table = _new_table(scaled, device)
    else:
        if cache.hashtable is None:
            cache.hashtable = _new_table(coords, device)
        table = cache.hashtable
    out_coords, new_shape, koff = build_out_coords(coords, spatial_shape, k, s, d, p, transposed=transposed,
                                                   submanifold=submanifold)
    koff._st_host = [v for o in kernel_offsets(k, d, p, transposed) for v in o]
    return table, out_coords, new_shape, koff


def _stored_geometry(cache, coords, spatial_shape, k, s, p, d, submanifold, transposed, batch_bound=0):
    """(out_coords, neighbor_indices, new_shape) of a layer under the stored-map algorithm, from the cache of the
    input's coordinate set or built and memoised there."""
    cache_key = (k, s, p, d, submanifold, transposed)
    cached = cache.neighbor_indices.get(cache_key)
    if cached is not None:
        return cached
    if not (submanifold and s == 1):
        # strided / transposed layer: coordinates and map come out of one pass over the candidates; no table over
        # the inputs is needed
        out_coords, new_shape, _, neighbor_indices = out_coords_and_map(coords, spatial_shape, k, s, d, p, transposed,
                                                                        batch_bound)
    else:
        table, out_coords, new_shape, koff = _table_and_out_coords(cache, coords, spatial_shape, k, s, p, d,
                                                                   submanifold, transposed)
        upsample = transposed and s > 1
        lookup_shape = tuple(v * s for v in spatial_shape) if upsample else tuple(spatial_shape)
        neighbor_indices = compute_neighbor_indices(table, out_coords, koff, lookup_shape, 1 if transposed else s, p, d,
                                                    queries_are_table_rows=out_coords is coords)
    if out_coords.shape[0] > 0:
        cache.neighbor_indices[cache_key] = (out_coords, neighbor_indices, new_shape)
    return out_coords, neighbor_indices, new_shape


class ConvPreparation:
    """Everything a stored-map layer derives from coordinates alone, built ahead of the features, in two halves (no
    reference counterpart).  Construction launches, on the current stream, the half that needs no size from the
    device (for a strided or transposed layer: counting and deduplicating the candidates; for a submanifold layer:
    table and map).  `finish()` waits for the output count alone, launches the rest on that same stream (output
    coordinates, neighbour map, tile plan and, with `backward`, what the feature gradient reads) and returns the
    TensorCache to hand to `SparseTensor(feats, coords, spatial_shape, batch_size, cache=...)`; `sparse_conv3d`
    with the same geometry then launches only its products.

    Built under a side stream it overlaps the products of another batch; a caller that constructs the preparation of
    batch j+2 before finishing that of batch j+1 never waits for the device.  Pass the stream the layer will run on as
    `consumer_stream` so that the allocator keeps the results alive for it, and make that stream wait for an event
    recorded after `finish()`.  `batch_size` (the number of samples, every batch index below it) is optional; with
    it the output coordinates are deduplicated by direct addressing instead of hashing."""

    def __init__(self, coords, spatial_shape, kernel_size, stride=1, dilation=1, padding=0, transposed=False,
                 submanifold=True, backward=True, cache=None, consumer_stream=None, batch_size=None):
        k = _scalar(kernel_size, "Only cubic kernels supported for now")
        s = _scalar(stride, "Only uniform stride supported for now")
        d = _scalar(dilation, "Only uniform dilation supported for now")
        if submanifold:
            padding = ((k - 1) * d) // 2
            assert not transposed, "Submanifold convolution does not support transposed=True"
        p = _scalar(padding, "Only uniform padding supported for now")
        _lib.require_cuda(coords, "prepare_conv3d")
        self.cache = TensorCache() if cache is None else cache
        self.coords, self.spatial_shape = coords, tuple(spatial_shape)
        self.geometry = (k, s, p, d, submanifold, transposed)
        self.backward, self.consumer_stream = backward, consumer_stream
        self.stream = torch.cuda.current_stream(coords.device)
        self.pending = None
        if self.geometry in self.cache.neighbor_indices:
            return
        if submanifold and s == 1:
            _stored_geometry(self.cache, coords, self.spatial_shape, k, s, p, d, submanifold, transposed)
        else:
            self.pending = PendingOutCoordsAndMap(coords, self.spatial_shape, k, s, d, p, transposed, batch_size or 0)

    def finish(self) -> TensorCache:
        cache, coords = self.cache, self.coords
        with torch.cuda.stream(self.stream):
            if self.pending is not None:
                out_coords, new_shape, _, nbr = self.pending.finish()
                self.pending = None
                if out_coords.shape[0] > 0:
                    cache.neighbor_indices[self.geometry] = (out_coords, nbr, new_shape)
            else:
                out_coords, nbr, new_shape = _stored_geometry(cache, coords, self.spatial_shape, *self.geometry)
            made = [out_coords, nbr]
            if nbr.shape[0] > 0:
                made += prepare_plans(nbr, coords.shape[0], self.backward)
        self.out_coords, self.neighbor_indices, self.new_shape = out_coords, nbr, _as_shape(new_shape)
        if cache.hashtable is not None:
            made += [cache.hashtable.table_keys, cache.hashtable.table_values]
        if self.consumer_stream is not None:
            for t in made:
                if t is not None and t.is_cuda and t.numel() > 0:
                    t.record_stream(self.consumer_stream)
        return cache


def prepare_conv3d(
    coords: torch.Tensor,
    spatial_shape: Tuple[int, int, int],
    kernel_size: Union[int, Tuple[int, int, int]],
    stride: Union[int, Tuple[int, int, int]] = 1,
    dilation: Union[int, Tuple[int, int, int]] = 1,
    padding: Union[int, Tuple[int, int, int]] = 0,
    transposed: bool = False,
    submanifold: bool = True,
    backward: bool = True,
    cache: TensorCache = None,
    consumer_stream: "torch.cuda.Stream" = None,
    batch_size: int = None,
) -> TensorCache:
    """Both halves of a ConvPreparation at once, on the current stream: returns the TensorCache holding output
    coordinates, neighbour map and tile plans of the layer (no reference counterpart)."""
    return ConvPreparation(coords, spatial_shape, kernel_size, stride, dilation, padding, transposed, submanifold,
                           backward, cache, consumer_stream, batch_size).finish()


def _scalar(value, what):
    if isinstance(value, tuple):
        assert value[0] == value[1] == value[2], what
        return value[0]
    return value


def sparse_conv3d(
    tensor: SparseTensor,
    weight: torch.Tensor,
    kernel_size: Union[int, Tuple[int, int, int]],
    bias: torch.Tensor = None,
    stride: Union[int, Tuple[int, int, int]] = 1,
    dilation: Union[int, Tuple[int, int, int]] = 1,
    padding: Union[int, Tuple[int, int, int]] = 0,
    transposed: bool = False,
    submanifold: bool = True,
) -> SparseTensor:
    """3-D sparse convolution of `tensor` with `weight` (K, C_in, C_out) (conv.py:77-239).

    submanifold=True keeps the input coordinate set (padding is forced to the centred value);
    otherwise output coordinates are every cell reached by the kernel, strided or transposed.
    Cubic kernels, uniform stride / dilation / padding only, as in the reference.
    """
    k = _scalar(kernel_size, "Only cubic kernels supported for now")
    s = _scalar(stride, "Only uniform stride supported for now")
    d = _scalar(dilation, "Only uniform dilation supported for now")
    if submanifold:
        padding = ((k - 1) * d) // 2
    p = _scalar(padding, "Only uniform padding supported for now")
    if submanifold:
        assert not transposed, "Submanifold convolution does not support transposed=True"

    feats, coords = tensor.F, tensor.C
    device = feats.device
    K, c_in, c_out = weight.shape
    assert c_in == feats.shape[1], f"Input channels in weight({c_in}) and tensor({feats.shape[1]}) must match"
    assert K == k ** 3, f"Kernel size in weight({K}) and argument({k ** 3}) must match"

    cache = tensor._cache
    algo = get_conv_algo()
    upsample = transposed and s > 1
    neighbor_indices = table = koff = None
    if algo == ConvAlgo.PrecomputedNeighborGEMM:
        out_coords, neighbor_indices, new_shape = _stored_geometry(cache, coords, tensor.spatial_shape, k, s, p, d,
                                                                   submanifold, transposed, tensor.batch_size)
    else:
        table, out_coords, new_shape, koff = _table_and_out_coords(cache, coords, tensor.spatial_shape, k, s, p, d,
                                                                   submanifold, transposed)

    if out_coords.shape[0] == 0:
        return SparseTensor(
            feats=torch.empty((0, c_out), device=device, dtype=feats.dtype),
            coords=torch.empty((0, 4), device=device, dtype=coords.dtype),
            spatial_shape=_as_shape(new_shape), batch_size=tensor.batch_size)

    if algo == ConvAlgo.PrecomputedNeighborGEMM:
        out_feats = ConvPrecomputedNeighborGEMM.apply(feats, weight, neighbor_indices)
    elif algo == ConvAlgo.ImplicitHashFlyGEMM:
        lookup_shape = tuple(v * s for v in tensor.spatial_shape) if upsample else tuple(tensor.spatial_shape)
        lookup_stride = 1 if transposed else s
        out_feats = ConvHashOnTheFlyImplicitGEMM.apply(feats, weight, out_coords, koff, table.table_keys,
                                                       table.table_values, lookup_shape, lookup_stride)
    else:  # pragma: no cover - ConvAlgo has two members
        raise ValueError(f"unknown convolution algorithm {algo}")

    if bias is not None:
        out_feats = out_feats + bias.to(out_feats.dtype)

    if submanifold and out_coords is coords:
        return tensor.replace(out_feats)
    # with a stored map the output coordinates are memoised per geometry, and so is the cache of what derives from them
    child = cache.child((k, s, p, d, submanifold, transposed)) if algo == ConvAlgo.PrecomputedNeighborGEMM else None
    return SparseTensor._trusted(out_feats, out_coords, _as_shape(new_shape), tensor.batch_size, child)


def _as_shape(shape):
    if isinstance(shape, torch.Tensor):
        host = getattr(shape, "_st_host", None)
        return tuple(int(v) for v in (host if host is not None else shape.tolist()))
    return tuple(int(v) for v in shape)
