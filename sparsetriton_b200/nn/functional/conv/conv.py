"""Functional sparse 3-D convolution (reference: nn/functional/conv/conv.py).

`compute_neighbor_indices` and `sparse_conv3d` keep the reference's signatures, argument
normalisation, assertion messages, caching rules and return types; the work is done by the CUDA
library through the two autograd Functions.
"""
from typing import Tuple, Union

import torch

from sparsetriton_b200 import _lib, trace
from sparsetriton_b200.config import ConvAlgo, get_conv_algo, get_h_table_f
from sparsetriton_b200.tensor import SparseTensor
from sparsetriton_b200.utils.hash import HashTable, round_up_capacity

from .funcs import ConvHashOnTheFlyImplicitGEMM, ConvPrecomputedNeighborGEMM
from .kmap import build_out_coords, kernel_offsets, out_coords_and_map

__all__ = ["compute_neighbor_indices", "sparse_conv3d"]


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
        with torch.cuda.device(device), trace.stage("map_build", 3):
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
    with torch.cuda.device(device), trace.stage("map_build", 1):
        rc = _lib.lib().st_map_build(_lib.ptr(coords), n_out, _lib.coord_code(coords), _lib.host_i32(host), K,
                                     int(stride), _lib.host_i32(int(v) for v in spatial_shape), _lib.ptr(keys),
                                     _lib.ptr(vals), keys.shape[0], _lib.ptr(nbr), _lib.stream_ptr())
    _lib.check(rc, "st_map_build")
    return nbr


def _new_table(coords, device):
    table = HashTable(round_up_capacity(coords.shape[0], get_h_table_f()), device=device)
    table.insert(coords)
    return table


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
    cache_key = (k, s, p, d, submanifold, transposed)
    algo = get_conv_algo()
    upsample = transposed and s > 1

    cached = cache.neighbor_indices.get(cache_key) if algo == ConvAlgo.PrecomputedNeighborGEMM else None
    shortcut = submanifold and s == 1                       # output coordinates are the input coordinates
    neighbor_indices = table = koff = None
    if cached is not None:
        out_coords, neighbor_indices, new_shape = cached
    elif algo == ConvAlgo.PrecomputedNeighborGEMM and not shortcut:
        # strided / transposed layer with a stored map: coordinates and map come out of one pass over
        # the candidates; no table over the inputs is needed
        out_coords, new_shape, koff, neighbor_indices = out_coords_and_map(coords, tensor.spatial_shape, k, s, d, p,
                                                                           transposed)
        if out_coords.shape[0] > 0:
            cache.neighbor_indices[cache_key] = (out_coords, neighbor_indices, new_shape)
    else:
        # Table over the coordinates the lookup is made in: the inputs themselves, or, for an
        # upsampling transposed conv, the inputs with their spatial columns scaled (conv.py:138-142).
        if upsample:
            scaled = coords.clone()
            scaled[:, 1:] *= s
            table = _new_table(scaled, device)
        else:
            if cache.hashtable is None:
                cache.hashtable = _new_table(coords, device)
            table = cache.hashtable
        out_coords, new_shape, koff = build_out_coords(coords, tensor.spatial_shape, k, s, d, p,
                                                       transposed=transposed, submanifold=submanifold)
        koff._st_host = [v for o in kernel_offsets(k, d, p, transposed) for v in o]

    if out_coords.shape[0] == 0:
        return SparseTensor(
            feats=torch.empty((0, c_out), device=device, dtype=feats.dtype),
            coords=torch.empty((0, 4), device=device, dtype=coords.dtype),
            spatial_shape=_as_shape(new_shape), batch_size=tensor.batch_size)

    lookup_shape = tuple(v * s for v in tensor.spatial_shape) if upsample else tuple(tensor.spatial_shape)
    lookup_stride = 1 if transposed else s

    if algo == ConvAlgo.PrecomputedNeighborGEMM:
        if neighbor_indices is None:
            neighbor_indices = compute_neighbor_indices(table, out_coords, koff, lookup_shape, lookup_stride, p, d,
                                                        queries_are_table_rows=shortcut and out_coords is coords)
            cache.neighbor_indices[cache_key] = (out_coords, neighbor_indices, new_shape)
        out_feats = ConvPrecomputedNeighborGEMM.apply(feats, weight, neighbor_indices)
    elif algo == ConvAlgo.ImplicitHashFlyGEMM:
        out_feats = ConvHashOnTheFlyImplicitGEMM.apply(feats, weight, out_coords, koff, table.table_keys,
                                                       table.table_values, lookup_shape, lookup_stride)
    else:  # pragma: no cover - ConvAlgo has two members
        raise ValueError(f"unknown convolution algorithm {algo}")

    if bias is not None:
        out_feats = out_feats + bias.to(out_feats.dtype)

    if submanifold and out_coords is coords:
        return tensor.replace(out_feats)
    return SparseTensor._trusted(out_feats, out_coords, _as_shape(new_shape), tensor.batch_size)


def _as_shape(shape):
    if isinstance(shape, torch.Tensor):
        host = getattr(shape, "_st_host", None)
        return tuple(int(v) for v in (host if host is not None else shape.tolist()))
    return tuple(int(v) for v in shape)
