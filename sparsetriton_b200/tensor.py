"""SparseTensor container, its cache and a seeded random generator.

Mirrors sparsetriton/tensor.py:27-457 of the reference: features (N,C), coordinates (N,4) in
(batch, x, y, z) order cast to the configured coordinate dtype, `spatial_shape` as torch.Size,
`batch_size`, and a TensorCache that travels through `replace` so that layers sharing
coordinates share the hash table and the neighbour maps.
"""
from typing import Any, Dict, Optional, Tuple

import torch

from sparsetriton_b200.config import get_coords_dtype
from sparsetriton_b200.utils.hash import HashTable
from sparsetriton_b200.utils.to_dense import to_dense

__all__ = ["SparseTensor", "randn", "TensorCache"]


class TensorCache:
    """Per-coordinate-set memo (tensor.py:27-52).

    hashtable         table over this tensor's coordinates
    neighbor_indices  (k, s, p, d, subm, transposed) -> (out_coords, nbr (N_out,K) int32, new_shape)
    kmaps             free-form; this implementation keeps derived maps here (inverse maps for
                      the gather-form dgrad) keyed by ("inv", <neighbor_indices key>)
    children          (no reference counterpart) neighbor_indices key -> TensorCache of the output coordinate set
                      of that layer: applying the same geometry to the same coordinates gives the same output
                      coordinates, so what was derived from those (maps of the next layers) is found again, and a
                      whole network's maps can be prepared ahead of its features
    """

    def __init__(self):
        self.kmaps: Dict[Tuple[Any, ...], Any] = {}
        self.hashtable: Optional[HashTable] = None
        self.neighbor_indices: Dict[Tuple[Any, ...], Tuple[torch.Tensor, torch.Tensor, Tuple]] = {}
        self.children: Dict[Tuple[Any, ...], "TensorCache"] = {}

    def child(self, key) -> "TensorCache":
        """The cache of the output coordinate set of the layer `key` (made on first use)."""
        c = self.children.get(key)
        if c is None:
            c = self.children[key] = TensorCache()
        return c


class SparseTensor:
    """Active voxels of a batch of 3-D grids: `feats` (N,C) and `coords` (N,4) (tensor.py:55-378)."""

    def __init__(self, feats, coords, spatial_shape=None, batch_size=None, cache=None):
        self.feats = feats
        self.coords = coords.to(device=feats.device, dtype=get_coords_dtype())
        assert self.feats.shape[0] == self.coords.shape[0], "The number of features and coordinates must match."
        assert self.coords.shape[1] == 4, "Coordinates must have shape (N, 4)."
        assert self.feats.ndim == 2 and self.coords.ndim == 2, "Features and coordinates must be 2D tensors."

        n = self.coords.shape[0]
        # one device->host transfer serves both derived quantities
        extent = self.coords.max(dim=0).values.tolist() if n > 0 else None
        if spatial_shape is None:
            self.spatial_shape = torch.Size([v + 1 for v in extent[1:]]) if n > 0 else torch.Size([0, 0, 0])
        else:
            self.spatial_shape = torch.Size(spatial_shape)
        if batch_size is None:
            self.batch_size = int(extent[0] + 1) if n > 0 else 0
        else:
            if n > 0:
                assert batch_size > extent[0], f"batch_size {batch_size} must be > max batch index {extent[0]}"
            self.batch_size = batch_size
        self._cache = TensorCache() if cache is None else cache
        # dense() sizes its batch axis by the largest batch index present, as the reference does
        self._dense_batch = int(extent[0] + 1) if n > 0 else 1

    @classmethod
    def _trusted(cls, feats, coords, spatial_shape, batch_size, cache=None):
        """Internal constructor for tensors produced by this library's own operators: the
        coordinates are already in range and of the right dtype, so the device->host read that the
        public constructor needs for validation is skipped."""
        self = cls.__new__(cls)
        self.feats = feats
        self.coords = coords
        self.spatial_shape = torch.Size(spatial_shape)
        self.batch_size = batch_size
        self._cache = TensorCache() if cache is None else cache
        self._dense_batch = None
        return self

    # feature / coordinate aliases -------------------------------------------------------------
    @property
    def F(self):
        return self.feats

    @F.setter
    def F(self, feats):
        self.feats = feats

    @property
    def C(self):
        return self.coords

    @C.setter
    def C(self, coords):
        self.coords = coords.to(get_coords_dtype())

    # movement / dtype ---------------------------------------------------------------------------
    def to(self, device, non_blocking=False):
        self.feats = self.feats.to(device, non_blocking=non_blocking)
        self.coords = self.coords.to(device, non_blocking=non_blocking)
        return self

    def cpu(self):
        return self.to("cpu")

    def half(self):
        self.feats = self.feats.half()
        return self

    def float(self):
        self.feats = self.feats.float()
        return self

    def dense(self):
        """(B, X, Y, Z, C) dense copy (tensor.py:296-312); differentiable.  B is the largest batch index + 1
        where the constructor has seen the coordinates, `batch_size` for tensors produced by the library's
        own operators (no device->host read either way)."""
        batch = self._dense_batch if self._dense_batch is not None else max(int(self.batch_size), 1)
        return to_dense(self.feats, self.coords, self.spatial_shape, batch_size=batch)

    def replace(self, feats):
        """Same coordinates, shape, batch size and cache; new features."""
        assert feats.shape[0] == self.coords.shape[0], "The number of features and coordinates must match."
        return SparseTensor._trusted(feats, self.coords, self.spatial_shape, self.batch_size, self._cache)

    def __repr__(self):
        return (
            "SparseTensor(\n"
            f"  feats=tensor(shape={self.feats.shape}, dtype={self.feats.dtype}, device={self.feats.device}),\n"
            f"  coords=tensor(shape={self.coords.shape}, dtype={self.coords.dtype}, device={self.coords.device}),\n"
            f"  spatial_shape={self.spatial_shape}\n"
            ")"
        )

    def __add__(self, other):
        if not isinstance(other, SparseTensor):
            raise NotImplementedError("Addition with dense tensors not yet supported")
        return self.replace(self.feats + other.feats)   # same coordinate set assumed (residual add)


def randn(spatial_shape, batch_size=1, channels=1, nnz=100, device="cpu", dtype=torch.float32):
    """Random SparseTensor with `nnz` distinct coordinates and N(0,1) features (tensor.py:381-457)."""
    cells = batch_size * spatial_shape[0] * spatial_shape[1] * spatial_shape[2]
    if nnz > cells:
        raise ValueError(f"nnz ({nnz}) exceeds total available voxels ({cells})")
    cdt = get_coords_dtype()
    limits = (batch_size, *spatial_shape)
    pool = None
    have = 0
    while have < nnz:
        draw = nnz if pool is None else int((nnz - have) * 1.2)
        cols = [torch.randint(0, hi, (draw, 1), device=device, dtype=cdt) for hi in limits]
        fresh = torch.cat(cols, dim=1)
        pool = fresh if pool is None else torch.cat([pool, fresh], dim=0)
        pool = torch.unique(pool, dim=0)
        have = pool.shape[0]
    coords = pool[:nnz].contiguous()
    feats = torch.randn(nnz, channels, device=device, dtype=dtype, requires_grad=True).contiguous()
    return SparseTensor(feats, coords, spatial_shape=spatial_shape)
