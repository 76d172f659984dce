"""Coordinate hash table (reference: sparsetriton/utils/hash.py).

Same class surface as the reference's ``HashTable`` (ctor arguments, ``insert``, ``query``,
``capacity``, ``device``, ``cpu``/``to``, public ``table_keys`` / ``table_values`` tensors with
-1 marking an empty slot), but the kernels behind it are CUDA kernels of
libsparsetriton_b200 and the stored key is the exact packed coordinate

    key = batch << 48 | x << 32 | y << 16 | z        (int64)

instead of the reference's second 31-bit hash (hash.py:136-152), so two different coordinates can
never be confused.  ``table_values`` holds int32 row indices.  A coordinate inserted more than once
keeps its largest row index.
"""
import torch

from sparsetriton_b200 import _lib, trace
from sparsetriton_b200.config import get_coords_dtype

__all__ = ["HashTable", "flatten_coord", "hash_coords", "unflatten_coord"]


def flatten_coord(coords):
    """(N,4) (batch,x,y,z) -> int64 with 16 bits per field (hash.py:25-53)."""
    c = coords.to(torch.int64)
    return (c[:, 0] << 48) | (c[:, 1] << 32) | (c[:, 2] << 16) | c[:, 3]


def unflatten_coord(flat_coords):
    """Inverse of flatten_coord, returned in the configured coordinate dtype (hash.py:56-84)."""
    fields = [(flat_coords >> shift) & 0xFFFF for shift in (48, 32, 16, 0)]
    return torch.stack(fields, dim=1).to(get_coords_dtype())


def hash_coords(coords):
    """Non-negative int32 spatial hash of (N,4) coordinates (hash.py:87-113)."""
    c = coords.to(torch.int32)
    mixed = (c[:, 1] * 73856093) ^ (c[:, 2] * 19349663) ^ (c[:, 3] * 83492791) ^ (c[:, 0] * 1000003)
    return mixed & 0x7FFFFFFF


def round_up_capacity(n_keys, factor):
    """Power-of-two slot count >= factor * n_keys (so the slot index is a mask, not a modulo)."""
    want = max(int(n_keys * factor), 1)
    return 1 << (want - 1).bit_length()


class HashTable:
    """Open-addressing table from voxel coordinate to row index (hash.py:369-580)."""

    def __init__(self, capacity=None, device="cpu", table_keys=None, table_values=None):
        assert capacity is not None or (table_keys is not None and table_values is not None), \
            "Either capacity or both table_keys and table_values must be provided."
        if table_keys is not None and table_values is not None:
            assert table_keys.shape == table_values.shape, "table_keys and table_values must have the same shape."
            self.table_keys, self.table_values = table_keys, table_values
            return
        dev = torch.device(device)
        if dev.type == "cuda" and capacity > 0:
            self.table_keys = torch.empty((capacity,), dtype=torch.int64, device=dev)
            self.table_values = torch.empty((capacity,), dtype=torch.int32, device=dev)
            with _lib.on_device(self.table_keys.device), trace.stage("hash_clear", 1):
                rc = _lib.lib().st_hash_clear(_lib.ptr(self.table_keys), _lib.ptr(self.table_values), capacity,
                                              _lib.stream_ptr())
            _lib.check(rc, "st_hash_clear")
        else:
            self.table_keys = torch.full((capacity,), -1, dtype=torch.int64, device=dev)
            self.table_values = torch.full((capacity,), -1, dtype=torch.int32, device=dev)

    @property
    def device(self):
        return self.table_keys.device

    @device.setter
    def device(self, device):
        self.table_keys = self.table_keys.to(device, non_blocking=True)
        self.table_values = self.table_values.to(device, non_blocking=True)

    def cpu(self):
        self.device = torch.device("cpu")
        return self

    def to(self, device):
        self.device = device
        return self

    @property
    def capacity(self):
        return self.table_keys.shape[0]

    def _kernel_ready(self, coords, what):
        _lib.require_cuda(self.table_keys, what)
        _lib.require_cuda(coords, what)
        if self.table_keys.dtype != torch.int64 or self.table_values.dtype != torch.int32:
            raise TypeError(f"{what}: table_keys must be int64 and table_values int32")
        assert coords.ndim == 2 and coords.shape[1] == 4, "coordinates must have shape (N, 4)"
        if coords.dtype not in (torch.int16, torch.int32):
            coords = coords.to(torch.int32)
        return coords.contiguous()

    def insert(self, keys):
        """Insert (N,4) coordinates; the stored value of row i is i (hash.py:516-544)."""
        assert self.capacity >= keys.shape[0], \
            "Hash table capacity should be at least twice the number of keys to ensure low collision rate."
        if keys.shape[0] == 0:
            return
        coords = self._kernel_ready(keys, "HashTable.insert")
        # one status word per table, kept across inserts: the kernels OR their ST_DEV_* conditions into it
        status = getattr(self, "_status", None)
        if status is None or status.device != coords.device:
            status = self._status = torch.zeros(1, dtype=torch.int32, device=coords.device)
        with _lib.on_device(coords.device), trace.stage("hash_build", 1):
            rc = _lib.lib().st_hash_build(_lib.ptr(coords), coords.shape[0], _lib.coord_code(coords),
                                          _lib.ptr(self.table_keys), _lib.ptr(self.table_values), self.capacity,
                                          _lib.ptr(status), _lib.stream_ptr())
        _lib.check(rc, "st_hash_build")

    def check(self):
        """Raise if an insert into this table ran out of slots (repeated inserts can exceed the capacity that
        each of them passed on its own) or met a coordinate outside [0, 65535], which has no key.  One
        device->host read; no reference counterpart (the reference drops such keys silently)."""
        status = getattr(self, "_status", None)
        flags = int(status.item()) if status is not None else 0
        if flags & _lib.DEV_TABLE_FULL:
            raise RuntimeError("HashTable: an insert found no free slot (capacity too small for all inserted keys)")
        if flags & _lib.DEV_BAD_INDEX:
            raise ValueError("HashTable: a coordinate outside [0, 65535] cannot be stored")

    def query(self, keys):
        """int32 row index of each (N,4) coordinate, -1 where absent (hash.py:546-580)."""
        n = keys.shape[0]
        if n == 0:
            return torch.empty((0,), dtype=torch.int32, device=self.device)
        coords = self._kernel_ready(keys, "HashTable.query")
        out = torch.empty((n,), dtype=torch.int32, device=coords.device)
        with _lib.on_device(coords.device), trace.stage("hash_query", 1):
            rc = _lib.lib().st_hash_query(_lib.ptr(coords), n, _lib.coord_code(coords), _lib.ptr(self.table_keys),
                                          _lib.ptr(self.table_values), self.capacity, _lib.ptr(out),
                                          _lib.stream_ptr())
        _lib.check(rc, "st_hash_query")
        return out
