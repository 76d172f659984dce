"""Process-wide switches of the sparse-convolution path.

Mirrors sparsetriton/config.py:21-201 of the reference: same names, defaults, accepted
inputs and error types.  `_STATE` is a plain dict because callers snapshot and restore it.
"""
from enum import Enum

import torch

__all__ = [
    "ConvAlgo", "set_coords_dtype", "get_coords_dtype", "set_conv_algo", "get_conv_algo",
    "set_h_table_f", "get_h_table_f", "set_h_table_max_p", "get_h_table_max_p",
    "set_row_order", "get_row_order", "set_hashfly_transient_map", "get_hashfly_transient_map",
]


class ConvAlgo(Enum):
    """Which form of the gather-GEMM-scatter convolution runs (config.py:21-35)."""
    ImplicitHashFlyGEMM = "Implicit_hashfly_gemm"          # probe the hash table inside the GEMM
    PrecomputedNeighborGEMM = "Precomputed_neighbor_gemm"  # stored (N_out, K) neighbour map


_STATE = {
    "coords_dtype": torch.int16,
    "algo": ConvAlgo.PrecomputedNeighborGEMM,
    "h_tbl_factor": 1.5,       # minimum slots per key; tables are rounded up to a power of two
    "h_tbl_max_probe_n": 16,   # kept for API parity; probing here is bounded by the capacity
    "row_order": True,         # stored-map products walk rows sorted by occupied offsets (no reference counterpart)
    "hashfly_transient_map": True,   # hash-on-the-fly probes once per call into scratch, not once per tile and kernel
}


def set_coords_dtype(dtype):
    if not isinstance(dtype, torch.dtype):
        raise TypeError(f"Expected torch.dtype, got {type(dtype)}")
    _STATE["coords_dtype"] = dtype


def get_coords_dtype():
    return _STATE["coords_dtype"]


def set_conv_algo(algo):
    if not isinstance(algo, ConvAlgo):
        raise TypeError(f"Expected ConvAlgo, got {type(algo)}")
    _STATE["algo"] = algo


def get_conv_algo():
    return _STATE["algo"]


def set_h_table_f(factor):
    try:
        value = float(factor)
    except (TypeError, ValueError):
        raise TypeError("factor must be a number")
    assert value >= 1, "factor must be >= 1"
    _STATE["h_tbl_factor"] = value


def get_h_table_f():
    return _STATE["h_tbl_factor"]


def set_h_table_max_p(probe_n):
    try:
        value = int(probe_n)
    except (TypeError, ValueError):
        raise TypeError("probe_n must be an integer")
    assert value > 0, "probe_n must be positive"
    _STATE["h_tbl_max_probe_n"] = value


def get_h_table_max_p():
    return _STATE["h_tbl_max_probe_n"]


def set_row_order(enabled):
    """Whether the stored-map products walk the rows of their map sorted by occupied offsets
    (fewer, denser 128-row tile steps).  Results of forward and feature gradient are the same
    either way.  No counterpart in the reference."""
    if not isinstance(enabled, bool):
        raise TypeError(f"Expected bool, got {type(enabled)}")
    _STATE["row_order"] = enabled


def get_row_order():
    return _STATE["row_order"]


def set_hashfly_transient_map(enabled):
    """How ImplicitHashFlyGEMM finds its neighbours.  True (default): each forward and each backward call probes
    the table once into a scratch map that lives for that call only (nothing is kept between calls, which is
    what distinguishes the algorithm from PrecomputedNeighborGEMM) and runs the tile-planned tensor-core kernels
    over it.  False: the kernels probe the table themselves, per tile and per kernel, as the reference's
    Triton kernels do; no scratch map exists at any time (lowest memory, several times slower).  Results are
    identical.  No counterpart in the reference."""
    if not isinstance(enabled, bool):
        raise TypeError(f"Expected bool, got {type(enabled)}")
    _STATE["hashfly_transient_map"] = enabled


def get_hashfly_transient_map():
    return _STATE["hashfly_transient_map"]
