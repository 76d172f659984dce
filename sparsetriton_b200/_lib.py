"""Loader and thin ctypes binding of libsparsetriton_b200.so.

The product has no CPU fallback: if the library is missing, or a tensor that reaches a
kernel is not a CUDA tensor, the call raises.  Pointers are taken from torch tensors; the
library itself knows nothing about torch.
"""
import contextlib
import ctypes
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "_native", "libsparsetriton_b200.so")

ST_I16, ST_I32 = 0, 1
ST_F32, ST_F16, ST_BF16 = 0, 1, 2
DEV_TABLE_FULL, DEV_OUT_OVERFLOW, DEV_BAD_INDEX, DEV_TIMEOUT = 1, 2, 4, 8

_COORD_CODES = {torch.int16: ST_I16, torch.int32: ST_I32}
_FEAT_CODES = {torch.float32: ST_F32, torch.float16: ST_F16, torch.bfloat16: ST_BF16}

_lib = None

_I64, _INT, _PTR = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p

_SIGNATURES = {
    "st_version": ([], _INT),
    "st_last_error_string": ([], ctypes.c_char_p),
    "st_launch_count": ([], ctypes.c_longlong),
    "st_conv_uses_tensor_cores": ([_INT, _INT, _INT], _INT),
    "st_set_dense_tiles": ([_INT], _INT),
    "st_concat_cols": ([_PTR, _PTR, _I64, _INT, _INT, _PTR, _PTR], _INT),
    "st_split_cols": ([_PTR, _I64, _INT, _INT, _PTR, _PTR, _PTR], _INT),
    "st_device_status": ([_PTR, _PTR], _INT),
    "st_device_status_enqueue": ([_PTR, _PTR], _INT),
    "st_device_status_clear": ([_PTR], _INT),
    "st_set_tensor_cores": ([_INT], _INT),
    "st_set_tma": ([_INT], _INT),
    "st_hash_clear": ([_PTR, _PTR, _I64, _PTR], _INT),
    "st_hash_build": ([_PTR, _I64, _INT, _PTR, _PTR, _I64, _PTR, _PTR], _INT),
    "st_hash_query": ([_PTR, _I64, _INT, _PTR, _PTR, _I64, _PTR, _PTR], _INT),
    "st_outcoords_workspace_bytes": ([_I64, _INT, _INT, _INT], _I64),
    "st_outcoords_count": ([_PTR, _I64, _INT, _PTR, _INT, _INT, _INT, _PTR, _INT, _PTR, _I64, _PTR, _PTR, _PTR], _INT),
    "st_outcoords_write": ([_PTR, _I64, _INT, _PTR, _INT, _INT, _INT, _PTR, _INT, _PTR, _I64, _PTR, _I64, _PTR, _PTR], _INT),
    "st_outcoords_map": ([_PTR, _I64, _INT, _PTR, _INT, _INT, _INT, _PTR, _PTR, _INT, _PTR, _I64, _PTR, _I64, _PTR], _INT),
    "st_map_build": ([_PTR, _I64, _INT, _PTR, _INT, _INT, _PTR, _PTR, _PTR, _I64, _PTR, _PTR], _INT),
    "st_map_build_symmetric": ([_PTR, _I64, _INT, _PTR, _INT, _PTR, _PTR, _PTR, _I64, _PTR, _PTR, _PTR], _INT),
    "st_conv_dgrad_mirrored": ([_INT, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _I64, _INT, _INT, _INT, _PTR, _I64, _PTR], _INT),
    "st_map_invert": ([_PTR, _I64, _INT, _I64, _PTR, _PTR], _INT),
    "st_map_pairs_workspace_bytes": ([_I64, _INT], _I64),
    "st_map_pairs_count": ([_PTR, _I64, _INT, _PTR, _I64, _PTR, _PTR], _INT),
    "st_map_pairs_write": ([_PTR, _I64, _INT, _PTR, _I64, _PTR, _I64, _PTR, _PTR], _INT),
    "st_conv_workspace_bytes": ([_INT, _I64, _I64, _INT, _INT, _INT], _I64),
    "st_conv_hashfly_workspace_bytes": ([_INT, _I64, _I64, _INT, _INT, _INT], _I64),
    "st_conv_fwd": ([_INT, _PTR, _PTR, _PTR, _PTR, _I64, _I64, _INT, _INT, _INT, _PTR, _I64, _PTR], _INT),
    "st_conv_dgrad": ([_INT, _PTR, _PTR, _PTR, _PTR, _I64, _I64, _INT, _INT, _INT, _PTR, _I64, _PTR], _INT),
    "st_conv_wgrad": ([_INT, _PTR, _PTR, _PTR, _PTR, _I64, _I64, _INT, _INT, _INT, _PTR, _I64, _PTR], _INT),
}
_PLANNED_SIG = ([_INT, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _I64, _I64, _INT, _INT, _INT, _PTR, _I64, _PTR], _INT)
for _n in ("st_conv_fwd_planned", "st_conv_dgrad_planned", "st_conv_wgrad_planned", "st_conv_wgrad_planned_presorted"):
    _SIGNATURES[_n] = _PLANNED_SIG
_SIGNATURES["st_conv_wgrad_presort"] = ([_INT, _PTR, _PTR, _I64, _INT, _INT, _INT, _PTR, _I64, _PTR], _INT)
_SIGNATURES["st_map_plan_workspace_bytes"] = ([_I64, _INT], _I64)
_SIGNATURES["st_map_plan_inverse_workspace_bytes"] = ([_I64, _INT], _I64)
_SIGNATURES["st_map_plan_inverse"] = ([_PTR, _I64, _INT, _I64, _PTR, _PTR, _PTR, _PTR, _I64, _PTR], _INT)
_SIGNATURES["st_map_plan"] = ([_PTR, _I64, _INT, _INT, _PTR, _PTR, _PTR, _PTR, _I64, _PTR], _INT)
_SIGNATURES["st_map_row_order_workspace_bytes"] = ([_I64, _INT], _I64)
_SIGNATURES["st_map_row_order"] = ([_PTR, _I64, _INT, _PTR, _PTR, _I64, _PTR], _INT)
_SIGNATURES["st_bn_sums"] = ([_INT, _PTR, _PTR, _I64, _INT, _INT, _PTR, _PTR, _PTR, _PTR], _INT)
_SIGNATURES["st_bn_apply"] = ([_INT, _PTR, _PTR, _I64, _INT, _INT, _PTR, _PTR, _PTR, _PTR, _INT, _PTR, _PTR, _PTR], _INT)
_SIGNATURES["st_bn_backward_sums"] = ([_INT, _PTR, _PTR, _PTR, _I64, _INT, _INT, _PTR, _PTR, _PTR, _PTR, _INT, _PTR, _PTR,
                                       _PTR], _INT)
_SIGNATURES["st_bn_backward_apply"] = ([_INT, _PTR, _PTR, _PTR, _I64, _INT, _INT, _PTR, _PTR, _PTR, _PTR, _INT, _PTR, _PTR,
                                        _PTR, _PTR, _PTR], _INT)
_F32 = ctypes.c_float
_SIGNATURES["st_conv_wgrad_inverse_workspace_bytes"] = ([_INT, _I64, _INT, _INT, _INT], _I64)
_SIGNATURES["st_conv_wgrad_inverse_planned"] = ([_INT, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _I64, _I64, _INT, _INT, _INT, _PTR, _I64,
                                                 _PTR], _INT)
_SIGNATURES["st_bn_first_rows"] = ([_PTR, _I64, _INT, _PTR, _PTR], _INT)
_SIGNATURES["st_bn_forward_stats"] = ([_INT, _PTR, _PTR, _PTR, _I64, _INT, _INT, _PTR, _F32, _F32, _PTR, _PTR, _PTR, _PTR, _PTR,
                                       _PTR, _PTR], _INT)
_SIGNATURES["st_bn_backward"] = ([_INT, _PTR, _PTR, _PTR, _I64, _INT, _INT, _PTR, _PTR, _PTR, _PTR, _INT, _INT, _PTR, _PTR, _PTR,
                                  _PTR, _PTR, _PTR, _PTR], _INT)
_SIGNATURES["st_conv_wgrad_static_max_bytes"] = ([], _I64)
_SIGNATURES["st_conv_wgrad_static"] = ([_INT, _PTR, _PTR, _PTR, _PTR, _I64, _I64, _INT, _INT, _INT, _PTR], _INT)
_SIGNATURES["st_to_dense_fwd"] = ([_INT, _PTR, _PTR, _INT, _I64, _INT, _INT, _PTR, _PTR, _PTR, _PTR], _INT)
_SIGNATURES["st_to_dense_bwd"] = ([_INT, _PTR, _PTR, _INT, _I64, _INT, _INT, _PTR, _PTR, _PTR], _INT)
_SIGNATURES["st_pool_workspace_bytes"] = ([_I64], _I64)
_SIGNATURES["st_pool_count"] = ([_PTR, _I64, _INT, _INT, _INT, _INT, _PTR, _INT, _PTR, _I64, _PTR, _PTR, _PTR], _INT)
_SIGNATURES["st_pool_write"] = ([_PTR, _I64, _INT, _INT, _INT, _INT, _PTR, _INT, _PTR, _I64, _PTR, _I64, _PTR, _PTR, _PTR,
                                 _PTR], _INT)
_SIGNATURES["st_pool_fwd"] = ([_INT, _PTR, _INT, _PTR, _PTR, _I64, _INT, _PTR, _PTR], _INT)
_SIGNATURES["st_pool_bwd"] = ([_INT, _PTR, _PTR, _PTR, _INT, _PTR, _PTR, _I64, _INT, _PTR, _PTR], _INT)
_SIGNATURES["st_upsample_fwd"] = ([_INT, _PTR, _PTR, _INT, _I64, _INT, _INT, _PTR, _PTR, _PTR], _INT)
_SIGNATURES["st_upsample_bwd"] = ([_INT, _PTR, _I64, _INT, _INT, _PTR, _PTR], _INT)
_HASHFLY_SIG = ([_INT, _PTR, _PTR, _PTR, _INT, _PTR, _PTR, _PTR, _I64, _PTR, _INT, _PTR, _I64, _I64, _INT, _INT, _INT,
                 _PTR, _I64, _PTR], _INT)
for _n in ("st_conv_fwd_hashfly", "st_conv_dgrad_hashfly", "st_conv_wgrad_hashfly"):
    _SIGNATURES[_n] = _HASHFLY_SIG

EXPORTED_SYMBOLS = tuple(_SIGNATURES)


def lib():
    """The loaded library; raises RuntimeError if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m sparsetriton_b200.build` "
                "(needs nvcc; there is no CPU fallback)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (argtypes, restype) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = handle
    return _lib


def check(rc, what):
    if rc != 0:
        msg = lib().st_last_error_string().decode()
        raise RuntimeError(f"{what} failed with status {rc}: {msg}")


def require_cuda(t, what):
    if not t.is_cuda:
        raise RuntimeError(f"{what}: expected a CUDA tensor, got device '{t.device}' "
                           "(sparsetriton_b200 has no CPU path)")


def coord_code(t):
    try:
        return _COORD_CODES[t.dtype]
    except KeyError:
        raise TypeError(f"coordinates must be int16 or int32 for the CUDA kernels, got {t.dtype}") from None


def feat_code(t):
    try:
        return _FEAT_CODES[t.dtype]
    except KeyError:
        raise TypeError(f"features must be float32, float16 or bfloat16, got {t.dtype}") from None


def ptr(t):
    """The address of a tensor's first element as a plain integer (None for no tensor): every entry point has its
    argument types declared, so ctypes converts it to `void*` itself, which costs less host time than building a
    c_void_p per argument (a training step passes about a thousand).  An empty tensor gives 0 or the address of its
    storage; the library reads nothing through either."""
    return None if t is None else t.data_ptr()


_NULL_CONTEXT = contextlib.nullcontext()


def on_device(device):
    """`torch.cuda.device(device)`, or nothing at all when `device` is the current one already (the usual case:
    the switch and the switch back cost more host time than many of the calls they guard)."""
    index = device.index if isinstance(device, torch.device) else device
    if index is None or index == torch.cuda.current_device():
        return _NULL_CONTEXT
    return torch.cuda.device(index)


def stream_ptr(device=None):
    """The current CUDA stream of `device` (a torch.device, an index or None) as a raw handle."""
    index = device.index if isinstance(device, torch.device) else device
    if index is None:
        index = torch.cuda.current_device()
    return torch._C._cuda_getCurrentRawStream(index)


def host_i32(values):
    """A ctypes int32 array (host) from a flat python sequence."""
    vals = [int(v) for v in values]
    return (ctypes.c_int32 * len(vals))(*vals)


def workspace(nbytes, device):
    """256-byte aligned scratch from torch's caching allocator."""
    return torch.empty((max(int(nbytes), 256),), dtype=torch.uint8, device=device)


def clear_device_status(device=None):
    """Clears the sticky status word of the tensor-core kernels on `device` (stream-ordered)."""
    with torch.cuda.device(device):
        check(lib().st_device_status_clear(stream_ptr()), "st_device_status_clear")


def raise_on_timeout(words, device):
    """`words`: the four status words read back from the device.  A bounded wait that expired means some earlier product
    returned partial results: clear the word (it is sticky) and raise."""
    if int(words[0]) & DEV_TIMEOUT:
        clear_device_status(device)
        raise RuntimeError("a bounded wait inside a tensor-core kernel expired earlier on this device (wait site %d, "
                           "block %d): results produced since the last check are incomplete" % (int(words[1]), int(words[2])))


def device_status(device=None):
    """[flags, wait site, block, reserved] of the tensor-core kernels on `device` (synchronises)."""
    out = (ctypes.c_int32 * 4)()
    with torch.cuda.device(device):
        check(lib().st_device_status(out, stream_ptr()), "st_device_status")
    return list(out)
