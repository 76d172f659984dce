"""Channel padding so that narrow layers still reach the tensor-core kernels.

The tcgen05 kernels need the reduction width to be a multiple of one MMA K-step (16 half-precision
or 8 fp32 channels) and the output width a multiple of 16.  A layer such as the 4-channel network
input or a 20-class head is therefore run on zero-padded copies of its operands: zero input channels
meet zero weight rows, padded output columns are cut off again, so the result is unchanged.
"""
import torch
import torch.nn.functional as F

from sparsetriton_b200 import _lib

__all__ = ["padded_widths", "pad_cols", "pad_weight"]


def _round_up(v, m):
    return (v + m - 1) // m * m


def padded_widths(dtype, c_in, c_out):
    """(c_in', c_out') to run the layer with: the widths themselves if the tensor-core kernels take
    them or padding would not help, else the next widths they take."""
    code = _lib._FEAT_CODES.get(dtype)
    if code is None:
        return c_in, c_out
    uses = _lib.lib().st_conv_uses_tensor_cores
    if uses(code, c_in, c_out) and uses(code, c_out, c_in):
        return c_in, c_out
    ci, co = _round_up(c_in, 16), _round_up(c_out, 16)
    if uses(code, ci, co) and uses(code, co, ci):
        return ci, co
    return c_in, c_out


def pad_cols(t, width):
    """(N, C) -> (N, width) with zero columns appended."""
    return t if t.shape[1] == width else F.pad(t, (0, width - t.shape[1]))


def pad_weight(w, c_in, c_out):
    """(K, Cin, Cout) -> (K, c_in, c_out) with zero rows / columns appended."""
    if w.shape[1] == c_in and w.shape[2] == c_out:
        return w
    return F.pad(w, (0, c_out - w.shape[2], 0, c_in - w.shape[1]))
