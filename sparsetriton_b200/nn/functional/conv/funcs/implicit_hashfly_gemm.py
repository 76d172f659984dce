"""Hash-on-the-fly form of the convolution: autograd Function over the C ABI.

Reference: nn/functional/conv/funcs/implicit_hashfly_gemm.py:330-452
(ConvHashOnTheFlyImplicitGEMM).  Same call signature and return values:

    out = ConvHashOnTheFlyImplicitGEMM.apply(features, weights, coords, kernel_offsets,
                                             hash_table_keys, hash_table_vals,
                                             spatial_shape, lookup_stride)
    backward -> (d_features, d_weights, None, None, None, None, None, None)

No neighbour map is stored between calls.  Two forms (config.set_hashfly_transient_map):

  transient map (default)  each forward and each backward call evaluates
        curr = out * lookup_stride - kernel_offsets[k]   (dropped when outside [0, spatial_shape))
      against the table once, into a scratch (N_out, K) map that is freed when the call returns, and runs the
      tile-planned tensor-core kernels of the stored-map form over it: one probe per (row, offset) and call
      instead of one per (row, offset), kernel and channel block;
  in-kernel probing        every tile of every kernel probes the table itself, as the reference's Triton kernels
      do; no scratch map at any time.

dgrad accumulates in fp32 without atomics (gather over the inverse of the probed map); wgrad reduces fp32
partials in a fixed order.  The weight-gradient kernel of the reference omits the upper bound check (:308);
the full check is applied here in all three products.
"""
import torch

from sparsetriton_b200 import _lib, trace

from sparsetriton_b200.config import get_hashfly_transient_map

from ._channels import pad_cols, pad_weight, padded_widths
from .implicit_precomputed_gemm import stored_map_dgrad, stored_map_forward, stored_map_wgrad

__all__ = ["ConvHashOnTheFlyImplicitGEMM"]


def _host_offsets(kernel_offsets):
    host = getattr(kernel_offsets, "_st_host", None)
    if host is None:
        host = [int(v) for v in kernel_offsets.reshape(-1).tolist()]
    return _lib.host_i32(host)


def _probe_map(c, offsets_h, keys, vals, shape_h, lookup_stride, K):
    """(N_out, K) int32 scratch map: row of (batch, out*stride - off[k]) in the table, or -1 (st_map_build)."""
    n_out = c.shape[0]
    nbr = torch.empty((n_out, K), dtype=torch.int32, device=c.device)
    if n_out > 0:
        with _lib.on_device(c.device), trace.stage("hashfly_probe", 1):
            rc = _lib.lib().st_map_build(_lib.ptr(c), n_out, _lib.coord_code(c), offsets_h, K, lookup_stride, shape_h,
                                         _lib.ptr(keys), _lib.ptr(vals), keys.shape[0], _lib.ptr(nbr), _lib.stream_ptr())
        _lib.check(rc, "st_map_build")
    return nbr


class ConvHashOnTheFlyImplicitGEMM(torch.autograd.Function):
    @staticmethod
    def forward(ctx, features, weights, coords, kernel_offsets, hash_table_keys, hash_table_vals, spatial_shape,
                lookup_stride):
        _lib.require_cuda(features, "ConvHashOnTheFlyImplicitGEMM")
        n_in, c_in = features.shape
        K, w_cin, c_out = weights.shape
        assert w_cin == c_in, f"weights expect {w_cin} input channels, features have {c_in}"
        assert kernel_offsets.shape[0] == K, "kernel_offsets must be (K, 3)"
        if hash_table_keys.dtype != torch.int64 or hash_table_vals.dtype != torch.int32:
            raise TypeError("hash table must hold int64 keys and int32 values")
        n_out = coords.shape[0]
        ctx.true_widths = (c_in, c_out)
        c_in, c_out = padded_widths(features.dtype, c_in, c_out)          # narrow layers: zero-padded operands
        x = pad_cols(features, c_in).contiguous()
        w = pad_weight(weights.to(x.dtype), c_in, c_out).contiguous()
        c = coords.contiguous()
        keys, vals = hash_table_keys.contiguous(), hash_table_vals.contiguous()
        ctx.offsets_h = _host_offsets(kernel_offsets)
        ctx.shape_h = _lib.host_i32(int(v) for v in spatial_shape)
        ctx.lookup_stride = int(lookup_stride)
        ctx.w_dtype = weights.dtype
        code = _lib.feat_code(x)
        ctx.transient = bool(get_hashfly_transient_map())
        if ctx.transient:
            nbr = _probe_map(c, ctx.offsets_h, keys, vals, ctx.shape_h, ctx.lookup_stride, K)
            y, _ = stored_map_forward(x, w, nbr, n_in)
            del nbr                                                   # the map and its plan die with the call
            ctx.save_for_backward(x, w, c, keys, vals)
            return y if c_out == ctx.true_widths[1] else y[:, :ctx.true_widths[1]].contiguous()
        y = torch.empty((n_out, c_out), device=x.device, dtype=x.dtype)
        if n_out > 0:
            with _lib.on_device(x.device), trace.stage("conv_fwd_hashfly", 1):
                rc = _lib.lib().st_conv_fwd_hashfly(
                    code, _lib.ptr(x), _lib.ptr(w), _lib.ptr(c), _lib.coord_code(c), ctx.offsets_h, _lib.ptr(keys),
                    _lib.ptr(vals), keys.shape[0], ctx.shape_h, ctx.lookup_stride, _lib.ptr(y), n_in, n_out, K, c_in,
                    c_out, None, 0, _lib.stream_ptr())
            _lib.check(rc, "st_conv_fwd_hashfly")
        ctx.save_for_backward(x, w, c, keys, vals)
        return y if c_out == ctx.true_widths[1] else y[:, :ctx.true_widths[1]].contiguous()

    @staticmethod
    def backward(ctx, grad_output):
        x, w, c, keys, vals = ctx.saved_tensors
        n_in, c_in = x.shape
        K, _, c_out = w.shape
        n_out = c.shape[0]
        t_in, t_out = ctx.true_widths
        dy = pad_cols(grad_output.to(x.dtype), c_out).contiguous()
        code, ccode = _lib.feat_code(x), _lib.coord_code(c)
        L = _lib.lib()
        dx = dw = None
        if ctx.transient:
            nbr = _probe_map(c, ctx.offsets_h, keys, vals, ctx.shape_h, ctx.lookup_stride, K)
            if ctx.needs_input_grad[0]:
                dx = stored_map_dgrad(dy, w, nbr, n_in)
            if ctx.needs_input_grad[1]:
                dw = stored_map_wgrad(x, dy, nbr, K).to(ctx.w_dtype)
            del nbr
            if dx is not None and t_in != c_in:
                dx = dx[:, :t_in].contiguous()
            if dw is not None and (t_in != c_in or t_out != c_out):
                dw = dw[:, :t_in, :t_out].contiguous()
            return dx, dw, None, None, None, None, None, None
        with _lib.on_device(x.device):
            stream = _lib.stream_ptr()
            ws = _lib.workspace(L.st_conv_hashfly_workspace_bytes(code, n_in, n_out, K, c_in, c_out), x.device)
            if ctx.needs_input_grad[0]:
                dx = torch.empty_like(x)
                with trace.stage("conv_dgrad_hashfly", 3):
                    rc = L.st_conv_dgrad_hashfly(
                        code, _lib.ptr(dy), _lib.ptr(w), _lib.ptr(c), ccode, ctx.offsets_h, _lib.ptr(keys),
                        _lib.ptr(vals), keys.shape[0], ctx.shape_h, ctx.lookup_stride, _lib.ptr(dx), n_in, n_out, K,
                        c_in, c_out, _lib.ptr(ws), ws.numel(), stream)
                _lib.check(rc, "st_conv_dgrad_hashfly")
            if ctx.needs_input_grad[1]:
                dw = torch.empty_like(w)
                with trace.stage("conv_wgrad_hashfly", 2):
                    rc = L.st_conv_wgrad_hashfly(
                        code, _lib.ptr(x), _lib.ptr(dy), _lib.ptr(c), ccode, ctx.offsets_h, _lib.ptr(keys),
                        _lib.ptr(vals), keys.shape[0], ctx.shape_h, ctx.lookup_stride, _lib.ptr(dw), n_in, n_out, K,
                        c_in, c_out, _lib.ptr(ws), ws.numel(), stream)
                _lib.check(rc, "st_conv_wgrad_hashfly")
                dw = dw.to(ctx.w_dtype)
        if dx is not None and t_in != c_in:
            dx = dx[:, :t_in].contiguous()
        if dw is not None and (t_in != c_in or t_out != c_out):
            dw = dw[:, :t_in, :t_out].contiguous()
        return dx, dw, None, None, None, None, None, None
