"""Pooling and nearest-neighbour upsampling of sparse tensors (reference: nn/functional/spatial.py).

`sparse_pooling(input, kernel_size, padding, stride, mode)` and `sparse_upsample(input, scale_factor)`
keep the reference's signatures, output order and shapes; the work is done by the CUDA library:

  pooling   out cell = floor((in + padding - kernel_size // 2) / stride) per axis; output rows are the
            distinct cells in ascending (batch, x, y, z) order (the reference's sorted `torch.unique` of
            the packed coordinates, spatial.py:123-129).  st_pool_count / st_pool_write sort the inputs
            by cell on the device, st_pool_fwd reduces every row over its own segment (mean or max, fp32,
            no atomics) and st_pool_bwd is a gather.  `mode="max"` works here; the reference's
            atomic-max kernel does not compile (its own test skips it).
  upsample  row i -> rows i*s^3 + (dx*s + dy)*s + dz at in*s + (dx, dy, dz) (spatial.py:305-396).

Cells are exact integers: inputs at coordinate 0 with padding < kernel_size // 2 land in cell -1, which
the reference's 16-bit packing aliases; here it stays -1.
"""
import torch

from sparsetriton_b200 import _lib, trace
from sparsetriton_b200.tensor import SparseTensor

__all__ = ["sparse_pooling", "sparse_upsample", "SparsePoolingFunction", "SparseUpsampleFunction"]


class SparsePoolingFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, in_feats, in_coords, spatial_shape, kernel_size, padding, stride, mode="max", batch_size=None):
        if mode not in ("max", "avg"):
            raise ValueError(f"Unsupported mode: {mode}")
        _lib.require_cuda(in_feats, "sparse_pooling")
        if stride is None:
            stride = kernel_size
        shape = tuple(int(v) for v in spatial_shape)
        new_shape = tuple((s - kernel_size + padding * 2) // stride + 1 for s in shape)          # spatial.py:116
        feats = in_feats.contiguous()
        coords = in_coords.contiguous()
        dev = feats.device
        n, C = feats.shape
        if batch_size is None:
            batch_size = int(coords[:, 0].max().item()) + 1 if n > 0 else 0
        L = _lib.lib()
        code, ccode = _lib.feat_code(feats), _lib.coord_code(coords)
        shape_h = _lib.host_i32(shape)
        ws = _lib.workspace(L.st_pool_workspace_bytes(n), dev)
        counters = torch.zeros(2, dtype=torch.int64, device=dev)          # [n_out, status]
        status = counters[1:].view(torch.int32)
        with _lib.on_device(dev), trace.stage("pool_map"):
            s = _lib.stream_ptr()
            _lib.check(L.st_pool_count(_lib.ptr(coords), n, ccode, kernel_size, padding, stride, shape_h, int(batch_size),
                                       _lib.ptr(ws), ws.numel(), _lib.ptr(counters), _lib.ptr(status), s), "st_pool_count")
            n_out, flags = counters.tolist()                               # the one device->host read
            if flags & _lib.DEV_BAD_INDEX:
                raise ValueError("sparse_pooling: a coordinate lies outside spatial_shape / batch_size")
            out_coords = torch.empty((n_out, 4), dtype=coords.dtype, device=dev)
            in_to_out = torch.empty((n,), dtype=torch.int32, device=dev)
            members = torch.empty((n,), dtype=torch.int32, device=dev)
            seg_start = torch.empty((n_out + 1,), dtype=torch.int32, device=dev)
            _lib.check(L.st_pool_write(_lib.ptr(coords), n, ccode, kernel_size, padding, stride, shape_h, int(batch_size),
                                       _lib.ptr(ws), ws.numel(), _lib.ptr(out_coords), n_out, _lib.ptr(in_to_out),
                                       _lib.ptr(members), _lib.ptr(seg_start), s), "st_pool_write")
        out_feats = torch.empty((n_out, C), dtype=feats.dtype, device=dev)
        with _lib.on_device(dev), trace.stage("pool_fwd"):
            _lib.check(L.st_pool_fwd(code, _lib.ptr(feats), C, _lib.ptr(members), _lib.ptr(seg_start), n_out,
                                     int(mode == "max"), _lib.ptr(out_feats), _lib.stream_ptr()), "st_pool_fwd")
        ctx.save_for_backward(feats, out_feats, in_to_out, seg_start)
        ctx.mode = mode
        ctx.mark_non_differentiable(out_coords)
        return out_feats, out_coords, new_shape

    @staticmethod
    def backward(ctx, grad_out_feats, grad_out_coords, grad_spatial_shape):
        feats, out_feats, in_to_out, seg_start = ctx.saved_tensors
        n, C = feats.shape
        g = grad_out_feats.to(feats.dtype).contiguous()
        grad_in = torch.empty_like(feats)
        with _lib.on_device(feats.device), trace.stage("pool_bwd"):
            _lib.check(_lib.lib().st_pool_bwd(_lib.feat_code(feats), _lib.ptr(g), _lib.ptr(feats), _lib.ptr(out_feats), C,
                                              _lib.ptr(in_to_out), _lib.ptr(seg_start), n, int(ctx.mode == "max"),
                                              _lib.ptr(grad_in), _lib.stream_ptr()), "st_pool_bwd")
        return grad_in, None, None, None, None, None, None, None


def sparse_pooling(input: SparseTensor, kernel_size: int, padding: int, stride: int, mode: str) -> SparseTensor:
    """Mean ("avg") or maximum ("max") of the voxels of every pooling cell (spatial.py:265-292)."""
    out_feats, out_coords, new_shape = SparsePoolingFunction.apply(
        input.F, input.C, input.spatial_shape, kernel_size, padding, stride, mode, input.batch_size)
    return SparseTensor._trusted(out_feats, out_coords, new_shape, input.batch_size)


class SparseUpsampleFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, feats, coords, spatial_shape, scale_factor):
        _lib.require_cuda(feats, "sparse_upsample")
        feats, coords = feats.contiguous(), coords.contiguous()
        n, C = feats.shape
        s3 = scale_factor ** 3
        dev = feats.device
        out_feats = torch.empty((n * s3, C), dtype=feats.dtype, device=dev)
        out_coords = torch.empty((n * s3, 4), dtype=coords.dtype, device=dev)
        with _lib.on_device(dev), trace.stage("upsample_fwd"):
            _lib.check(_lib.lib().st_upsample_fwd(_lib.feat_code(feats), _lib.ptr(feats), _lib.ptr(coords),
                                                  _lib.coord_code(coords), n, C, int(scale_factor), _lib.ptr(out_feats),
                                                  _lib.ptr(out_coords), _lib.stream_ptr()), "st_upsample_fwd")
        ctx.geometry = (n, C, int(scale_factor))
        ctx.mark_non_differentiable(out_coords)
        return out_feats, out_coords, tuple(int(v) * scale_factor for v in spatial_shape)

    @staticmethod
    def backward(ctx, grad_output, grad_coords, grad_shape):
        n, C, scale = ctx.geometry
        g = grad_output.contiguous()
        grad_in = torch.empty((n, C), dtype=g.dtype, device=g.device)
        with _lib.on_device(g.device), trace.stage("upsample_bwd"):
            _lib.check(_lib.lib().st_upsample_bwd(_lib.feat_code(g), _lib.ptr(g), n, C, scale, _lib.ptr(grad_in),
                                                  _lib.stream_ptr()), "st_upsample_bwd")
        return grad_in, None, None, None


def sparse_upsample(input: SparseTensor, scale_factor: int = None) -> SparseTensor:
    """Every voxel replicated to scale_factor^3 voxels (spatial.py:508-535)."""
    out_feats, out_coords, new_shape = SparseUpsampleFunction.apply(input.F, input.C, input.spatial_shape, scale_factor)
    return SparseTensor._trusted(out_feats, out_coords, new_shape, input.batch_size)
