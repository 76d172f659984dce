"""Per-sample batch normalisation of sparse features (reference: nn/functional/norm.py:20-112).

Statistics are taken per (batch index, channel), exactly as in the reference, so sharding a batch by
sample over GPUs needs no cross-GPU statistics.  On the GPU the layer runs as four streaming kernels
behind the C ABI (st_bn_forward_stats + st_bn_apply forward, st_bn_backward backward: one pass over the features
for the statistics, one for the output, two for the gradient; no elementwise torch ops in between), with the
ReLU that follows it in the reference's networks optionally folded in (`relu=True`; the reference has
no fused form, its ReLU is a separate module).  Unlike the reference, half / bfloat16 features are
accepted: statistics are fp32 and the result is cast back to the feature dtype.
"""
import torch

from sparsetriton_b200 import _lib, trace
from sparsetriton_b200.tensor import SparseTensor

__all__ = ["sparse_batch_norm"]


def _batch_info(tensor: SparseTensor):
    """(int32 batch index per row, fp32 1/count per sample, int32 status word, int32 first row per sample), memoised with the coordinate
    set.  The kernels OR ST_DEV_BAD_INDEX into the status word for rows whose batch index is not in
    [0, batch_size) -- such rows join no statistic and come out as zeros; `bad_batch_index(tensor)` reads it."""
    cache = tensor._cache.kmaps
    hit = cache.get("batch_info")
    if hit is None or hit[0].shape[0] != tensor.C.shape[0]:
        ids = tensor.C[:, 0].to(torch.int32).contiguous()
        if tensor.batch_size <= 64:
            # compare-and-sum: a plain reduction, where bincount's atomics all land on a handful of addresses
            samples = torch.arange(tensor.batch_size, dtype=torch.int32, device=ids.device)
            counts = (ids.view(-1, 1) == samples.view(1, -1)).sum(0)
        else:
            counts = torch.bincount(ids.long(), minlength=tensor.batch_size)
        counts = counts.clamp(min=1).to(torch.float32)
        # first row of every sample (-1 for an empty one): the statistics are summed around that row's values
        first = torch.empty((tensor.batch_size,), dtype=torch.int32, device=ids.device)
        with _lib.on_device(ids.device):
            _lib.check(_lib.lib().st_bn_first_rows(_lib.ptr(ids), ids.shape[0], tensor.batch_size, _lib.ptr(first),
                                                   _lib.stream_ptr()), "st_bn_first_rows")
        hit = (ids, (1.0 / counts).contiguous(), torch.zeros(1, dtype=torch.int32, device=ids.device), first)
        cache["batch_info"] = hit
    return hit


def bad_batch_index(tensor: SparseTensor) -> bool:
    """True if a batch-norm kernel has met a batch index outside [0, batch_size) on this tensor's
    coordinate set (one device->host read)."""
    hit = tensor._cache.kmaps.get("batch_info")
    return bool(hit is not None and int(hit[2].item()) & _lib.DEV_BAD_INDEX)


class _BatchNormFn(torch.autograd.Function):
    """y = relu?((x - mean_b) * rstd_b * weight + bias) with statistics per sample b."""

    @staticmethod
    def forward(ctx, x, weight, bias, batch, inv_count, n_samples, eps, relu, mean_in, rstd_in, status, first_row,
                running_mean, running_var, momentum):
        _lib.require_cuda(x, "sparse_batch_norm")
        x = x.contiguous()
        n, C = x.shape
        L = _lib.lib()
        code = _lib.feat_code(x)
        dev = x.device
        w = weight.detach().float().contiguous() if weight is not None else None
        b = bias.detach().float().contiguous() if bias is not None else None
        with _lib.on_device(dev), trace.stage("bn_fwd"):
            s = _lib.stream_ptr()
            if mean_in is None:
                sums = torch.empty((n_samples, C, 2), dtype=torch.float32, device=dev)
                mean = torch.empty((n_samples, C), dtype=torch.float32, device=dev)
                rstd = torch.empty((n_samples, C), dtype=torch.float32, device=dev)
                _lib.check(L.st_bn_forward_stats(code, _lib.ptr(x), _lib.ptr(batch), _lib.ptr(first_row), n, C, n_samples,
                                                 _lib.ptr(inv_count), float(eps), float(momentum), _lib.ptr(sums),
                                                 _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(running_mean),
                                                 _lib.ptr(running_var), _lib.ptr(status), s), "st_bn_forward_stats")
            else:
                mean, rstd = mean_in, rstd_in
            y = torch.empty_like(x)
            _lib.check(L.st_bn_apply(code, _lib.ptr(x), _lib.ptr(batch), n, C, n_samples, _lib.ptr(mean), _lib.ptr(rstd),
                                     _lib.ptr(w), _lib.ptr(b), 1 if relu else 0, _lib.ptr(y), _lib.ptr(status), s),
                       "st_bn_apply")
        ctx.save_for_backward(x, batch, inv_count, mean, rstd, w, b)
        ctx.status = status
        ctx.meta = (n_samples, relu, weight is not None, bias is not None, mean_in is None)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, batch, inv_count, mean, rstd, w, b = ctx.saved_tensors
        n_samples, relu, has_w, has_b, batch_stats = ctx.meta
        n, C = x.shape
        L = _lib.lib()
        code = _lib.feat_code(x)
        dy = dy.to(x.dtype).contiguous()
        dev = x.device
        with _lib.on_device(dev), trace.stage("bn_bwd"):
            sums = torch.empty((n_samples, C, 2), dtype=torch.float32, device=dev)
            dw = torch.empty((C,), dtype=torch.float32, device=dev) if has_w else None
            db = torch.empty((C,), dtype=torch.float32, device=dev) if has_b else None
            dx = torch.empty_like(x) if ctx.needs_input_grad[0] else None
            _lib.check(L.st_bn_backward(code, _lib.ptr(x), _lib.ptr(dy), _lib.ptr(batch), n, C, n_samples, _lib.ptr(mean),
                                        _lib.ptr(rstd), _lib.ptr(w), _lib.ptr(b), 1 if relu else 0, 1 if batch_stats else 0,
                                        _lib.ptr(inv_count), _lib.ptr(sums), _lib.ptr(dx), _lib.ptr(dw), _lib.ptr(db),
                                        _lib.ptr(ctx.status), _lib.stream_ptr()), "st_bn_backward")
        return (dx, dw, db) + (None,) * 12


def sparse_batch_norm(tensor: SparseTensor, weight=None, bias=None, running_mean=None, running_var=None,
                      training=True, eps=1e-5, momentum=0.1, relu=False) -> SparseTensor:
    feats = tensor.F
    if feats.shape[0] == 0:
        return tensor.replace(feats)
    C = feats.shape[1]
    if training:
        batch, inv_count, status, first_row = _batch_info(tensor)
        rm = running_mean if running_mean is not None and running_mean.dtype == torch.float32 else None
        rv = running_var if running_var is not None and running_var.dtype == torch.float32 else None
        if (running_mean is not None and rm is None) or (running_var is not None and rv is None):
            raise TypeError("running_mean / running_var must be float32 tensors")
        # the running buffers are updated by the statistics kernel itself (norm.py:91-94)
        y = _BatchNormFn.apply(feats, weight, bias, batch, inv_count, tensor.batch_size, float(eps), bool(relu), None, None,
                               status, first_row, rm, rv, float(momentum))
    else:
        mean = running_mean.detach().float().view(1, C).contiguous()
        rstd = torch.rsqrt(running_var.detach().float() + eps).view(1, C).contiguous()
        one = torch.ones(1, dtype=torch.float32, device=feats.device)
        y = _BatchNormFn.apply(feats, weight, bias, None, one, 1, float(eps), bool(relu), mean, rstd, None, None, None, None,
                               0.0)
    return tensor.replace(y)
