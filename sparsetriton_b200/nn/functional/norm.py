"""Per-sample batch normalisation of sparse features (reference: nn/functional/norm.py:20-112).

Statistics are taken per (batch index, channel), exactly as in the reference, so sharding a batch by
sample over GPUs needs no cross-GPU statistics.  On the GPU the layer runs as four streaming kernels
behind the C ABI (st_bn_sums / st_bn_apply / st_bn_backward_sums / st_bn_backward_apply), with the
ReLU that follows it in the reference's networks optionally folded in (`relu=True`; the reference has
no fused form, its ReLU is a separate module).  Unlike the reference, half / bfloat16 features are
accepted: statistics are fp32 and the result is cast back to the feature dtype.
"""
import torch

from sparsetriton_b200 import _lib, trace
from sparsetriton_b200.tensor import SparseTensor

__all__ = ["sparse_batch_norm"]


def _batch_info(tensor: SparseTensor):
    """(int32 batch index per row, fp32 1/count per sample, int32 status word), memoised with the coordinate
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
        hit = (ids, (1.0 / counts).contiguous(), torch.zeros(1, dtype=torch.int32, device=ids.device))
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
    def forward(ctx, x, weight, bias, batch, inv_count, n_samples, eps, relu, mean_in, rstd_in, status):
        _lib.require_cuda(x, "sparse_batch_norm")
        x = x.contiguous()
        n, C = x.shape
        L = _lib.lib()
        code = _lib.feat_code(x)
        dev = x.device
        w = weight.detach().float().contiguous() if weight is not None else None
        b = bias.detach().float().contiguous() if bias is not None else None
        with torch.cuda.device(dev), trace.stage("bn_fwd"):
            s = _lib.stream_ptr()
            if mean_in is None:
                sums = torch.empty((n_samples, C, 2), dtype=torch.float32, device=dev)
                _lib.check(L.st_bn_sums(code, _lib.ptr(x), _lib.ptr(batch), n, C, n_samples, None, _lib.ptr(sums),
                                        _lib.ptr(status), s), "st_bn_sums")
                mean = (sums[:, :, 0] * inv_count.view(-1, 1)).contiguous()
                _lib.check(L.st_bn_sums(code, _lib.ptr(x), _lib.ptr(batch), n, C, n_samples, _lib.ptr(mean),
                                        _lib.ptr(sums), _lib.ptr(status), s), "st_bn_sums")
                var = sums[:, :, 1] * inv_count.view(-1, 1)
                rstd = torch.rsqrt(var + eps).contiguous()
            else:
                mean, rstd, var = mean_in.clone(), rstd_in, None
            y = torch.empty_like(x)
            _lib.check(L.st_bn_apply(code, _lib.ptr(x), _lib.ptr(batch), n, C, n_samples, _lib.ptr(mean), _lib.ptr(rstd),
                                     _lib.ptr(w), _lib.ptr(b), 1 if relu else 0, _lib.ptr(y), _lib.ptr(status), s),
                       "st_bn_apply")
        ctx.save_for_backward(x, batch, inv_count, mean, rstd, w, b)
        ctx.status = status
        ctx.meta = (n_samples, relu, weight is not None, bias is not None, mean_in is None)
        ctx.mark_non_differentiable(mean)
        if var is None:
            var = torch.empty(0, device=dev)
        ctx.mark_non_differentiable(var)
        return y, mean, var

    @staticmethod
    def backward(ctx, dy, _dmean, _dvar):
        x, batch, inv_count, mean, rstd, w, b = ctx.saved_tensors
        n_samples, relu, has_w, has_b, batch_stats = ctx.meta
        n, C = x.shape
        L = _lib.lib()
        code = _lib.feat_code(x)
        dy = dy.to(x.dtype).contiguous()
        dev = x.device
        with torch.cuda.device(dev), trace.stage("bn_bwd"):
            s = _lib.stream_ptr()
            sums = torch.empty((n_samples, C, 2), dtype=torch.float32, device=dev)
            _lib.check(L.st_bn_backward_sums(code, _lib.ptr(x), _lib.ptr(dy), _lib.ptr(batch), n, C, n_samples,
                                             _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(w), _lib.ptr(b), 1 if relu else 0,
                                             _lib.ptr(sums), _lib.ptr(ctx.status), s), "st_bn_backward_sums")
            dw = sums[:, :, 1].sum(0) if has_w else None
            db = sums[:, :, 0].sum(0) if has_b else None
            dx = None
            if ctx.needs_input_grad[0]:
                dx = torch.empty_like(x)
                # with fixed (running) statistics the two correction terms vanish
                corr = sums if batch_stats else torch.zeros_like(sums)
                _lib.check(L.st_bn_backward_apply(code, _lib.ptr(x), _lib.ptr(dy), _lib.ptr(batch), n, C, n_samples,
                                                  _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(w), _lib.ptr(b),
                                                  1 if relu else 0, _lib.ptr(corr), _lib.ptr(inv_count), _lib.ptr(dx),
                                                  _lib.ptr(ctx.status), s), "st_bn_backward_apply")
        return dx, dw, db, None, None, None, None, None, None, None, None


def sparse_batch_norm(tensor: SparseTensor, weight=None, bias=None, running_mean=None, running_var=None,
                      training=True, eps=1e-5, momentum=0.1, relu=False) -> SparseTensor:
    feats = tensor.F
    if feats.shape[0] == 0:
        return tensor.replace(feats)
    C = feats.shape[1]
    if training:
        batch, inv_count, status = _batch_info(tensor)
        y, mean, var = _BatchNormFn.apply(feats, weight, bias, batch, inv_count, tensor.batch_size, float(eps), bool(relu),
                                          None, None, status)
        if running_mean is not None:
            running_mean.mul_(1 - momentum).add_(momentum * mean.mean(0).detach())
        if running_var is not None:
            running_var.mul_(1 - momentum).add_(momentum * var.mean(0).detach())
    else:
        mean = running_mean.detach().float().view(1, C).contiguous()
        rstd = torch.rsqrt(running_var.detach().float() + eps).view(1, C).contiguous()
        one = torch.ones(1, dtype=torch.float32, device=feats.device)
        y, _, _ = _BatchNormFn.apply(feats, weight, bias, None, one, 1, float(eps), bool(relu), mean, rstd, None)
    return tensor.replace(y)
