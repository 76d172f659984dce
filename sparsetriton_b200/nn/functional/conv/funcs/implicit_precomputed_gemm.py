"""Stored-map form of the convolution: autograd Function over the C ABI.

Reference: nn/functional/conv/funcs/implicit_precomputed_gemm.py:233-324
(ConvPrecomputedNeighborGEMM).  Same call signature and return values:

    out = ConvPrecomputedNeighborGEMM.apply(features, weights, neighbor_indices)
    backward -> (d_features, d_weights, None)

Forward   Y[o]  = sum_k X[nbr[o,k]] . W[k]                 st_conv_fwd
dgrad     dX[i] = sum_k dY[inv[i,k]] . W[k]^T              st_map_invert + st_conv_dgrad
wgrad     dW[k] = sum_o X[nbr[o,k]]^T . dY[o]              st_conv_wgrad
All three accumulate in fp32 and run without atomics, so results are reproducible run to run
(the reference scatters dX and dW with atomic adds in the storage dtype).
"""
import torch

from sparsetriton_b200 import _lib, trace

from ._channels import pad_cols, pad_weight, padded_widths

__all__ = ["ConvPrecomputedNeighborGEMM", "inverse_map", "map_plan", "MapPlan", "stored_map_forward", "stored_map_dgrad",
           "stored_map_wgrad", "prepare_plans"]

# below this many rows the sort costs more than the denser tiles save
_MIN_ROWS_FOR_ORDER = 16384

# Walk the weight gradient of a strided layer over the INVERSE map's plan (st_conv_wgrad_inverse_planned)?  Its
# tiles are better filled (all rows of a tile share their few offsets), but measured slower on the 64 -> 128
# k3 s2 layer of 1.2 M voxels (0.68 ms against 0.55 ms over the forward plan): each CTA then meets only one or
# two offsets of its group per tile and long runs of tiles without any, so its copy rings run nearly empty.
WGRAD_OVER_INVERSE_PLAN = False


def inverse_map(neighbor_indices, n_in):
    """inv (n_in, K) with inv[nbr[o,k], k] = o.  Memoised on the map tensor: layers that share a
    neighbour map share its inverse."""
    cached = getattr(neighbor_indices, "_st_inverse", None)
    if cached is not None and cached.shape[0] == n_in:
        return cached
    n_out, K = neighbor_indices.shape
    inv = torch.empty((n_in, K), dtype=torch.int32, device=neighbor_indices.device)
    with _lib.on_device(neighbor_indices.device), trace.stage("map_invert", 2):
        rc = _lib.lib().st_map_invert(_lib.ptr(neighbor_indices), n_out, K, n_in, _lib.ptr(inv), _lib.stream_ptr())
    _lib.check(rc, "st_map_invert")
    neighbor_indices._st_inverse = inv
    return inv


class MapPlan:
    """Tile plan of a (forward or inverse) neighbour map: row order, re-laid map, tile masks
    (st_map_plan).  `ptrs()` are the three pointers the *_planned entry points take."""
    __slots__ = ("order", "tmap", "tmask")

    def __init__(self, order, tmap, tmask):
        self.order, self.tmap, self.tmask = order, tmap, tmask

    def ptrs(self):
        return _lib.ptr(self.order), _lib.ptr(self.tmap), _lib.ptr(self.tmask)


_NO_PLAN = MapPlan(None, None, None)


def map_plan(map_tensor):
    """The tile plan of a map, memoised on the map tensor like the inverse (layers that share a
    map share its plan).  Rows are sorted by occupied offsets unless config.set_row_order(False)
    or the map is small."""
    from sparsetriton_b200.config import get_row_order
    n_rows, K = map_tensor.shape
    if n_rows == 0:
        return _NO_PLAN
    sort_rows = bool(get_row_order()) and n_rows >= _MIN_ROWS_FOR_ORDER
    cached = getattr(map_tensor, "_st_plan", None)
    if cached is not None and cached[0] == sort_rows:
        return cached[1]
    L = _lib.lib()
    dev = map_tensor.device
    n_tiles = (n_rows + 127) // 128
    order = torch.empty((n_rows,), dtype=torch.int32, device=dev) if sort_rows else None
    tmap = torch.empty((n_tiles * K * 128,), dtype=torch.int32, device=dev)
    tmask = torch.empty((n_tiles * ((K + 31) // 32),), dtype=torch.int32, device=dev)
    ws = _lib.workspace(L.st_map_plan_workspace_bytes(n_rows, K), dev) if sort_rows else None
    with _lib.on_device(dev), trace.stage("map_plan"):
        rc = L.st_map_plan(_lib.ptr(map_tensor), n_rows, K, 1 if sort_rows else 0, _lib.ptr(order), _lib.ptr(tmap),
                           _lib.ptr(tmask), _lib.ptr(ws), ws.numel() if ws is not None else 0, _lib.stream_ptr())
    _lib.check(rc, "st_map_plan")
    plan = MapPlan(order, tmap, tmask)
    map_tensor._st_plan = (sort_rows, plan)
    return plan


def inverse_plan(neighbor_indices, n_in):
    """Tile plan of the inverse map built straight from the forward map (st_map_plan_inverse), or None
    when that form does not apply (more than 32 offsets, row order switched off, small maps).  Memoised
    on the map tensor."""
    from sparsetriton_b200.config import get_row_order
    n_out, K = neighbor_indices.shape
    if K > 32 or not get_row_order() or n_in < _MIN_ROWS_FOR_ORDER:
        return None
    cached = getattr(neighbor_indices, "_st_inverse_plan", None)
    if cached is not None and cached.order.shape[0] == n_in:
        return cached
    L = _lib.lib()
    dev = neighbor_indices.device
    n_tiles = (n_in + 127) // 128
    order = torch.empty((n_in,), dtype=torch.int32, device=dev)
    tmap = torch.empty((n_tiles * K * 128,), dtype=torch.int32, device=dev)
    tmask = torch.empty((n_tiles,), dtype=torch.int32, device=dev)
    ws = _lib.workspace(L.st_map_plan_inverse_workspace_bytes(n_in, K), dev)
    with _lib.on_device(dev), trace.stage("map_plan_inverse"):
        rc = L.st_map_plan_inverse(_lib.ptr(neighbor_indices), n_out, K, n_in, _lib.ptr(order), _lib.ptr(tmap),
                                   _lib.ptr(tmask), _lib.ptr(ws), ws.numel(), _lib.stream_ptr())
    _lib.check(rc, "st_map_plan_inverse")
    plan = MapPlan(order, tmap, tmask)
    neighbor_indices._st_inverse_plan = plan
    return plan


def _is_symmetric(map_tensor, n_in):
    """True for a submanifold map whose builder found every row under its own coordinate
    (st_map_build_symmetric): then nbr[o,k] = i <=> nbr[i,K-1-k] = o.  The builder's count was copied to pinned
    host memory when the map was built; this waits for that copy only (not for the stream) and memoises."""
    flag = getattr(map_tensor, "_st_asymmetric_rows", None)
    if flag is None or map_tensor.shape[0] != n_in:
        return False
    if not isinstance(flag, bool):
        host, arrived = flag
        arrived.synchronize()
        flag = int(host[0]) == 0
        map_tensor._st_asymmetric_rows = flag
    return flag


_AUX_STREAMS = {}


def _aux_stream(device, like):
    """A second stream per device (and priority of the stream it helps) for work that is independent of what the
    current stream does next."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), like.priority)
    s = _AUX_STREAMS.get(key)
    if s is None:
        s = _AUX_STREAMS[key] = torch.cuda.Stream(device=device, priority=like.priority)
    return s


def prepare_plans(nbr, n_in, backward=True):
    """Builds (and memoises on the map) what the tensor-core products read besides the map: the tile plan, and with
    `backward` the feature gradient's side (nothing more for a symmetric submanifold map, else the inverse map's plan).
    The two plans depend on the map alone and each is a chain of short kernels, so the inverse map's plan is built on
    a second stream beside the forward one; the current stream waits for it before this returns.
    Returns the tensors made, for callers that manage streams."""
    made = []
    fork = None
    if backward and not _is_symmetric(nbr, n_in) and getattr(nbr, "_st_inverse_plan", None) is None \
            and getattr(nbr, "_st_inverse", None) is None:
        cur = torch.cuda.current_stream(nbr.device)
        aux = _aux_stream(nbr.device, cur)
        aux.wait_stream(cur)
        with torch.cuda.stream(aux):
            inv_plan = inverse_plan(nbr, n_in)
            if inv_plan is None:
                inv = inverse_map(nbr, n_in)
                inv_plan = map_plan(inv)
                made.append(inv)
        fork = (cur, aux)
        made += [inv_plan.order, inv_plan.tmap, inv_plan.tmask]
    plan = map_plan(nbr)
    made += [plan.order, plan.tmap, plan.tmask]
    if fork is not None:
        cur, aux = fork
        cur.wait_stream(aux)
        for t in made:
            if t is not None and t.is_cuda and t.numel() > 0:
                t.record_stream(cur)
    return made


def stored_map_forward(x, w, nbr, n_in):
    """Y = sum_k X[nbr[:, k]] . W[k] over a stored map; x, w already padded and contiguous.  Returns (y, flops)."""
    K, c_in, c_out = w.shape
    n_out = nbr.shape[0]
    code = _lib.feat_code(x)
    y = torch.empty((n_out, c_out), device=x.device, dtype=x.dtype)
    flops = 2.0 * trace.map_pairs(nbr) * c_in * c_out if trace.active() else 0.0
    if n_out > 0:
        # the plan only serves the tensor-core kernels
        plan = map_plan(nbr) if _lib.lib().st_conv_uses_tensor_cores(code, c_in, c_out) else _NO_PLAN
        with _lib.on_device(x.device), trace.stage("conv_fwd", work=flops, tag=(c_in, c_out)):
            rc = _lib.lib().st_conv_fwd_planned(code, _lib.ptr(x), _lib.ptr(w), _lib.ptr(nbr), *plan.ptrs(),
                                                _lib.ptr(y), n_in, n_out, K, c_in, c_out, None, 0, _lib.stream_ptr())
        _lib.check(rc, "st_conv_fwd_planned")
    return y, flops


def stored_map_dgrad(dy, w, nbr, n_in, flops=0.0):
    """dX = sum_k dY[inv[:, k]] . W[k]^T; the inverse map is read through its plan (built straight from `nbr`) or,
    for a symmetric submanifold map, is `nbr` itself with the offsets reversed."""
    K, c_in, c_out = w.shape
    n_out = nbr.shape[0]
    code = _lib.feat_code(dy)
    L = _lib.lib()
    dx = torch.empty((n_in, c_in), device=dy.device, dtype=dy.dtype)
    if n_in == 0:
        return dx
    with _lib.on_device(dy.device):
        stream = _lib.stream_ptr()
        tc = bool(L.st_conv_uses_tensor_cores(code, c_out, c_in))
        if tc and _is_symmetric(nbr, n_in):
            # submanifold layer: the map is its own inverse with the offsets reversed
            plan = map_plan(nbr)
            with trace.stage("conv_dgrad", work=flops, tag=(c_in, c_out)):
                rc = L.st_conv_dgrad_mirrored(code, _lib.ptr(dy), _lib.ptr(w), _lib.ptr(nbr), *plan.ptrs(),
                                              _lib.ptr(dx), n_in, K, c_in, c_out, None, 0, stream)
            _lib.check(rc, "st_conv_dgrad_mirrored")
        elif tc and inverse_plan(nbr, n_in) is not None:
            # the kernels read the inverse map only through its plan, which comes straight from nbr
            plan = inverse_plan(nbr, n_in)
            with trace.stage("conv_dgrad", work=flops, tag=(c_in, c_out)):
                rc = L.st_conv_dgrad_planned(code, _lib.ptr(dy), _lib.ptr(w), None, *plan.ptrs(),
                                             _lib.ptr(dx), n_in, n_out, K, c_in, c_out, None, 0, stream)
            _lib.check(rc, "st_conv_dgrad_planned")
        else:
            inv = inverse_map(nbr, n_in)
            plan = map_plan(inv) if tc else _NO_PLAN
            with trace.stage("conv_dgrad", work=flops, tag=(c_in, c_out)):
                rc = L.st_conv_dgrad_planned(code, _lib.ptr(dy), _lib.ptr(w), _lib.ptr(inv), *plan.ptrs(),
                                             _lib.ptr(dx), n_in, n_out, K, c_in, c_out, None, 0, stream)
            _lib.check(rc, "st_conv_dgrad_planned")
    return dx


_NO_PRESORT = set()          # (dtype code, K, c_in, c_out) of layers whose weight gradient makes no sorted copy of dY
# A second stream costs the host some 30 us (two waits, an event, the stream switch): worth it when the copy is long
# enough to hide something -- 32 MB of dY are 13 us of copy at 5 TB/s.  Below that the copy stays inside the one call.
_PRESORT_MIN_BYTES = 32 << 20


def start_wgrad_presort(x, dy, nbr, K):
    """First half of the weight gradient, on a second stream: the copy of dY in the plan's row order, which depends on
    dY and the plan alone, so that it runs beside the feature gradient instead of before the weight gradient's
    product.  Returns (workspace, event) for stored_map_wgrad, or None when the layer makes no such copy."""
    n_in, c_in = x.shape
    n_out, c_out = dy.shape
    code = _lib.feat_code(x)
    key = (code, K, c_in, c_out)
    if n_out == 0 or key in _NO_PRESORT or WGRAD_OVER_INVERSE_PLAN or dy.numel() * dy.element_size() < _PRESORT_MIN_BYTES:
        return None
    L = _lib.lib()
    if not L.st_conv_uses_tensor_cores(code, c_in, c_out):
        _NO_PRESORT.add(key)
        return None
    with _lib.on_device(x.device):
        plan = map_plan(nbr)
        if plan.order is None:
            return None
        ws = _lib.workspace(L.st_conv_workspace_bytes(code, n_in, n_out, K, c_in, c_out), x.device)
        cur = torch.cuda.current_stream(x.device)
        aux = _aux_stream(x.device, cur)
        aux.wait_stream(cur)
        with torch.cuda.stream(aux):
            with trace.stage("conv_wgrad_presort", tag=(c_in, c_out)):
                rc = L.st_conv_wgrad_presort(code, _lib.ptr(dy), _lib.ptr(plan.order), n_out, K, c_in, c_out, _lib.ptr(ws),
                                             ws.numel(), _lib.stream_ptr())
            if rc == -5:                      # ST_ERR_UNSUPPORTED: no copy for this shape; nothing was launched
                _NO_PRESORT.add(key)
                return None
            _lib.check(rc, "st_conv_wgrad_presort")
            done = torch.cuda.Event()
            done.record(aux)
    # no record_stream on ws / dy: the caller's stream waits for `done` before the product, and both tensors are
    # released on that stream after it, so their memory is never handed out while the second stream still reads it
    return ws, done


def stored_map_wgrad(x, dy, nbr, K, flops=0.0, presorted=None):
    """dW[k] = sum_o X[nbr[o, k]]^T . dY[o], in the dtype of x.  Walks the plan of the forward map; with
    WGRAD_OVER_INVERSE_PLAN, a layer with more input than output rows walks the inverse plan instead.
    `presorted`: what start_wgrad_presort returned for the same operands."""
    n_in, c_in = x.shape
    n_out, c_out = dy.shape
    code = _lib.feat_code(x)
    L = _lib.lib()
    dw = torch.empty((K, c_in, c_out), device=x.device, dtype=x.dtype)
    tc = bool(L.st_conv_uses_tensor_cores(code, c_in, c_out))
    with _lib.on_device(x.device):
        inv_plan = None
        if WGRAD_OVER_INVERSE_PLAN and tc and n_in > n_out > 0 and not _is_symmetric(nbr, n_in):
            inv_plan = inverse_plan(nbr, n_in)
        if inv_plan is not None:
            ws = _lib.workspace(L.st_conv_wgrad_inverse_workspace_bytes(code, n_in, K, c_in, c_out), x.device)
            with trace.stage("conv_wgrad", work=flops, tag=(c_in, c_out)):
                rc = L.st_conv_wgrad_inverse_planned(code, _lib.ptr(x), _lib.ptr(dy), *inv_plan.ptrs(), _lib.ptr(dw), n_in,
                                                     n_out, K, c_in, c_out, _lib.ptr(ws), ws.numel(), _lib.stream_ptr())
            if rc != -5:                      # ST_ERR_UNSUPPORTED: unaligned tensors or TMA switched off -> forward plan
                _lib.check(rc, "st_conv_wgrad_inverse_planned")
                return dw
        plan = map_plan(nbr) if tc else _NO_PLAN
        if presorted is not None:
            ws, done = presorted
            torch.cuda.current_stream(x.device).wait_event(done)
            entry = L.st_conv_wgrad_planned_presorted
        else:
            ws = _lib.workspace(L.st_conv_workspace_bytes(code, n_in, n_out, K, c_in, c_out), x.device)
            entry = L.st_conv_wgrad_planned
        with trace.stage("conv_wgrad", work=flops, tag=(c_in, c_out)):
            rc = entry(code, _lib.ptr(x), _lib.ptr(dy), _lib.ptr(nbr), *plan.ptrs(), _lib.ptr(dw), n_in, n_out, K, c_in,
                       c_out, _lib.ptr(ws), ws.numel(), _lib.stream_ptr())
        _lib.check(rc, "st_conv_wgrad_planned")
    return dw


class ConvPrecomputedNeighborGEMM(torch.autograd.Function):
    @staticmethod
    def forward(ctx, features, weights, neighbor_indices):
        _lib.require_cuda(features, "ConvPrecomputedNeighborGEMM")
        n_in, c_in = features.shape
        K, w_cin, c_out = weights.shape
        assert w_cin == c_in, f"weights expect {w_cin} input channels, features have {c_in}"
        assert neighbor_indices.shape[1] == K, "neighbor_indices must be (N_out, K)"

        ctx.true_widths = (c_in, c_out)
        c_in, c_out = padded_widths(features.dtype, c_in, c_out)          # narrow layers: zero-padded operands
        x = pad_cols(features, c_in).contiguous()
        w = pad_weight(weights.to(x.dtype), c_in, c_out).contiguous()
        nbr = neighbor_indices if neighbor_indices.is_contiguous() else neighbor_indices.contiguous()
        assert nbr.dtype == torch.int32, "neighbor_indices must be int32"
        y, ctx.flops = stored_map_forward(x, w, nbr, n_in)
        ctx.save_for_backward(x, w, nbr)
        ctx.w_dtype = weights.dtype
        return y if c_out == ctx.true_widths[1] else y[:, :ctx.true_widths[1]].contiguous()

    @staticmethod
    def backward(ctx, grad_output):
        x, w, nbr = ctx.saved_tensors
        n_in, c_in = x.shape
        K, _, c_out = w.shape
        t_in, t_out = ctx.true_widths
        dy = pad_cols(grad_output.to(x.dtype), c_out).contiguous()
        dx = dw = None
        presorted = None
        if ctx.needs_input_grad[0] and ctx.needs_input_grad[1]:
            presorted = start_wgrad_presort(x, dy, nbr, K)     # beside the feature gradient, on a second stream
        if ctx.needs_input_grad[0]:
            dx = stored_map_dgrad(dy, w, nbr, n_in, ctx.flops)
        if ctx.needs_input_grad[1]:
            dw = stored_map_wgrad(x, dy, nbr, K, ctx.flops, presorted).to(ctx.w_dtype)
        if dx is not None and t_in != c_in:
            dx = dx[:, :t_in].contiguous()
        if dw is not None and (t_in != c_in or t_out != c_out):
            dw = dw[:, :t_in, :t_out].contiguous()
        return dx, dw, None
