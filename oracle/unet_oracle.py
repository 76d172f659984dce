"""CPU composition of the benchmark U-Net out of the oracle's pieces.  TEST INFRASTRUCTURE ONLY.

Every layer of `sparsetriton_b200.unet.SparseUNet` restated on the host:

  convolutions   oracle.kernel_map + oracle.conv_fwd / conv_dgrad / conv_wgrad (oracle.c, fp32), wrapped in a
                 torch.autograd.Function so that torch's CPU autograd chains them
  batch norm     the reference's own formulation, nn/functional/norm.py:73-112, written with the same torch
                 ops (index_add_ sums per (batch index, channel), counts clamped to 1, biased variance, eps
                 inside the square root), followed by ReLU as the reference's blocks apply it
  skip           decoder coordinate looked up in the encoder level's table; that row or zeros
  head           torch.nn.functional.linear on the fp32 features

`prune=False` is the literal composition (SparseConvTransposed3D output = every child); `prune=True`
evaluates the transposed convolution and keeps the rows at the encoder's coordinates (children without
a parent get zeros: the benchmark network's up-convolutions have no bias).

`store` mimics the feature storage type of the GPU run: after every convolution and normalisation the
activations are rounded to it (and back to fp32), so that what remains between the two runs is summation
order, not storage precision.
"""
import numpy as np
import torch

from . import cpu_oracle as O


class _OracleConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, nbr, n_in):
        ctx.save_for_backward(x, w)
        ctx.nbr, ctx.n_in = nbr, n_in
        return torch.from_numpy(O.conv_fwd(x.detach().numpy(), w.detach().numpy(), nbr))

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        K, cin, cout = w.shape
        dyn = dy.contiguous().numpy()
        dx = torch.from_numpy(O.conv_dgrad(dyn, w.detach().numpy(), ctx.nbr, ctx.n_in))
        dw = torch.from_numpy(O.conv_wgrad(x.detach().numpy(), dyn, ctx.nbr, K, cin, cout))
        return dx, dw, None, None


class _Round(torch.autograd.Function):
    """Round to the storage dtype on the way forward and round the gradient on the way back, as a tensor
    stored in that dtype (and its gradient) would be."""

    @staticmethod
    def forward(ctx, t, store):
        ctx.store = store
        return t.to(store).float()

    @staticmethod
    def backward(ctx, g):
        return g.to(ctx.store).float(), None


def _rounded(t, store):
    return t if store == torch.float32 else _Round.apply(t, store)


def conv(x, coords, shape, weight, k, s, p, transposed, subm, store, w_store):
    """Returns (features, out_coords, new_shape)."""
    oc, ns, _, nbr = O.kernel_map(coords, shape, k, s, 1, p, transposed, subm)
    w = _rounded(weight, w_store)
    y = _OracleConv.apply(x, w, nbr, x.shape[0])
    return _rounded(y, store), oc, tuple(int(v) for v in ns)


def batch_norm(x, batch_idx, n_samples, weight, bias, eps):
    """nn/functional/norm.py:73-112, training branch, with the reference's own torch ops."""
    C = x.shape[1]
    sums = torch.zeros(n_samples, C).index_add_(0, batch_idx, x)
    counts = torch.bincount(batch_idx, minlength=n_samples).float().view(-1, 1).clamp(min=1)
    mean = sums / counts
    cen = x - mean[batch_idx]
    var = torch.zeros(n_samples, C).index_add_(0, batch_idx, cen.pow(2)) / counts
    y = cen / torch.sqrt(var[batch_idx] + eps)
    return y * weight + bias


def batch_norm_relu(x, batch_idx, n_samples, weight, bias, eps, store, decisions=None):
    """batch_norm + ReLU.  `decisions`: see unet_forward."""
    z = batch_norm(x, batch_idx, n_samples, weight, bias, eps)
    if decisions is None:
        return _rounded(torch.relu(z), store)
    mask = decisions.take(z)
    return _rounded(z * mask, store)


class ReluDecisions:
    """ReLU on/off decisions taken elsewhere (by the run under test), consumed layer by layer.

    The gradient of a ReLU network is discontinuous in its pre-activations: where two runs' z differ in sign
    (|z| below the arithmetic noise between them), one whole term of every gradient sum upstream appears or
    disappears -- a single such element moves a small layer's gradient by 1e-3..1e-2 relative.  To compare
    gradients to arithmetic accuracy the host composition can therefore take the on/off decision of every
    element from the other run, and it records how far from zero its own pre-activation was wherever the two
    disagree (`worst_disagreement`): the caller asserts that this stays within the arithmetic noise."""

    def __init__(self, masks):
        self.masks = list(masks)
        self.next = 0
        self.worst_disagreement = 0.0
        self.disagreements = 0

    def take(self, z):
        mask = self.masks[self.next]
        self.next += 1
        assert mask.shape == z.shape, "ReLU decisions do not line up with the layers"
        differ = (z.detach() > 0) != mask
        if bool(differ.any()):
            self.disagreements += int(differ.sum())
            self.worst_disagreement = max(self.worst_disagreement, float(z.detach()[differ].abs().max()))
        return mask.to(z.dtype)


def _block(x, coords, shape, n_samples, params, prefix, store, w_store, decisions):
    b = torch.from_numpy(coords[:, 0].astype(np.int64))
    for i in (1, 2):
        x, _, _ = conv(x, coords, shape, params[f"{prefix}.conv{i}.weight"], 3, 1, 1, False, True, store, w_store)
        x = batch_norm_relu(x, b, n_samples, params[f"{prefix}.bn{i}.weight"], params[f"{prefix}.bn{i}.bias"], 1e-5, store,
                            decisions)
    return x


def unet_forward(params, coords, feats, shape, n_samples, n_levels, prune, store=torch.float32, decisions=None):
    """`params`: name -> fp32 CPU tensor (requires_grad where gradients are wanted), named as the module's
    state_dict.  `decisions`: optional ReluDecisions holding one boolean (rows, channels) mask per batch-norm
    layer in call order.  Returns (logits (N_out, classes) fp32, out_coords)."""
    w_store = store
    coords = np.ascontiguousarray(coords, dtype=np.int32)
    x = _rounded(feats, store)
    skips = []
    for lvl in range(n_levels):
        if lvl > 0:
            x, coords, shape = conv(x, coords, shape, params[f"down.{lvl - 1}.weight"], 2, 2, 0, False, False, store, w_store)
        x = _block(x, coords, shape, n_samples, params, f"enc.{lvl}", store, w_store, decisions)
        skips.append((x, coords, shape))
    for j in range(n_levels - 1):
        sx, sc, ss = skips[n_levels - 2 - j]
        y, oc, ns = conv(x, coords, shape, params[f"up.{j}.weight"], 2, 2, 0, True, False, store, w_store)
        if prune:
            idx = torch.from_numpy(O.Table(oc).query(sc).astype(np.int64))
            found = (idx >= 0).unsqueeze(1).float()
            y = y.index_select(0, idx.clamp(min=0)) * found
            x, coords, shape = torch.cat([y, sx], dim=1), sc, ss
        else:
            idx = torch.from_numpy(O.Table(sc).query(oc).astype(np.int64))
            found = (idx >= 0).unsqueeze(1).float()
            rows = sx.index_select(0, idx.clamp(min=0)) * found
            x, coords, shape = torch.cat([y, rows], dim=1), oc, ns
        x = _block(x, coords, shape, n_samples, params, f"dec.{j}", store, w_store, decisions)
    logits = torch.nn.functional.linear(x, params["head.weight"], params["head.bias"])
    return logits, coords
