"""Parity at the sizes of the benchmark configurations, against the CPU oracle (never against another CUDA path).

  config 2   2 M random cells of 4 x 2048^3: table, submanifold maps k3 / k5, the k3 s2 p1 downsample (ordered
             output coordinates + map) and the transposed k3 s2 p1 map built from its output coordinates; every
             map entry identical to oracle.neighbor_map (compared a few million rows at a time)
  config 3   SparseConv3D 64 -> 128, k3 s2 p1, 4 x 300 k surface voxels, both algorithms (hash-on-the-fly in both of its forms)
             x {fp16, bf16}: Y, dX, dW
             within 1e-2 of the fp32 oracle in max-norm, RMS and row-wise relative error (gpu_util.check_close)
  configs 4/5  the U-Net on a small two-sample scene, fp32 and bf16, literal and pruned decoder, against the
             host composition oracle/unet_oracle.py: logits and every parameter gradient
"""
import numpy as np
import pytest
import torch

import sparsetriton_b200 as st
from gpu_util import ALGOS, check_close, map_triples, rel_err, rms_err, t2n
from sparsetriton_b200 import _lib, synthetic
from sparsetriton_b200.config import ConvAlgo, set_conv_algo, set_coords_dtype, set_h_table_f
from sparsetriton_b200.nn.functional import sparse_conv3d
from sparsetriton_b200.nn.functional.conv.conv import compute_neighbor_indices
from sparsetriton_b200.nn.functional.conv.kmap import build_out_coords, out_coords_and_map
from sparsetriton_b200.nn.modules import SparseBatchNorm
from sparsetriton_b200.unet import SparseUNet
from sparsetriton_b200.utils.hash import HashTable

pytestmark = pytest.mark.gpu

ROWS = 4_000_000                       # rows of a map compared per step (host memory stays below ~2 GB)


def _assert_map_equals_oracle(oracle, table, out_coords_np, off, stride, lookup_shape, nbr_gpu, what):
    K = off.shape[0]
    step = max(ROWS * 27 // K, 1)
    pairs = 0
    for r0 in range(0, out_coords_np.shape[0], step):
        want = oracle.neighbor_map(table, out_coords_np[r0:r0 + step], off, stride, lookup_shape)
        got = nbr_gpu[r0:r0 + step].cpu().numpy()
        assert np.array_equal(got, want), f"{what}: map rows {r0}..{r0 + step} differ"
        pairs += int((want >= 0).sum())
    return pairs


def _gpu_pair_count(nbr):
    L = _lib.lib()
    n_out, K = nbr.shape
    ws = _lib.workspace(L.st_map_pairs_workspace_bytes(n_out, K), nbr.device)
    total = torch.zeros(1, dtype=torch.int64, device=nbr.device)
    _lib.check(L.st_map_pairs_count(_lib.ptr(nbr), n_out, K, _lib.ptr(ws), ws.numel(), _lib.ptr(total), _lib.stream_ptr()),
               "st_map_pairs_count")
    return int(total.item())


def test_config2_maps_at_2m_cells(cuda_device, oracle):
    dev = cuda_device
    set_coords_dtype(torch.int32)
    n, grid = 2_000_000, 2048
    shape = (grid,) * 3
    coords_h = synthetic.random_cells(n, 4, grid, seed=2001)
    coords_np = coords_h.numpy()
    coords = coords_h.to(dev)
    with torch.cuda.device(dev):
        table = HashTable(1 << 22, device=dev)                         # load factor 0.48
        table.insert(coords)
        assert torch.equal(table.query(coords), torch.arange(n, dtype=torch.int32, device=dev))
        o_table = oracle.Table(coords_np)
        for k in (3, 5):
            _, _, ko = build_out_coords(coords, shape, k, 1, 1, (k - 1) // 2, submanifold=True)
            nbr = compute_neighbor_indices(table, coords, ko, shape, 1, queries_are_table_rows=True)
            off = oracle.offsets(k, 1, (k - 1) // 2, False)
            pairs = _assert_map_equals_oracle(oracle, o_table, coords_np, off, 1, shape, nbr, f"subm k{k}")
            assert pairs == _gpu_pair_count(nbr) and pairs >= n            # at least every centre entry
            del nbr
        # downsample k3 s2 p1: ordered output coordinates and map
        oc, ns, ko, nbr = out_coords_and_map(coords, shape, 3, 2, 1, 1, False)
        woc, wns, woff = oracle.out_coords(coords_np, shape, 3, 2, 1, 1, False, False)
        assert list(ns) == wns.tolist() and np.array_equal(oc.cpu().numpy(), woc), "downsample: ordered coordinates differ"
        pairs = _assert_map_equals_oracle(oracle, o_table, woc, woff, 2, shape, nbr, "down k3 s2")
        assert pairs == _gpu_pair_count(nbr)
        tri = map_triples(nbr[:200_000].contiguous())                     # the triple form of the first rows
        assert np.array_equal(tri, oracle.pairs(oracle.neighbor_map(o_table, woc[:200_000], woff, 2, shape)))
        del nbr
        # the transposed k3 s2 p1 map from the downsample's output coordinates
        oc2, ns2, ko2, nbr2 = out_coords_and_map(oc, ns, 3, 2, 1, 1, True)
        woc2, wns2, woff2 = oracle.out_coords(woc, tuple(wns), 3, 2, 1, 1, True, False)
        assert list(ns2) == wns2.tolist() and oc2.shape[0] == woc2.shape[0]
        for r0 in range(0, woc2.shape[0], 4 * ROWS):
            assert np.array_equal(oc2[r0:r0 + 4 * ROWS].cpu().numpy(), woc2[r0:r0 + 4 * ROWS]), "transposed: coordinates differ"
        scaled = woc.copy()
        scaled[:, 1:] *= 2                                                # conv.py:138-142: lookup in the scaled inputs
        t_table = oracle.Table(scaled)
        pairs = _assert_map_equals_oracle(oracle, t_table, woc2, woff2, 1, tuple(v * 2 for v in wns), nbr2, "up k3 s2")
        assert pairs == _gpu_pair_count(nbr2)


# --------------------------------------------------------------------------------------- config 3
_C3 = {}


def _c3_inputs():
    if not _C3:
        scenes = [synthetic.surface_scene(3000 + b, grid=512, target=300_000) for b in range(4)]
        _C3["coords"] = synthetic.batch_of(scenes, dtype=torch.int32)
    return _C3["coords"]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_config3_layer_full_size(cuda_device, oracle, dtype):
    dev = cuda_device
    set_coords_dtype(torch.int32)
    set_h_table_f(2.0)
    coords = _c3_inputs()
    n_in = coords.shape[0]
    assert 1_100_000 < n_in < 1_300_000
    gen = torch.Generator().manual_seed(9000)
    feats = torch.randn(n_in, 64, generator=gen).to(dtype)
    weight = ((torch.rand(27, 64, 128, generator=gen) * 2 - 1) / (64 * 27) ** 0.5).to(dtype)
    shape = (512, 512, 512)
    woc, wns, _, wnbr = oracle.kernel_map(coords.numpy(), shape, 3, 2, 1, 1, False, False)
    dy = torch.randn(woc.shape[0], 128, generator=gen).to(dtype)
    f32 = lambda t: t.float().numpy()
    want_y = oracle.conv_fwd(f32(feats), f32(weight), wnbr)
    want_dx = oracle.conv_dgrad(f32(dy), f32(weight), wnbr, n_in)
    want_dw = oracle.conv_wgrad(f32(feats), f32(dy), wnbr, 27, 64, 128)
    for algo in ALGOS:                                  # stored map, hash-on-the-fly with a scratch map, and probing in the kernels
        algo.use()
        x = feats.to(dev).requires_grad_(True)
        w = weight.to(dev).requires_grad_(True)
        sp = st.SparseTensor(x, coords.to(dev), spatial_shape=shape, batch_size=4)
        out = sparse_conv3d(sp, w, kernel_size=3, stride=2, padding=1, submanifold=False)
        assert np.array_equal(t2n(out.C), woc), "output coordinates (ordered) differ from the oracle"
        dx, dw = torch.autograd.grad(out.F, [x, w], dy.to(dev))
        check_close(t2n(out.F), want_y, 1e-2, f"{algo.name} Y")
        check_close(t2n(dx), want_dx, 1e-2, f"{algo.name} dX")
        check_close(t2n(dw).reshape(27 * 64, 128), want_dw.reshape(27 * 64, 128), 1e-2, f"{algo.name} dW")
        if algo.algo == ConvAlgo.PrecomputedNeighborGEMM:
            nbr = sp._cache.neighbor_indices[(3, 2, 1, 1, False, False)][1]
            assert np.array_equal(nbr.cpu().numpy(), wnbr), "neighbour map differs from the oracle"
        del out, dx, dw, sp
    assert _lib.device_status(dev)[0] == 0


# --------------------------------------------------------------------------------------- configs 4 / 5
UNET_SHAPE = (64, 64, 41)


def _unet_scene():
    samples = []
    for b in range(2):
        c = synthetic.surface_scene(70 + b, grid=64, target=5000, n_spheres=3, n_boxes=3)
        samples.append(c[c[:, 2] < UNET_SHAPE[2]])
    coords = synthetic.batch_of(samples)
    g = torch.Generator().manual_seed(5)
    feats = torch.cat([coords[:, 1:].float() / torch.tensor([64.0, 64.0, 41.0]), torch.rand(coords.shape[0], 1, generator=g)], 1)
    return coords, feats


@pytest.mark.parametrize("prune", [False, True], ids=["literal", "pruned"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_unet_against_host_composition(cuda_device, dtype, prune):
    """Logits and all parameter gradients of the training step (cross-entropy over random labels) against the
    host composition.  fp32 runs with the tensor cores off (exact fp32 products); bf16 with them on, the host
    side rounding activations, weights and their gradients to bf16 where the GPU stores them.  Bars (RMS relative):
    logits 1e-4 fp32 / 2e-2 bf16 on the host's own ReLU decisions; gradients 2e-4 / 2e-2 over all parameters and
    4x that for the worst single parameter, on the GPU run's ReLU decisions, which must agree with the host's
    wherever the host's pre-activation is further than 1e-4 / 1e-1 from zero."""
    from oracle import unet_oracle as U
    dev = cuda_device
    set_coords_dtype(torch.int32)
    set_conv_algo(ConvAlgo.PrecomputedNeighborGEMM)
    widths = (16, 32, 64, 128)
    torch.manual_seed(4100)
    model = SparseUNet(widths=widths, prune=prune).to(dev)
    with torch.no_grad():                                              # non-trivial affine parameters
        for name, p_ in model.named_parameters():
            if ".bn" in name:
                p_.add_(torch.randn_like(p_) * 0.1)
    coords, feats = _unet_scene()
    g = torch.Generator().manual_seed(1)

    # the run under test; the on/off decision of every ReLU element is recorded for the host run (see ReluDecisions)
    masks = []
    hooks = [m.register_forward_hook(lambda mod, inp, out: masks.append((out.F > 0).cpu()))
             for m in model.modules() if isinstance(m, SparseBatchNorm)]
    _lib.lib().st_set_tensor_cores(0 if dtype == torch.float32 else 1)
    try:
        x = st.SparseTensor(feats.to(dev, dtype), coords.to(dev), spatial_shape=UNET_SHAPE, batch_size=2)
        out = model(x)
        labels = torch.randint(0, 20, (out.F.shape[0],), generator=g)
        loss = torch.nn.functional.cross_entropy(out.F.float(), labels.to(dev))
        loss.backward()
    finally:
        _lib.lib().st_set_tensor_cores(1)
        for h in hooks:
            h.remove()

    params = {k: v.detach().cpu().clone().requires_grad_(True) for k, v in model.named_parameters()}
    # forward on the host's own ReLU decisions: logits and coordinates
    with torch.no_grad():
        logits_own, oc_w = U.unet_forward(params, coords.numpy(), feats, UNET_SHAPE, 2, len(widths), prune, store=dtype)
    assert np.array_equal(t2n(out.C), oc_w), "output coordinates differ from the host composition"
    tol_y = 1e-4 if dtype == torch.float32 else 2e-2
    assert rel_err(t2n(out.F), logits_own.numpy()) < tol_y and rms_err(t2n(out.F), logits_own.numpy()) < tol_y
    # forward + backward on the recorded decisions: they may differ from the host's own only where the host's
    # pre-activation is within the arithmetic noise of zero
    decisions = U.ReluDecisions(masks)
    logits_w, _ = U.unet_forward(params, coords.numpy(), feats, UNET_SHAPE, 2, len(widths), prune, store=dtype,
                                 decisions=decisions)
    torch.nn.functional.cross_entropy(logits_w, labels).backward()
    assert decisions.next == len(masks)
    assert decisions.worst_disagreement < (1e-4 if dtype == torch.float32 else 1e-1), decisions.worst_disagreement

    tol_g = 2e-4 if dtype == torch.float32 else 2e-2
    names = [n for n, _ in model.named_parameters()]
    got_all = np.concatenate([t2n(p_.grad).reshape(-1) for _, p_ in model.named_parameters()])
    want_all = np.concatenate([params[n].grad.numpy().reshape(-1) for n in names])
    errs = {n: rms_err(t2n(p_.grad), params[n].grad.numpy()) for n, p_ in model.named_parameters()}
    worst = max((e, n) for n, e in errs.items())
    print(f"logits rel {rel_err(t2n(out.F), logits_own.numpy()):.2e}; ReLU decisions differing {decisions.disagreements} "
          f"(largest |z| among them {decisions.worst_disagreement:.2e}); gradients: all {rms_err(got_all, want_all):.2e}, "
          f"worst parameter {worst[1]} {worst[0]:.2e}")
    assert rms_err(got_all, want_all) < tol_g
    assert worst[0] < 4 * tol_g, f"gradient of {worst[1]}: rms relative error {worst[0]:.2e}"
    if not prune:
        assert out.C.shape[0] > coords.shape[0]                        # every child is materialised
    assert _lib.device_status(dev)[0] == 0
