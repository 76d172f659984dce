"""The benchmark U-Net on small lidar-like scenes: both convolution algorithms, tensor-core and
CUDA-core kernels, must give the same network output and gradients within the feature tolerances."""
import numpy as np
import pytest
import torch

import sparsetriton_b200 as st
from gpu_util import rel_err
from sparsetriton_b200 import _lib, synthetic
from sparsetriton_b200.config import ConvAlgo, set_conv_algo, set_coords_dtype, set_hashfly_transient_map
from sparsetriton_b200.unet import SparseUNet, skip_concat, up_conv_onto

pytestmark = pytest.mark.gpu


SHAPE = (64, 64, 41)                      # odd z extent: the k2 s2 layers drop the last slab, as in the benchmark grid


def _scene(dev, batch=2):
    samples = []
    for b in range(batch):
        c = synthetic.surface_scene(70 + b, grid=64, target=7000, n_spheres=3, n_boxes=3)
        samples.append(c[c[:, 2] < SHAPE[2]])
    coords = synthetic.batch_of(samples)
    g = torch.Generator().manual_seed(5)
    feats = torch.cat([coords[:, 1:].float() / torch.tensor([64.0, 64.0, 41.0]), torch.rand(coords.shape[0], 1, generator=g)], 1)
    return coords.to(dev), feats.to(dev)


def _run(model, coords, feats, labels_seed, dtype, algo, tensor_cores, transient=True):
    set_conv_algo(algo)
    set_hashfly_transient_map(transient)
    _lib.lib().st_set_tensor_cores(int(tensor_cores))
    model.zero_grad(set_to_none=True)
    x = st.SparseTensor(feats.to(dtype), coords, spatial_shape=SHAPE, batch_size=2)
    out = model(x)
    g = torch.Generator().manual_seed(labels_seed)
    labels = torch.randint(0, 20, (out.F.shape[0],), generator=g).to(out.F.device)
    loss = torch.nn.functional.cross_entropy(out.F.float(), labels)
    loss.backward()
    grads = torch.cat([p.grad.reshape(-1).float() for p in model.parameters()])
    _lib.lib().st_set_tensor_cores(1)
    return out.C.cpu().numpy(), out.F.detach().float().cpu().numpy(), float(loss.detach()), grads.cpu().numpy()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_unet_algorithms_and_kernels_agree(cuda_device, dtype):
    set_coords_dtype(torch.int32)
    torch.manual_seed(4100)
    model = SparseUNet(widths=(16, 32, 64, 128)).to(cuda_device)
    coords, feats = _scene(cuda_device)
    ref = _run(model, coords, feats, 1, dtype, ConvAlgo.PrecomputedNeighborGEMM, tensor_cores=False)
    assert ref[0].shape[0] >= coords.shape[0] and np.isfinite(ref[1]).all() and np.isfinite(ref[3]).all()
    assert (np.abs(ref[3]) > 0).mean() > 0.5
    # network-level bounds (20 layers deep, tf32 products against exact fp32 ones); the per-layer parity bars
    # live in test_gpu_conv.py.  The gradient bound leaves room for the run-to-run spread of the batch-norm
    # sums (fp32 atomics): 1.9e-2 .. 2.1e-2 was observed.
    tol_out, tol_grad = (5e-3, 3e-2) if dtype == torch.float32 else (5e-2, 1.5e-1)
    for algo, tcores, transient in [(ConvAlgo.PrecomputedNeighborGEMM, True, True), (ConvAlgo.ImplicitHashFlyGEMM, True, True),
                                    (ConvAlgo.ImplicitHashFlyGEMM, True, False), (ConvAlgo.ImplicitHashFlyGEMM, False, False)]:
        got = _run(model, coords, feats, 1, dtype, algo, tcores, transient)
        assert np.array_equal(got[0], ref[0]), "output coordinates differ between algorithms"
        assert rel_err(got[1], ref[1]) < tol_out, (algo, tcores, rel_err(got[1], ref[1]))
        assert abs(got[2] - ref[2]) < tol_out * max(1.0, abs(ref[2]))
        assert rel_err(got[3], ref[3]) < tol_grad, (algo, tcores, rel_err(got[3], ref[3]))
    assert _lib.device_status(cuda_device)[0] == 0


def test_conv_stack_is_reproducible(cuda_device):
    """Stored-map convolutions use no atomics anywhere (forward, dgrad over the inverse map, wgrad with a
    fixed-order reduction): running the same layers twice gives bit-identical outputs and gradients.
    (The U-Net as a whole is not bit-reproducible because the batch-norm sums are added with fp32 atomics.)"""
    from sparsetriton_b200.nn import SparseConv3D, SparseConvTransposed3D, SubMConv3D
    set_coords_dtype(torch.int32)
    set_conv_algo(ConvAlgo.PrecomputedNeighborGEMM)
    torch.manual_seed(1)
    layers = torch.nn.Sequential(SubMConv3D(16, 32, 3), SparseConv3D(32, 64, 2, stride=2),
                                 SubMConv3D(64, 64, 3), SparseConvTransposed3D(64, 32, 2, stride=2)).to(cuda_device)
    coords, _ = _scene(cuda_device)
    feats = torch.randn(coords.shape[0], 16, device=cuda_device).bfloat16()
    results = []
    for _ in range(2):
        layers.zero_grad(set_to_none=True)
        x = feats.clone().requires_grad_(True)
        out = layers(st.SparseTensor(x, coords, spatial_shape=SHAPE, batch_size=2))
        out.F.float().square().mean().backward()
        results.append((out.F.detach().clone(), x.grad.clone(), torch.cat([p.grad.reshape(-1) for p in layers.parameters()])))
    for a, b in zip(*results):
        assert torch.equal(a, b), "reruns must be bit-identical"


@pytest.mark.parametrize("algo", [ConvAlgo.PrecomputedNeighborGEMM, ConvAlgo.ImplicitHashFlyGEMM], ids=lambda a: a.name)
def test_up_conv_onto_equals_transposed_conv_then_lookup(cuda_device, algo):
    """The pruned decoder's up-conv (gather over the inverse of the down-conv's map) against the literal
    SparseConvTransposed3D followed by picking the rows at the encoder's coordinates."""
    from sparsetriton_b200.nn import SparseConv3D, SparseConvTransposed3D
    from sparsetriton_b200.utils.hash import HashTable
    set_coords_dtype(torch.int32)
    set_conv_algo(algo)
    torch.manual_seed(3)
    coords, _ = _scene(cuda_device)
    enc = st.SparseTensor(torch.randn(coords.shape[0], 32, device=cuda_device).bfloat16(), coords,
                          spatial_shape=SHAPE, batch_size=2)
    down = SparseConv3D(32, 64, 2, stride=2, bias=False).to(cuda_device)
    up = SparseConvTransposed3D(64, 32, 2, stride=2, bias=True).to(cuda_device)
    low = down(enc)
    got = up_conv_onto(low, up, enc)
    assert torch.equal(got.C, enc.C) and got._cache is enc._cache
    full = up(low)
    table = HashTable(2 * full.C.shape[0], device=cuda_device)
    table.insert(full.C)
    idx = table.query(enc.C).long()
    found = idx >= 0
    # under the even-kernel rule child c has parent ceil(c/2), which must lie inside the coarse grid
    # (S-2)//2+1: the last slab(s) of each axis (x, y = 63; z = 39, 40) are orphans.  The literal
    # transposed conv never produces them, the restricted one gives them the bias alone.
    coarse = torch.tensor([(v - 2) // 2 + 1 for v in SHAPE], device=cuda_device)
    orphan = (((enc.C[:, 1:].long() + 1) // 2) >= coarse).any(dim=1)
    assert torch.equal(orphan, ~found) and found.float().mean() > 0.9
    want = full.F[idx[found]]
    assert rel_err(got.F[found].detach().float().cpu().numpy(), want.detach().float().cpu().numpy()) < 1e-2
    assert torch.equal(got.F[~found], up.bias.to(got.F.dtype).expand_as(got.F[~found]))


def test_skip_concat(cuda_device):
    set_coords_dtype(torch.int32)
    enc = st.SparseTensor(torch.arange(6.0, device=cuda_device).view(3, 2),
                          torch.tensor([[0, 1, 1, 1], [0, 2, 2, 2], [1, 1, 1, 1]], device=cuda_device))
    dec = st.SparseTensor(torch.ones(4, 1, device=cuda_device),
                          torch.tensor([[1, 1, 1, 1], [0, 9, 9, 9], [0, 2, 2, 2], [0, 1, 1, 1]], device=cuda_device))
    out = skip_concat(dec, enc)
    assert out.F.tolist() == [[1, 4, 5], [1, 0, 0], [1, 2, 3], [1, 0, 1]]


@pytest.mark.parametrize("backward", [False, True], ids=["forward", "forward_backward"])
def test_prepared_network_matches(cuda_device, backward):
    """SparseUNet.prepare on a second stream, then the network on the first: the same results as the network alone, and
    the network then launches no coordinate work.  The normalisation layers use their running statistics here, which
    leaves the products and every feature gradient free of atomics, so those must agree bit for bit; the gradients of
    the normalisation parameters are sums by atomic adds and agree to rounding."""
    from sparsetriton_b200 import trace
    set_conv_algo(ConvAlgo.PrecomputedNeighborGEMM)
    set_coords_dtype(torch.int32)
    coords, feats = _scene(cuda_device)
    feats = feats.to(torch.bfloat16)
    shape, batch = SHAPE, 2
    assert coords.shape[0] > 10_000
    torch.manual_seed(14)
    model = SparseUNet(widths=(16, 32, 64), num_classes=5).to(cuda_device)
    model.train(False)
    names = ["logits"] + [n for n, _ in model.named_parameters()]

    def run(cache):
        model.zero_grad(set_to_none=True)
        x = st.SparseTensor(feats, coords, shape, batch, cache=cache)
        if not backward:
            with torch.no_grad():
                return [model(x).F]
        out = model(x)
        out.F.float().square().mean().backward()
        return [out.F.detach()] + [p.grad.clone() for p in model.parameters()]

    want = run(None)
    main, side = torch.cuda.current_stream(cuda_device), torch.cuda.Stream(cuda_device)
    side.wait_stream(main)
    with torch.cuda.stream(side):
        cache = model.prepare(coords, shape, batch, backward=backward, consumer_stream=main)
        ready = torch.cuda.Event()
        ready.record(side)
    main.wait_event(ready)
    with trace.recording() as rec:
        got = run(cache)
        torch.cuda.synchronize(cuda_device)
        stages = set(rec.summary())
    assert {"conv_fwd", "bn_fwd"} <= stages <= {"conv_fwd", "conv_dgrad", "conv_wgrad", "bn_fwd", "bn_bwd"}, stages
    assert len(got) == len(want)
    for name, a, b in zip(names, got, want):
        if ".bn" in name:
            assert torch.allclose(a, b, rtol=1e-4, atol=1e-7 + 1e-5 * float(b.abs().max())), name
        else:
            assert torch.equal(a, b), name
