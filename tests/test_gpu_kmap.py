"""Kernel-map construction on the GPU: ordered output coordinates and (in, out, offset) triples
must be bit-identical to the reference's golden vectors and to the oracle."""
import numpy as np
import pytest
import torch

from conftest import case_id, golden_files, load_golden
from gpu_util import map_triples
from sparsetriton_b200 import synthetic
from sparsetriton_b200.config import set_coords_dtype
from sparsetriton_b200.nn.functional.conv.conv import compute_neighbor_indices
from sparsetriton_b200.nn.functional.conv.funcs.implicit_precomputed_gemm import inverse_map
from sparsetriton_b200.nn.functional.conv.kmap import build_out_coords, out_coords_and_map
from sparsetriton_b200.utils.hash import HashTable

pytestmark = pytest.mark.gpu


def gpu_kernel_map(dev, coords, shape, k, s, d, p, transposed, subm, dtype=torch.int32, factor=2.0):
    """Same call sequence as sparse_conv3d up to the neighbour map."""
    set_coords_dtype(dtype)
    c = torch.as_tensor(coords).to(dev, dtype)
    if subm:
        p = ((k - 1) * d) // 2
    keyc = c.clone()
    if transposed and s > 1:
        keyc[:, 1:] *= s
    table = HashTable(capacity=max(int(c.shape[0] * factor), 1), device=dev)
    table.insert(keyc)
    oc, ns, ko = build_out_coords(c, tuple(int(v) for v in shape), k, s, d, p, transposed=transposed,
                                  submanifold=subm)
    look = tuple(int(v) * s for v in shape) if (transposed and s > 1) else tuple(int(v) for v in shape)
    nbr = compute_neighbor_indices(table, oc, ko, look, 1 if transposed else s, p, d)
    ns = [int(v) for v in (ns.tolist() if isinstance(ns, torch.Tensor) else ns)]
    return oc, ns, ko, nbr


@pytest.mark.parametrize("path", golden_files("kmap_"), ids=case_id)
def test_golden(cuda_device, oracle, path):
    g = load_golden(path)
    dtype = getattr(torch, str(g["coord_dtype"]))
    oc, ns, ko, nbr = gpu_kernel_map(cuda_device, g["coords"], g["shape"], int(g["k"]), int(g["s"]), int(g["d"]),
                                     int(g["p"]), bool(g["transposed"]), bool(g["subm"]), dtype)
    assert oc.dtype == dtype
    assert np.array_equal(ko.cpu().numpy().astype(np.int32), g["kernel_offsets"])
    assert ns == g["new_shape"].tolist()
    assert np.array_equal(oc.cpu().numpy().astype(np.int32), g["out_coords"]), "ordered output coordinates differ"
    assert np.array_equal(nbr.cpu().numpy(), g["nbr"])
    assert np.array_equal(map_triples(nbr), oracle.pairs(g["nbr"]))


def gpu_fused_map(dev, coords, shape, k, s, d, p, transposed, dtype=torch.int32):
    """Coordinates and map from the single-pass form used by sparse_conv3d for strided / transposed layers."""
    set_coords_dtype(dtype)
    c = torch.as_tensor(coords).to(dev, dtype)
    oc, ns, ko, nbr = out_coords_and_map(c, tuple(int(v) for v in shape), k, s, d, p, transposed)
    return oc, list(ns), ko, nbr


@pytest.mark.parametrize("path", [p for p in golden_files("kmap_") if "subm_k" not in p or "_s2" in p], ids=case_id)
def test_golden_single_pass_map(cuda_device, oracle, path):
    g = load_golden(path)
    dtype = getattr(torch, str(g["coord_dtype"]))
    k, s, d, subm = int(g["k"]), int(g["s"]), int(g["d"]), bool(g["subm"])
    p = ((k - 1) * d) // 2 if subm else int(g["p"])
    oc, ns, ko, nbr = gpu_fused_map(cuda_device, g["coords"], g["shape"], k, s, d, p, bool(g["transposed"]), dtype)
    assert ns == g["new_shape"].tolist()
    assert np.array_equal(oc.cpu().numpy().astype(np.int32), g["out_coords"])
    assert np.array_equal(nbr.cpu().numpy(), g["nbr"])
    assert np.array_equal(map_triples(nbr), oracle.pairs(g["nbr"]))


CASES = [
    # k, s, p, d, transposed, subm
    (3, 1, 1, 1, False, True),
    (5, 1, 2, 1, False, True),
    (3, 1, 2, 2, False, True),
    (3, 2, 1, 1, False, False),
    (2, 2, 0, 1, False, False),
    (3, 1, 1, 1, False, False),
    (5, 2, 2, 1, False, False),
    (2, 2, 0, 1, True, False),
    (3, 2, 1, 1, True, False),
]


@pytest.mark.parametrize("k,s,p,d,transposed,subm", CASES)
@pytest.mark.parametrize("dtype", [torch.int32, torch.int16])
def test_random_vs_oracle(cuda_device, oracle, k, s, p, d, transposed, subm, dtype):
    n = 20_000 if (transposed or (k == 3 and s == 1 and not subm)) else 60_000
    coords = synthetic.random_cells(n, 3, 40, seed=100 + k + s)
    if transposed:                                   # batched transposed: rows grouped by sample or not,
        coords = coords[torch.argsort(coords[:, 0], stable=True)]   # the exact rule is order-independent
    shape = (40, 40, 40)
    oc, ns, ko, nbr = gpu_kernel_map(cuda_device, coords, shape, k, s, d, p, transposed, subm, dtype)
    woc, wns, woff, wnbr = oracle.kernel_map(coords.numpy(), shape, k, s, d, p, transposed, subm)
    assert ns == wns.tolist()
    assert np.array_equal(oc.cpu().numpy().astype(np.int32), woc)
    assert np.array_equal(nbr.cpu().numpy(), wnbr)
    assert np.array_equal(map_triples(nbr), oracle.pairs(wnbr))
    if not (subm and s == 1):
        oc2, ns2, _, nbr2 = gpu_fused_map(cuda_device, coords, shape, k, s, d, p, transposed, dtype)
        assert np.array_equal(oc2.cpu().numpy().astype(np.int32), woc) and np.array_equal(nbr2.cpu().numpy(), wnbr)


def test_single_pass_map_duplicates_and_out_of_grid(cuda_device, oracle):
    """Rows with equal coordinates keep the largest row (as the table does); inputs outside the
    declared grid produce output coordinates but no map entry (as the bounds-checked lookup does)."""
    base = synthetic.random_cells(3000, 2, 20, seed=9).numpy()
    coords = np.concatenate([base, base[:500], np.array([[0, 25, 3, 3], [1, 3, 30, 3]], np.int32)])
    shape = (20, 20, 20)
    oc, ns, _, nbr = gpu_fused_map(cuda_device, coords, shape, 3, 2, 1, 1, False)
    woc, wns, _, wnbr = oracle.kernel_map(coords, shape, 3, 2, 1, 1, False, False)
    assert np.array_equal(oc.cpu().numpy(), woc) and np.array_equal(nbr.cpu().numpy(), wnbr)


def test_surface_scene_downsample_and_back(cuda_device, oracle):
    """A contiguous surface (duplicate-heavy candidates): k3 s2 p1 map, then the transposed map
    built from its output coordinates."""
    cells = synthetic.surface_scene(3000, grid=128, target=40_000, n_spheres=3, n_boxes=4)
    coords = synthetic.batch_of([cells, synthetic.surface_scene(3001, grid=128, target=30_000, n_spheres=2, n_boxes=2)])
    shape = (128, 128, 128)
    oc, ns, ko, nbr = gpu_kernel_map(cuda_device, coords, shape, 3, 2, 1, 1, False, False)
    woc, wns, _, wnbr = oracle.kernel_map(coords.numpy(), shape, 3, 2, 1, 1, False, False)
    assert np.array_equal(oc.cpu().numpy(), woc) and np.array_equal(nbr.cpu().numpy(), wnbr)
    oc2, ns2, _, nbr2 = gpu_kernel_map(cuda_device, oc, ns, 3, 2, 1, 1, True, False)
    woc2, wns2, _, wnbr2 = oracle.kernel_map(woc, tuple(wns), 3, 2, 1, 1, True, False)
    assert ns2 == wns2.tolist()
    assert np.array_equal(oc2.cpu().numpy(), woc2) and np.array_equal(nbr2.cpu().numpy(), wnbr2)


def test_edge_cases(cuda_device, oracle):
    set_coords_dtype(torch.int32)
    empty = torch.empty((0, 4), dtype=torch.int32, device=cuda_device)
    oc, ns, ko = build_out_coords(empty, (8, 8, 8), 3, 2, 1, 1, submanifold=False)
    assert oc.shape == (0, 4) and ns.tolist() == [4, 4, 4] and ko.shape == (27, 3)
    # single voxel in the far corner, every kind of map
    one = np.array([[1, 7, 7, 7]], np.int32)
    for (k, s, p, d, tr, subm) in CASES:
        oc, ns, _, nbr = gpu_kernel_map(cuda_device, one, (8, 8, 8), k, s, d, p, tr, subm)
        woc, wns, _, wnbr = oracle.kernel_map(one, (8, 8, 8), k, s, d, p, tr, subm)
        assert np.array_equal(oc.cpu().numpy(), woc) and np.array_equal(nbr.cpu().numpy(), wnbr), (k, s, p, d, tr)
    # fully occupied small grid: every candidate is duplicated up to 27 times
    xs = torch.arange(6)
    full = torch.stack(torch.meshgrid(torch.zeros(1, dtype=torch.long), xs, xs, xs, indexing="ij"), -1).reshape(-1, 4)
    oc, ns, _, nbr = gpu_kernel_map(cuda_device, full.numpy().astype(np.int32), (6, 6, 6), 3, 2, 1, 1, False, False)
    woc, wns, _, wnbr = oracle.kernel_map(full.numpy(), (6, 6, 6), 3, 2, 1, 1, False, False)
    assert np.array_equal(oc.cpu().numpy(), woc) and np.array_equal(nbr.cpu().numpy(), wnbr)


def test_inverse_map(cuda_device):
    coords = synthetic.random_cells(5000, 2, 24, seed=5)
    oc, ns, ko, nbr = gpu_kernel_map(cuda_device, coords, (24, 24, 24), 3, 2, 1, 1, False, False)
    inv = inverse_map(nbr, coords.shape[0]).cpu().numpy()
    want = np.full((coords.shape[0], 27), -1, np.int32)
    n = nbr.cpu().numpy()
    o, k = np.nonzero(n >= 0)
    want[n[o, k], k] = o
    assert np.array_equal(inv, want)


@pytest.mark.parametrize("k,d", [(3, 1), (3, 2), (5, 1), (1, 1)])
@pytest.mark.parametrize("dtype", [torch.int32, torch.int16], ids=["i32", "i16"])
def test_submanifold_map_by_symmetry_equals_full_probing(cuda_device, oracle, k, d, dtype):
    """st_map_build_symmetric probes half of the offsets and mirrors the hits; the result must equal the
    fully probed map entry for entry, also for rows with duplicate coordinates (the largest row wins, the
    smaller ones still get their own entries) and for rows outside the declared grid."""
    base = synthetic.random_cells(6000, 2, 24, seed=31).numpy()
    coords = np.concatenate([base, base[:700], base[100:300],
                             np.array([[0, 30, 3, 3], [1, 3, 40, 3], [0, 23, 23, 24]], np.int32)])
    shape = (24, 24, 24)
    set_coords_dtype(dtype)
    c = torch.as_tensor(coords).to(cuda_device, dtype)
    p = ((k - 1) * d) // 2
    table = HashTable(capacity=2 * c.shape[0], device=cuda_device)
    table.insert(c)
    oc, _, ko = build_out_coords(c, shape, k, 1, d, p, transposed=False, submanifold=True)
    assert oc is c
    full = compute_neighbor_indices(table, c, ko, shape, 1, p, d)
    half = compute_neighbor_indices(table, c, ko, shape, 1, p, d, queries_are_table_rows=True)
    assert torch.equal(full, half)
    want = oracle.kernel_map(coords, shape, k, 1, d, p, False, True)[3]
    assert np.array_equal(half.cpu().numpy(), want)


@pytest.mark.parametrize("cdt", [torch.int32, torch.int16], ids=["int32", "int16"])
@pytest.mark.parametrize("k,s,p,d,transposed", [(3, 2, 1, 1, False), (2, 2, 0, 1, False), (3, 1, 0, 1, False), (5, 2, 2, 1, False),
                                                (3, 2, 1, 1, True), (2, 2, 0, 1, True), (3, 3, 0, 2, False)])
def test_direct_addressing_equals_the_hash_table(cuda_device, k, s, p, d, transposed, cdt):
    """With the batch size given, output coordinates are deduplicated by direct addressing (cell bitmap); without,
    through the hash table: ordered coordinates and map must be identical, duplicates in the input included."""
    from sparsetriton_b200.nn.functional.conv.kmap import out_coords_and_map
    set_coords_dtype(cdt)
    batch, grid = 3, 40
    coords = synthetic.random_cells(20_000, batch, grid, 321, dtype=cdt)
    coords = torch.cat([coords, coords[:500]]).to(cuda_device)                # 500 duplicated rows
    want = out_coords_and_map(coords, (grid,) * 3, k, s, d, p, transposed, batch_bound=0)
    got = out_coords_and_map(coords, (grid,) * 3, k, s, d, p, transposed, batch_bound=batch)
    assert got[0].shape[0] > 0 and got[1] == want[1]
    assert torch.equal(got[0], want[0]) and torch.equal(got[3], want[3])


def test_direct_addressing_flags_a_batch_index_beyond_the_batch(cuda_device):
    from sparsetriton_b200.nn.functional.conv.kmap import out_coords_and_map
    set_coords_dtype(torch.int32)
    coords = synthetic.random_cells(5_000, 3, 32, 322).to(cuda_device)
    with pytest.raises(ValueError, match="batch index"):
        out_coords_and_map(coords, (32,) * 3, 3, 2, 1, 1, False, batch_bound=2)


def test_direct_addressing_edge_cases(cuda_device):
    """No candidate at all (every input falls outside the output grid), a single voxel, and a batch bound larger
    than the samples present."""
    from sparsetriton_b200.nn.functional.conv.kmap import out_coords_and_map
    set_coords_dtype(torch.int32)
    one = torch.tensor([[1, 5, 6, 7]], dtype=torch.int32, device=cuda_device)
    for bound in (0, 2, 64):
        oc, shape, _, nbr = out_coords_and_map(one, (16, 16, 16), 3, 2, 1, 1, False, batch_bound=bound)
        # (5,6,7) + off is even on every axis for four offsets, in ascending k: 3, 5, 21, 23
        assert oc.tolist() == [[1, 3, 3, 4], [1, 3, 3, 3], [1, 2, 3, 4], [1, 2, 3, 3]]
        assert nbr.shape == (4, 27) and [int(nbr[r, k]) for r, k in enumerate((3, 5, 21, 23))] == [0, 0, 0, 0]
        assert int((nbr >= 0).sum()) == 4
    # k2 s2 on a 1-cell-wide grid: the output grid is empty
    thin = torch.tensor([[0, 0, 0, 0]], dtype=torch.int32, device=cuda_device)
    for bound in (0, 1):
        oc, shape, _, nbr = out_coords_and_map(thin, (1, 1, 1), 2, 2, 1, 0, False, batch_bound=bound)
        assert oc.shape[0] == 0 and nbr.shape[0] == 0
