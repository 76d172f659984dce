"""CPU-only checks: host-side integer logic against the oracle, the mirrored Python surface
(config / SparseTensor / HashTable construction and error messages), the C-ABI exports, and the
rule that nothing runs without the CUDA library."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import sparsetriton_b200 as st
from sparsetriton_b200 import _lib, config
from sparsetriton_b200.nn.functional.conv.kmap import kernel_offsets, output_shape
from sparsetriton_b200.utils.hash import HashTable, flatten_coord, hash_coords, round_up_capacity, unflatten_coord

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("k", [1, 2, 3, 5])
@pytest.mark.parametrize("d", [1, 2])
@pytest.mark.parametrize("p", [0, 1, 2])
@pytest.mark.parametrize("transposed", [False, True])
def test_offsets_and_shapes_match_oracle(oracle, k, d, p, transposed):
    assert np.array_equal(np.array(kernel_offsets(k, d, p, transposed), np.int32).reshape(-1, 3),
                          oracle.offsets(k, d, p, transposed))
    for s in (1, 2, 4):
        for shape in ((8, 8, 8), (9, 8, 7), (41, 1440, 3)):
            assert list(output_shape(shape, k, s, d, p, transposed)) == \
                oracle.new_shape(shape, k, s, d, p, transposed).tolist()


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "sparsetriton_b200.h")).read()
    declared = sorted(set(re.findall(r"\b(st_[a-z0-9_]+)\s*\(", header)))
    assert len(declared) >= 20
    assert os.path.exists(_lib.LIB_PATH), "library not built: python -m sparsetriton_b200.build"
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
    assert sorted(_lib.EXPORTED_SYMBOLS) == declared, "ctypes binding and header disagree"
    assert _lib.lib().st_version() >= 1


def test_abi_argument_errors_need_no_gpu():
    L = _lib.lib()
    assert L.st_hash_clear(None, None, -1, None) == -1
    assert b"st_hash_clear" in L.st_last_error_string()
    assert L.st_conv_fwd(7, None, None, None, None, 0, 0, 27, 4, 4, None, 0, None) == -2      # bad dtype
    assert L.st_conv_fwd(0, None, None, None, None, 0, 0, 1000, 4, 4, None, 0, None) == -1    # K too large
    assert L.st_map_build(None, 0, 1, None, 27, 1, None, None, None, 0, None, None) == -1
    assert L.st_outcoords_workspace_bytes(1000, 27, 2, 0) > 1000 * 8


def test_no_cpu_fallback():
    sp = st.randn((8, 8, 8), channels=4, nnz=20, device="cpu")
    conv = st.nn.SubMConv3D(4, 8, 3)
    with pytest.raises(RuntimeError, match="no CPU path"):
        conv(sp)
    t = HashTable(capacity=100, device="cpu")
    with pytest.raises(RuntimeError, match="no CPU path"):
        t.insert(torch.zeros(3, 4, dtype=torch.int32))
    with pytest.raises(RuntimeError, match="no CPU path"):
        t.query(torch.zeros(3, 4, dtype=torch.int32))


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "sparsetriton_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(base, f)).read()
                assert "oracle" not in text.replace("oracle-", ""), f"{f} mentions the oracle"


# ---- mirrored surface: the assertions of the reference's CPU tests -------------------------

def test_config_surface():
    assert config.get_coords_dtype() == torch.int16 and config.get_h_table_f() == 1.5
    assert config.get_conv_algo() == config.ConvAlgo.PrecomputedNeighborGEMM and config.get_h_table_max_p() == 16
    assert config.ConvAlgo.ImplicitHashFlyGEMM.value == "Implicit_hashfly_gemm" and len(config.ConvAlgo) == 2
    config.set_h_table_f("3.5")
    assert config.get_h_table_f() == 3.5
    config.set_h_table_max_p("64")
    assert config.get_h_table_max_p() == 64
    for bad in ("int32", 32, None):
        with pytest.raises(TypeError):
            config.set_coords_dtype(bad)
    for bad in ("Implicit_hashmap_gemm", 1, None):
        with pytest.raises(TypeError):
            config.set_conv_algo(bad)
    with pytest.raises(AssertionError, match="factor must be >= 1"):
        config.set_h_table_f(0.5)
    with pytest.raises(TypeError, match="factor must be a number"):
        config.set_h_table_f(None)
    with pytest.raises(AssertionError, match="probe_n must be positive"):
        config.set_h_table_max_p(0)
    with pytest.raises(TypeError, match="probe_n must be an integer"):
        config.set_h_table_max_p("x")


def test_sparse_tensor_surface():
    coords = torch.tensor([[0, 1, 2, 3], [0, 1, 2, 4], [0, 1, 3, 3], [1, 0, 0, 0], [1, 1, 1, 1]])
    sp = st.SparseTensor(torch.randn(5, 3), coords)
    assert sp.spatial_shape == torch.Size([2, 4, 5]) and sp.batch_size == 2 and sp.coords.dtype == torch.int16
    assert st.SparseTensor(torch.empty(0, 3), torch.empty(0, 4, dtype=torch.int16)).batch_size == 0
    with pytest.raises(AssertionError, match="must match"):
        st.SparseTensor(torch.randn(5, 3), torch.tensor([[0, 1, 2, 3]]))
    with pytest.raises(AssertionError, match="shape .*N, 4.*"):
        st.SparseTensor(torch.randn(5, 3), torch.randn(5, 3))
    with pytest.raises(AssertionError, match="must be 2D"):
        st.SparseTensor(torch.randn(5, 3, 2), torch.randn(5, 4))
    with pytest.raises(AssertionError, match="batch_size .* must be >"):
        st.SparseTensor(torch.randn(3, 4), torch.tensor([[0, 1, 2, 3], [0, 1, 2, 4], [5, 1, 3, 3]]), batch_size=3)
    sp2 = sp.replace(torch.randn(5, 7))
    assert sp2._cache is sp._cache and sp2.spatial_shape == sp.spatial_shape and sp2.batch_size == 2
    assert "spatial_shape=" in repr(sp) and sp.half().F.dtype == torch.float16 and sp.float().F.dtype == torch.float32
    with pytest.raises(RuntimeError, match="no CPU path"):      # dense() is a CUDA scatter like every other operator
        st.SparseTensor(torch.tensor([[1.0], [2.0], [3.0]]), torch.tensor([[0, 0, 0, 0], [0, 0, 0, 1], [1, 0, 0, 0]])).dense()
    r = st.randn((16, 16, 16), batch_size=2, nnz=100, channels=4)
    assert torch.unique(r.coords, dim=0).shape[0] == 100 and r.F.shape == (100, 4)
    with pytest.raises(ValueError, match="nnz .* exceeds"):
        st.randn((2, 2, 2), nnz=10)


def test_hash_helpers_and_cpu_construction():
    c = torch.tensor([[0, 1, 2, 3], [0, 1, 2, 4], [0, 1, 3, 3], [1, 100, 200, 50]])
    assert flatten_coord(c)[0].item() == (1 << 32) | (2 << 16) | 3 and flatten_coord(c).dtype == torch.int64
    config.set_coords_dtype(torch.int64)
    assert torch.equal(unflatten_coord(flatten_coord(c)), c)
    h = hash_coords(torch.randint(0, 100, (1000, 4)))
    assert h.dtype == torch.int32 and torch.all(h >= 0) and torch.unique(h).shape[0] > 500
    t = HashTable(capacity=1000, device="cpu")
    assert t.capacity == 1000 and torch.all(t.table_keys == -1) and torch.all(t.table_values == -1)
    assert HashTable(table_keys=torch.full((100,), -1), table_values=torch.full((100,), -1)).capacity == 100
    with pytest.raises(AssertionError, match="must have the same shape"):
        HashTable(table_keys=torch.ones(100), table_values=torch.ones(50))
    with pytest.raises(AssertionError, match="capacity should be at least"):
        HashTable(capacity=10, device="cpu").insert(torch.randint(0, 10, (20, 4), dtype=torch.int32))
    assert round_up_capacity(1000, 1.5) == 2048 and round_up_capacity(0, 2.0) == 1


def test_module_surface_and_compat_alias():
    m = st.nn.SparseConvTransposed3D(4, 8, 3, stride=2, padding=1)
    assert m.weight.shape == (27, 4, 8) and m.transposed and not m.subm and m.stride == (2, 2, 2)
    assert st.nn.SubMConv3D(4, 8, 3, bias=False).bias is None and st.nn.SparseConv3D(4, 8, 5).kernel_volume == 125
    bound = 1.0 / (4 * 27) ** 0.5
    assert m.weight.abs().max() <= bound
    import sparsetriton_b200.compat as compat
    compat.install()
    from sparsetriton import SparseTensor as Aliased
    from sparsetriton.nn.functional.conv.funcs import ConvHashOnTheFlyImplicitGEMM  # noqa: F401
    from sparsetriton.nn.functional.conv.funcs.implicit_precomputed_gemm import ConvPrecomputedNeighborGEMM  # noqa: F401
    assert Aliased is st.SparseTensor


def test_preparation_surface_needs_cuda_and_caches_children():
    """ConvPreparation / prepare_conv3d refuse CPU coordinates (no CPU path), and a TensorCache hands out one child
    cache per layer geometry."""
    from sparsetriton_b200.nn.functional import ConvPreparation, prepare_conv3d
    from sparsetriton_b200.tensor import TensorCache
    coords = torch.zeros((4, 4), dtype=torch.int32)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ConvPreparation(coords, (8, 8, 8), 3, stride=2, padding=1, submanifold=False)
    with pytest.raises(RuntimeError, match="no CPU path"):
        prepare_conv3d(coords, (8, 8, 8), 3)
    with pytest.raises(AssertionError, match="transposed"):
        ConvPreparation(coords, (8, 8, 8), 3, transposed=True, submanifold=True)
    cache = TensorCache()
    key = (2, 2, 0, 1, False, False)
    child = cache.child(key)
    assert cache.child(key) is child and cache.child((3, 2, 1, 1, False, False)) is not child
    assert child.neighbor_indices == {} and child.hashtable is None and child.children == {}


def test_tall_linear_gradients_on_the_host():
    """The split weight gradient of SparseLinear's tall form equals torch's on the same numbers (the Function itself is
    device-agnostic; the module only routes CUDA inputs of 65 536 rows or more through it)."""
    import sparsetriton_b200.nn.modules.simple as simple
    torch.manual_seed(0)
    lin = simple.SparseLinear(7, 5).double()
    ref = torch.nn.Linear(7, 5).double()
    ref.load_state_dict(lin.state_dict())
    n = 2 * simple._SPLIT_ROWS + 333                      # two whole pieces and a remainder
    x = torch.randn(n, 7, dtype=torch.float64, requires_grad=True)
    x2 = x.detach().clone().requires_grad_(True)
    y, y2 = simple._TallLinear.apply(x, lin.weight, lin.bias), ref(x2)
    g = torch.randn_like(y)
    y.backward(g)
    y2.backward(g)
    assert torch.allclose(y, y2) and torch.allclose(x.grad, x2.grad)
    assert torch.allclose(lin.weight.grad, ref.weight.grad) and torch.allclose(lin.bias.grad, ref.bias.grad)
    # a CPU input takes nn.Linear's own path
    assert torch.equal(lin(x.detach()), ref(x.detach()))


def test_concat_features_is_torch_cat_for_host_tensors():
    """The reference's networks call torch.cat here; the library's copy kernels only take over for CUDA matrices whose rows
    are whole 16-byte pieces."""
    from sparsetriton_b200.utils.concat import concat_features
    a, b = torch.randn(5, 8), torch.randn(5, 4)
    assert torch.equal(concat_features(a, b), torch.cat([a, b], dim=1))
