"""Hash table build/query on the GPU against the oracle and the reference's golden answers."""
import numpy as np
import pytest
import torch

from conftest import golden_files, load_golden
from sparsetriton_b200 import synthetic
from sparsetriton_b200.utils.hash import HashTable

pytestmark = pytest.mark.gpu


def test_golden_insert_query(cuda_device):
    g = load_golden(golden_files("hash_basic")[0])
    t = HashTable(capacity=int(g["capacity"]), device=cuda_device)
    assert torch.all(t.table_keys == -1) and torch.all(t.table_values == -1)
    t.insert(torch.as_tensor(g["insert"]).to(cuda_device))
    assert torch.any(t.table_keys != -1)
    out = t.query(torch.as_tensor(g["query"]).to(cuda_device))
    assert out.dtype == torch.int32
    assert np.array_equal(out.cpu().numpy(), g["result"])


def test_golden_duplicates_keep_last_row(cuda_device):
    g = load_golden(golden_files("hash_basic")[0])
    t = HashTable(capacity=int(g["dup_capacity"]), device=cuda_device)
    t.insert(torch.as_tensor(g["dup_insert"]).to(cuda_device))
    out = t.query(torch.as_tensor(g["dup_query"]).to(cuda_device))
    assert np.array_equal(out.cpu().numpy(), g["dup_result"])


@pytest.mark.parametrize("dtype", [torch.int16, torch.int32])
@pytest.mark.parametrize("capacity_factor", [1.0, 1.5, 2.0, "pow2"])
def test_random_vs_oracle(cuda_device, oracle, dtype, capacity_factor):
    n = 200_000
    coords = synthetic.random_cells(n + 50_000, 4, 128, seed=11)
    present, absent = coords[:n], coords[n:]
    cap = 1 << 19 if capacity_factor == "pow2" else int(n * capacity_factor)
    t = HashTable(capacity=cap, device=cuda_device)
    t.insert(present.to(cuda_device, dtype))
    q = torch.cat([present[::3], absent])
    got = t.query(q.to(cuda_device, dtype)).cpu().numpy()
    want = oracle.Table(present.numpy()).query(q.numpy())
    assert np.array_equal(got, want)
    assert (got[: present[::3].shape[0]] == np.arange(0, n, 3)).all()
    assert (got[present[::3].shape[0]:] == -1).all()


def test_edge_cases(cuda_device):
    t = HashTable(capacity=64, device=cuda_device)
    t.insert(torch.empty((0, 4), dtype=torch.int32, device=cuda_device))
    assert torch.all(t.table_keys == -1)
    q = torch.tensor([[0, 1, 2, 3], [0, -1, 0, 0], [0, 0, 0, 70000]], dtype=torch.int32, device=cuda_device)
    assert t.query(q).tolist() == [-1, -1, -1]
    assert t.query(q[:0]).shape == (0,)
    t.insert(torch.tensor([[0, 0, 0, 0], [3, 65535, 65535, 65535]], dtype=torch.int32, device=cuda_device))
    q2 = torch.tensor([[3, 65535, 65535, 65535], [0, 0, 0, 0], [0, 0, 0, 1]], dtype=torch.int32, device=cuda_device)
    assert t.query(q2).tolist() == [1, 0, -1]
    # a full table still terminates: capacity == number of keys, then a miss
    full = HashTable(capacity=4, device=cuda_device)
    c = torch.tensor([[0, 1, 1, 1], [0, 2, 2, 2], [0, 3, 3, 3], [0, 4, 4, 4]], dtype=torch.int32, device=cuda_device)
    full.insert(c)
    assert full.query(c).tolist() == [0, 1, 2, 3]
    assert full.query(torch.tensor([[0, 9, 9, 9]], dtype=torch.int32, device=cuda_device)).tolist() == [-1]


def test_reference_suite_cases(cuda_device):
    """The assertions of the reference's tests/test_utils_hash.py:61-129 on this implementation."""
    t = HashTable(capacity=1000, device=cuda_device)
    assert t.capacity == 1000 and t.device.type == "cuda"
    coords = torch.tensor([[0, 1, 2, 3], [0, 1, 2, 4], [0, 1, 3, 3], [1, 0, 0, 0]], dtype=torch.int32,
                          device=cuda_device)
    t.insert(coords)
    assert t.query(coords).tolist() == [0, 1, 2, 3]
    assert t.query(torch.tensor([[0, 5, 5, 5]], dtype=torch.int32, device=cuda_device))[0].item() == -1
    assert t.cpu().device.type == "cpu"
    with pytest.raises(AssertionError, match="capacity should be at least"):
        HashTable(capacity=10, device=cuda_device).insert(
            torch.randint(0, 10, (20, 4), dtype=torch.int32, device=cuda_device))


def test_large_scale_roundtrip(cuda_device):
    """2M keys at load factor 0.5: every key finds its own row, a disjoint set misses."""
    n = 2_000_000
    coords = synthetic.random_cells(n + 100_000, 4, 2048, seed=2001).to(cuda_device)
    t = HashTable(capacity=2 * n, device=cuda_device)
    t.insert(coords[:n])
    got = t.query(coords[:n])
    assert torch.equal(got, torch.arange(n, dtype=torch.int32, device=cuda_device))
    assert torch.all(t.query(coords[n:]) == -1)
    assert int((t.table_keys != -1).sum().item()) == n
