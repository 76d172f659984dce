"""World-size-2 checks of the data-parallel plumbing on CPU (gloo): sample sharding, batch
relabelling, the flat gradient bucket and the loss scaling that makes summed gradients equal the
single-process mean-loss gradients."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sparsetriton_b200.distributed import GradientBucket, global_mean_scale, relabel_batch, shard_samples


def test_shard_and_relabel():
    assert [shard_samples(16, r, 8) for r in range(8)] == [[2 * r, 2 * r + 1] for r in range(8)]
    assert sum((shard_samples(10, r, 4) for r in range(4)), []) == list(range(10))
    coords = torch.tensor([[0, 1, 1, 1], [2, 5, 5, 5], [1, 2, 2, 2], [2, 6, 6, 6], [3, 0, 0, 0]])
    got = relabel_batch(coords, [2, 3])
    assert got.tolist() == [[0, 5, 5, 5], [0, 6, 6, 6], [1, 0, 0, 0]]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.ReLU(), torch.nn.Linear(5, 3))
    data = torch.randn(10, 6, generator=torch.Generator().manual_seed(1))
    target = torch.randint(0, 3, (10,), generator=torch.Generator().manual_seed(2))
    mine = slice(0, 7) if rank == 0 else slice(7, 10)              # uneven shards on purpose
    bucket = GradientBucket(model.parameters())
    bucket.zero()
    scale = global_mean_scale(data[mine].shape[0])
    loss = torch.nn.functional.cross_entropy(model(data[mine]), target[mine], reduction="sum") * scale
    loss.backward()
    flat = bucket.all_reduce().clone()
    if rank == 0:
        ref = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.ReLU(), torch.nn.Linear(5, 3))
        ref.load_state_dict(model.state_dict())
        torch.nn.functional.cross_entropy(ref(data), target).backward()
        want = torch.cat([p.grad.reshape(-1) for p in ref.parameters()])
        out.put((flat, want, abs(scale - 0.1) < 1e-12))
    dist.barrier()
    dist.destroy_process_group()


def test_bucket_allreduce_equals_single_process_gradients():
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    flat, want, scale_ok = out.get()
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert scale_ok
    torch.testing.assert_close(flat, want, rtol=1e-5, atol=1e-6)
