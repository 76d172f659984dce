"""Data parallelism by batch sample: one process per GPU, no collective on the data path.

Samples are independent through every operator of the path (hash keys carry the batch index, maps
never cross samples, batch norm is per sample), so each rank builds its own tables and maps.  The
only exchange of a training step is one all-reduce of a single flat fp32 gradient bucket.
"""
import torch
import torch.distributed as dist

__all__ = ["shard_samples", "relabel_batch", "GradientBucket", "global_mean_scale"]


def shard_samples(n_samples, rank, world):
    """Indices of the samples rank `rank` owns: contiguous blocks, sizes differing by at most one."""
    base, extra = divmod(n_samples, world)
    start = rank * base + min(rank, extra)
    return list(range(start, start + base + (1 if rank < extra else 0)))


def relabel_batch(coords, samples):
    """Rows of `coords` (N,4) whose batch index is in `samples`, relabelled 0..len(samples)-1."""
    out = []
    for new, old in enumerate(samples):
        rows = coords[coords[:, 0] == old].clone()
        rows[:, 0] = new
        out.append(rows)
    return torch.cat(out) if out else coords[:0]


def global_mean_scale(local_count, device=None):
    """1 / (total number of voxels over all ranks): multiply the local SUM of per-voxel losses by it
    and the summed gradients equal those of the single-process mean loss."""
    total = torch.tensor([float(local_count)], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(total)
    return 1.0 / max(total.item(), 1.0)


class GradientBucket:
    """All parameters' gradients as views of one flat fp32 buffer, reduced with one collective."""

    def __init__(self, parameters):
        self.params = [p for p in parameters if p.requires_grad]
        n = sum(p.numel() for p in self.params)
        dev = self.params[0].device if self.params else None
        self.flat = torch.zeros(n, dtype=torch.float32, device=dev)
        offset = 0
        for p in self.params:
            p.grad = self.flat[offset:offset + p.numel()].view_as(p)
            offset += p.numel()

    def zero(self):
        self.flat.zero_()

    def all_reduce(self):
        """Sum over ranks, in place.  Parameters whose .grad was replaced by autograd are copied back in."""
        offset = 0
        for p in self.params:
            view = self.flat[offset:offset + p.numel()].view_as(p)
            if p.grad is None:
                view.zero_()
                p.grad = view
            elif p.grad.data_ptr() != view.data_ptr():
                view.copy_(p.grad)
                p.grad = view
            offset += p.numel()
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(self.flat)
        return self.flat
