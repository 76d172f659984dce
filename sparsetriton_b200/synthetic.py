"""Seeded synthetic inputs with the shapes and value distributions of the benchmark workloads.

Every generator uses its own `torch.Generator(device="cpu")`, returns CPU tensors and is
deterministic in its seed, so the same voxels can be handed to any implementation.

    random_cells        uniformly random distinct cells of a batch of grids (hash / map microbenchmarks)
    surface_scene       ground sheet + spherical shells + box shells in a 512^3 grid
    lidar_scene         one spinning-lidar sweep over a ground plane and boxes in a 1440x1440x41 grid
    batch_of            stack per-sample scenes into one (N,4) coordinate tensor
"""
import math

import torch

__all__ = ["random_cells", "surface_scene", "lidar_scene", "batch_of"]


def random_cells(n, batch, grid, seed, dtype=torch.int32):
    """`n` distinct cells of `batch` cubic grids of side `grid`, shuffled; rows (b, x, y, z)."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    total = batch * grid ** 3
    if n > total:
        raise ValueError("more cells requested than the grids hold")
    if total <= 1 << 24:
        flat = torch.randperm(total, generator=gen)[:n]
    else:
        flat = torch.empty(0, dtype=torch.int64)
        while flat.numel() < n:
            draw = torch.randint(0, total, (int((n - flat.numel()) * 1.05) + 16,), generator=gen)
            flat = torch.unique(torch.cat([flat, draw]))
        flat = flat[torch.randperm(flat.numel(), generator=gen)[:n]]
    z = flat % grid
    y = (flat // grid) % grid
    x = (flat // (grid * grid)) % grid
    b = flat // (grid ** 3)
    return torch.stack([b, x, y, z], dim=1).to(dtype)


def _unique_cells(xyz, grid):
    """Deduplicate (M,3) integer cells inside [0,grid)^3; returns sorted unique rows."""
    keep = ((xyz >= 0) & (xyz < grid)).all(dim=1)
    xyz = xyz[keep]
    flat = torch.unique((xyz[:, 0] * grid + xyz[:, 1]) * grid + xyz[:, 2])
    return torch.stack([flat // (grid * grid), (flat // grid) % grid, flat % grid], dim=1)


def _sphere_shell(centre, radius, grid):
    """Cells p with | |p - c| - r | < 0.5, clipped to the grid."""
    lo = [max(int(math.floor(c - radius - 1)), 0) for c in centre]
    hi = [min(int(math.ceil(c + radius + 1)), grid - 1) for c in centre]
    if any(l > h for l, h in zip(lo, hi)):
        return torch.empty((0, 3), dtype=torch.int64)
    ax = [torch.arange(l, h + 1, dtype=torch.float32) for l, h in zip(lo, hi)]
    d2 = ((ax[0] - centre[0]) ** 2)[:, None, None] + ((ax[1] - centre[1]) ** 2)[None, :, None] \
        + ((ax[2] - centre[2]) ** 2)[None, None, :]
    hit = (d2.sqrt() - radius).abs() < 0.5
    idx = hit.nonzero()
    return idx + torch.tensor(lo, dtype=torch.int64)


def _box_shell(centre, half, grid):
    """One-voxel-thick faces of an axis-aligned box, clipped to the grid."""
    lo = [int(round(c - h)) for c, h in zip(centre, half)]
    hi = [int(round(c + h)) for c, h in zip(centre, half)]
    rng = [torch.arange(l, h + 1, dtype=torch.int64) for l, h in zip(lo, hi)]
    faces = []
    for axis in range(3):
        others = [a for a in range(3) if a != axis]
        u, v = torch.meshgrid(rng[others[0]], rng[others[1]], indexing="ij")
        for w in (lo[axis], hi[axis]):
            cols = [None, None, None]
            cols[axis] = torch.full_like(u, w)
            cols[others[0]], cols[others[1]] = u, v
            faces.append(torch.stack([c.reshape(-1) for c in cols], dim=1))
    cells = torch.cat(faces)
    keep = ((cells >= 0) & (cells < grid)).all(dim=1)
    return cells[keep]


def surface_scene(seed, grid=512, target=300_000, n_spheres=12, n_boxes=20):
    """(M,3) int64 cells of one sample: a ground sheet z = 20 + {-1,0,1} (one voxel per (x,y)
    column), `n_spheres` one-voxel spherical shells (radius U[20,120]) and `n_boxes` box shells
    (half sizes U[5,60]), centres uniform in the grid.  Objects are added whole, in drawing order,
    while the total stays within `target`; the first object that would overflow is cut (in
    lexicographic cell order) to land on `target`, the rest are dropped.  Surfaces therefore stay
    contiguous sheets.  With the defaults M == target."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    xs, ys = torch.meshgrid(torch.arange(grid), torch.arange(grid), indexing="ij")
    zs = 20 + torch.randint(-1, 2, (grid, grid), generator=gen)
    cells = torch.stack([xs.reshape(-1), ys.reshape(-1), zs.reshape(-1)], dim=1)
    objects = []
    for _ in range(n_spheres):
        c = (torch.rand(3, generator=gen) * grid).tolist()
        r = float(torch.rand(1, generator=gen)) * 100 + 20
        objects.append(("sphere", c, r))
    for _ in range(n_boxes):
        c = (torch.rand(3, generator=gen) * grid).tolist()
        h = (torch.rand(3, generator=gen) * 55 + 5).tolist()
        objects.append(("box", c, h))
    order = torch.randperm(len(objects), generator=gen).tolist()
    for i in order:
        kind, c, size = objects[i]
        new = _sphere_shell(c, size, grid) if kind == "sphere" else _box_shell(c, size, grid)
        merged = _unique_cells(torch.cat([cells, new]), grid)
        if merged.shape[0] <= target:
            cells = merged
            continue
        # keep only as many new cells as fit, in lexicographic order
        have = _unique_cells(cells, grid)
        flat_have = (have[:, 0] * grid + have[:, 1]) * grid + have[:, 2]
        flat_all = (merged[:, 0] * grid + merged[:, 1]) * grid + merged[:, 2]
        fresh = merged[~torch.isin(flat_all, flat_have)]
        cells = _unique_cells(torch.cat([have, fresh[: target - have.shape[0]]]), grid)
        break
    return _unique_cells(cells, grid)


def lidar_scene(seed, grid=(1440, 1440, 41), rings=64, azimuths=2048, n_boxes=40):
    """(M,3) int64 cells hit by one sweep of a spinning lidar at the grid centre (height 38):
    `rings` elevation rings x `azimuths` headings; each ray stops at the nearest of the ground
    plane z = 2 and `n_boxes` axis-aligned boxes standing on it (centres uniform in [100,1340]^2,
    footprint half sizes U[4,40], heights U[4,30]); rays that leave the grid hit nothing; duplicate
    cells are merged.  The ring elevations are spaced so that their ground ranges are uniform in
    [250, 715] cells (elevations about -8 deg to -2.8 deg): with one-cell voxels this is what
    makes most of the 131 072 rays land in distinct cells (about 105k voxels per sample); a low
    sensor with rings linear in angle piles the hits up within a few tens of cells and leaves
    about 20k."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    gx, gy, gz = grid
    origin = torch.tensor([gx / 2.0, gy / 2.0, 38.0])
    el = -torch.atan((origin[2] - 2.5) / torch.linspace(250.0, 715.0, rings))
    az = torch.arange(azimuths, dtype=torch.float32) * (2 * math.pi / azimuths)
    ce, se = torch.cos(el)[:, None], torch.sin(el)[:, None]
    d = torch.stack([ce * torch.cos(az)[None, :], ce * torch.sin(az)[None, :], se.expand(-1, azimuths)], dim=-1)
    d = d.reshape(-1, 3)
    inf = torch.full((d.shape[0],), float("inf"))
    # ground plane z = 2 (top face of the ground voxels)
    t_hit = torch.where(d[:, 2] < -1e-6, (2.5 - origin[2]) / d[:, 2], inf)
    centre_xy = torch.rand(n_boxes, 2, generator=gen) * 1240 + 100
    half_xy = torch.rand(n_boxes, 2, generator=gen) * 36 + 4
    height = torch.rand(n_boxes, generator=gen) * 26 + 4
    lo = torch.cat([centre_xy - half_xy, torch.full((n_boxes, 1), 2.0)], dim=1)
    hi = torch.cat([centre_xy + half_xy, 2.0 + height[:, None]], dim=1)
    # the sensor must not sit inside a box
    inside = ((origin >= lo) & (origin <= hi)).all(dim=1)
    lo, hi = lo[~inside], hi[~inside]
    inv = 1.0 / torch.where(d.abs() < 1e-9, torch.full_like(d, 1e-9), d)
    t1 = (lo[None, :, :] - origin) * inv[:, None, :]
    t2 = (hi[None, :, :] - origin) * inv[:, None, :]
    t_near = torch.minimum(t1, t2).amax(dim=2)
    t_far = torch.maximum(t1, t2).amin(dim=2)
    box_t = torch.where((t_near <= t_far) & (t_near > 0), t_near, torch.full_like(t_near, float("inf")))
    t_hit = torch.minimum(t_hit, box_t.amin(dim=1))
    ok = torch.isfinite(t_hit)
    p = origin + d[ok] * (t_hit[ok][:, None] + 1e-3)
    cells = torch.floor(p).to(torch.int64)
    keep = (cells[:, 0] >= 0) & (cells[:, 0] < gx) & (cells[:, 1] >= 0) & (cells[:, 1] < gy) \
        & (cells[:, 2] >= 0) & (cells[:, 2] < gz)
    cells = cells[keep]
    flat = torch.unique((cells[:, 0] * gy + cells[:, 1]) * gz + cells[:, 2])
    return torch.stack([flat // (gy * gz), (flat // gz) % gy, flat % gz], dim=1)


def batch_of(samples, dtype=torch.int32):
    """Concatenate per-sample (M_i,3) cells into (N,4) rows (b, x, y, z), sample-major."""
    rows = [torch.cat([torch.full((s.shape[0], 1), b, dtype=torch.int64), s], dim=1) for b, s in enumerate(samples)]
    return torch.cat(rows).to(dtype)
