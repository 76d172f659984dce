"""Generate golden vectors by running the UNMODIFIED reference on CPU.

The reference (ptj0225/SparseTriton) has no native CPU path: its kernels are
Triton programs.  They execute here through the Triton interpreter
(``TRITON_INTERPRET=1``) with one harness-side adjustment made *before* the
reference is imported: ``triton.autotune`` keeps only the first config of each
list, because triton 3.6's autotuner asks the (absent) GPU driver for a
benchmarker even in interpreter mode.  No reference file is modified or copied.

Usage (only where the reference checkout is mounted; the fixtures travel, this
script's inputs do not):

    python tests/golden/make_golden.py --ref /path/to/SparseTriton [--only NAME] [--c1]

Every fixture stores its own inputs (coords, feats, weights, upstream gradient)
so no implementation has to reproduce a random stream.

What each ``.npz`` pins (reference file:line):
  hash_*      HashTable.insert/query                     sparsetriton/utils/hash.py:516-580
  kmap_*      build_out_coords + compute_neighbor_indices nn/functional/conv/kmap.py:213-495,
                                                          nn/functional/conv/conv.py:12-75
  conv_*      sparse_conv3d forward + autograd backward   nn/functional/conv/conv.py:77-239,
              (both ConvAlgo values)                      funcs/implicit_precomputed_gemm.py:233-324,
                                                          funcs/implicit_hashfly_gemm.py:330-452
  dense_*     to_dense forward + autograd backward        utils/to_dense.py:143-282
  pool_*      sparse_pooling (avg) forward + backward     nn/functional/spatial.py:26-292
  upsample_*  sparse_upsample forward + backward          nn/functional/spatial.py:294-535
  bn_*        sparse_batch_norm, training and inference   nn/functional/norm.py:20-112

Batched transposed convolution with stride > 1 is run one sample at a time
(rows of a sample relabelled to batch 0) and concatenated, because the reference
scales the batch column together with the spatial ones (kmap.py:407).
"""
import argparse
import os
import sys
import time

os.environ.setdefault("TRITON_INTERPRET", "1")
sys.dont_write_bytecode = True

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _install_autotune_shim():
    import triton

    original = triton.autotune

    def first_config_only(configs, key, **kw):
        return original(configs[:1], key, **kw)

    triton.autotune = first_config_only


def _rand_coords(gen, n, batch, shape, sort_rows=False):
    """n distinct (b,x,y,z) rows; shuffled unless sort_rows."""
    total = batch * shape[0] * shape[1] * shape[2]
    assert n <= total
    flat = torch.randperm(total, generator=gen)[:n]
    if sort_rows:
        flat = torch.sort(flat).values
    z = flat % shape[2]
    y = (flat // shape[2]) % shape[1]
    x = (flat // (shape[2] * shape[1])) % shape[0]
    b = flat // (shape[2] * shape[1] * shape[0])
    return torch.stack([b, x, y, z], dim=1).to(torch.int32)


KMAP_CASES = [
    # name, N, batch, shape, k, s, p, d, transposed, subm, coord dtype
    ("subm_k3", 300, 2, (16, 16, 16), 3, 1, 1, 1, False, True, "int32"),
    ("subm_k3_i16", 200, 2, (12, 12, 12), 3, 1, 1, 1, False, True, "int16"),
    ("subm_k5", 150, 1, (10, 10, 10), 5, 1, 2, 1, False, True, "int32"),
    ("subm_k3_d2", 200, 2, (12, 12, 12), 3, 1, 2, 2, False, True, "int32"),
    ("subm_k1", 100, 2, (8, 8, 8), 1, 1, 0, 1, False, True, "int32"),
    ("subm_k3_s2", 200, 2, (12, 12, 12), 3, 2, 1, 1, False, True, "int32"),
    ("conv_k3_s2_p1", 300, 2, (16, 16, 16), 3, 2, 1, 1, False, False, "int32"),
    ("conv_k2_s2_p0", 300, 2, (9, 8, 7), 2, 2, 0, 1, False, False, "int32"),
    ("conv_k5_s2_p2", 150, 1, (10, 10, 10), 5, 2, 2, 1, False, False, "int32"),
    ("conv_k3_s1_p1", 120, 2, (8, 8, 8), 3, 1, 1, 1, False, False, "int32"),
    ("conv_k3_s1_p0", 200, 1, (10, 10, 10), 3, 1, 0, 1, False, False, "int32"),
    ("conv_k3_s1_p2", 60, 1, (6, 6, 6), 3, 1, 2, 1, False, False, "int32"),
    ("conv_k3_s2_p1_d2", 200, 2, (12, 12, 12), 3, 2, 1, 2, False, False, "int32"),
    ("conv_k3_s4_p1", 300, 1, (16, 16, 16), 3, 4, 1, 1, False, False, "int16"),
    ("tconv_k2_s2_p0", 100, 1, (8, 8, 8), 2, 2, 0, 1, True, False, "int32"),
    ("tconv_k3_s2_p1", 80, 1, (8, 8, 8), 3, 2, 1, 1, True, False, "int32"),
    ("tconv_k3_s4_p1", 40, 1, (6, 6, 6), 3, 4, 1, 1, True, False, "int32"),
    ("tconv_k3_s1_p1", 100, 1, (8, 8, 8), 3, 1, 1, 1, True, False, "int32"),
    ("tconv_k5_s1_p2", 60, 1, (8, 8, 8), 5, 1, 2, 1, True, False, "int32"),
    ("tconv_k2_s2_p0_b3", 120, 3, (6, 6, 6), 2, 2, 0, 1, True, False, "int32"),
    ("tconv_k3_s2_p1_b2", 80, 2, (6, 6, 6), 3, 2, 1, 1, True, False, "int32"),
]

CONV_CASES = [
    # name, kmap case name, Cin, Cout, bias
    ("conv_subm_k3_c16_32", "subm_k3", 16, 32, False),
    ("conv_subm_k3_i16_c4_8", "subm_k3_i16", 4, 8, True),
    ("conv_subm_k5_c8_16", "subm_k5", 8, 16, False),
    ("conv_down_k3s2_c16_16", "conv_k3_s2_p1", 16, 16, True),
    ("conv_down_k2s2_c32_64", "conv_k2_s2_p0", 32, 64, False),
    ("conv_full_k3s1p1_c8_8", "conv_k3_s1_p1", 8, 8, False),
    ("conv_up_k2s2_c16_8", "tconv_k2_s2_p0", 16, 8, False),
    ("conv_up_k3s2_c4_8", "tconv_k3_s2_p1", 4, 8, True),
    ("conv_up_k2s2_b3_c8_8", "tconv_k2_s2_p0_b3", 8, 8, False),
]


def _case_inputs(case):
    name, n, batch, shape = case[0], case[1], case[2], case[3]
    seed = 1000 + [c[0] for c in KMAP_CASES].index(name)
    gen = torch.Generator(device="cpu").manual_seed(seed)
    # batched transposed cases keep rows grouped by sample (sorted), the rest are shuffled
    grouped = case[8] and batch > 1
    coords = _rand_coords(gen, n, batch, shape, sort_rows=grouped)
    return coords, seed


def _ref_kmap(st, coords, shape, batch, k, s, p, d, transposed, subm, cdtype):
    """out_coords, new_shape, kernel_offsets, nbr from the reference, per its own call sequence
    in sparse_conv3d (conv.py:137-188)."""
    from sparsetriton.nn.functional.conv.kmap import build_out_coords
    from sparsetriton.nn.functional.conv.conv import compute_neighbor_indices
    from sparsetriton.utils.hash import HashTable
    from sparsetriton.config import set_coords_dtype

    set_coords_dtype(cdtype)
    c = coords.to(cdtype)
    if subm:
        p = ((k - 1) * d) // 2
    table = HashTable(int(c.shape[0] * 2) + 1, device="cpu")
    keyc = c.clone()
    if transposed and s > 1:
        keyc[:, 1:] *= s
    table.insert(keyc)
    oc, ns, ko = build_out_coords(c, shape, k, s, d, p, transposed=transposed, submanifold=subm)
    look = tuple(v * s for v in shape) if (transposed and s > 1) else tuple(shape)
    if oc.shape[0] == 0:
        nbr = torch.empty((0, ko.shape[0]), dtype=torch.int32)
    else:
        nbr = compute_neighbor_indices(table, oc, ko, look, s if not transposed else 1, p, d)
    ns = [int(v) for v in ns]
    return oc.clone(), ns, ko.clone(), nbr


def _check_no_alias(coords):
    """The reference stores a 31-bit hash as key (hash.py:136-152); make sure this fixture has
    no two coordinates that share it, so the reference's answer is the exact one."""
    c = coords.to(torch.int32)
    h2 = ((c[:, 0] * 1000003) ^ (c[:, 1] * 100003) ^ (c[:, 2] * 10007) ^ c[:, 3]) & 0x7FFFFFFF
    assert torch.unique(h2).shape[0] == torch.unique(c, dim=0).shape[0], "31-bit key alias in fixture"


def make_kmap(case):
    name, n, batch, shape, k, s, p, d, transposed, subm, dt = case
    cdtype = getattr(torch, dt)
    coords, seed = _case_inputs(case)
    _check_no_alias(coords)
    t0 = time.time()
    if transposed and s > 1 and batch > 1:
        ocs, nbrs = [], []
        row0 = 0
        for b in range(batch):
            rows = coords[coords[:, 0] == b].clone()
            rows[:, 0] = 0
            oc, ns, ko, nbr = _ref_kmap(None, rows, shape, 1, k, s, p, d, transposed, subm, cdtype)
            oc = oc.clone()
            oc[:, 0] = b
            nbr = torch.where(nbr >= 0, nbr + row0, nbr)
            row0 += rows.shape[0]
            ocs.append(oc)
            nbrs.append(nbr)
        oc, nbr = torch.cat(ocs), torch.cat(nbrs)
    else:
        oc, ns, ko, nbr = _ref_kmap(None, coords, shape, batch, k, s, p, d, transposed, subm, cdtype)
    print(f"  kmap {name}: N={n} N_out={oc.shape[0]} pairs={int((nbr >= 0).sum())} new_shape={ns} ({time.time() - t0:.1f}s)")
    np.savez_compressed(
        os.path.join(HERE, f"kmap_{name}.npz"),
        coords=coords.numpy(), shape=np.array(shape), batch=batch,
        k=k, s=s, p=p, d=d, transposed=transposed, subm=subm, coord_dtype=dt,
        out_coords=oc.to(torch.int32).numpy(), new_shape=np.array(ns),
        kernel_offsets=ko.to(torch.int32).numpy(), nbr=nbr.numpy(),
    )


def make_hash():
    from sparsetriton.utils.hash import HashTable
    from sparsetriton.config import set_coords_dtype

    set_coords_dtype(torch.int32)
    gen = torch.Generator(device="cpu").manual_seed(77)
    allc = _rand_coords(gen, 700, 2, (32, 32, 32))
    _check_no_alias(allc)
    present, absent = allc[:500], allc[500:]
    table = HashTable(capacity=1000, device="cpu")
    table.insert(present)
    query = torch.cat([present[torch.randperm(500, generator=gen)[:300]], absent])
    out = table.query(query)
    # duplicate insert: the reference's sequential interpreter leaves the LAST row of a duplicated
    # coordinate in the table (hash.py:251 unconditional store)
    dup = torch.cat([present[:50], present[:50]])
    t2 = HashTable(capacity=300, device="cpu")
    t2.insert(dup)
    dup_out = t2.query(present[:50])
    np.savez_compressed(
        os.path.join(HERE, "hash_basic.npz"),
        insert=present.numpy(), capacity=1000, query=query.numpy(), result=out.numpy(),
        dup_insert=dup.numpy(), dup_capacity=300, dup_query=present[:50].numpy(), dup_result=dup_out.numpy(),
    )
    print("  hash_basic: hits", int((out >= 0).sum()), "misses", int((out < 0).sum()))


def _ref_conv(coords, feats, weight, bias, dy, shape, batch, k, s, p, d, transposed, subm, cdtype, algo):
    from sparsetriton import SparseTensor
    from sparsetriton.nn.functional import sparse_conv3d
    from sparsetriton.config import set_coords_dtype, set_conv_algo

    set_coords_dtype(cdtype)
    set_conv_algo(algo)
    x = feats.detach().clone().requires_grad_(True)
    w = weight.detach().clone().requires_grad_(True)
    bvec = None if bias is None else bias.detach().clone().requires_grad_(True)
    sp = SparseTensor(x, coords.to(cdtype), spatial_shape=shape, batch_size=batch)
    out = sparse_conv3d(sp, w, kernel_size=k, bias=bvec, stride=s, dilation=d, padding=p,
                        transposed=transposed, submanifold=subm)
    g = dy(out.F.shape)
    (out.F * g).sum().backward()
    return (out.C.to(torch.int32).clone(), out.F.detach().clone(), x.grad.clone(), w.grad.clone(),
            None if bvec is None else bvec.grad.clone(), g, [int(v) for v in out.spatial_shape])


def make_conv(case):
    from sparsetriton.config import ConvAlgo

    name, kname, cin, cout, has_bias = case
    kcase = [c for c in KMAP_CASES if c[0] == kname][0]
    _, n, batch, shape, k, s, p, d, transposed, subm, dt = kcase
    cdtype = getattr(torch, dt)
    coords, seed = _case_inputs(kcase)
    gen = torch.Generator(device="cpu").manual_seed(seed + 500)
    feats = torch.randn(n, cin, generator=gen)
    stdv = 1.0 / (cin * k ** 3) ** 0.5
    weight = (torch.rand(k ** 3, cin, cout, generator=gen) * 2 - 1) * stdv
    bias = (torch.rand(cout, generator=gen) * 2 - 1) * stdv if has_bias else None
    gstate = gen.get_state()

    def dy(shape_):
        g2 = torch.Generator(device="cpu")
        g2.set_state(gstate)
        return torch.randn(shape_, generator=g2)

    res = {}
    for algo in (ConvAlgo.PrecomputedNeighborGEMM, ConvAlgo.ImplicitHashFlyGEMM):
        t0 = time.time()
        if transposed and s > 1 and batch > 1:
            # per-sample run; gradients of shared weight/bias are summed over samples
            ocs, ys, dxs, gs = [], [], [], []
            dw = torch.zeros_like(weight)
            db = None if bias is None else torch.zeros_like(bias)
            # upstream gradient drawn once for the concatenated output
            sizes = []
            per = []
            for b in range(batch):
                sel = coords[:, 0] == b
                rows = coords[sel].clone()
                rows[:, 0] = 0
                per.append((rows, feats[sel]))
            # first pass to learn output sizes
            from sparsetriton.nn.functional.conv.kmap import build_out_coords
            from sparsetriton.config import set_coords_dtype
            set_coords_dtype(cdtype)
            for rows, _ in per:
                oc, _, _ = build_out_coords(rows.to(cdtype), shape, k, s, d, p, transposed=True, submanifold=False)
                sizes.append(oc.shape[0])
            gfull = dy((sum(sizes), cout))
            start = 0
            ns = None
            for b, (rows, f) in enumerate(per):
                gslice = gfull[start:start + sizes[b]]
                start += sizes[b]
                oc, y, dx, dwb, dbb, _, ns = _ref_conv(rows, f, weight, bias, lambda sh, gs_=gslice: gs_, shape, 1,
                                                       k, s, p, d, transposed, subm, cdtype, algo)
                oc[:, 0] = b
                ocs.append(oc); ys.append(y); dxs.append(dx)
                dw += dwb
                if db is not None:
                    db += dbb
            out = (torch.cat(ocs), torch.cat(ys), torch.cat(dxs), dw, db, gfull, ns)
        else:
            out = _ref_conv(coords, feats, weight, bias, dy, shape, batch, k, s, p, d, transposed, subm, cdtype, algo)
        res[algo.name] = out
        print(f"  conv {name} [{algo.name}]: N_out={out[0].shape[0]} ({time.time() - t0:.1f}s)")
    a, h = res["PrecomputedNeighborGEMM"], res["ImplicitHashFlyGEMM"]
    assert torch.equal(a[0], h[0])
    np.savez_compressed(
        os.path.join(HERE, f"{name}.npz"),
        kmap_case=kname, cin=cin, cout=cout,
        coords=coords.numpy(), shape=np.array(shape), batch=batch, k=k, s=s, p=p, d=d,
        transposed=transposed, subm=subm, coord_dtype=dt,
        feats=feats.numpy(), weight=weight.numpy(),
        bias=(np.zeros(0, np.float32) if bias is None else bias.numpy()),
        dy=a[5].numpy(), out_coords=a[0].numpy(), new_shape=np.array(a[6]),
        y=a[1].numpy(), dx=a[2].numpy(), dw=a[3].numpy(),
        db=(np.zeros(0, np.float32) if a[4] is None else a[4].numpy()),
        y_hashfly=h[1].numpy(), dx_hashfly=h[2].numpy(), dw_hashfly=h[3].numpy(),
    )


def make_c1():
    """The reference's CPU-runnable headline case: SubMConv3D 16->32, k3, B=2, 64^3, N=4096,
    loss = sum of outputs; PrecomputedNeighborGEMM only (the hash-fly run takes ~17 min here)."""
    from sparsetriton import SparseTensor
    from sparsetriton.nn.modules import SubMConv3D
    from sparsetriton.config import set_coords_dtype, set_conv_algo, ConvAlgo

    set_coords_dtype(torch.int32)
    set_conv_algo(ConvAlgo.PrecomputedNeighborGEMM)
    gen = torch.Generator(device="cpu").manual_seed(1234)
    flat = torch.randperm(2 * 64 ** 3, generator=gen)[:4096]
    coords = torch.stack([flat // 64 ** 3, (flat // 4096) % 64, (flat // 64) % 64, flat % 64], 1).to(torch.int32)
    # 4096 coordinates do contain pairs with equal 31-bit keys (hash.py:136-152); whether one of
    # them ever meets the other on a probe path is checked after the run, against the exact map.
    feats = torch.randn(4096, 16, generator=gen)
    stdv = 1.0 / (16 * 27) ** 0.5
    weight = (torch.rand(27, 16, 32, generator=gen) * 2 - 1) * stdv
    conv = SubMConv3D(16, 32, 3, bias=False)
    with torch.no_grad():
        conv.weight.copy_(weight)
    x = feats.clone().requires_grad_(True)
    sp = SparseTensor(x, coords, spatial_shape=(64, 64, 64), batch_size=2)
    t0 = time.time()
    out = conv(sp)
    t1 = time.time()
    out.F.sum().backward()
    t2 = time.time()
    key = list(sp._cache.neighbor_indices.keys())[0]
    nbr = sp._cache.neighbor_indices[key][1]
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle import cpu_oracle
    exact = cpu_oracle.kernel_map(coords.numpy(), (64, 64, 64), 3, 1, 1, 1, False, True)[3]
    n_diff = int((exact != nbr.numpy()).sum())
    print(f"  c1: fwd {t1 - t0:.1f}s bwd {t2 - t1:.1f}s pairs={int((nbr >= 0).sum())} "
          f"map entries differing from the exact map (31-bit key aliasing): {n_diff}")
    np.savez_compressed(
        os.path.join(HERE, "c1_subm_16_32.npz"),
        coords=coords.numpy(), feats=feats.numpy(), weight=weight.numpy(), nbr=nbr.numpy(),
        y=out.F.detach().numpy(), dx=x.grad.numpy(), dw=conv.weight.grad.numpy(),
        ref_fwd_seconds=t1 - t0, ref_bwd_seconds=t2 - t1, ref_threads=torch.get_num_threads(),
        ref_map_entries_differing_from_exact=n_diff,
    )


def make_dense():
    """to_dense on a batch-2 tensor: dense volume and the gradient that comes back for a random upstream."""
    from sparsetriton.utils.to_dense import to_dense
    from sparsetriton.config import set_coords_dtype

    set_coords_dtype(torch.int32)
    gen = torch.Generator(device="cpu").manual_seed(4242)
    shape = (6, 5, 7)
    coords = _rand_coords(gen, 90, 2, shape)
    feats = torch.randn(90, 5, generator=gen, requires_grad=True)
    dense = to_dense(feats, coords, shape)
    g = torch.randn(dense.shape, generator=gen)
    (dense * g).sum().backward()
    np.savez_compressed(os.path.join(HERE, "dense_b2_c5.npz"), coords=coords.numpy(), shape=np.array(shape),
                        feats=feats.detach().numpy(), dense=dense.detach().numpy(), upstream=g.numpy(),
                        grad_feats=feats.grad.numpy())
    print("  dense_b2_c5:", tuple(dense.shape))


POOL_CASES = [
    # name, N, batch, shape, kernel, padding, stride, channels
    ("pool_avg_k2s2", 160, 2, (8, 8, 8), 2, 1, 2, 6),
    ("pool_avg_k3s2p1", 200, 2, (9, 7, 8), 3, 1, 2, 4),
    ("pool_avg_k4s4", 150, 1, (12, 12, 12), 4, 2, 4, 3),
]


def make_pool(case):
    """sparse_pooling(mode="avg"): output coordinates (sorted cells), features, gradient.  Paddings are chosen
    so that no cell index is negative (the reference's 16-bit packing aliases negative cells).  mode="max"
    is tried and its failure recorded: the reference's own test skips it for a known compile issue."""
    from sparsetriton import SparseTensor
    from sparsetriton.nn.functional import sparse_pooling
    from sparsetriton.config import set_coords_dtype

    name, n, batch, shape, k, p, s, ch = case
    set_coords_dtype(torch.int32)
    gen = torch.Generator(device="cpu").manual_seed(600 + [c[0] for c in POOL_CASES].index(name))
    coords = _rand_coords(gen, n, batch, shape)
    feats = torch.randn(n, ch, generator=gen, requires_grad=True)
    sp = SparseTensor(feats, coords, spatial_shape=shape, batch_size=batch)
    out = sparse_pooling(sp, kernel_size=k, padding=p, stride=s, mode="avg")
    g = torch.randn(out.F.shape, generator=gen)
    (out.F * g).sum().backward()
    try:
        sparse_pooling(SparseTensor(feats.detach(), coords, spatial_shape=shape, batch_size=batch), kernel_size=k,
                       padding=p, stride=s, mode="max")
        max_note = "ran"
    except Exception as e:  # noqa: BLE001 - recorded, not handled
        max_note = type(e).__name__
    np.savez_compressed(os.path.join(HERE, f"{name}.npz"), coords=coords.numpy(), shape=np.array(shape), batch=batch,
                        k=k, p=p, s=s, feats=feats.detach().numpy(), out_coords=out.C.to(torch.int32).numpy(),
                        new_shape=np.array([int(v) for v in out.spatial_shape]), y=out.F.detach().numpy(),
                        upstream=g.numpy(), grad_feats=feats.grad.numpy(), reference_max_mode=max_note)
    print(f"  {name}: N_out={out.F.shape[0]} new_shape={tuple(out.spatial_shape)} max mode: {max_note}")


def make_upsample(scale):
    from sparsetriton import SparseTensor
    from sparsetriton.nn.functional import sparse_upsample
    from sparsetriton.config import set_coords_dtype

    set_coords_dtype(torch.int32)
    gen = torch.Generator(device="cpu").manual_seed(700 + scale)
    shape = (5, 6, 4)
    coords = _rand_coords(gen, 70, 2, shape)
    feats = torch.randn(70, 5, generator=gen, requires_grad=True)
    sp = SparseTensor(feats, coords, spatial_shape=shape, batch_size=2)
    out = sparse_upsample(sp, scale_factor=scale)
    g = torch.randn(out.F.shape, generator=gen)
    (out.F * g).sum().backward()
    np.savez_compressed(os.path.join(HERE, f"upsample_s{scale}.npz"), coords=coords.numpy(), shape=np.array(shape),
                        scale=scale, feats=feats.detach().numpy(), out_coords=out.C.to(torch.int32).numpy(),
                        new_shape=np.array([int(v) for v in out.spatial_shape]), y=out.F.detach().numpy(),
                        upstream=g.numpy(), grad_feats=feats.grad.numpy())
    print(f"  upsample_s{scale}: N_out={out.F.shape[0]}")


def make_bn():
    """sparse_batch_norm (plain torch in the reference): training forward + backward with the running buffers
    it leaves behind, and the inference form on the updated buffers."""
    from sparsetriton import SparseTensor
    from sparsetriton.nn.functional import sparse_batch_norm
    from sparsetriton.config import set_coords_dtype

    set_coords_dtype(torch.int32)
    gen = torch.Generator(device="cpu").manual_seed(808)
    shape = (8, 8, 8)
    coords = _rand_coords(gen, 300, 3, shape)
    coords = coords[coords[:, 0] != 1]                  # sample 1 is empty: its count clamps to 1
    n, ch = coords.shape[0], 6
    feats = (torch.randn(n, ch, generator=gen) * 2.0 + 0.7).requires_grad_(True)
    weight = (torch.rand(ch, generator=gen) + 0.5).requires_grad_(True)
    bias = torch.randn(ch, generator=gen).requires_grad_(True)
    rm, rv = torch.zeros(ch), torch.ones(ch)
    sp = SparseTensor(feats, coords, spatial_shape=shape, batch_size=3)
    out = sparse_batch_norm(sp, weight=weight, bias=bias, running_mean=rm, running_var=rv, training=True, eps=1e-5,
                            momentum=0.1)
    g = torch.randn(out.F.shape, generator=gen)
    (out.F * g).sum().backward()
    with torch.no_grad():
        ev = sparse_batch_norm(SparseTensor(feats.detach(), coords, spatial_shape=shape, batch_size=3), weight=weight,
                               bias=bias, running_mean=rm.detach().clone(), running_var=rv.detach().clone(), training=False, eps=1e-5)
    np.savez_compressed(os.path.join(HERE, "bn_b3_c6.npz"), coords=coords.numpy(), shape=np.array(shape), batch=3,
                        feats=feats.detach().numpy(), weight=weight.detach().numpy(), bias=bias.detach().numpy(),
                        eps=1e-5, momentum=0.1, y_train=out.F.detach().numpy(), upstream=g.numpy(),
                        grad_feats=feats.grad.numpy(), grad_weight=weight.grad.numpy(), grad_bias=bias.grad.numpy(),
                        running_mean=rm.detach().numpy(), running_var=rv.detach().numpy(), y_eval=ev.F.detach().numpy())
    print("  bn_b3_c6: rows", n)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="checkout of the unmodified reference (the directory that holds sparsetriton/)")
    ap.add_argument("--only", default=None, help="substring filter on fixture names")
    ap.add_argument("--c1", action="store_true", help="also run the 4096-voxel headline case (minutes)")
    args = ap.parse_args()
    _install_autotune_shim()
    sys.path.insert(0, args.ref)
    import sparsetriton  # noqa: F401  (the reference)

    assert os.path.realpath(os.path.dirname(sparsetriton.__file__)).startswith(os.path.realpath(args.ref))

    def want(n):
        return args.only is None or args.only in n

    if want("hash"):
        make_hash()
    for case in KMAP_CASES:
        if want("kmap_" + case[0]):
            make_kmap(case)
    for case in CONV_CASES:
        if want(case[0]):
            make_conv(case)
    if want("dense"):
        make_dense()
    for case in POOL_CASES:
        if want(case[0]):
            make_pool(case)
    for scale in (2, 3):
        if want(f"upsample_s{scale}"):
            make_upsample(scale)
    if want("bn"):
        make_bn()
    if args.c1:
        make_c1()


if __name__ == "__main__":
    main()
