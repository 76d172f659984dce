"""Benchmark of the sparse-convolution hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Other workloads: `hash_map_c2` (hash table + kernel-map microbenchmark, 2M or 8M random cells in a
2048^3 grid), `unet_infer` / `unet_train` (the lidar-like sparse U-Net, batch 8 / 16 sharded by sample
over the ranks; training all-reduces one flat gradient bucket over NCCL and applies SGD with momentum).

Workload (default `conv_layer_c3`): one SparseConv3D downsample layer, batch 4, grid 512^3,
300 000 surface voxels per sample, 64 -> 128 channels, kernel 3, stride 2, padding 1, bf16,
PrecomputedNeighborGEMM.  One step is one pass of the whole hot path over one batch:

    hash build -> output coordinates -> neighbour map -> forward -> dgrad -> wgrad

`value` is input voxels per second with inputs resident in HBM; `e2e` is the same step through the
public Python API starting from pinned HOST buffers (coordinates, features, upstream gradient are
copied host->device and Y, dX, dW device->host inside the timed region).  With N > 1 every rank
runs its own batch of the same shape (weak scaling) and the weight gradient is all-reduced over
NCCL inside the step.  Inputs are synthetic (seeded procedural surfaces) and larger than L2.

`--impl reference` times the CPU restatement of the reference's algorithm (the oracle port; the
reference itself is Triton code that only runs on CPU through the Triton interpreter, at minutes per
4k voxels) on the host cores, one sample of the same workload per step.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CIN, COUT, KS, STRIDE, PAD, GRID, BATCH, PER_SAMPLE = 64, 128, 3, 2, 1, 512, 4, 300_000


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def make_batch(rank, batch=BATCH, per_sample=PER_SAMPLE, grid=GRID):
    """(N,4) int32 CPU coordinates of `batch` surface scenes; seeds 3000 + rank*batch + sample."""
    from sparsetriton_b200 import synthetic
    scenes = [synthetic.surface_scene(3000 + rank * batch + b, grid=grid, target=per_sample) for b in range(batch)]
    return synthetic.batch_of(scenes, dtype=torch.int32)


class ClockSampler:
    """Polls nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm = [float(r[1]) for r in self.rows if len(r) >= 7 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 7 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 7 and r[3 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ ours
def run_ours(args):
    import torch.distributed as dist
    import sparsetriton_b200 as st
    from sparsetriton_b200 import trace
    from sparsetriton_b200.config import ConvAlgo, set_conv_algo, set_coords_dtype, set_h_table_f
    from sparsetriton_b200.nn.functional import sparse_conv3d

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    set_coords_dtype(torch.int32)
    set_h_table_f(2.0)
    algo = ConvAlgo.ImplicitHashFlyGEMM if args.algo == "hashfly" else ConvAlgo.PrecomputedNeighborGEMM
    set_conv_algo(algo)
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]

    coords_h = make_batch(rank, args.batch, args.per_sample, args.grid).pin_memory()
    n_in = coords_h.shape[0]
    gen = torch.Generator(device="cpu").manual_seed(9000 + rank)
    feats_h = torch.randn(n_in, CIN, generator=gen).to(dtype).pin_memory()
    bound = 1.0 / (CIN * KS ** 3) ** 0.5
    weight = ((torch.rand(KS ** 3, CIN, COUT, generator=torch.Generator().manual_seed(7)) * 2 - 1) * bound).to(dtype).to(dev)
    shape = (args.grid,) * 3

    def step(coords, feats, dy, w):
        """One pass of the hot path; returns (y, dx, dw, out_tensor)."""
        x = feats.detach().requires_grad_(True)
        wp = w.detach().requires_grad_(True)
        sp = st.SparseTensor._trusted(x, coords, shape, args.batch)
        out = sparse_conv3d(sp, wp, kernel_size=KS, stride=STRIDE, padding=PAD, submanifold=False)
        g = dy if dy is not None else torch.ones_like(out.F)
        dx, dw = torch.autograd.grad(out.F, [x, wp], g)
        if world > 1:
            dist.all_reduce(dw)
        return out.F, dx, dw, out

    coords_d, feats_d = coords_h.to(dev), feats_h.to(dev)
    # first pass: learn N_out and the pair count, prepare the upstream gradient
    y0, _, _, out0 = step(coords_d, feats_d, None, weight)
    n_out = y0.shape[0]
    dy_h = torch.randn(n_out, COUT, generator=gen).to(dtype).pin_memory()
    dy_d = dy_h.to(dev)
    # pair count of the map (for the flop figures): one probe pass with the stored-map algorithm
    set_conv_algo(ConvAlgo.PrecomputedNeighborGEMM)
    sp_probe = st.SparseTensor._trusted(feats_d, coords_d, shape, args.batch)
    sparse_conv3d(sp_probe, weight, kernel_size=KS, stride=STRIDE, padding=PAD, submanifold=False)
    pairs = int((sp_probe._cache.neighbor_indices[(KS, STRIDE, PAD, 1, False, False)][1] >= 0).sum().item())
    del sp_probe
    set_conv_algo(algo)
    del y0, out0

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step(coords_d, feats_d, dy_d, weight)
    sync_all()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    ev0.record()
    for _ in range(args.steps):
        step(coords_d, feats_d, dy_d, weight)
    ev1.record()
    sync_all()
    dev_ms = ev0.elapsed_time(ev1)
    # the per-stage breakdown and the launch count come from a second pass over the same steps with the
    # stage recorder on (its event pairs cost host time, so it stays out of the timed pass)
    with trace.recording() as rec:
        for _ in range(args.steps):
            step(coords_d, feats_d, dy_d, weight)
        sync_all()
        stages = rec.summary()
        launches = rec.total_launches()

    # end to end: host buffers in, host results out, through the same public API
    y_h = torch.empty((n_out, COUT), dtype=dtype).pin_memory()
    dx_h = torch.empty((n_in, CIN), dtype=dtype).pin_memory()
    dw_h = torch.empty((KS ** 3, CIN, COUT), dtype=dtype).pin_memory()

    # Three streams: the copy of step i+1's inputs (pinned host -> device, double-buffered) and the read-back
    # of step i-1's results run beside step i's kernels.  Every step still moves all of its inputs and results.
    s_comp = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    in_bufs = [(torch.empty_like(coords_d), torch.empty_like(feats_d), torch.empty_like(dy_d)) for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]

    def upload(i):
        b = i % 2
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_free[b])                 # step i-2 has finished reading this buffer
            for dst, src in zip(in_bufs[b], (coords_h, feats_h, dy_h)):
                dst.copy_(src, non_blocking=True)
            ev_in[b].record(s_in)

    def e2e_run(n_steps):
        upload(0)
        for i in range(n_steps):
            b = i % 2
            if i + 1 < n_steps:
                upload(i + 1)
            s_comp.wait_event(ev_in[b])
            c, f, g = in_bufs[b]
            y, dx, dw, _ = step(c, f, g, weight)
            ev_free[b].record(s_comp)
            done = torch.cuda.Event()
            done.record(s_comp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                y_h.copy_(y, non_blocking=True)
                dx_h.copy_(dx, non_blocking=True)
                dw_h.copy_(dw, non_blocking=True)
            for t in (y, dx, dw):
                t.record_stream(s_out)
        s_comp.wait_stream(s_out)

    e2e_run(max(2, args.warmup // 2))
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_run(args.steps)
    e1.record()
    sync_all()
    e2e_ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None

    times = torch.tensor([dev_ms, e2e_ms, float(n_in)], dtype=torch.float64, device=dev)
    if world > 1:
        tmax = times.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = times.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        dev_ms, e2e_ms, total_voxels = tmax[0].item(), tmax[1].item(), tsum[2].item()
    else:
        total_voxels = float(n_in)

    if rank == 0:
        pk = peaks()
        ms_per_step = dev_ms / args.steps
        value = total_voxels / (ms_per_step * 1e-3)
        per_stage = {k: {"ms_per_step": v["ms"] / args.steps, "launches_per_step": v["launches"] / args.steps}
                     for k, v in stages.items()}
        roof = roofline(per_stage, n_in, n_out, pairs, pk, dtype)
        if roof is not None:
            roof["traffic"], roof["traffic_source"] = ncu_traffic(roof["kernel"], args, algo, n_in)
        h2d = coords_h.numel() * 4 + feats_h.numel() * feats_h.element_size() + dy_h.numel() * dy_h.element_size()
        d2h = (y_h.numel() + dx_h.numel() + dw_h.numel()) * y_h.element_size()
        line = {
            "metric": "sparse_conv_layer_fwd_bwd_voxels_per_s", "value": value, "unit": "voxels/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": args.dtype, "data": "synthetic",
            "config": {"workload": "conv_layer_c3: SparseConv3D 64->128 k3 s2 p1, batch %d x %d voxels, grid %d^3, "
                                   "hash+outcoords+map+fwd+dgrad+wgrad per step" % (args.batch, args.per_sample, args.grid),
                       "algo": algo.value, "n_in_per_gpu": n_in, "n_out_per_gpu": n_out, "pairs_per_gpu": pairs,
                       "l2_policy": "inputs larger than L2 (features+map+outputs > 400 MB per step)",
                       "parallelism": "dp%d by sample, NCCL all-reduce of dW" % world},
            "e2e": {"value": total_voxels / (e2e_ms / args.steps * 1e-3), "unit": "voxels/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": launches,
            "stages": per_stage,
            "roofline": roof,
            "clocks": clocks,
        }
        if pairs:
            gemm_ms = sum(per_stage.get(s, {}).get("ms_per_step", 0.0) for s in ("conv_fwd", "conv_dgrad", "conv_wgrad"))
            line["gemm_tflops"] = 3 * 2.0 * pairs * CIN * COUT / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_leg(args, seconds_budget=20.0)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of the dominant kernels, from the ncu
# captures summarised under profiles/ (default workload: 4 x 300 k voxels, bf16, stored-map algorithm).
NCU_TRAFFIC_C3 = {
    "conv_fwd": (466.4e6 + 187.8e6, "profiles/planned_gather_kernel_c3.md"),
    "conv_dgrad": (820.9e6 + 143.0e6, "profiles/planned_gather_kernel_c3.md"),
    "conv_wgrad": (899.5e6 + 43.6e6, "profiles/planned_wgrad_kernel_c3.md"),
}


def ncu_traffic(kernel, args, algo, n_in):
    """Measured DRAM traffic per launch when this run is the configuration the capture was taken on, scaled
    by the voxel count of this rank otherwise (traffic of these kernels grows with the rows); None where no
    capture exists."""
    from sparsetriton_b200.config import ConvAlgo
    if kernel not in NCU_TRAFFIC_C3 or algo != ConvAlgo.PrecomputedNeighborGEMM or args.dtype == "fp32":
        return None, None
    nbytes, src = NCU_TRAFFIC_C3[kernel]
    return nbytes * n_in / 1.2e6, src


def roofline(per_stage, n_in, n_out, pairs, pk, dtype):
    """Roofline entry of the stage that takes the largest share of the step.

    Algorithmic work per launch:
      conv_*      2 * pairs * Cin * Cout flop against the bf16 GEMM peak, and
                  (gathered rows + streamed rows + weights) * element size + map rows * 4 K bytes against the
                  copy bandwidth: the ceiling that takes longer is reported as the bound
      map_build   N_out * (16 + 12 K) + 4 * pairs bytes             (coords + key probe + map write + value)
      map_plan    8 K rows bytes (read the map, write its plan); the inverse plan also reads the forward map
      out_coords  N * (16 + 12 c) + 16 N_out bytes, c = 27/8        (candidates inserted + coords written)
      hash_build  52 N bytes at capacity 2N
    """
    K = KS ** 3
    if not per_stage:
        return None
    top = max(per_stage, key=lambda k: per_stage[k]["ms_per_step"])
    ms = per_stage[top]["ms_per_step"]
    total = sum(v["ms_per_step"] for v in per_stage.values())
    entry = {"kernel": top, "share_of_step": ms / total if total else None, "traffic": None}
    if top.startswith("conv_") and pairs:
        # Both ceilings of the product; the one that takes longer at its measured peak is the bound.
        flops = 2.0 * pairs * CIN * COUT
        es = 4 if dtype == torch.float32 else 2
        kind = top.replace("_hashfly", "")
        gathered = {"conv_fwd": pairs * CIN, "conv_dgrad": pairs * COUT, "conv_wgrad": pairs * CIN}[kind]
        streamed = {"conv_fwd": n_out * COUT, "conv_dgrad": n_in * CIN, "conv_wgrad": n_out * COUT}[kind]
        map_rows = n_in if kind == "conv_dgrad" else n_out
        nbytes = (gathered + streamed + K * CIN * COUT) * es + map_rows * K * 4
        tc_peak = pk["bf16_tflops"] * (0.5 if dtype == torch.float32 else 1.0)
        t_tc = flops / (tc_peak * 1e12)
        t_hbm = nbytes / (pk["hbm_gbs"] * 1e9)
        if t_hbm >= t_tc:
            ach = nbytes / (ms * 1e-3) / 1e9
            entry.update({"bound": "hbm", "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s",
                          "frac": ach / pk["hbm_gbs"], "peak_source": pk["source"],
                          "algorithmic_bytes_per_launch": nbytes, "algorithmic_flops_per_launch": flops,
                          "tensor_frac": flops / (ms * 1e-3) / 1e12 / tc_peak})
        else:
            ach = flops / (ms * 1e-3) / 1e12
            entry.update({"bound": "tensor", "achieved": ach, "peak": tc_peak, "unit": "TFLOP/s", "frac": ach / tc_peak,
                          "peak_source": pk["source"], "algorithmic_flops_per_launch": flops,
                          "algorithmic_bytes_per_launch": nbytes})
    else:
        if top == "map_build":
            nbytes = n_out * (16 + 12 * K) + 4 * (pairs or 0)
        elif top in ("map_plan", "map_plan_inverse"):
            nbytes = 8 * K * (n_out if top == "map_plan" else n_in) + (4 * K * n_out if top == "map_plan_inverse" else 0)
        elif top == "map_scatter":
            nbytes = 4 * (pairs or 0) + 4 * n_out * K
        elif top == "out_coords":
            nbytes = n_in * (16 + 12 * K / 8.0) + 16 * n_out
        else:
            nbytes = 52 * n_in
        ach = nbytes / (ms * 1e-3) / 1e9
        entry.update({"bound": "hbm", "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": ach / pk["hbm_gbs"],
                      "peak_source": pk["source"], "algorithmic_bytes_per_launch": nbytes})
    return entry


# ------------------------------------------------------------------------------------ CPU baseline
def cpu_step(O, coords, feats, weight, dy_seed):
    """The same step on the host through the oracle port; returns (seconds, n_in, n_out)."""
    t0 = time.perf_counter()
    oc, ns, off, nbr = O.kernel_map(coords, (GRID,) * 3, KS, STRIDE, 1, PAD, False, False)
    y = O.conv_fwd(feats, weight, nbr)
    dy = np.full_like(y, 1.0) if dy_seed is None else dy_seed(y.shape)
    O.conv_dgrad(dy, weight, nbr, feats.shape[0])
    O.conv_wgrad(feats, dy, nbr, KS ** 3, CIN, COUT)
    return time.perf_counter() - t0, coords.shape[0], oc.shape[0]


def cpu_inputs(per_sample, grid):
    from sparsetriton_b200 import synthetic
    coords = synthetic.batch_of([synthetic.surface_scene(3000, grid=grid, target=per_sample)]).numpy()
    rng = np.random.default_rng(9000)
    feats = rng.standard_normal((coords.shape[0], CIN), dtype=np.float32)
    weight = ((rng.random((KS ** 3, CIN, COUT), dtype=np.float32) * 2 - 1) / (CIN * KS ** 3) ** 0.5).astype(np.float32)
    return coords, feats, weight


def cpu_baseline_leg(args, seconds_budget):
    from oracle import cpu_oracle as O
    O.build()
    O.set_threads(os.cpu_count() or 1)            # launchers such as torchrun export OMP_NUM_THREADS=1
    coords, feats, weight = cpu_inputs(args.per_sample, args.grid)
    secs, n_in, n_out = cpu_step(O, coords, feats, weight, None)
    reps = 1
    while secs * (reps + 1) < seconds_budget and reps < 3:
        s2, _, _ = cpu_step(O, coords, feats, weight, None)
        secs = min(secs, s2)
        reps += 1
    return {"value": n_in / secs, "unit": "voxels/s", "cores": O.num_threads(), "kind": "port",
            "sample": "1 of the %d samples of the batch (%d voxels), same layer and step, fp32, best of %d" %
                      (args.batch, n_in, reps),
            "seconds_per_sample_step": secs}


def run_reference(args):
    """CPU arm: the oracle port (C + OpenMP restatement of the reference's algorithm) on all host
    threads; each step processes one sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import cpu_oracle as O
    O.build()
    O.set_threads(os.cpu_count() or 1)            # launchers such as torchrun export OMP_NUM_THREADS=1
    coords, feats, weight = cpu_inputs(args.per_sample, args.grid)
    for _ in range(min(args.warmup, 1)):
        cpu_step(O, coords, feats, weight, None)
    steps = min(args.steps, 5)
    t = 0.0
    for _ in range(steps):
        s, n_in, n_out = cpu_step(O, coords, feats, weight, None)
        t += s
    value = n_in * steps / t
    sample = "each step = 1 of the %d samples of the batch (%d voxels); %d steps timed" % (args.batch, n_in, steps)
    print(json.dumps({
        "impl": "reference", "metric": "sparse_conv_layer_fwd_bwd_voxels_per_s", "value": value, "unit": "voxels/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": t / steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "conv_layer_c3 on host cores (oracle port of the reference's algorithm; the reference's "
                               "own Triton-interpreter CPU path needs minutes per 4k voxels)", "sample": sample},
        "cpu_baseline": {"value": value, "unit": "voxels/s", "cores": O.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "voxels/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# --------------------------------------------------------------------------------- other workloads
def _dist_setup(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    return dist, world, rank, local, dev


def run_hash_map(args):
    """BASELINE config 2: table build at load factor 0.5, submanifold maps for k3 (27) and k5 (125),
    a k3 s2 p1 downsample (output coordinates + map) and the transposed map from its output."""
    from sparsetriton_b200 import synthetic, trace
    from sparsetriton_b200.config import set_coords_dtype
    from sparsetriton_b200.nn.functional.conv.conv import compute_neighbor_indices
    from sparsetriton_b200.nn.functional.conv.kmap import build_out_coords, out_coords_and_map
    from sparsetriton_b200.utils.hash import HashTable

    dist, world, rank, local, dev = _dist_setup(args)
    set_coords_dtype(torch.int32)
    n, grid = args.cells, 2048
    coords = synthetic.random_cells(n, 4, grid, seed=2001 + rank).to(dev)
    shape = (grid,) * 3
    cap = 1 << (2 * n - 1).bit_length()

    def step():
        t = HashTable(cap, device=dev)
        t.insert(coords)
        res = {}
        for k in (3, 5):
            _, _, ko = build_out_coords(coords, shape, k, 1, 1, (k - 1) // 2, submanifold=True)
            with trace.stage(f"subm_map_k{k}"):
                res[k] = compute_neighbor_indices(t, coords, ko, shape, 1, queries_are_table_rows=True)
        oc, ns, ko, nbr = out_coords_and_map(coords, shape, 3, 2, 1, 1, False)
        oc2, ns2, ko2, nbr2 = out_coords_and_map(oc, ns, 3, 2, 1, 1, True)
        return res, nbr, nbr2, oc, oc2

    res, nbr, nbr2, oc, oc2 = step()
    def count_pairs(m, rows=1 << 22):
        """Valid entries of a map, a few million rows at a time (the transposed map has > 3e9 entries)."""
        return sum(int((m[i:i + rows] >= 0).sum()) for i in range(0, m.shape[0], rows))

    pairs = {"k3": count_pairs(res[3]), "k5": count_pairs(res[5]), "down": count_pairs(nbr), "up": count_pairs(nbr2)}
    n_down, n_up = oc.shape[0], oc2.shape[0]
    del res, nbr, nbr2, oc, oc2
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with trace.recording() as rec:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        stages = rec.summary()
        launches = rec.total_launches()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        pk = peaks()
        per = {k: v["ms"] / args.steps for k, v in stages.items()}
        # algorithmic bytes (coords 16 B, one 8 B key probe + 4 B map entry per (voxel, offset), 4 B value per hit)
        algo = {
            "hash_build": 52.0 * n,
            "subm_map_k3": n * (16 + 12 * 27) + 4.0 * pairs["k3"],
            "subm_map_k5": n * (16 + 12 * 125) + 4.0 * pairs["k5"],
        }
        roof = {}
        for name, nbytes in algo.items():
            if name in per and per[name] > 0:
                gbs = nbytes / (per[name] * 1e-3) / 1e9
                roof[name] = {"ms": per[name], "algorithmic_bytes": nbytes, "achieved_gbs": gbs, "frac": gbs / pk["hbm_gbs"]}
        top = max(roof, key=lambda k: roof[k]["ms"])
        ms_step = t.item() / args.steps
        print(json.dumps({
            "metric": "hash_and_kernel_map_voxels_per_s", "value": world * n / (ms_step * 1e-3), "unit": "voxels/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int64 keys / int32 coords",
            "data": "synthetic",
            "config": {"workload": "hash_map_c2: %d random cells, batch 4, grid 2048^3, table capacity %d; build + subm k3 + "
                                   "subm k5 + k3s2p1 down (coords+map) + transposed map" % (n, cap),
                       "pairs": pairs, "n_out_down": n_down, "n_out_up": n_up, "l2_policy": "tables and maps larger than L2"},
            "gpu_launches": launches, "stages": per, "stage_rooflines": roof,
            "roofline": {"kernel": top, "bound": "hbm", "achieved": roof[top]["achieved_gbs"], "peak": pk["hbm_gbs"],
                         "unit": "GB/s", "frac": roof[top]["frac"], "traffic": None, "peak_source": pk["source"]},
            "clocks": clocks,
        }))
    if world > 1:
        dist.destroy_process_group()


def make_lidar_batch(samples):
    """(coords (N,4) int32 with batch relabelled from 0, feats (N,4) fp32) of the given scene seeds."""
    from sparsetriton_b200 import synthetic
    scenes = [synthetic.lidar_scene(seed) for seed in samples]
    coords = synthetic.batch_of(scenes, dtype=torch.int32)
    g = torch.Generator().manual_seed(samples[0] + 17)
    xyz = coords[:, 1:].float() / torch.tensor([1440.0, 1440.0, 41.0])
    feats = torch.cat([xyz, torch.rand(coords.shape[0], 1, generator=g)], dim=1)
    return coords, feats


def run_unet(args, train):
    """BASELINE configs 4 / 5: lidar-like sparse U-Net, bf16 features, fp32 master weights."""
    from sparsetriton_b200 import trace
    from sparsetriton_b200.config import ConvAlgo, set_conv_algo, set_coords_dtype, set_h_table_f
    from sparsetriton_b200.distributed import GradientBucket, global_mean_scale, shard_samples
    from sparsetriton_b200.tensor import SparseTensor
    from sparsetriton_b200.unet import SparseUNet

    dist, world, rank, local, dev = _dist_setup(args)
    set_coords_dtype(torch.int32)
    set_h_table_f(2.0)
    set_conv_algo(ConvAlgo.ImplicitHashFlyGEMM if args.algo == "hashfly" else ConvAlgo.PrecomputedNeighborGEMM)
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    total_batch = 16 if train else 8
    base_seed = 5000 if train else 4000
    mine = shard_samples(total_batch, rank, world)
    coords_h, feats_h = make_lidar_batch([base_seed + i for i in mine])
    coords_h, feats_h = coords_h.pin_memory(), feats_h.to(dtype).pin_memory()
    shape = (1440, 1440, 41)
    torch.manual_seed(5100 if train else 4100)
    model = SparseUNet().to(dev)
    model.train(train)
    n_in = coords_h.shape[0]
    opt = bucket = None
    if train:
        bucket = GradientBucket(model.parameters())
        opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)

    state = {"labels": None, "scale": None, "n_out": None}

    def step(coords, feats):
        x = SparseTensor._trusted(feats, coords, shape, len(mine))
        if not train:
            with torch.no_grad():
                out = model(x)
            return out.F
        out = model(x)
        if state["labels"] is None:
            g = torch.Generator().manual_seed(base_seed + 99 + rank)
            state["labels"] = torch.randint(0, 20, (out.F.shape[0],), generator=g).to(dev)
            state["scale"] = global_mean_scale(out.F.shape[0], dev)
            state["n_out"] = out.F.shape[0]
        # per-row losses summed by a parallel reduction: torch's fused "sum" reduction of nll_loss runs in one block
        loss = torch.nn.functional.cross_entropy(out.F.float(), state["labels"], reduction="none").sum() * state["scale"]
        bucket.zero()
        loss.backward()
        bucket.all_reduce()
        opt.step()
        return loss.detach()

    coords_d, feats_d = coords_h.to(dev), feats_h.to(dev)
    for _ in range(args.warmup):
        step(coords_d, feats_d)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sync_all()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    for _ in range(args.steps):
        step(coords_d, feats_d)
    e1.record()
    sync_all()
    dev_ms = e0.elapsed_time(e1)
    # stage breakdown and launch count: a second pass with the stage recorder on (kept out of the timed pass)
    with trace.recording() as rec:
        for _ in range(args.steps):
            step(coords_d, feats_d)
        sync_all()
        stages = rec.summary()
        launches = rec.total_launches()

    result_h = torch.zeros(1, dtype=torch.float32).pin_memory()

    def e2e_step():
        c = coords_h.to(dev, non_blocking=True)
        f = feats_h.to(dev, non_blocking=True)
        r = step(c, f)
        result_h.copy_(r.float().sum().reshape(1), non_blocking=True)

    for _ in range(2):
        e2e_step()
    sync_all()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        e2e_step()
    f1.record()
    sync_all()
    e2e_ms = f0.elapsed_time(f1)
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([dev_ms, e2e_ms, float(n_in)], dtype=torch.float64, device=dev)
    if world > 1:
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = t.clone()
        dist.all_reduce(tsum)
        dev_ms, e2e_ms, total_voxels = tmax[0].item(), tmax[1].item(), tsum[2].item()
    else:
        total_voxels = float(n_in)
    if rank == 0:
        pk = peaks()
        ms_step = dev_ms / args.steps
        per = {k: {"ms_per_step": v["ms"] / args.steps, "launches_per_step": v["launches"] / args.steps,
                   "calls_per_step": v["calls"] / args.steps,
                   "tflops": (v["work"] / (v["ms"] * 1e-3) / 1e12) if v["work"] and v["ms"] > 0 else None}
               for k, v in stages.items()}
        conv = [k for k in per if k.startswith("conv_")]
        top = max(conv, key=lambda k: per[k]["ms_per_step"]) if conv else None
        roof = None
        if top and per[top]["tflops"]:
            peak = pk["bf16_tflops_sustained"] * (0.5 if dtype == torch.float32 else 1.0)
            roof = {"kernel": top + " (all layers)", "bound": "tensor", "achieved": per[top]["tflops"], "peak": peak,
                    "unit": "TFLOP/s", "frac": per[top]["tflops"] / peak, "traffic": None, "peak_source": pk["source"],
                    "share_of_step": per[top]["ms_per_step"] / ms_step}
        print(json.dumps({
            "metric": "sparse_unet_%s_voxels_per_s" % ("train_step" if train else "inference"),
            "value": total_voxels / (ms_step * 1e-3), "unit": "voxels/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "config": {"workload": "%s: lidar-like U-Net 4->32/64/128/256->...->32->20, grid 1440x1440x41, batch %d "
                                   "(%d samples on this rank, %d voxels)" % (args.workload, total_batch, len(mine), n_in),
                       "algo": args.algo, "parallelism": "dp%d by sample%s" % (world, ", NCCL all-reduce of one flat gradient bucket" if train else ""),
                       "l2_policy": "activations of every level exceed L2"},
            "e2e": {"value": total_voxels / (e2e_ms / args.steps * 1e-3), "unit": "voxels/s",
                    "h2d_bytes_per_step": coords_h.numel() * 4 + feats_h.numel() * feats_h.element_size(),
                    "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": launches, "stages": per, "roofline": roof, "clocks": clocks,
        }))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--algo", default="precomputed", choices=["precomputed", "hashfly"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--per-sample", type=int, default=PER_SAMPLE, dest="per_sample")
    ap.add_argument("--grid", type=int, default=GRID)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="conv_layer_c3",
                    choices=["conv_layer_c3", "hash_map_c2", "unet_infer", "unet_train"])
    ap.add_argument("--cells", type=int, default=8_000_000, help="hash_map_c2: number of coordinates")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "hash_map_c2":
        run_hash_map(args)
    elif args.workload in ("unet_infer", "unet_train"):
        run_unet(args, train=args.workload == "unet_train")
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
