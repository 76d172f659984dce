"""Benchmark of the sparse-convolution hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

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
    with trace.recording() as rec:
        sync_all()
        ev0.record()
        for _ in range(args.steps):
            step(coords_d, feats_d, dy_d, weight)
        ev1.record()
        sync_all()
        stages = rec.summary()
        launches = rec.total_launches()
    dev_ms = ev0.elapsed_time(ev1)

    # end to end: host buffers in, host results out, through the same public API
    y_h = torch.empty((n_out, COUT), dtype=dtype).pin_memory()
    dx_h = torch.empty((n_in, CIN), dtype=dtype).pin_memory()
    dw_h = torch.empty((KS ** 3, CIN, COUT), dtype=dtype).pin_memory()

    def e2e_step():
        c = coords_h.to(dev, non_blocking=True)
        f = feats_h.to(dev, non_blocking=True)
        g = dy_h.to(dev, non_blocking=True)
        y, dx, dw, _ = step(c, f, g, weight)
        y_h.copy_(y, non_blocking=True)
        dx_h.copy_(dx, non_blocking=True)
        dw_h.copy_(dw, non_blocking=True)

    for _ in range(max(1, args.warmup // 2)):
        e2e_step()
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        e2e_step()
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


def roofline(per_stage, n_in, n_out, pairs, pk, dtype):
    """Roofline entry of the stage that takes the largest share of the step.

    Algorithmic work per launch:
      conv_*      2 * pairs * Cin * Cout flop                       (tensor bound, vs bf16 GEMM peak)
      map_build   N_out * (16 + 12 K) + 4 * pairs bytes             (coords + key probe + map write + value)
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
        flops = 2.0 * pairs * CIN * COUT
        peak = pk["bf16_tflops"] * (0.5 if dtype == torch.float32 else 1.0)
        ach = flops / (ms * 1e-3) / 1e12
        entry.update({"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                      "peak_source": pk["source"], "algorithmic_flops_per_launch": flops})
    else:
        if top == "map_build":
            nbytes = n_out * (16 + 12 * K) + 4 * (pairs or 0)
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
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
