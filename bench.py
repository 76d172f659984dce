"""Benchmark of the sparse-convolution hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload `conv_layer_c3` (BASELINE config 3): one SparseConv3D downsample layer, batch 4, grid 512^3,
300 000 surface voxels per sample, 64 -> 128 channels, kernel 3, stride 2, padding 1, bf16, PrecomputedNeighborGEMM.
One PASS is the whole hot path over one batch,

    output coordinates -> neighbour map -> tile plans -> forward -> dgrad -> wgrad

and one STEP is `--passes` such passes cycling over `--batches` distinct seeded batches, so that the timed region
of a default run lasts most of a second.  `value` is input voxels per second with inputs resident in HBM; `e2e` is
the same passes through the public Python API starting from pinned HOST buffers (coordinates, features, upstream
gradient copied host->device and Y, dX, dW device->host inside the timed region).  With N > 1 every rank runs its
own batches of the same shape (weak scaling) and the weight gradient is all-reduced over NCCL inside the pass.

The same JSON line carries, from short legs run after the timed regions: the layer with ImplicitHashFlyGEMM and in
fp16, the hash / kernel-map microbenchmark at 2 M cells (config 2), the U-Net inference and training steps
(configs 4 / 5, sharded by sample over the ranks of this run), the reference's own Triton kernels on this GPU
(from baseline/_ref when it travelled, N = 1 only) and the CPU baseline (oracle port, N = 1 only).

Other workloads, each printing its own line: `hash_map_c2`, `unet_infer`, `unet_train`.

`--impl reference` times the CPU restatement of the reference's algorithm (the oracle port; the reference itself
is Triton code whose only CPU path is the Triton interpreter, at minutes per 4k voxels) on the host cores, one
sample of the same workload per step.
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
K = KS ** 3
DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def make_batch(seed0, batch=BATCH, per_sample=PER_SAMPLE, grid=GRID):
    """(N,4) int32 CPU coordinates of `batch` surface scenes; seeds seed0 + sample."""
    from sparsetriton_b200 import synthetic
    scenes = [synthetic.surface_scene(seed0 + b, grid=grid, target=per_sample) for b in range(batch)]
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


def _dist_setup(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        # NCCL announces its version on the process's stdout when the first communicator comes up: keep stdout
        # for the one JSON line by pointing file descriptor 1 at stderr until that has happened
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)
    return dist, world, rank, local, dev


def _sync_all(dist, world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def _max_over_ranks(dist, world, dev, values):
    t = torch.tensor(values, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def _sum_over_ranks(dist, world, dev, values):
    t = torch.tensor(values, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t)
    return t.tolist()


def _event_ms(dist, world, fn, reps):
    """Device time of `reps` calls of fn, bracketed by barrier + synchronize on both sides."""
    _sync_all(dist, world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        fn(i)
    e1.record()
    _sync_all(dist, world)
    return e0.elapsed_time(e1)


# ------------------------------------------------------------------------------------------------ the layer
class C3Layer:
    """The config-3 layer over a few resident batches; `one_pass(j)` runs the whole hot path on batch j."""

    def __init__(self, args, dist, world, rank, dev, dtype, algo_name, n_batches):
        import sparsetriton_b200 as st
        from sparsetriton_b200.config import ConvAlgo, set_conv_algo
        from sparsetriton_b200.nn.functional import sparse_conv3d
        self.st, self.conv, self.dist, self.world, self.dev = st, sparse_conv3d, dist, world, dev
        self.args, self.dtype = args, dtype
        self.algo = ConvAlgo.ImplicitHashFlyGEMM if algo_name == "hashfly" else ConvAlgo.PrecomputedNeighborGEMM
        self.set_algo = lambda: set_conv_algo(self.algo)
        self.shape = (args.grid,) * 3
        bound = 1.0 / (CIN * K) ** 0.5
        self.weight = ((torch.rand(K, CIN, COUT, generator=torch.Generator().manual_seed(7)) * 2 - 1) * bound).to(dtype).to(dev)
        self.host, self.resident, self.n_in, self.n_out, self.pairs = [], [], [], [], []
        self.steps_fwd, self.steps_inv = [], []
        for j in range(n_batches):
            coords_h = make_batch(3000 + (rank * n_batches + j) * args.batch, args.batch, args.per_sample, args.grid).pin_memory()
            gen = torch.Generator(device="cpu").manual_seed(9000 + rank * n_batches + j)
            feats_h = torch.randn(coords_h.shape[0], CIN, generator=gen).to(dtype).pin_memory()
            coords_d, feats_d = coords_h.to(dev), feats_h.to(dev)
            # learn N_out and the pair count of this batch with the stored-map form (one probe pass)
            set_conv_algo(ConvAlgo.PrecomputedNeighborGEMM)
            sp = st.SparseTensor._trusted(feats_d, coords_d, self.shape, args.batch)
            out = sparse_conv3d(sp, self.weight, kernel_size=KS, stride=STRIDE, padding=PAD, submanifold=False)
            nbr = sp._cache.neighbor_indices[(KS, STRIDE, PAD, 1, False, False)][1]
            n_out = out.F.shape[0]
            self.pairs.append(int((nbr >= 0).sum().item()))
            # (tile, offset) steps of the two tile plans = 128-row gather slots the products issue (one per step and
            # 128-byte line of a row): what their copy time is proportional to, absent rows of a slot included
            from sparsetriton_b200.nn.functional.conv.funcs.implicit_precomputed_gemm import inverse_plan, map_plan

            def popcount(t):
                b = t.view(torch.uint8)
                lut = torch.tensor([bin(i).count("1") for i in range(256)], dtype=torch.int64, device=b.device)
                return int(lut[b.long()].sum().item())
            fwd_plan, inv_plan = map_plan(nbr), inverse_plan(nbr, coords_d.shape[0])
            self.steps_fwd.append(popcount(fwd_plan.tmask) if fwd_plan.tmask is not None else 0)
            self.steps_inv.append(popcount(inv_plan.tmask) if inv_plan is not None else 0)
            del sp, out, nbr, fwd_plan, inv_plan
            dy_h = torch.randn(n_out, COUT, generator=gen).to(dtype).pin_memory()
            self.host.append((coords_h, feats_h, dy_h))
            self.resident.append((coords_d, feats_d, dy_h.to(dev)))
            self.n_in.append(coords_h.shape[0])
            self.n_out.append(n_out)
        self.set_algo()

    def prepare(self, coords, consumer):
        """First half of the coordinate side of one pass (candidates counted and deduplicated) on the current stream;
        `.finish()` launches the rest (output coordinates, map, tile plans) and returns the cache for `run`."""
        from sparsetriton_b200.nn.functional import ConvPreparation
        return ConvPreparation(coords, self.shape, kernel_size=KS, stride=STRIDE, padding=PAD, submanifold=False,
                               consumer_stream=consumer, batch_size=self.args.batch)

    def run(self, coords, feats, dy, cache=None):
        """One pass; returns (y, dx, dw).  With `cache` (from `prepare`) only the three products are left to do."""
        x = feats.detach().requires_grad_(True)
        wp = self.weight.detach().requires_grad_(True)
        sp = self.st.SparseTensor._trusted(x, coords, self.shape, self.args.batch, cache)
        out = self.conv(sp, wp, kernel_size=KS, stride=STRIDE, padding=PAD, submanifold=False)
        dx, dw = torch.autograd.grad(out.F, [x, wp], dy)
        if self.world > 1:
            self.dist.all_reduce(dw)
        return out.F, dx, dw

    def one_pass(self, j):
        return self.run(*self.resident[j % len(self.resident)])

    def pipelined(self, passes, side, keep=None):
        """`passes` passes with the coordinate side of the passes ahead on stream `side`, beside the products of pass j:
        while pass j's products run, the second half of pass j+1's preparation and the first half of pass j+2's are
        launched, so the host never waits for a count that is not already there.  Every pass still builds its own
        coordinates, map and plans; nothing is carried from one pass to another."""
        main = torch.cuda.current_stream()
        side.wait_stream(main)

        def begin(j):
            with torch.cuda.stream(side):
                return self.prepare(self.resident[j % len(self.resident)][0], main)

        def finish(prep):
            with torch.cuda.stream(side):
                cache = prep.finish()
                ready = torch.cuda.Event()
                ready.record(side)
            return cache, ready

        current = finish(begin(0))
        ahead = begin(1) if passes > 1 else None
        for j in range(passes):
            cache, ready = current
            main.wait_event(ready)
            out = self.run(*self.resident[j % len(self.resident)], cache=cache)
            if keep is not None:
                keep.append(out)
            if ahead is not None:
                current = finish(ahead)
                ahead = begin(j + 2) if j + 2 < passes else None
        main.wait_stream(side)

    def overlapped_equals_serial(self, side, passes=5):
        """The overlapped form must give, bit for bit, what the passes give on one stream (nothing in the path is
        order-dependent: no atomics in the products, deterministic maps and plans)."""
        got = []
        self.pipelined(passes, side, keep=got)
        torch.cuda.synchronize()
        for j, out in enumerate(got):
            want = self.one_pass(j)
            torch.cuda.synchronize()
            if not (torch.equal(out[0], want[0]) and torch.equal(out[1], want[1])):
                return False
            # dW went through the all-reduce when there are several ranks: equal up to the collective's own rounding
            if not (torch.equal(out[2], want[2]) if self.world == 1 else
                    torch.allclose(out[2].float(), want[2].float(), rtol=2e-2, atol=1e-3)):
                return False
        return True

    def voxels(self, passes):
        return sum(self.n_in[j % len(self.n_in)] for j in range(passes))


GATHER_CEILING_GBS = 4400.0      # measured row-gather rate of one B200 (see stage_rooflines)


def conv_bytes(kind, n_in, n_out, pairs, es):
    """Compulsory traffic of one product, e*(N_in*Cin + N_out*Cout + K*Cin*Cout) + 4*rows*K (the map is read once:
    the forward map for fwd and wgrad, the (N_in, K) inverse map for dgrad), and the bytes the kernel gathers."""
    rows = n_in if kind == "conv_dgrad" else n_out
    compulsory = es * (n_in * CIN + n_out * COUT + K * CIN * COUT) + 4 * rows * K
    gathered = {"conv_fwd": pairs * CIN + n_out * COUT, "conv_dgrad": pairs * COUT + n_in * CIN,
                "conv_wgrad": pairs * CIN + n_out * COUT}[kind] * es + K * CIN * COUT * es + 4 * rows * K
    return compulsory, gathered


def stage_rooflines(per_stage, n_in, n_out, pairs, pk, dtype, steps_fwd=0, steps_inv=0):
    """Roofline entry of every stage of the pass.  Algorithmic bytes:
      out_coords        N_in*(16 + 12*c) + 16*N_out, c = 27/8 candidates per input of a k3 s2 layer
      map_scatter       N_out*(16 + 12 K) + 4 P   (the kernel-map figure for N_out rows; the scatter form executes less)
      map_plan          8 K N_out (read the map, write its plan);  map_plan_inverse  8 K N_in + 4 K N_out
      conv_*            compulsory bytes (conv_bytes) against the copy bandwidth and 2 P Cin Cout flop against the GEMM
                        peak; the ceiling that takes longer is the bound
    """
    es = 4 if dtype == torch.float32 else 2
    tc_peak = pk["bf16_tflops"] * (0.5 if dtype == torch.float32 else 1.0)
    out = {}
    for name, st in per_stage.items():
        ms = st["ms_per_pass"]
        if ms <= 0:
            continue
        kind = name.replace("_hashfly", "")
        entry = {"ms": ms}
        if kind in ("conv_fwd", "conv_dgrad", "conv_wgrad"):
            nbytes, gathered = conv_bytes(kind, n_in, n_out, pairs, es)
            flops = 2.0 * pairs * CIN * COUT
            t_hbm, t_tc = nbytes / (pk["hbm_gbs"] * 1e9), flops / (tc_peak * 1e12)
            gbs = nbytes / (ms * 1e-3) / 1e9
            entry.update({"bound": "hbm" if t_hbm >= t_tc else "tensor", "algorithmic_bytes": nbytes,
                          "gathered_bytes": gathered, "algorithmic_flops": flops, "achieved_gbs": gbs,
                          "frac": gbs / pk["hbm_gbs"], "tflops": flops / (ms * 1e-3) / 1e12,
                          "tensor_frac": flops / (ms * 1e-3) / 1e12 / tc_peak})
            if t_hbm < t_tc:
                entry["frac"] = entry["tensor_frac"]
            # what these kernels are bound by in practice: rows pulled into shared memory per second.  A microbenchmark
            # on this pool's B200 (one 16 KB slot = 128 rows of 128 bytes per tile::gather4 burst, ring of slots,
            # 148 CTAs) tops out at 15.7 B/clk/SM = 4.4 TB/s for random rows out of DRAM
            # Slots issued: one per (tile, offset) step of the plan the product walks and per 128-byte line of the
            # gathered row (fwd and wgrad gather X rows over the forward plan, dgrad gathers dY rows over the inverse
            # plan).  wgrad also loads a dY tile per (tile, offset group): not counted here.
            steps = steps_inv if kind == "conv_dgrad" else steps_fwd
            lines = -(-(COUT if kind == "conv_dgrad" else CIN) * es // 128)
            if steps:
                slot_bytes = steps * lines * 128 * 128
                entry["gather_slot_bytes"] = slot_bytes
                entry["gather_gbs"] = slot_bytes / (ms * 1e-3) / 1e9
                entry["gather_ceiling_gbs"] = GATHER_CEILING_GBS
                entry["gather_frac"] = entry["gather_gbs"] / GATHER_CEILING_GBS
        else:
            if kind == "out_coords":
                nbytes = n_in * (16 + 12 * K / 8.0) + 16 * n_out
            elif kind in ("map_scatter", "map_build"):
                nbytes = n_out * (16 + 12 * K) + 4 * pairs
            elif kind == "conv_wgrad_presort":
                nbytes = 2 * n_out * COUT * es + 4 * n_out          # dY read and written once, the row order read
            elif kind == "map_plan":
                nbytes = 8 * K * n_out
            elif kind == "map_plan_inverse":
                nbytes = 8 * K * n_in + 4 * K * n_out
            elif kind == "map_invert":
                nbytes = 4 * K * (n_in + n_out)
            elif kind in ("hash_build", "hash_clear"):
                nbytes = 52 * n_in
            else:
                continue
            gbs = nbytes / (ms * 1e-3) / 1e9
            entry.update({"bound": "hbm", "algorithmic_bytes": nbytes, "achieved_gbs": gbs, "frac": gbs / pk["hbm_gbs"]})
        out[name] = entry
    return out


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of the dominant kernels, from the ncu
# captures summarised under profiles/ (default workload: 4 x 300 k voxels, bf16, stored-map algorithm).
NCU_TRAFFIC_C3 = {
    "conv_fwd": (466.4e6 + 187.8e6, "profiles/planned_gather_kernel_c3.md"),
    "conv_dgrad": (820.9e6 + 143.0e6, "profiles/planned_gather_kernel_c3.md"),
    # the stage's two kernels: the product and the sum of the partials (the copy of dY into tile order, 216.9 + 169.8 MB,
    # runs on a second stream beside the feature gradient: stage conv_wgrad_presort)
    "conv_wgrad": ((976.2e6 + 46.5e6) + (65.5e6 + 0.2e6), "profiles/planned_wgrad_kernel_c3.md"),
}


def run_ours(args):
    from sparsetriton_b200 import trace
    from sparsetriton_b200.config import set_coords_dtype, set_h_table_f

    dist, world, rank, local, dev = _dist_setup(args)
    set_coords_dtype(torch.int32)
    set_h_table_f(2.0)
    dtype = DTYPES[args.dtype]
    if args.hashfly_in_kernel:
        from sparsetriton_b200.config import set_hashfly_transient_map
        set_hashfly_transient_map(False)
    layer = C3Layer(args, dist, world, rank, dev, dtype, args.algo, args.batches)
    passes = args.passes

    def serial_step(_i=0):
        for j in range(passes):
            layer.one_pass(j)

    # Timed form: the coordinate side of pass j+1 (output coordinates, map, tile plans: prepare_conv3d on a second
    # stream) runs beside the three products of pass j.  The serial form is timed as well and reported next to it.
    pipelined = args.algo == "precomputed" and not args.no_pipeline
    # the side stream's small kernels go ahead of the products' queued CTAs (higher priority), or they would wait
    # behind every wave of a product
    side = torch.cuda.Stream(priority=-1) if pipelined else None

    def step(_i=0):
        if pipelined:
            layer.pipelined(passes, side)
        else:
            serial_step()

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    allocs_before = torch.cuda.memory_stats()["num_device_alloc"]
    dev_ms = _event_ms(dist, world, step, args.steps)
    device_allocs = torch.cuda.memory_stats()["num_device_alloc"] - allocs_before      # cudaMalloc calls inside the timed steps
    serial_ms = _event_ms(dist, world, serial_step, args.steps) if pipelined else dev_ms
    same = layer.overlapped_equals_serial(side) if pipelined else None
    step = serial_step
    # the per-stage breakdown and the launch count come from one more step with the stage recorder on (its event
    # pairs cost host time, so it stays out of the timed steps)
    with trace.recording() as rec:
        step()
        _sync_all(dist, world)
        stages, launches_per_step = rec.summary(), rec.total_launches()

    # ---- end to end: host buffers in, host results out, through the same public API.  Three streams: the copy of
    # pass i+1's inputs (pinned host -> device, double-buffered) and the read-back of pass i-1's results run beside
    # pass i's kernels.  Every pass still moves all of its inputs and results.
    big = max(range(len(layer.host)), key=lambda j: layer.n_out[j])
    y_h = torch.empty((layer.n_out[big], COUT), dtype=dtype).pin_memory()
    dx_h = torch.empty((max(layer.n_in), CIN), dtype=dtype).pin_memory()
    dw_h = torch.empty((K, CIN, COUT), dtype=dtype).pin_memory()
    s_comp = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    in_bufs = [(torch.empty((max(layer.n_in), 4), dtype=torch.int32, device=dev),
                torch.empty((max(layer.n_in), CIN), dtype=dtype, device=dev),
                torch.empty((max(layer.n_out), COUT), dtype=dtype, device=dev)) for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]

    def views(b, j):
        return (in_bufs[b][0][:layer.n_in[j]], in_bufs[b][1][:layer.n_in[j]], in_bufs[b][2][:layer.n_out[j]])

    def upload(i):
        b, j = i % 2, i % len(layer.host)
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_free[b])                 # pass i-2 has finished reading this buffer
            for dst, src in zip(views(b, j), layer.host[j]):
                dst.copy_(src, non_blocking=True)
            ev_in[b].record(s_in)

    def e2e_run(n_passes):
        upload(0)
        for i in range(n_passes):
            b, j = i % 2, i % len(layer.host)
            if i + 1 < n_passes:
                upload(i + 1)
            s_comp.wait_event(ev_in[b])
            y, dx, dw = layer.run(*views(b, j))
            ev_free[b].record(s_comp)
            done = torch.cuda.Event()
            done.record(s_comp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                y_h[:y.shape[0]].copy_(y, non_blocking=True)
                dx_h[:dx.shape[0]].copy_(dx, non_blocking=True)
                dw_h.copy_(dw, non_blocking=True)
            for t in (y, dx, dw):
                t.record_stream(s_out)
        s_comp.wait_stream(s_out)

    e2e_passes = args.steps * passes
    e2e_run(min(4, e2e_passes))
    e2e_ms = _event_ms(dist, world, lambda _i: e2e_run(e2e_passes), 1)
    clocks = sampler.stop() if rank == 0 else None
    del in_bufs

    dev_ms, e2e_ms, serial_ms = _max_over_ranks(dist, world, dev, [dev_ms, e2e_ms, serial_ms])
    (voxels_per_step,) = _sum_over_ranks(dist, world, dev, [float(layer.voxels(passes))])

    # ---- legs (same process, after the timed regions)
    legs = {}
    if not args.no_legs:
        legs.update(c3_variant_legs(args, dist, world, rank, dev))
        legs.update(unet_legs(args, dist, world, rank, dev))
        if rank == 0:
            legs["c2_2m"] = c2_leg(args, dev)
        if world == 1:
            legs["reference_gpu_triton"] = reference_gpu_leg(args)

    if rank == 0:
        pk = peaks()
        ms_per_step = dev_ms / args.steps
        ms_per_pass = ms_per_step / passes
        value = voxels_per_step / (ms_per_step * 1e-3)
        n_in, n_out, pairs = (statistics.mean(v) for v in (layer.n_in, layer.n_out, layer.pairs))
        per_stage = {k: {"ms_per_pass": v["ms"] / passes, "launches_per_pass": v["launches"] / passes}
                     for k, v in stages.items()}
        roofs = stage_rooflines(per_stage, n_in, n_out, pairs, pk, dtype, statistics.mean(layer.steps_fwd),
                                statistics.mean(layer.steps_inv))
        # the dominant stage among those on the pass's own stream (conv_wgrad_presort runs on a second stream beside
        # conv_dgrad: its elapsed time is not a share of the pass)
        in_line = {k: v for k, v in roofs.items() if k != "conv_wgrad_presort"}
        top = max(in_line, key=lambda k: in_line[k]["ms"]) if in_line else None
        roof = None
        if top:
            r = roofs[top]
            bound = r["bound"]
            traffic, src = None, None
            if top in NCU_TRAFFIC_C3 and args.algo == "precomputed" and args.dtype != "fp32":
                traffic, src = NCU_TRAFFIC_C3[top][0] * n_in / 1.2e6, NCU_TRAFFIC_C3[top][1]
            roof = {"kernel": top, "bound": bound,
                    "achieved": r["achieved_gbs"] if bound == "hbm" else r["tflops"],
                    "peak": pk["hbm_gbs"] if bound == "hbm" else pk["bf16_tflops"],
                    "unit": "GB/s" if bound == "hbm" else "TFLOP/s", "frac": r["frac"], "traffic": traffic,
                    "traffic_source": src, "peak_source": pk["source"],
                    "algorithmic_bytes_per_launch": r["algorithmic_bytes"], "gathered_bytes": r.get("gathered_bytes"),
                    "algorithmic_flops_per_launch": r.get("algorithmic_flops"), "tensor_frac": r.get("tensor_frac"),
                    "ms_per_launch": r["ms"], "share_of_pass": r["ms"] / sum(v["ms"] for v in in_line.values())}
        h2d = sum(sum(t.numel() * t.element_size() for t in layer.host[j % len(layer.host)]) for j in range(passes))
        d2h = sum((layer.n_out[j % len(layer.host)] * COUT + layer.n_in[j % len(layer.host)] * CIN + K * CIN * COUT)
                  * y_h.element_size() for j in range(passes))
        line = {
            "metric": "sparse_conv_layer_fwd_bwd_voxels_per_s", "value": value, "unit": "voxels/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": args.dtype, "data": "synthetic",
            "config": {"workload": "conv_layer_c3: SparseConv3D 64->128 k3 s2 p1, batch %d x %d voxels, grid %d^3; one pass = "
                                   "output coordinates + neighbour map (one sweep over the candidates, no hash table of the "
                                   "inputs) + tile plans + fwd + dgrad + wgrad; one step = %d passes over %d distinct seeded "
                                   "batches" % (args.batch, args.per_sample, args.grid, passes, len(layer.host)),
                       "algo": layer.algo.value, "passes_per_step": passes, "ms_per_pass": ms_per_pass,
                       "pipelining": ("coordinate side of passes j+1 and j+2 on a second stream beside the products of pass j "
                                      "(prepare_conv3d); every pass builds its own coordinates, map and plans"
                                      if pipelined else "none: one stream"),
                       "serial_ms_per_pass": serial_ms / args.steps / passes,
                       "overlapped_results_equal_serial_bitwise": same,
                       "device_allocs_in_timed_steps": device_allocs,
                       "n_in_per_pass": n_in, "n_out_per_pass": n_out, "pairs_per_pass": pairs,
                       "constructor": "SparseTensor._trusted (the library's internal constructor: no validation read of the "
                                      "coordinates; the public one adds one device->host read per tensor)",
                       "l2_policy": "inputs larger than L2 (features + map + outputs > 400 MB per pass, %d batches cycled)"
                                    % len(layer.host),
                       "parallelism": "dp%d by sample, NCCL all-reduce of dW" % world},
            "e2e": {"value": voxels_per_step / (e2e_ms / args.steps * 1e-3), "unit": "voxels/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps,
                    "h2d_gbs": h2d / (e2e_ms / args.steps * 1e-3) / 1e9, "d2h_gbs": d2h / (e2e_ms / args.steps * 1e-3) / 1e9,
                    "bound": "host<->device copies: both directions busy at once (this pool's boxes copy 48 GB/s per "
                             "direction when both run, 55 GB/s alone: PCIe 5 x16)",
                    "ms_per_pass": e2e_ms / e2e_passes},
            "gpu_launches": launches_per_step * args.steps, "gpu_launches_per_pass": launches_per_step / passes,
            "stages": per_stage, "stage_rooflines": roofs, "roofline": roof, "clocks": clocks,
        }
        if pairs:
            gemm_ms = sum(per_stage.get(s, {}).get("ms_per_pass", 0.0) for s in ("conv_fwd", "conv_dgrad", "conv_wgrad"))
            line["gemm_tflops"] = 3 * 2.0 * pairs * CIN * COUT / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
        line.update(legs)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_leg(args, seconds_budget=20.0)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()                     # rank 0 ran legs of its own: leave together
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------ legs
def c3_variant_legs(args, dist, world, rank, dev):
    """The same layer with the hash-on-the-fly algorithm (scratch map per call, and probing inside the kernels) and in
    fp16: ms per pass (max over ranks), one batch."""
    out = {}
    from sparsetriton_b200.config import set_hashfly_transient_map
    for key, algo, dt, transient in (("c3_hashfly_ms_per_step", "hashfly", args.dtype, True),
                                     ("c3_hashfly_in_kernel_probing_ms_per_step", "hashfly", args.dtype, False),
                                     ("c3_fp16_ms_per_step", "precomputed", "fp16", True)):
        try:
            set_hashfly_transient_map(transient)
            layer = C3Layer(args, dist, world, rank, dev, DTYPES[dt], algo, 1)
            for _ in range(3):
                layer.one_pass(0)
            reps = 5
            ms = _event_ms(dist, world, layer.one_pass, reps) / reps
            (ms,) = _max_over_ranks(dist, world, dev, [ms])
            out[key] = ms
            out[key.replace("_ms_per_step", "_voxels_per_s")] = world * layer.n_in[0] / (ms * 1e-3)
            del layer
        except Exception as e:  # noqa: BLE001 - a leg must not take the headline down
            out[key] = "failed: %r" % (e,)
        torch.cuda.empty_cache()
    from sparsetriton_b200.config import ConvAlgo, set_conv_algo
    set_conv_algo(ConvAlgo.PrecomputedNeighborGEMM)
    set_hashfly_transient_map(True)
    return out


def c2_leg(args, dev, cells=2_000_000, steps=3):
    """BASELINE config 2 at 2 M cells on one GPU: per-stage ms and fraction of the measured copy bandwidth."""
    try:
        res = hash_map_measure(dev, cells, 2001, warmup=2, steps=steps)
        res.pop("launches", None)
        return res
    except Exception as e:  # noqa: BLE001
        return "failed: %r" % (e,)
    finally:
        torch.cuda.empty_cache()


def unet_legs(args, dist, world, rank, dev):
    out = {}
    for key, train in (("unet_infer", False), ("unet_train", True)):
        try:
            # ten warm-up steps: with the preparation on a second stream the caching allocator keeps growing its pools
            # (cudaMalloc inside a step) for about that long; detail.device_allocs_in_timed_steps says what was left
            r = unet_measure(args, dist, world, rank, dev, train, steps=8, warmup=10, prune=True, e2e=False)
            out[key + "_ms_per_step"] = r["ms_per_step"]
            out[key + "_detail"] = {"prune": True, "batch": r["total_batch"], "voxels": r["total_voxels"],
                                    "launches_per_step": r["launches"], "kernel_ms_per_step": r["kernel_ms"],
                                    "serial_ms_per_step": r["serial_ms_per_step"],
                       "device_allocs_in_timed_steps": r["device_allocs_in_timed_steps"],
                                    "device_allocs_in_timed_steps": r["device_allocs_in_timed_steps"],
                                    "conv_by_width": r["conv_by_width"],
                                    "pipelining": ("coordinate side of step i+1 (SparseUNet.prepare) on a second stream "
                                                   "beside step i" if r["pipelined"] else "none: one stream"),
                                    "decoder": "up-convolution evaluated at the encoder's coordinates (prune=True)"}
        except Exception as e:  # noqa: BLE001
            out[key + "_ms_per_step"] = "failed: %r" % (e,)
        torch.cuda.empty_cache()
    if rank == 0:
        # the literal decoder (every child of the transposed convolution kept, skip by lookup) on two samples
        try:
            r = unet_measure(args, None, 1, 0, dev, False, steps=3, warmup=2, prune=False, e2e=False, samples=[4000, 4001])
            out["unet_infer_literal_2_samples_ms_per_step"] = r["ms_per_step"]
            out["unet_infer_literal_detail"] = {"prune": False, "batch": 2, "voxels_in": r["total_voxels"],
                                                "voxels_out": r["n_out"], "launches_per_step": r["launches"]}
        except Exception as e:  # noqa: BLE001
            out["unet_infer_literal_2_samples_ms_per_step"] = "failed: %r" % (e,)
        torch.cuda.empty_cache()
    return out


REF_GPU_SCRIPT = r"""
import json, os, sys, time
root = sys.argv[1]
sys.path.insert(0, os.path.join(root, "baseline", "_ref"))
sys.path.insert(0, root)
import torch
try:
    import triton                                                       # noqa: F401
    import sparsetriton
    from sparsetriton import SparseTensor
    from sparsetriton.nn.modules import SparseConv3D
    from sparsetriton.config import set_conv_algo, ConvAlgo
    assert os.path.realpath(sparsetriton.__file__).startswith(os.path.realpath(os.path.join(root, "baseline", "_ref")))
except Exception as e:
    print(json.dumps({"unavailable": "reference-on-GPU unavailable on this box: %r" % (e,)}))
    sys.exit(0)
from sparsetriton_b200 import synthetic
dev = torch.device("cuda")
batch, per_sample, grid, warm, iters = int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), int(sys.argv[5]), int(sys.argv[6])
coords = synthetic.batch_of([synthetic.surface_scene(3000 + b, grid=grid, target=per_sample) for b in range(batch)],
                            dtype=torch.int32).to(dev)
n = coords.shape[0]
feats = torch.randn(n, 64, generator=torch.Generator().manual_seed(9000)).to(torch.bfloat16).to(dev)
res = {"n_in": n, "protocol": "%d warm-up + %d timed iterations of SparseConv3D(64,128,3,stride=2,padding=1) forward + backward "
                              "on a fresh SparseTensor per iteration (benchmark_spconv_vs_sparsetriton.py:45-64), bf16, CUDA events"
                              % (warm, iters)}
for algo in (ConvAlgo.PrecomputedNeighborGEMM, ConvAlgo.ImplicitHashFlyGEMM):
    try:
        set_conv_algo(algo)
        torch.manual_seed(7)
        conv = SparseConv3D(64, 128, 3, stride=2, padding=1, bias=False).to(dev).to(torch.bfloat16)
        def step():
            x = feats.detach().requires_grad_(True)
            out = conv(SparseTensor(x, coords, spatial_shape=(grid,) * 3, batch_size=batch))
            out.F.backward(torch.ones_like(out.F))
            return out.F.shape[0]
        for _ in range(warm):
            n_out = step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        res[algo.name] = {"ms_per_step": ms, "voxels_per_s": n / (ms * 1e-3), "n_out": n_out}
    except Exception as e:
        res[algo.name] = "failed: %r" % (e,)
print(json.dumps(res))
"""


def reference_gpu_leg(args, warm=10, iters=30):
    """The UNMODIFIED reference package (installed into baseline/_ref in the build container) timed on this GPU on the
    shapes of the default workload, in a child process with a time limit; or the reason it cannot run here."""
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "sparsetriton")):
        return "reference-on-GPU unavailable on this box: baseline/_ref/sparsetriton is not present"
    try:
        p = subprocess.run([sys.executable, "-c", REF_GPU_SCRIPT, ROOT, str(args.batch), str(args.per_sample), str(args.grid),
                            str(warm), str(iters)], capture_output=True, text=True, timeout=600)
        lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
        if p.returncode != 0 or not lines:
            return "reference-on-GPU unavailable on this box: exit %d: %s" % (p.returncode, (p.stderr or p.stdout)[-300:])
        res = json.loads(lines[-1])
        return res.get("unavailable", res)
    except subprocess.TimeoutExpired:
        return "reference-on-GPU unavailable on this box: no result within 600 s"


# ------------------------------------------------------------------------------------ CPU baseline
def cpu_step(O, coords, feats, weight, dy_seed):
    """The same pass on the host through the oracle port; returns (seconds, n_in, n_out)."""
    t0 = time.perf_counter()
    oc, ns, off, nbr = O.kernel_map(coords, (GRID,) * 3, KS, STRIDE, 1, PAD, False, False)
    y = O.conv_fwd(feats, weight, nbr)
    dy = np.full_like(y, 1.0) if dy_seed is None else dy_seed(y.shape)
    O.conv_dgrad(dy, weight, nbr, feats.shape[0])
    O.conv_wgrad(feats, dy, nbr, K, CIN, COUT)
    return time.perf_counter() - t0, coords.shape[0], oc.shape[0]


def cpu_inputs(per_sample, grid):
    from sparsetriton_b200 import synthetic
    coords = synthetic.batch_of([synthetic.surface_scene(3000, grid=grid, target=per_sample)]).numpy()
    rng = np.random.default_rng(9000)
    feats = rng.standard_normal((coords.shape[0], CIN), dtype=np.float32)
    weight = ((rng.random((K, CIN, COUT), dtype=np.float32) * 2 - 1) / (CIN * K) ** 0.5).astype(np.float32)
    return coords, feats, weight


CPU_NOTE = ("oracle port (C + OpenMP restatement of the reference's algorithm, fp32); the three products, the candidate "
            "count and the neighbour map run on all threads, the first-occurrence dedupe of the output coordinates and the "
            "inverse-map build of dgrad are sequential loops (their order defines the result)")


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
            "sample": "1 of the %d samples of a batch (%d voxels), same layer and pass, best of %d; %s" %
                      (args.batch, n_in, reps, CPU_NOTE),
            "seconds_per_sample_pass": secs}


def run_reference(args):
    """CPU arm: the oracle port on all host threads; each step processes one sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import cpu_oracle as O
    O.build()
    O.set_threads(os.cpu_count() or 1)            # launchers such as torchrun export OMP_NUM_THREADS=1
    coords, feats, weight = cpu_inputs(args.per_sample, args.grid)
    warm = min(args.warmup, 1)
    for _ in range(warm):
        cpu_step(O, coords, feats, weight, None)
    steps = min(args.steps, 5)
    t = 0.0
    for _ in range(steps):
        s, n_in, n_out = cpu_step(O, coords, feats, weight, None)
        t += s
    value = n_in * steps / t
    sample = ("each step = 1 of the %d samples of a batch (%d voxels); %d steps timed after %d warm-up (asked for %d / %d: a "
              "host step takes ~0.4 s and repeats to within a few per cent, so the arm caps itself at 5 timed steps and 1 "
              "warm-up to stay within its time budget); %s" % (args.batch, n_in, steps, warm, args.steps, args.warmup, CPU_NOTE))
    print(json.dumps({
        "impl": "reference", "metric": "sparse_conv_layer_fwd_bwd_voxels_per_s", "value": value, "unit": "voxels/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": t / steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "conv_layer_c3 on host cores (oracle port of the reference's algorithm; the reference's "
                               "own Triton-interpreter CPU path needs minutes per 4k voxels)", "sample": sample},
        "cpu_baseline": {"value": value, "unit": "voxels/s", "cores": O.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "voxels/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# --------------------------------------------------------------------------------- hash / kernel-map workload
def hash_map_measure(dev, n, seed, warmup, steps):
    """BASELINE config 2: table build at load factor <= 0.5, submanifold maps for k3 (27) and k5 (125), a k3 s2 p1
    downsample (output coordinates + map) and the transposed map from its output.  Returns per-stage ms and
    rooflines (algorithmic bytes: coords 16 B, one 8-byte key probe + 4-byte map entry per (voxel, offset), 4 bytes
    per hit; strided / transposed add 16 N_out for the coordinates written and 12 bytes per candidate inserted)."""
    from sparsetriton_b200 import synthetic, trace
    from sparsetriton_b200.config import set_coords_dtype
    from sparsetriton_b200.nn.functional.conv.conv import compute_neighbor_indices
    from sparsetriton_b200.nn.functional.conv.kmap import build_out_coords, out_coords_and_map
    from sparsetriton_b200.utils.hash import HashTable

    set_coords_dtype(torch.int32)
    grid = 2048
    coords = synthetic.random_cells(n, 4, grid, seed=seed).to(dev)
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
        with trace.stage("down_k3s2"):
            oc, ns, ko, nbr = out_coords_and_map(coords, shape, 3, 2, 1, 1, False)
        with trace.stage("up_k3s2"):
            oc2, ns2, ko2, nbr2 = out_coords_and_map(oc, ns, 3, 2, 1, 1, True)
        return res, nbr, nbr2, oc, oc2

    def count_pairs(m, rows=1 << 22):
        """Valid entries of a map, a few million rows at a time (the transposed map has > 3e9 entries at 8 M cells)."""
        return sum(int((m[i:i + rows] >= 0).sum()) for i in range(0, m.shape[0], rows))

    res, nbr, nbr2, oc, oc2 = step()
    pairs = {"k3": count_pairs(res[3]), "k5": count_pairs(res[5]), "down": count_pairs(nbr), "up": count_pairs(nbr2)}
    n_down, n_up = oc.shape[0], oc2.shape[0]
    del res, nbr, nbr2, oc, oc2
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with trace.recording() as rec:
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        stages = rec.summary()
        launches = rec.total_launches()
    ms = e0.elapsed_time(e1)
    pk = peaks()
    per = {k: v["ms"] / steps for k, v in stages.items()}
    cand_down = n * 27 / 8.0
    algo = {
        "hash_build": 52.0 * n,
        "subm_map_k3": n * (16 + 12 * 27) + 4.0 * pairs["k3"],
        "subm_map_k5": n * (16 + 12 * 125) + 4.0 * pairs["k5"],
        "down_k3s2": 16.0 * n + 12.0 * cand_down + 16.0 * n_down + n_down * (16 + 12 * 27) + 4.0 * pairs["down"],
        "up_k3s2": 16.0 * n_down + 12.0 * 27 * n_down + 16.0 * n_up + n_up * (16 + 12 * 27) + 4.0 * pairs["up"],
    }
    roof = {}
    for name, nbytes in algo.items():
        if name in per and per[name] > 0:
            gbs = nbytes / (per[name] * 1e-3) / 1e9
            roof[name] = {"ms": per[name], "algorithmic_bytes": nbytes, "achieved_gbs": gbs, "frac": gbs / pk["hbm_gbs"]}
    return {"cells": n, "table_capacity": cap, "ms_per_step": ms / steps, "pairs": pairs, "n_out_down": n_down,
            "n_out_up": n_up, "stages_ms": per, "stage_rooflines": roof, "launches": launches / steps}


def run_hash_map(args):
    dist, world, rank, local, dev = _dist_setup(args)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    r = hash_map_measure(dev, args.cells, 2001 + rank, max(args.warmup, 3), args.steps)
    clocks = sampler.stop() if rank == 0 else None
    (ms_step,) = _max_over_ranks(dist, world, dev, [r["ms_per_step"]])
    if rank == 0:
        pk = peaks()
        roof = r["stage_rooflines"]
        top = max(roof, key=lambda k: roof[k]["ms"])
        print(json.dumps({
            "metric": "hash_and_kernel_map_voxels_per_s", "value": world * r["cells"] / (ms_step * 1e-3), "unit": "voxels/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int64 keys / int32 coords",
            "data": "synthetic",
            "config": {"workload": "hash_map_c2: %d random cells, batch 4, grid 2048^3, table capacity %d; build + subm k3 + "
                                   "subm k5 + k3s2p1 down (coords+map) + transposed map" % (r["cells"], r["table_capacity"]),
                       "pairs": r["pairs"], "n_out_down": r["n_out_down"], "n_out_up": r["n_out_up"],
                       "l2_policy": "tables and maps larger than L2"},
            "gpu_launches": r["launches"] * args.steps, "stages": r["stages_ms"], "stage_rooflines": roof,
            "roofline": {"kernel": top, "bound": "hbm", "achieved": roof[top]["achieved_gbs"], "peak": pk["hbm_gbs"],
                         "unit": "GB/s", "frac": roof[top]["frac"], "traffic": None, "peak_source": pk["source"]},
            "clocks": clocks,
        }))
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------- U-Net workloads
def make_lidar_batch(samples):
    """(coords (N,4) int32 with batch relabelled from 0, feats (N,4) fp32) of the given scene seeds."""
    from sparsetriton_b200 import synthetic
    scenes = [synthetic.lidar_scene(seed) for seed in samples]
    coords = synthetic.batch_of(scenes, dtype=torch.int32)
    g = torch.Generator().manual_seed(samples[0] + 17)
    xyz = coords[:, 1:].float() / torch.tensor([1440.0, 1440.0, 41.0])
    feats = torch.cat([xyz, torch.rand(coords.shape[0], 1, generator=g)], dim=1)
    return coords, feats


def unet_measure(args, dist, world, rank, dev, train, steps, warmup, prune=True, e2e=True, samples=None):
    """BASELINE configs 4 / 5: lidar-like sparse U-Net, bf16 features, fp32 master weights; batch 8 (inference) or 16
    (training) sharded by sample over the ranks.  Returns ms per step (max over ranks) and the stage breakdown."""
    from sparsetriton_b200 import trace
    from sparsetriton_b200.config import ConvAlgo, set_conv_algo, set_coords_dtype, set_h_table_f
    from sparsetriton_b200.distributed import GradientBucket, global_mean_scale, shard_samples
    from sparsetriton_b200.tensor import SparseTensor
    from sparsetriton_b200.unet import SparseUNet

    set_coords_dtype(torch.int32)
    set_h_table_f(2.0)
    set_conv_algo(ConvAlgo.ImplicitHashFlyGEMM if args.algo == "hashfly" else ConvAlgo.PrecomputedNeighborGEMM)
    dtype = DTYPES[args.dtype]
    total_batch = 16 if train else 8
    base_seed = 5000 if train else 4000
    if samples is None:
        mine = shard_samples(total_batch, rank, world)
        seeds = [base_seed + i for i in mine]
    else:
        seeds, total_batch = list(samples), len(samples)
    coords_h, feats_h = make_lidar_batch(seeds)
    coords_h, feats_h = coords_h.pin_memory(), feats_h.to(dtype).pin_memory()
    shape = (1440, 1440, 41)
    torch.manual_seed(5100 if train else 4100)
    model = SparseUNet(prune=prune).to(dev)
    model.train(train)
    n_in = coords_h.shape[0]
    opt = bucket = None
    if train:
        bucket = GradientBucket(model.parameters())
        opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
    state = {"labels": None, "scale": None, "n_out": None}

    def step(coords, feats, cache=None):
        x = SparseTensor._trusted(feats, coords, shape, len(seeds), cache)
        if not train:
            with torch.no_grad():
                out = model(x)
            state["n_out"] = out.F.shape[0]
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

    # Timed form (stored maps, pruned decoder): while step i runs, the coordinate side of step i+1 (SparseUNet.prepare:
    # every level's maps, plans and row counts) is built on a second stream from that step's coordinates; the
    # step itself then launches no coordinate work and reads nothing back.  Every step still builds all of its maps.
    pipelined = prune and args.algo != "hashfly" and not args.no_pipeline
    main = torch.cuda.current_stream()
    side = torch.cuda.Stream(priority=-1) if pipelined else None

    def prefetch(coords=None):
        """Coordinate side of the next step on the side stream; uploads the coordinates there first when none are given
        (resident coordinates were uploaded and waited for before the first step)."""
        with torch.cuda.stream(side):
            if coords is None:
                coords = coords_h.to(dev, non_blocking=True)
                coords.record_stream(main)
            cache = model.prepare(coords, shape, len(seeds), backward=train, consumer_stream=main)
            ready = torch.cuda.Event()
            ready.record(side)
        return coords, cache, ready

    coords_d, feats_d = coords_h.to(dev), feats_h.to(dev)
    torch.cuda.synchronize()
    pending = {"next": None}

    def run_step(_i=0):
        if not pipelined:
            return step(coords_d, feats_d)
        coords, cache, ready = pending["next"] or prefetch(coords_d)
        main.wait_event(ready)
        r = step(coords, feats_d, cache)
        pending["next"] = prefetch(coords_d)
        return r

    for _ in range(warmup):
        run_step()
    allocs_before = torch.cuda.memory_stats()["num_device_alloc"]
    dev_ms = _event_ms(dist, world, run_step, steps)
    # cudaMalloc calls inside the timed steps (the caching allocator still growing): such a run is not steady state
    device_allocs = torch.cuda.memory_stats()["num_device_alloc"] - allocs_before
    pending["next"] = None
    serial_ms = _event_ms(dist, world, lambda _i: step(coords_d, feats_d), steps) if pipelined else dev_ms
    # stage breakdown and launch count: one more step (one stream) with the stage recorder on, outside the timed steps
    with trace.recording() as rec:
        step(coords_d, feats_d)
        _sync_all(dist, world)
        stages, launches = rec.summary(), rec.total_launches()
        # the three products by channel widths: ms, TFLOP/s and the fraction of the sustained dense bf16 peak
        pk = peaks()
        peak_tf = pk["bf16_tflops_sustained"] * (0.5 if dtype == torch.float32 else 1.0)
        widths = {}
        for (name, tag), v in rec.by_tag().items():
            e = widths.setdefault("%dx%d" % tag, {"ms": 0.0, "flops": 0.0, "launches": 0})
            e["ms"] += v["ms"]
            e["flops"] += v["work"]
            e["launches"] += v["calls"]
        for e in widths.values():
            e["tflops"] = e["flops"] / (e["ms"] * 1e-3) / 1e12 if e["ms"] > 0 else None
            e["tensor_frac"] = e["tflops"] / peak_tf if e["tflops"] else None
    e2e_ms = None
    if e2e:
        result_h = torch.zeros(1, dtype=torch.float32).pin_memory()

        def e2e_step(_i):
            if pipelined:
                coords, cache, ready = pending["next"] or prefetch()
                main.wait_event(ready)
            else:
                coords, cache = coords_h.to(dev, non_blocking=True), None
            f = feats_h.to(dev, non_blocking=True)
            r = step(coords, f, cache)
            result_h.copy_(r.float().sum().reshape(1), non_blocking=True)
            if pipelined:
                pending["next"] = prefetch()

        for i in range(2):
            e2e_step(i)
        e2e_ms = _event_ms(dist, world, e2e_step, steps)
        pending["next"] = None
    vals = _max_over_ranks(dist, world, dev, [dev_ms, e2e_ms or 0.0, serial_ms])
    (total_voxels,) = _sum_over_ranks(dist, world, dev, [float(n_in)])
    del model, opt, bucket
    return {"ms_per_step": vals[0] / steps, "e2e_ms_per_step": (vals[1] / steps) if e2e else None, "stages": stages,
            "serial_ms_per_step": vals[2] / steps, "pipelined": pipelined, "conv_by_width": widths,
            "device_allocs_in_timed_steps": device_allocs,
            "launches": launches, "kernel_ms": sum(v["ms"] for v in stages.values()), "total_voxels": total_voxels,
            "total_batch": total_batch, "n_in": n_in, "n_out": state["n_out"], "local_samples": len(seeds),
            "h2d": coords_h.numel() * 4 + feats_h.numel() * feats_h.element_size()}


def run_unet(args, train):
    dist, world, rank, local, dev = _dist_setup(args)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    samples = None
    if args.unet_samples:
        base = 5000 if train else 4000
        samples = [base + rank * args.unet_samples + i for i in range(args.unet_samples)]
    r = unet_measure(args, dist, world, rank, dev, train, args.steps, max(args.warmup, 3 if args.no_pipeline else 10),
                     prune=not args.literal_decoder, samples=samples)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        pk = peaks()
        dtype = DTYPES[args.dtype]
        ms_step = r["ms_per_step"]
        per = {k: {"ms_per_step": v["ms"], "launches_per_step": v["launches"], "calls_per_step": v["calls"],
                   "tflops": (v["work"] / (v["ms"] * 1e-3) / 1e12) if v["work"] and v["ms"] > 0 else None}
               for k, v in r["stages"].items()}
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
            "value": r["total_voxels"] / (ms_step * 1e-3), "unit": "voxels/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3 if args.no_pipeline else 10), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "config": {"workload": "%s: lidar-like U-Net 4->32/64/128/256->...->32->20, grid 1440x1440x41, batch %d "
                                   "(%d samples on this rank, %d voxels)" % (args.workload, r["total_batch"], r["local_samples"],
                                                                             r["n_in"]),
                       "decoder": "literal (every child of the transposed convolution)" if args.literal_decoder
                                  else "up-convolution evaluated at the encoder's coordinates (prune=True)",
                       "algo": args.algo, "parallelism": "dp%d by sample%s" % (world, ", NCCL all-reduce of one flat gradient bucket" if train else ""),
                       "pipelining": ("coordinate side of step i+1 (SparseUNet.prepare) on a second stream beside step i"
                                      if r["pipelined"] else "none: one stream"),
                       "serial_ms_per_step": r["serial_ms_per_step"],
                       "device_allocs_in_timed_steps": r["device_allocs_in_timed_steps"],
                       "l2_policy": "activations of every level exceed L2"},
            "e2e": {"value": r["total_voxels"] / (r["e2e_ms_per_step"] * 1e-3), "unit": "voxels/s",
                    "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": 4, "ms_per_step": r["e2e_ms_per_step"]},
            "gpu_launches": r["launches"] * args.steps, "stages": per, "roofline": roof, "clocks": clocks,
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
    ap.add_argument("--passes", type=int, default=32, help="conv_layer_c3: passes of the hot path per step")
    ap.add_argument("--batches", type=int, default=4, help="conv_layer_c3: distinct seeded batches cycled through")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-pipeline", action="store_true",
                    help="conv_layer_c3: time the passes on one stream (no overlap of the next pass's coordinate side)")
    ap.add_argument("--no-legs", action="store_true", help="conv_layer_c3: skip the extra legs (variants, config 2, U-Net, reference on GPU)")
    ap.add_argument("--hashfly-in-kernel", action="store_true",
                    help="with --algo hashfly: probe the table inside the GEMM kernels instead of into a scratch map per call")
    ap.add_argument("--literal-decoder", action="store_true", help="unet_*: keep every child of the transposed convolutions")
    ap.add_argument("--unet-samples", type=int, default=0, dest="unet_samples",
                    help="unet_*: samples per rank instead of the BASELINE batch (8 inference / 16 training) split over the ranks")
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
