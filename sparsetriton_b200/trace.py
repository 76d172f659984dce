"""Per-stage device timing of the hot path.

    with trace.recording() as rec:
        ... run convolutions ...
    rec.summary()  -> {stage: {"calls": n, "ms": total, "launches": n_kernels, "work": flops or bytes}}

Each C-ABI call site is wrapped in `trace.stage(name)`.  When no recording is active the wrapper
does nothing; when one is, it brackets the call with CUDA events on the current stream (the stream
the kernels are launched on) and reads the library's own launch counter before and after, so
"launches" is the number of kernels the library really enqueued.
"""
import contextlib

import torch

from sparsetriton_b200 import _lib

_active = None


class Recording:
    def __init__(self):
        self.spans = []          # (name, start_event, end_event, launches, algorithmic work, tag)

    def summary(self):
        torch.cuda.synchronize()
        out = {}
        for name, a, b, launches, work, _tag in self.spans:
            e = out.setdefault(name, {"calls": 0, "ms": 0.0, "launches": 0, "work": 0.0})
            e["calls"] += 1
            e["ms"] += a.elapsed_time(b)
            e["launches"] += launches
            e["work"] += work
        return out

    def by_tag(self):
        """{(stage, tag): {"calls", "ms", "work"}} over the spans that carry a tag (the products tag their channel widths)."""
        torch.cuda.synchronize()
        out = {}
        for name, a, b, _launches, work, tag in self.spans:
            if tag is None:
                continue
            e = out.setdefault((name, tag), {"calls": 0, "ms": 0.0, "work": 0.0})
            e["calls"] += 1
            e["ms"] += a.elapsed_time(b)
            e["work"] += work
        return out

    def total_launches(self):
        return sum(s[3] for s in self.spans)


@contextlib.contextmanager
def recording():
    global _active
    prev, _active = _active, Recording()
    try:
        yield _active
    finally:
        _active = prev


def active():
    """True while a recording is open (call sites use it to skip bookkeeping that costs a sync)."""
    return _active is not None


def map_pairs(neighbor_indices):
    """Number of valid entries of a neighbour map, memoised on the tensor (one device->host read)."""
    n = getattr(neighbor_indices, "_st_pairs", None)
    if n is None:
        n = int((neighbor_indices >= 0).sum().item())
        neighbor_indices._st_pairs = n
    return n


_NULL_CONTEXT = contextlib.nullcontext()


def stage(name, launches=None, work=0.0, tag=None):
    """Context manager around one C-ABI call site: nothing when no recording is open."""
    if _active is None:
        return _NULL_CONTEXT
    return _recorded_stage(name, launches, work, tag)


@contextlib.contextmanager
def _recorded_stage(name, launches, work, tag):
    rec = _active
    counter = _lib.lib().st_launch_count
    a = torch.cuda.Event(enable_timing=True)
    b = torch.cuda.Event(enable_timing=True)
    before = counter()
    a.record()
    try:
        yield
    finally:
        b.record()
        rec.spans.append((name, a, b, counter() - before, float(work), tag))
