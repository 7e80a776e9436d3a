"""Per-component device timing of a decoder step with CUDA events — what the reference's hook timer does around its
modules (test/test_flh_inference.py:10-100, 195-216), here around named regions of the wiring.

    with timing.collect() as t:
        model(ids)
    t.summary()   ->  {"quant": ms, "gemm": ms, "allreduce": ms, "attention": ms, "glue": ms, "total": ms, "gaps": ms}

Outside `collect()` a region costs one `is None` test.  Events are recorded on the current stream; `gaps` is the part
of the step's device time that no region covers (idle time between launches: the host was not ahead of the GPU).
"""
from __future__ import annotations

import contextlib

import torch

_active = None


class Collector:
    def __init__(self):
        self.spans = []           # (name, start event, end event)
        self.t0 = self.t1 = None

    @contextlib.contextmanager
    def region(self, name):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        try:
            yield
        finally:
            b.record()
            self.spans.append((name, a, b))

    def summary(self):
        torch.cuda.synchronize()
        out = {}
        for name, a, b in self.spans:
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        total = self.t0.elapsed_time(self.t1)
        out["total"] = total
        out["gaps"] = total - sum(v for k, v in out.items() if k != "total")
        return out


@contextlib.contextmanager
def collect():
    global _active
    c = Collector()
    c.t0, c.t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    _active = c
    c.t0.record()
    try:
        yield c
    finally:
        c.t1.record()
        _active = None


_NULL = contextlib.nullcontext()


def region(name):
    return _NULL if _active is None else _active.region(name)
