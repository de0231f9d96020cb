"""Named ranges and per-phase device timing.

``range(name)`` is a context manager that opens an NVTX range (visible in any NVTX-aware timeline
tool) when ``ERI_B200_NVTX=1`` and does nothing otherwise; ``annotate_blocks(model)`` wraps every
transformer block's forward in one. ``PhaseTimer`` is the device-timed equivalent of the
reference's ``SDXL_PHASE_TIMING`` breakdown (crates/training/src/sdxl/runtime.rs:323-361, which
wraps phases in host timers after a device sync): phases are bracketed by CUDA events on the
current stream, nothing synchronises until ``summary()`` is read.
"""
from __future__ import annotations

import contextlib
import os
from collections import OrderedDict

import torch

builtins_range = range          # the module defines its own ``range`` context manager below

_NVTX = os.environ.get("ERI_B200_NVTX") == "1"


def nvtx_enabled() -> bool:
    return _NVTX and torch.cuda.is_available()


def enable_nvtx(on: bool = True) -> None:
    global _NVTX
    _NVTX = on


@contextlib.contextmanager
def range(name: str):                                     # noqa: A001 - mirrors torch.cuda.nvtx.range
    if nvtx_enabled():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


def annotate_blocks(model, attrs=("double_blocks", "single_blocks", "blocks", "layers")):
    """Forward pre/post hooks that open one range per block, named ``<list>.<index>``.
    Returns the hook handles (call ``.remove()`` on each to undo)."""
    handles = []
    for a in attrs:
        for i, blk in enumerate(getattr(model, a, []) or []):
            name = f"{a}.{i}"
            handles.append(blk.register_forward_pre_hook(
                lambda m, inp, _n=name: torch.cuda.nvtx.range_push(_n) if nvtx_enabled() else None))
            handles.append(blk.register_forward_hook(
                lambda m, inp, out: torch.cuda.nvtx.range_pop() if nvtx_enabled() else None))
    return handles


class PhaseTimer:
    """``with timer.phase("forward"): ...`` records the phase between two events (host clock on a
    machine without a GPU). ``summary()`` synchronises once and returns total milliseconds, call
    count and share per phase."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled
        self._cuda = torch.cuda.is_available()
        self._pending = []                                # (name, start, end)
        self._acc = OrderedDict()                         # name -> [ms, calls]

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        with range(name):
            if self._cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                try:
                    yield
                finally:
                    e1.record()
                    self._pending.append((name, e0, e1))
            else:
                import time
                t0 = time.perf_counter()
                try:
                    yield
                finally:
                    self._add(name, (time.perf_counter() - t0) * 1e3)

    def _add(self, name, ms):
        a = self._acc.setdefault(name, [0.0, 0])
        a[0] += ms
        a[1] += 1

    def summary(self, reset: bool = False):
        if self._pending:
            torch.cuda.synchronize()
            for name, e0, e1 in self._pending:
                self._add(name, e0.elapsed_time(e1))
            self._pending = []
        total = sum(v[0] for v in self._acc.values()) or 1.0
        out = {k: {"ms": v[0], "calls": v[1], "share": v[0] / total} for k, v in self._acc.items()}
        if reset:
            self._acc = OrderedDict()
        return out

    def format(self):
        s = self.summary()
        return "  ".join(f"{k} {v['ms'] / max(1, v['calls']):.2f} ms ({100 * v['share']:.0f}%)" for k, v in s.items())


def profile_steps(step_fn, n_steps: int, out_path, warmup: int = 1, with_stack: bool = False):
    """Run ``step_fn()`` ``warmup + n_steps`` times under ``torch.profiler`` (CPU activity, plus CUDA
    when a GPU is present), write a Chrome trace to ``out_path`` and return the per-kernel / per-op
    table as text. A diagnostic: timings taken under the profiler are not benchmark numbers."""
    from torch.profiler import ProfilerActivity, profile
    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
    for _ in builtins_range(warmup):
        step_fn()
    with profile(activities=acts, with_stack=with_stack) as prof:
        for i in builtins_range(n_steps):
            with range(f"step {i}"):
                step_fn()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
    prof.export_chrome_trace(str(out_path))
    key = "cuda_time_total" if torch.cuda.is_available() else "cpu_time_total"
    return prof.key_averages().table(sort_by=key, row_limit=30)
