"""Strict-bf16 guard: counts the events that silently cost memory or precision inside a block —
extra copies made to fix a layout (``layout_fixes``), clones (``clone_allocs``), and bf16 -> fp32
up-casts of whole activations (``f32_graph_casts``) — so tests can assert they stay zero.

The reference exposes the same three counters through flame-core's ``strict::scope`` /
``telemetry_snapshot`` / ``reset_counters`` and asserts them in tests/strict_mmdit_block.rs:8-80.
Here the counters are fed by a ``TorchDispatchMode`` that watches the dispatched ATen ops while
the scope is active; ``GuardMode.PANIC`` raises at the first event instead of counting."""
from __future__ import annotations

import contextlib
from dataclasses import dataclass, field

import torch
from torch.utils._python_dispatch import TorchDispatchMode


@dataclass
class StrictCounters:
    clone_allocs: int = 0
    f32_graph_casts: int = 0
    layout_fixes: int = 0
    events: list = field(default_factory=list)

    def reset(self):
        self.clone_allocs = self.f32_graph_casts = self.layout_fixes = 0
        self.events.clear()

    def snapshot(self) -> dict:
        return {"clone_allocs": self.clone_allocs, "f32_graph_casts": self.f32_graph_casts,
                "layout_fixes": self.layout_fixes}


strict_counters = StrictCounters()


class StrictViolation(RuntimeError):
    pass


class StrictScope(TorchDispatchMode):
    """Counts (or rejects) clones, layout-fixing copies and activation up-casts of tensors with at
    least ``min_numel`` elements (small scalars and statistics are not activations)."""

    def __init__(self, panic=False, min_numel=4096, counters: StrictCounters | None = None):
        super().__init__()
        self.panic, self.min_numel = panic, min_numel
        self.counters = counters or strict_counters

    def _hit(self, kind, op, t):
        setattr(self.counters, kind, getattr(self.counters, kind) + 1)
        self.counters.events.append((kind, str(op), tuple(t.shape)))
        if self.panic:
            raise StrictViolation(f"{kind}: {op} on tensor {tuple(t.shape)} {t.dtype}")

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        name = func.overloadpacket.__name__ if hasattr(func, "overloadpacket") else str(func)
        src = args[0] if args and isinstance(args[0], torch.Tensor) else None
        if src is not None and src.numel() >= self.min_numel:
            if name == "clone":
                fmt = kwargs.get("memory_format")
                if fmt in (torch.contiguous_format, torch.channels_last) and not src.is_contiguous(
                        memory_format=fmt):
                    self._hit("layout_fixes", name, src)      # .contiguous() of a strided view
                else:
                    self._hit("clone_allocs", name, src)
            elif name in ("_to_copy", "to"):
                dt = kwargs.get("dtype")
                if dt is None and len(args) > 1 and isinstance(args[1], torch.dtype):
                    dt = args[1]
                if dt == torch.float32 and src.dtype in (torch.bfloat16, torch.float16):
                    self._hit("f32_graph_casts", name, src)
        return func(*args, **kwargs)


@contextlib.contextmanager
def strict_scope(panic=False, min_numel=4096, reset=True):
    """``with strict_scope() as c: block(x)``; then ``c.snapshot()``."""
    if reset:
        strict_counters.reset()
    with StrictScope(panic=panic, min_numel=min_numel):
        yield strict_counters
