"""Block rotation of the trainable adapters (Chroma's ``LayerRotator``,
crates/training/src/chroma/train.rs:338-362): only a window of consecutive transformer blocks is
trained at a time and the window moves every ``period`` optimizer steps, which bounds the
activation-gradient work and spreads a fixed budget over a deep model. Here a rotated-out block is
frozen through the optimizer's per-block learning-rate multiplier (0 = parameters and moments
untouched), so no module is re-wrapped and the parameter arena keeps its layout."""
from __future__ import annotations

import re

from ..optim.arena import block_lr_scale

_BLOCK_RE = re.compile(r"(?:double_blocks|single_blocks|blocks|layers)\.(\d+)\.")


def block_index(name: str, single_offset: int = 0):
    """Depth index of the block a parameter belongs to, or None (embedders, final layer). Single-
    stream blocks are numbered after the double-stream ones."""
    m = _BLOCK_RE.search(name)
    if not m:
        return None
    i = int(m.group(1))
    return i + single_offset if "single_blocks" in name else i


class LayerRotator:
    def __init__(self, names, window: int, period: int, single_offset: int = 0, always=()):
        self.names = list(names)
        self.window, self.period = window, max(1, period)
        self.idx = [block_index(n, single_offset) for n in self.names]
        self.depth = max((i for i in self.idx if i is not None), default=-1) + 1
        self.always = tuple(always)          # substrings of parameter names that always train
        self._last = None

    def active_range(self, step: int):
        if self.depth <= self.window:
            return 0, self.depth
        start = ((step // self.period) * self.window) % self.depth
        return start, start + self.window

    def is_active(self, name_index: int, step: int):
        i = self.idx[name_index]
        if i is None or any(a in self.names[name_index] for a in self.always):
            return True
        lo, hi = self.active_range(step)
        return lo <= i < hi or (hi > self.depth and i < hi - self.depth)      # window wraps around

    def apply(self, optimizer, arena, step: int, rules=None, shard=None):
        """Refresh ``optimizer.lr_scale`` when the window moved. Returns True when it changed."""
        key = self.active_range(step)
        if key == self._last:
            return False
        self._last = key
        active = {n for k, n in enumerate(self.names) if self.is_active(k, step)}
        optimizer.lr_scale = block_lr_scale(arena, self.names, rules, frozen=lambda n: n not in active,
                                            shard=shard)
        return True
