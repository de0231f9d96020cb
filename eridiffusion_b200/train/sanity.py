"""Training sanity checks: what is trainable, what is finite, what the optimizer touches.

Reference: ``ModelSanityChecker`` / ``run_training_sanity_checks`` / ``assert_optimizer_only_
touches_lora`` (src/trainers/trainer_sanity_checks.rs:24-172): base weights frozen and adapter
weights trainable, all weights finite and not extreme, no all-zero adapter pair, loss finite and
positive, gradients only on adapter tensors. The reference panics; here every check raises
``SanityError`` with the offending name, and the expensive ones (full scans of the weights) run at
step 0 and every ``expensive_every`` steps, as in the reference (every 100).

Finite checks reduce on the device (one ``isfinite().all()`` and one ``abs().max()`` per tensor)
instead of copying each tensor to the host.
"""
from __future__ import annotations

import math

import torch


class SanityError(AssertionError):
    pass


def _is_adapter(name: str, markers) -> bool:
    return any(m in name for m in markers)


class ModelSanityChecker:
    def __init__(self, named_tensors, adapter_markers=("lora", "adapter", "hada", "lokr", "ia3", "dora"),
                 extreme=1e4):
        self.named = list(named_tensors)
        self.markers, self.extreme = adapter_markers, extreme

    @classmethod
    def from_module(cls, module, **kw):
        return cls(module.named_parameters(), **kw)

    def assert_trainable_is_only_lora(self):
        for name, t in self.named:
            ad = _is_adapter(name, self.markers)
            if not ad and t.requires_grad:
                raise SanityError(f"base weight `{name}` is not frozen")
            if ad and not t.requires_grad:
                raise SanityError(f"adapter weight `{name}` is frozen")

    def assert_all_weights_finite(self):
        for name, t in self.named:
            if not t.is_floating_point() or t.numel() == 0:
                continue
            if not bool(torch.isfinite(t).all()):
                raise SanityError(f"weight `{name}` contains NaN or Inf")
            m = float(t.detach().abs().max())
            if m > self.extreme:
                raise SanityError(f"weight `{name}` has an extreme value {m:.3g} (limit {self.extreme:g})")

    def assert_no_zero_lora(self):
        """An adapter whose down- AND up-projection are both zero can never learn (the gradient of
        each is proportional to the other). One zero side is the normal initialisation."""
        pairs = {}
        for name, t in self.named:
            if not _is_adapter(name, self.markers):
                continue
            for a, b in ((".lora_A", ".lora_B"), (".lora_down", ".lora_up"), (".A", ".B")):
                for side, tag in ((0, a), (1, b)):
                    if name.endswith(tag) or name.endswith(tag + ".weight"):
                        key = name[: name.rindex(tag)]
                        pairs.setdefault(key, [None, None])[side] = bool((t == 0).all())
        for key, (za, zb) in pairs.items():
            if za and zb:
                raise SanityError(f"adapter `{key}` has both matrices at zero")

    def assert_loss_is_valid(self, loss):
        v = float(loss)
        if not math.isfinite(v):
            raise SanityError(f"loss is {v}")
        if v < 0:
            raise SanityError(f"loss is negative ({v})")

    def assert_only_lora_has_gradients(self, grads=None):
        """``grads``: optional {name: tensor}; defaults to the ``.grad`` fields."""
        for name, t in self.named:
            g = grads.get(name) if grads is not None else t.grad
            if g is None:
                continue
            if not _is_adapter(name, self.markers) and bool((g != 0).any()):
                raise SanityError(f"base weight `{name}` received a gradient")
            if not bool(torch.isfinite(g).all()):
                raise SanityError(f"gradient of `{name}` contains NaN or Inf")


def run_training_sanity_checks(checker: ModelSanityChecker, loss, step: int, grads=None, expensive_every=100):
    if step == 0 or (expensive_every and step % expensive_every == 0):
        checker.assert_trainable_is_only_lora()
        checker.assert_all_weights_finite()
        checker.assert_no_zero_lora()
    checker.assert_loss_is_valid(loss)
    checker.assert_only_lora_has_gradients(grads)


def assert_optimizer_only_touches_lora(optimizer_param_names, adapter_markers=("lora", "adapter", "hada", "lokr",
                                                                               "ia3", "dora")):
    for name in optimizer_param_names:
        if not _is_adapter(name, adapter_markers):
            raise SanityError(f"optimizer includes non-adapter weight `{name}`")
