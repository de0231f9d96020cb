"""Mixed-precision policy objects: configuration, master-weight optimizer wrapper, autocast
context, memory estimate.

Reference: ``MixedPrecisionConfig{enabled, dtype, loss_scale (static | dynamic), gradient_clipping,
opt_level O0..O3}``, ``GradScaler`` (in ``optim/schedulers.py`` here), ``MixedPrecisionOptimizer``
with fp32 master parameters, ``AMPContext`` with white / black lists of ops and ``MemoryEstimate``
(crates/training/src/mixed_precision.rs:12-429).

On B200 the training path stores bf16 parameters and computes in bf16 with fp32 accumulation inside
every kernel; the 8-bit optimizer applies its update with stochastic rounding, so the default
policy needs neither a loss scale nor master copies. These classes exist for the other policies the
reference names: fp16 parameters with dynamic loss scaling, or bf16 parameters with fp32 masters
when bit-exact accumulation of tiny updates matters more than memory.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass, field

import torch

from ..optim import GradScaler

OPT_LEVELS = ("O0", "O1", "O2", "O3")


@dataclass
class LossScaleConfig:
    kind: str = "dynamic"                   # dynamic | static
    init_scale: float = 2048.0
    growth_factor: float = 2.0
    backoff_factor: float = 0.5
    growth_interval: int = 2000

    @classmethod
    def static(cls, scale: float):
        return cls("static", scale)


@dataclass
class MixedPrecisionConfig:
    enabled: bool = False
    dtype: str = "float16"                  # float16 | bfloat16
    loss_scale: LossScaleConfig = field(default_factory=LossScaleConfig)
    gradient_clipping: float | None = 1.0
    opt_level: str = "O1"

    def __post_init__(self):
        if self.dtype not in ("float16", "bfloat16"):
            raise ValueError(f"mixed-precision dtype {self.dtype!r}")
        if self.opt_level not in OPT_LEVELS:
            raise ValueError(f"opt_level {self.opt_level!r} not in {OPT_LEVELS}")

    @property
    def torch_dtype(self):
        return torch.float16 if self.dtype == "float16" else torch.bfloat16

    def make_scaler(self) -> GradScaler:
        ls = self.loss_scale
        needs_scale = self.enabled and self.dtype == "float16" and self.opt_level != "O0"
        if ls.kind == "static":
            return GradScaler(init_scale=ls.init_scale, growth_factor=1.0, backoff_factor=1.0,
                              growth_interval=1 << 62, enabled=needs_scale)
        return GradScaler(ls.init_scale, ls.growth_factor, ls.backoff_factor, ls.growth_interval, enabled=needs_scale)


class MixedPrecisionOptimizer:
    """fp32 master copies of low-precision parameters. ``step()``: un-scale the gradients into the
    masters' ``.grad``, skip on inf / NaN (the scaler backs off), clip, step the wrapped optimizer
    (which must have been built over ``master_params``) and copy the masters back."""

    def __init__(self, optimizer_factory, model_params, scaler: GradScaler | None = None,
                 gradient_clipping: float | None = None):
        self.model_params = [p for p in model_params if p.requires_grad]
        self.master_params = [p.detach().float().clone().requires_grad_(True) for p in self.model_params]
        self.optimizer = optimizer_factory(self.master_params)
        self.scaler = scaler or GradScaler(enabled=False)
        self.gradient_clipping = gradient_clipping
        self.skipped_steps = 0

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    def scale_loss(self, loss):
        return self.scaler.scale_loss(loss)

    @torch.no_grad()
    def step(self) -> bool:
        inv = 1.0 / self.scaler.scale if self.scaler.enabled else 1.0
        sumsq = torch.zeros((), dtype=torch.float32, device=self.master_params[0].device)
        for m, p in zip(self.master_params, self.model_params):
            m.grad = None if p.grad is None else p.grad.float() * inv
            if m.grad is not None:
                sumsq += m.grad.pow(2).sum()
        ok = self.scaler.check(sumsq)
        self.scaler.update()
        if not ok:
            self.skipped_steps += 1
            self.zero_grad()
            return False
        if self.gradient_clipping:
            torch.nn.utils.clip_grad_norm_(self.master_params, self.gradient_clipping)
        self.optimizer.step()
        for m, p in zip(self.master_params, self.model_params):
            p.copy_(m.to(p.dtype))
        return True

    def zero_grad(self):
        for p in self.model_params:
            p.grad = None
        for m in self.master_params:
            m.grad = None

    def state_dict(self):
        return {"optimizer": self.optimizer.state_dict(), "scaler": self.scaler.state_dict(),
                "master_params": [m.detach().clone() for m in self.master_params]}

    def load_state_dict(self, sd):
        self.optimizer.load_state_dict(sd["optimizer"])
        self.scaler.load_state_dict(sd["scaler"])
        with torch.no_grad():
            for m, s in zip(self.master_params, sd["master_params"]):
                m.copy_(s)


class AMPContext:
    """Which ops run in the low-precision dtype. ``autocast()`` is a context manager for library
    (non-kernel) code paths such as VAE or text-encoder passes; the framework's own kernels take
    bf16 inputs directly and ignore it."""

    def __init__(self, config: MixedPrecisionConfig, device="cuda"):
        self.enabled = config.enabled and config.opt_level != "O0"
        self.dtype = config.torch_dtype
        self.device_type = torch.device(device).type
        self.whitelist = ["matmul", "conv2d", "linear", "attention"]
        self.blacklist = ["softmax", "layer_norm", "group_norm", "loss", "exp", "log"]
        if config.opt_level in ("O2", "O3"):
            self.whitelist += ["layer_norm", "group_norm"]
            self.blacklist = [b for b in self.blacklist if b not in ("layer_norm", "group_norm")]

    def should_cast(self, op_name: str) -> bool:
        if not self.enabled:
            return False
        if any(b in op_name for b in self.blacklist):
            return False
        return any(w in op_name for w in self.whitelist)

    def cast(self, op_name: str, *tensors):
        dt = self.dtype if self.should_cast(op_name) else torch.float32
        out = tuple(t.to(dt) if torch.is_tensor(t) and t.is_floating_point() else t for t in tensors)
        return out[0] if len(out) == 1 else out

    def autocast(self):
        if not self.enabled:
            return contextlib.nullcontext()
        return torch.autocast(self.device_type, dtype=self.dtype)


@dataclass
class MemoryEstimate:
    fp32_total: int
    mp_total: int
    savings_percent: float


def estimate_memory(num_params: int, activation_elems: int, config: MixedPrecisionConfig, optimizer_state_per_param=8,
                    master_weights: bool = True) -> MemoryEstimate:
    """fp32: 4 B weights + 4 B grads + optimizer state + 4 B activations. Mixed: 2 B weights and
    grads (+ 4 B masters), the same optimizer state, 2 B activations."""
    fp32 = num_params * (8 + optimizer_state_per_param) + activation_elems * 4
    if not config.enabled or config.opt_level == "O0":
        return MemoryEstimate(fp32, fp32, 0.0)
    mp = num_params * (4 + (4 if master_weights else 0) + optimizer_state_per_param) + activation_elems * 2
    return MemoryEstimate(fp32, mp, 100.0 * (fp32 - mp) / max(1, fp32))
