"""Optimizers beyond 8-bit AdamW, a factory keyed by the reference's config strings, gradient
clipping and a multi-group wrapper.

The reference ships trait impls whose parameter writes are dropped
(crates/training/src/optimizer.rs:238-241, 305-308, 380-381, 441-444); these are working versions
with its defaults (lr 1e-4, wd 0.01, betas (0.9, 0.999), eps 1e-8; optimizer.rs:151-164) and its
name-substring weight-decay exclusion (optimizer.rs:278-297).
"""
from __future__ import annotations

import math

import torch
from torch.optim import Optimizer

from ..ops import _native as N
from ..ops import functional as F
from .adamw8bit import AdamW8bit
from .arena import ParamArena


class AdamWArena:
    """fp32-moment AdamW over a flat arena (single fused launch on CUDA)."""

    def __init__(self, params, lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                 stochastic_rounding=False, seed=0, shard=None):
        self.arena = params if isinstance(params, ParamArena) else ParamArena(list(params))
        self.betas, self.eps, self.weight_decay = betas, eps, weight_decay
        self.stochastic_rounding, self.seed, self.shard = stochastic_rounding, seed, shard
        self.step_count = 0
        data, _ = self._slices()
        self.m = torch.zeros(data.numel(), dtype=torch.float32, device=data.device)
        self.v = torch.zeros_like(self.m)
        self.param_groups = [{"lr": lr}]

    def _slices(self):
        return (self.arena.data, self.arena.grad) if self.shard is None else self.arena.shard(*self.shard)

    def zero_grad(self, set_to_none=False):
        self.arena.zero_grad()

    @torch.no_grad()
    def step(self, grad_sumsq=None, max_grad_norm=0.0, grad_scale=1.0):
        self.step_count += 1
        lr = self.param_groups[0]["lr"]
        data, grad = self._slices()
        b1, b2 = self.betas
        if data.is_cuda and F.get_backend() == "fused" and data.dtype in (torch.bfloat16, torch.float32):
            N.check(N.require().eri_adamw32_step(
                data.data_ptr(), grad.data_ptr(), self.m.data_ptr(), self.v.data_ptr(),
                N.ptr(grad_sumsq), data.numel(), 1 if data.dtype == torch.bfloat16 else 0, lr, b1,
                b2, self.eps, self.weight_decay, self.step_count, max_grad_norm, grad_scale,
                self.seed, 1 if self.stochastic_rounding else 0, N.stream_ptr()), "adamw32_step")
            return
        gs = grad_scale
        if grad_sumsq is not None and max_grad_norm > 0:
            gs *= min(1.0, max_grad_norm / (float(grad_sumsq) ** 0.5 * grad_scale + 1e-6))
        g = grad.float() * gs
        self.m.mul_(b1).add_(g, alpha=1 - b1)
        self.v.mul_(b2).addcmul_(g, g, value=1 - b2)
        bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
        upd = (self.m / bc1) / ((self.v / bc2).sqrt() + self.eps)
        data.copy_((data.float() * (1 - lr * self.weight_decay) - lr * upd).to(data.dtype))

    def state_dict(self):
        return {"step": self.step_count, "lr": self.param_groups[0]["lr"], "m": self.m, "v": self.v}

    def load_state_dict(self, sd):
        self.step_count = int(sd["step"])
        self.param_groups[0]["lr"] = float(sd["lr"])
        self.m.copy_(sd["m"]); self.v.copy_(sd["v"])

    def export_moments(self):
        return self.m, self.v


class Lion(Optimizer):
    """Sign-momentum optimizer (presets only in the reference: crates/training/src/optimizers/lion.rs)."""

    def __init__(self, params, lr=1e-4, betas=(0.9, 0.99), weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["m"] = torch.zeros_like(p, dtype=torch.float32)
                gr = p.grad.float()
                m = st["m"]
                upd = (m * b1 + gr * (1 - b1)).sign_()
                pf = p.float() * (1 - g["lr"] * g["weight_decay"]) - g["lr"] * upd
                p.copy_(pf.to(p.dtype))
                m.mul_(b2).add_(gr, alpha=1 - b2)


class Adafactor(Optimizer):
    """Factored second-moment optimizer (row/column statistics for matrices)."""

    def __init__(self, params, lr=1e-3, eps=(1e-30, 1e-3), clip_threshold=1.0, decay_rate=-0.8,
                 weight_decay=0.0):
        super().__init__(params, dict(lr=lr, eps=eps, clip_threshold=clip_threshold,
                                      decay_rate=decay_rate, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                gr = p.grad.float()
                st = self.state[p]
                factored = gr.dim() >= 2
                if not st:
                    st["step"] = 0
                    if factored:
                        st["row"] = torch.zeros(gr.shape[:-1], device=gr.device)
                        st["col"] = torch.zeros(gr.shape[:-2] + gr.shape[-1:], device=gr.device)
                    else:
                        st["v"] = torch.zeros_like(gr)
                st["step"] += 1
                beta2 = 1.0 - st["step"] ** g["decay_rate"]
                upd = gr * gr + g["eps"][0]
                if factored:
                    st["row"].mul_(beta2).add_(upd.mean(-1), alpha=1 - beta2)
                    st["col"].mul_(beta2).add_(upd.mean(-2), alpha=1 - beta2)
                    r = (st["row"] / st["row"].mean(-1, keepdim=True)).rsqrt().unsqueeze(-1)
                    c = st["col"].rsqrt().unsqueeze(-2)
                    u = gr * r * c
                else:
                    st["v"].mul_(beta2).add_(upd, alpha=1 - beta2)
                    u = gr * st["v"].rsqrt()
                u.div_((u.pow(2).mean().sqrt() / g["clip_threshold"]).clamp_(min=1.0))
                pf = p.float()
                if g["weight_decay"]:
                    pf.mul_(1 - g["lr"] * g["weight_decay"])
                p.copy_((pf - g["lr"] * u).to(p.dtype))


class Prodigy(Optimizer):
    """Adam with a distance estimate ``d`` that sets the step size automatically
    (the reference has the d-estimate and a stub step: crates/training/src/optimizers/prodigy.rs:496)."""

    def __init__(self, params, lr=1.0, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, d0=1e-6,
                 d_coef=1.0, growth_rate=float("inf")):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                      d=d0, d0=d0, d_max=d0, d_coef=d_coef, growth_rate=growth_rate,
                                      k=0))

    @torch.no_grad()
    def step(self, closure=None):
        g0 = self.param_groups[0]
        b1, b2 = g0["betas"]
        d, lr, k = g0["d"], g0["lr"], g0["k"]
        dlr = d * lr
        d_numer = g0.get("d_numer", 0.0) * math.sqrt(b2)
        d_denom = 0.0
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                gr = p.grad.float()
                st = self.state[p]
                if not st:
                    st["p0"] = p.detach().float().clone()
                    st["m"] = torch.zeros_like(gr)
                    st["v"] = torch.zeros_like(gr)
                    st["s"] = torch.zeros_like(gr)
                d_numer += (d / g0["d0"]) * dlr * torch.dot(gr.flatten(), (st["p0"] - p.float()).flatten()).item()
                st["m"].mul_(b1).add_(gr, alpha=d * (1 - b1))
                st["v"].mul_(b2).addcmul_(gr, gr, value=d * d * (1 - b2))
                st["s"].mul_(math.sqrt(b2)).add_(gr, alpha=(d / g0["d0"]) * dlr)
                d_denom += st["s"].abs().sum().item()
        if d_denom > 0:
            d_hat = g0["d_coef"] * d_numer / d_denom
            if d == g0["d0"]:
                d = max(d, d_hat)
            g0["d_max"] = max(g0["d_max"], d_hat)
            d = min(g0["d_max"], d * g0["growth_rate"])
        for g in self.param_groups:
            g["d"], g["d_numer"], g["k"] = d, d_numer, k + 1
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                denom = st["v"].sqrt().add_(d * g["eps"])
                pf = p.float()
                if g["weight_decay"]:
                    pf.mul_(1 - dlr * g["weight_decay"])
                p.copy_((pf - dlr * st["m"] / denom).to(p.dtype))


class RAdamScheduleFree(Optimizer):
    """Schedule-free RAdam: keeps a base sequence ``z`` and an averaged sequence ``x``; gradients
    are taken at the interpolation ``y``. ``train()`` / ``eval()`` swap the stored point
    (crates/training/src/optimizers/radam_schedulefree.rs:8-189)."""

    def __init__(self, params, lr=2.5e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                      k=0, train_mode=True, lr_sum=0.0))

    @torch.no_grad()
    def _swap(self, to_train):
        for g in self.param_groups:
            if g["train_mode"] == to_train:
                continue
            b1 = g["betas"][0]
            for p in g["params"]:
                st = self.state[p]
                if "z" in st:
                    w = (1 - b1) if to_train else (1 - 1 / b1)
                    p.copy_(torch.lerp(p.float(), st["z"], w).to(p.dtype))
            g["train_mode"] = to_train

    def train(self):
        self._swap(True)

    def eval(self):
        self._swap(False)

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            g["k"] += 1
            k = g["k"]
            bc2 = 1 - b2 ** k
            rho_inf = 2 / (1 - b2) - 1
            rho = rho_inf - 2 * k * b2 ** k / bc2
            rect = math.sqrt((rho - 4) * (rho - 2) * rho_inf / ((rho_inf - 4) * (rho_inf - 2) * rho)) \
                if rho > 4 else 0.0
            lr = g["lr"] * (rect if rho > 4 else 1.0)
            g["lr_sum"] += lr ** 2
            ckp1 = lr ** 2 / g["lr_sum"] if g["lr_sum"] > 0 else 0.0
            for p in g["params"]:
                if p.grad is None:
                    continue
                gr = p.grad.float()
                st = self.state[p]
                if not st:
                    st["z"] = p.detach().float().clone()
                    st["v"] = torch.zeros_like(gr)
                st["v"].mul_(b2).addcmul_(gr, gr, value=1 - b2)
                gn = gr / ((st["v"] / bc2).sqrt() + g["eps"]) if rho > 4 else gr
                y = p.float()
                if g["weight_decay"]:
                    gn = gn + g["weight_decay"] * y
                y = torch.lerp(y, st["z"], ckp1).add_(gn, alpha=lr * (b1 * (1 - ckp1) - 1))
                st["z"].sub_(gn, alpha=lr)
                p.copy_(y.to(p.dtype))


class CPUOffloadedAdamW:
    """AdamW whose moments live in pinned host memory; gradients are copied down, updated on the
    host and the parameters copied back (src/trainers/cpu_offload_manager.rs:188-311)."""

    def __init__(self, params, lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01):
        self.params = [p for p in params if p.requires_grad]
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        pin = torch.cuda.is_available()
        self.m = [torch.zeros(p.shape, dtype=torch.float32, pin_memory=pin) for p in self.params]
        self.v = [torch.zeros(p.shape, dtype=torch.float32, pin_memory=pin) for p in self.params]
        self.master = [p.detach().float().cpu() for p in self.params]
        self.step_count = 0
        self.param_groups = [{"lr": lr}]

    def zero_grad(self, set_to_none=True):
        for p in self.params:
            p.grad = None

    @torch.no_grad()
    def step(self):
        self.step_count += 1
        b1, b2 = self.betas
        lr = self.param_groups[0]["lr"]
        bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
        for p, m, v, w in zip(self.params, self.m, self.v, self.master):
            if p.grad is None:
                continue
            g = p.grad.detach().float().cpu()
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            w.mul_(1 - lr * self.wd).addcdiv_(m / bc1, (v / bc2).sqrt() + self.eps, value=-lr)
            p.copy_(w.to(p.device, p.dtype, non_blocking=True))


class MultiOptimizer:
    """Several optimizers stepped together, one per parameter group
    (src/flame_training.rs:110-186)."""

    def __init__(self, optimizers: dict):
        self.optimizers = optimizers

    def step(self, *a, **kw):
        for o in self.optimizers.values():
            o.step(*a, **kw)

    def zero_grad(self, set_to_none=False):
        for o in self.optimizers.values():
            o.zero_grad(set_to_none)

    @property
    def param_groups(self):
        return [g for o in self.optimizers.values() for g in o.param_groups]

    def state_dict(self):
        return {k: o.state_dict() for k, o in self.optimizers.items()}

    def load_state_dict(self, sd):
        for k, o in self.optimizers.items():
            o.load_state_dict(sd[k])


def split_weight_decay(named_params, exclude=("bias", "norm", "scale", "ln_", "embedding")):
    """Two groups: decayed and non-decayed, by name substring (optimizer.rs:278-297)."""
    decay, no_decay = [], []
    for n, p in named_params:
        if not p.requires_grad:
            continue
        (no_decay if any(s in n.lower() for s in exclude) or p.dim() < 2 else decay).append(p)
    return decay, no_decay


def create_optimizer(name, params, lr=1e-4, weight_decay=0.01, betas=(0.9, 0.999), eps=1e-8, **kw):
    """Factory keyed by the reference's strings: adamw8bit / adamw_8bit (block-wise 8-bit), adamw,
    adam, sgd, lion, adafactor, prodigy, radam_schedulefree, adamw_cpu
    (src/optimizers/memory_efficient_optimizers.rs:285-308, crates/training/src/optimizer.rs:179-192)."""
    n = name.lower().replace("-", "_")
    if n in ("adamw8bit", "adamw_8bit", "adam8bit", "adam_8bit"):
        return AdamW8bit(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, **kw)
    if n in ("adamw", "adamw_fused", "adamw_arena"):
        return AdamWArena(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, **kw)
    plist = params.params if isinstance(params, ParamArena) else list(params)
    if n == "adam":
        return torch.optim.Adam(plist, lr=lr, betas=betas, eps=eps, weight_decay=0.0)
    if n == "sgd":
        return torch.optim.SGD(plist, lr=lr, momentum=kw.get("momentum", 0.9), weight_decay=weight_decay)
    if n == "lion":
        return Lion(plist, lr=lr, betas=kw.get("lion_betas", (0.9, 0.99)), weight_decay=weight_decay)
    if n == "adafactor":
        return Adafactor(plist, lr=lr, weight_decay=weight_decay)
    if n == "prodigy":
        return Prodigy(plist, lr=kw.get("prodigy_lr", 1.0), betas=betas, eps=eps, weight_decay=weight_decay)
    if n in ("radam_schedulefree", "radam_schedule_free", "schedulefree"):
        return RAdamScheduleFree(plist, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
    if n in ("adamw_cpu", "adamw_cpu_offload"):
        return CPUOffloadedAdamW(plist, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
    raise ValueError(f"unknown optimizer {name!r}")


@torch.no_grad()
def clip_grad_norm_(params, max_norm: float, arena: ParamArena | None = None):
    """Global L2 clip. With an arena: one sum-of-squares launch and one scale launch, the norm stays
    on the device. Returns the (device) norm tensor. (The reference copies one scalar to the host
    per tensor: crates/training/src/optimizer.rs:88-123.)"""
    if arena is not None:
        ss = F.sumsq(arena.grad)
        if arena.grad.is_cuda and arena.grad.dtype == torch.bfloat16 and F.get_backend() == "fused":
            N.check(N.require().eri_scale_bf16(arena.grad.data_ptr(), arena.grad.numel(),
                                               ss.data_ptr(), max_norm, 1.0, N.stream_ptr()), "scale")
        else:
            arena.grad.mul_(torch.clamp(max_norm / (ss.sqrt() + 1e-6), max=1.0).to(arena.grad.dtype))
        return ss.sqrt()
    grads = [p.grad for p in params if p.grad is not None]
    norm = torch.sqrt(sum(g.float().pow(2).sum() for g in grads))
    coef = torch.clamp(max_norm / (norm + 1e-6), max=1.0)
    for g in grads:
        g.mul_(coef.to(g.dtype))
    return norm
