"""Block-wise 8-bit AdamW over a flat parameter arena.

State per 256-element block: int8 first-moment codes, uint8 second-moment codes and one fp32
absmax per moment. Codes are power-law companded: ``m = sign(q) (|q|/127)^2 absmax_m`` and
``v = (q/255)^4 absmax_v`` — square-root / fourth-root spacing keeps relative precision over the
wide dynamic range of Adam moments without a lookup table. Update order per step: dequantise,
AdamW in fp32 (decoupled weight decay, bias correction), requantise, write the parameter
(bf16, optional stochastic rounding since there is no fp32 master copy).

On CUDA the whole step is one kernel launch (``csrc/optim.cu``) that also applies the global-norm
clip coefficient from a device scalar; the PyTorch statement below is the oracle and CPU path.

Reference: tensor-wise absmax/127.5 symmetric codes updated with a dequant -> fp32 Adam -> requant
round trip (src/trainers/adam8bit.rs:101-241); the "enhanced" variant declares ``block_wise`` but
implements none (src/trainers/adam8bit_enhanced.rs:373-395). State-dict contract kept: per-arena
``m``/``v`` codes + scales, ``step``, lr/betas/eps/weight_decay (adam8bit.rs:38-47, 269-329).
"""
from __future__ import annotations

import torch

from ..ops import _native as N
from ..ops import functional as F
from .arena import ParamArena

BLOCK = 256


def quantize_m(m, block=BLOCK):
    mb = m.view(-1, block)
    amax = mb.abs().amax(1)
    inv = torch.where(amax > 0, 1.0 / amax, torch.zeros_like(amax))
    a = (mb.abs() * inv[:, None]).clamp(max=1.0).sqrt()
    q = torch.round(a * 127.0) * torch.sign(mb)
    return q.to(torch.int8).view(-1), amax


def dequantize_m(q, amax, block=BLOCK):
    qf = q.view(-1, block).float()
    a = qf.abs() / 127.0
    return (torch.sign(qf) * a * a * amax[:, None]).view(-1)


def quantize_v(v, block=BLOCK):
    vb = v.view(-1, block)
    amax = vb.amax(1)
    inv = torch.where(amax > 0, 1.0 / amax, torch.zeros_like(amax))
    a = (vb * inv[:, None]).clamp(max=1.0).sqrt().sqrt()
    q = torch.round(a * 255.0)
    q = torch.where((q == 0) & (vb > 0), torch.ones_like(q), q)
    return q.to(torch.uint8).view(-1), amax


def dequantize_v(q, amax, block=BLOCK):
    a = q.view(-1, block).float() / 255.0
    a = a * a
    return (a * a * amax[:, None]).view(-1)


class AdamW8bit:
    """optimizer over ``ParamArena`` (or a list of parameters, which is packed into one)."""

    def __init__(self, params, lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                 stochastic_rounding=True, seed=0, shard=None):
        self.arena = params if isinstance(params, ParamArena) else ParamArena(list(params))
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.stochastic_rounding = stochastic_rounding
        self.seed = seed
        self.step_count = 0
        # `shard` = (rank, world): state covers this rank's slice of the arena only (ZeRO-1/2)
        self.shard = shard
        data, _ = self._slices()
        n = data.numel()
        dev = data.device
        self.m_q = torch.zeros(n, dtype=torch.int8, device=dev)
        self.v_q = torch.zeros(n, dtype=torch.uint8, device=dev)
        self.m_absmax = torch.zeros(n // BLOCK, dtype=torch.float32, device=dev)
        self.v_absmax = torch.zeros(n // BLOCK, dtype=torch.float32, device=dev)
        self.param_groups = [{"lr": lr}]       # so LR schedulers can drive it
        self.lr_scale = None                   # optional fp32 [n / 256] per-block LR multiplier

    def _slices(self):
        if self.shard is None:
            return self.arena.data, self.arena.grad
        return self.arena.shard(*self.shard)

    def zero_grad(self, set_to_none=False):
        self.arena.zero_grad()

    @torch.no_grad()
    def step(self, grad_sumsq=None, max_grad_norm=0.0, grad_scale=1.0):
        """One update. ``grad_sumsq``: optional device fp32 scalar with the squared global gradient
        norm (before ``grad_scale``); with ``max_grad_norm > 0`` the clip happens inside the
        kernel, with no host synchronisation."""
        self.step_count += 1
        lr = self.param_groups[0]["lr"]
        data, grad = self._slices()
        b1, b2 = self.betas
        if data.is_cuda and data.dtype == torch.bfloat16 and F.get_backend() == "fused":
            lib = N.require()
            N.check(lib.eri_adamw8bit_step_scaled(
                data.data_ptr(), grad.data_ptr(), self.m_q.data_ptr(), self.v_q.data_ptr(),
                self.m_absmax.data_ptr(), self.v_absmax.data_ptr(), N.ptr(grad_sumsq),
                data.numel(), lr, b1, b2, self.eps, self.weight_decay, self.step_count,
                max_grad_norm, grad_scale, self.seed, 1 if self.stochastic_rounding else 0,
                N.ptr(self.lr_scale), N.stream_ptr()), "adamw8bit_step")
            return
        self._step_reference(data, grad, lr, grad_sumsq, max_grad_norm, grad_scale)

    def _step_reference(self, data, grad, lr, grad_sumsq, max_grad_norm, grad_scale):
        b1, b2 = self.betas
        gs = grad_scale
        if grad_sumsq is not None and max_grad_norm > 0:
            norm = float(grad_sumsq) ** 0.5 * grad_scale
            gs *= min(1.0, max_grad_norm / (norm + 1e-6))
        g = grad.float() * gs
        m0 = dequantize_m(self.m_q, self.m_absmax)
        v0 = dequantize_v(self.v_q, self.v_absmax)
        m = b1 * m0 + (1 - b1) * g
        v = b2 * v0 + (1 - b2) * g * g
        bc1 = 1 - b1 ** self.step_count
        bc2 = 1 - b2 ** self.step_count
        upd = (m / bc1) / ((v / bc2).sqrt() + self.eps)
        lr_e = lr
        if self.lr_scale is not None:          # per-block multiplier; zero freezes the block
            lr_e = lr * self.lr_scale.to(data.device).repeat_interleave(BLOCK)[: data.numel()]
            frozen = lr_e == 0
            m, v = torch.where(frozen, m0, m), torch.where(frozen, v0, v)
        p = data.float() * (1 - lr_e * self.weight_decay) - lr_e * upd
        data.copy_(p.to(data.dtype))
        mq, ma = quantize_m(m)
        vq, va = quantize_v(v)
        self.m_q.copy_(mq); self.m_absmax.copy_(ma)
        self.v_q.copy_(vq); self.v_absmax.copy_(va)

    # ------------------------------------------------------------------ state
    def state_dict(self):
        return {"step": self.step_count, "lr": self.param_groups[0]["lr"], "betas": self.betas,
                "eps": self.eps, "weight_decay": self.weight_decay, "block": BLOCK,
                "m_q": self.m_q, "v_q": self.v_q, "m_absmax": self.m_absmax,
                "v_absmax": self.v_absmax, "shard": self.shard}

    def load_state_dict(self, sd):
        self.step_count = int(sd["step"])
        self.param_groups[0]["lr"] = float(sd["lr"])
        for k in ("m_q", "v_q", "m_absmax", "v_absmax"):
            getattr(self, k).copy_(sd[k].to(getattr(self, k).device))

    def state_bytes(self):
        return self.m_q.numel() * 2 + self.m_absmax.numel() * 8

    # moments as fp32 maps, the reference's checkpoint contract
    # (crates/training/src/optimizer.rs:40-54 export_mv_as_map / import_mv_from_map)
    def export_moments(self):
        return dequantize_m(self.m_q, self.m_absmax), dequantize_v(self.v_q, self.v_absmax)

    def import_moments(self, m, v):
        mq, ma = quantize_m(m.float())
        vq, va = quantize_v(v.float())
        self.m_q.copy_(mq); self.m_absmax.copy_(ma)
        self.v_q.copy_(vq); self.v_absmax.copy_(va)
