"""Adapter family attached to ``models.layers.Linear`` (and Conv2d for LoCon).

LoRA runs through the fused linear kernel (down-projection launch + rank-r K-step inside the base
GEMM); the other kinds build a weight-space delta ``W' = W + dW(params)`` and run one GEMM, which
is how the reference's adapter crate defines them (crates/adapters/src/kinds/lora.rs:16-46,
loha.rs:19-27, lokr.rs:13-15, dora.rs:23-28, ia3.rs:12-17, locon2d.rs:19-42).
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..ops import functional as F
from ..models.layers import Linear


@dataclass
class AdapterConfig:
    kind: str = "lora"            # lora | dora | loha | lokr | ia3 | locon | glora
    rank: int = 16
    alpha: float | None = None    # default: rank (scale 1)
    dropout: float = 0.0
    init: str = "kaiming"         # "kaiming" | "reference" (A ~ N(0, 1/sqrt(r)), flux/lora.rs:22-44) | "nonzero" (B small, not zero)
    target: list[str] = field(default_factory=lambda: [r".*"])   # regexes on module paths
    exclude: list[str] = field(default_factory=list)
    rank_pattern: dict[str, int] = field(default_factory=dict)   # regex -> rank override
    lokr_factor: int = 8
    dtype: torch.dtype = torch.bfloat16


class LoRA(nn.Module):
    """y = x W^T + b + (alpha/r) (x A^T) B^T ; A [r, in], B [out, r] (B starts at zero)."""

    kind = "lora"

    def __init__(self, base: Linear, rank, alpha=None, dropout=0.0, init="kaiming",
                 dtype=torch.bfloat16, gen=None):
        super().__init__()
        dev = base.weight.device
        self.rank, self.alpha = rank, float(alpha if alpha is not None else rank)
        self.scale = self.alpha / rank
        self.dropout = dropout
        a = torch.empty(rank, base.in_features, dtype=torch.float32, device=dev)
        std = 1.0 / math.sqrt(rank) if init == "reference" else 1.0 / math.sqrt(base.in_features)
        a.normal_(0.0, std, generator=gen)
        self.lora_A = nn.Parameter(a.to(dtype))
        b = torch.zeros(base.out_features, rank, dtype=torch.float32, device=dev)
        if init == "nonzero":
            # ``lora_zero_init: false`` (crates/training/src/lora_keys.rs:31, flux_trainer.rs:59): the
            # up-projection starts small instead of at zero, so the adapter acts from the first step
            b.normal_(0.0, 0.01, generator=gen)
        self.lora_B = nn.Parameter(b.to(dtype))

    def forward(self, base: Linear, x, act=None, residual=None, gate=None):
        wt = base.frozen_transpose() if torch.is_grad_enabled() else None
        if self.dropout > 0 and self.training:
            y = F.linear(x, base.weight, base.bias, wt=wt)
            xd = TF.dropout(x, self.dropout)
            y = y + TF.linear(TF.linear(xd, self.lora_A), self.lora_B) * self.scale
            if act is not None:
                y = F.gelu_tanh(y) if act == "gelu" else F.silu(y)
            if gate is not None or residual is not None:
                y = F.gate_residual(residual, y, gate)
            return y
        return F.linear(x, base.weight, base.bias, lora=(self.lora_A, self.lora_B, self.scale),
                        act=act, residual=residual, gate=gate, wt=wt)

    def delta_weight(self, base=None):
        return (self.lora_B.float() @ self.lora_A.float()) * self.scale

    def export_tensors(self):
        return {"lora_down.weight": self.lora_A, "lora_up.weight": self.lora_B,
                "alpha": torch.tensor(self.alpha)}


class _MergedAdapter(nn.Module):
    """Adapters defined by a weight delta: one GEMM on W + dW."""

    def effective_weight(self, base):
        return (base.weight.float() + self.delta_weight(base)).to(base.weight.dtype)

    def forward(self, base, x, act=None, residual=None, gate=None):
        w = self.effective_weight(base)
        return F.linear(x, w, base.bias, act=act, residual=residual, gate=gate)


class LoHa(_MergedAdapter):
    """dW = (A B) o (C D) * alpha / r  (Hadamard product of two rank-r factors)."""

    kind = "loha"

    def __init__(self, base, rank, alpha=None, dtype=torch.bfloat16, gen=None, **_):
        super().__init__()
        dev, o, i = base.weight.device, base.out_features, base.in_features
        self.rank, self.alpha = rank, float(alpha if alpha is not None else rank)
        self.scale = self.alpha / rank
        mk = lambda *s, z=False: nn.Parameter(
            (torch.zeros(*s, device=dev) if z else
             torch.empty(*s, device=dev).normal_(0, 0.1, generator=gen)).to(dtype))
        self.hada_w1_a, self.hada_w1_b = mk(o, rank), mk(rank, i)
        self.hada_w2_a, self.hada_w2_b = mk(o, rank, z=True), mk(rank, i)

    def delta_weight(self, base=None):
        return ((self.hada_w1_a.float() @ self.hada_w1_b.float()) *
                (self.hada_w2_a.float() @ self.hada_w2_b.float())) * self.scale

    def export_tensors(self):
        return {"hada_w1_a": self.hada_w1_a, "hada_w1_b": self.hada_w1_b,
                "hada_w2_a": self.hada_w2_a, "hada_w2_b": self.hada_w2_b,
                "alpha": torch.tensor(self.alpha)}


def _factor(n, f):
    """Split n = a*b with a the largest divisor <= f (Kronecker factorisation helper)."""
    a = 1
    for c in range(1, min(f, n) + 1):
        if n % c == 0:
            a = c
    return a, n // a


class LoKr(_MergedAdapter):
    """dW = kron(W1, W2a W2b) * alpha / r (reference keeps a Kronecker LoKr in
    crates/networks/src/lokr.rs:222-285)."""

    kind = "lokr"

    def __init__(self, base, rank, alpha=None, factor=8, dtype=torch.bfloat16, gen=None, **_):
        super().__init__()
        dev, o, i = base.weight.device, base.out_features, base.in_features
        self.rank, self.alpha = rank, float(alpha if alpha is not None else rank)
        self.scale = self.alpha / rank
        o1, o2 = _factor(o, factor)
        i1, i2 = _factor(i, factor)
        self.lokr_w1 = nn.Parameter(torch.empty(o1, i1, device=dev).normal_(0, 0.1, generator=gen).to(dtype))
        self.lokr_w2_a = nn.Parameter(torch.zeros(o2, rank, device=dev, dtype=dtype))
        self.lokr_w2_b = nn.Parameter(torch.empty(rank, i2, device=dev).normal_(0, 0.1, generator=gen).to(dtype))

    def delta_weight(self, base=None):
        w2 = self.lokr_w2_a.float() @ self.lokr_w2_b.float()
        return torch.kron(self.lokr_w1.float(), w2) * self.scale

    def export_tensors(self):
        return {"lokr_w1": self.lokr_w1, "lokr_w2_a": self.lokr_w2_a, "lokr_w2_b": self.lokr_w2_b,
                "alpha": torch.tensor(self.alpha)}


class DoRA(_MergedAdapter):
    """W' = m * (W + dW) / ||W + dW||_col ; m starts at the column norms of W."""

    kind = "dora"

    def __init__(self, base, rank, alpha=None, dtype=torch.bfloat16, gen=None, **_):
        super().__init__()
        dev = base.weight.device
        self.rank, self.alpha = rank, float(alpha if alpha is not None else rank)
        self.scale = self.alpha / rank
        a = torch.empty(rank, base.in_features, device=dev).normal_(0, 1 / math.sqrt(base.in_features), generator=gen)
        self.lora_A = nn.Parameter(a.to(dtype))
        self.lora_B = nn.Parameter(torch.zeros(base.out_features, rank, dtype=dtype, device=dev))
        self.dora_scale = nn.Parameter(base.weight.detach().float().norm(dim=1, keepdim=True).to(dtype))

    def delta_weight(self, base=None):
        return (self.lora_B.float() @ self.lora_A.float()) * self.scale

    def effective_weight(self, base):
        w = base.weight.float() + self.delta_weight()
        norm = w.norm(dim=1, keepdim=True).detach()
        return (self.dora_scale.float() * w / (norm + 1e-12)).to(base.weight.dtype)

    def export_tensors(self):
        return {"lora_down.weight": self.lora_A, "lora_up.weight": self.lora_B,
                "dora_scale": self.dora_scale, "alpha": torch.tensor(self.alpha)}


class IA3(nn.Module):
    """Learned output scaling y = (x W^T + b) * l  (crates/adapters/src/kinds/ia3.rs:12-17)."""

    kind = "ia3"

    def __init__(self, base, dtype=torch.bfloat16, **_):
        super().__init__()
        self.ia3_out = nn.Parameter(torch.ones(base.out_features, dtype=dtype, device=base.weight.device))

    def forward(self, base, x, act=None, residual=None, gate=None):
        y = F.linear(x, base.weight, base.bias, wt=base.frozen_transpose()) * self.ia3_out
        if act is not None:
            y = F.gelu_tanh(y) if act == "gelu" else F.silu(y)
        if gate is not None or residual is not None:
            y = F.gate_residual(residual, y, gate)
        return y

    def delta_weight(self, base):
        return base.weight.float() * (self.ia3_out.float()[:, None] - 1.0)

    def export_tensors(self):
        return {"ia3_out": self.ia3_out}


class GLoRA(_MergedAdapter):
    """Generalised LoRA: W' = W + W o (A1 B1) + A2 B2, b' = b + bias delta
    (crates/networks/src/glora.rs:61-290 describes the same decomposition)."""

    kind = "glora"

    def __init__(self, base, rank, alpha=None, dtype=torch.bfloat16, gen=None, **_):
        super().__init__()
        dev, o, i = base.weight.device, base.out_features, base.in_features
        self.rank, self.alpha = rank, float(alpha if alpha is not None else rank)
        self.scale = self.alpha / rank
        z = lambda *s: nn.Parameter(torch.zeros(*s, dtype=dtype, device=dev))
        n = lambda *s: nn.Parameter(torch.empty(*s, device=dev).normal_(0, 0.02, generator=gen).to(dtype))
        self.a1, self.b1 = z(o, rank), n(rank, i)
        self.a2, self.b2 = z(o, rank), n(rank, i)

    def delta_weight(self, base):
        w = base.weight.float()
        return (w * (self.a1.float() @ self.b1.float()) + self.a2.float() @ self.b2.float()) * self.scale

    def export_tensors(self):
        return {"glora_a1": self.a1, "glora_b1": self.b1, "glora_a2": self.a2, "glora_b2": self.b2,
                "alpha": torch.tensor(self.alpha)}


class LoConConv2d(nn.Module):
    """LoRA for convolutions: dK = reshape(B[OC, r] A[r, IC*KH*KW]) added to the kernel
    (crates/adapters/src/kinds/locon2d.rs:19-42)."""

    kind = "locon"

    def __init__(self, conv: nn.Conv2d, rank, alpha=None, dtype=None, gen=None):
        super().__init__()
        dtype = dtype or conv.weight.dtype
        dev = conv.weight.device
        oc, ic, kh, kw = conv.weight.shape
        self.rank, self.alpha = rank, float(alpha if alpha is not None else rank)
        self.scale = self.alpha / rank
        self.conv_down = nn.Parameter(
            torch.empty(rank, ic * kh * kw, device=dev).normal_(0, 1 / math.sqrt(ic * kh * kw), generator=gen).to(dtype))
        self.conv_up = nn.Parameter(torch.zeros(oc, rank, dtype=dtype, device=dev))
        self.shape = (oc, ic, kh, kw)

    def delta_weight(self, conv=None):
        return (self.conv_up.float() @ self.conv_down.float()).view(self.shape) * self.scale

    def export_tensors(self):
        return {"conv_down": self.conv_down, "conv_up": self.conv_up, "alpha": torch.tensor(self.alpha)}


class AdaptedConv2d(nn.Module):
    def __init__(self, conv, adapter):
        super().__init__()
        self.conv, self.adapter = conv, adapter

    def forward(self, x):
        w = (self.conv.weight.float() + self.adapter.delta_weight()).to(self.conv.weight.dtype)
        return TF.conv2d(x, w, self.conv.bias, self.conv.stride, self.conv.padding,
                         self.conv.dilation, self.conv.groups)


_KINDS = {"lora": LoRA, "loha": LoHa, "lokr": LoKr, "dora": DoRA, "ia3": IA3, "glora": GLoRA}


def _matches(name, pats):
    return any(re.fullmatch(p, name) or re.search(p, name) for p in pats)


def inject_adapters(model: nn.Module, cfg: AdapterConfig, seed: int = 0):
    """Freeze the model, attach one adapter per matching ``Linear`` and return
    ``{module_path: adapter}`` (ordered by path; the order defines the parameter arena layout)."""
    for p in model.parameters():
        p.requires_grad_(False)
    gen_cpu = torch.Generator().manual_seed(seed)
    out = {}
    for name, mod in sorted(model.named_modules(), key=lambda kv: kv[0]):
        if not isinstance(mod, Linear) or type(mod).__name__ == "SmallLinear":
            continue
        if not _matches(name, cfg.target) or (cfg.exclude and _matches(name, cfg.exclude)):
            continue
        rank = cfg.rank
        for pat, r in cfg.rank_pattern.items():
            if re.search(pat, name):
                rank = r
        gen = gen_cpu if mod.weight.device.type == "cpu" else \
            torch.Generator(device=mod.weight.device).manual_seed(seed + len(out))
        cls = _KINDS[cfg.kind]
        kw = dict(rank=rank, alpha=cfg.alpha, dtype=cfg.dtype, gen=gen)
        if cfg.kind == "lora":
            kw.update(dropout=cfg.dropout, init=cfg.init)
        if cfg.kind == "lokr":
            kw.update(factor=cfg.lokr_factor)
        ad = cls(mod, **kw) if cfg.kind != "ia3" else cls(mod, dtype=cfg.dtype)
        mod.adapter = ad
        out[name] = ad
    return out


def adapter_parameters(adapters: dict):
    ps = []
    for name in sorted(adapters):
        ps += list(adapters[name].parameters())
    return ps


def adapter_state_dict(adapters: dict, layout: str = "eri", model=None, strict: bool = True):
    """Flatten adapter tensors under one of the supported key layouts:

    * ``phase4`` / ``stable`` / ``sdxl`` : the reference's per-site names (``lora.block{NN}.attn.q.
      lora.A`` ...; see ``adapters.reference_keys``); these need ``model`` to number the blocks and
      split the fused projections
    * ``eri``   : ``lora.{path}.lora.A`` / ``.lora.B`` (phase-4 layout,
      crates/training/src/flux_trainer.rs:633-666); non-LoRA kinds use ``lora.{path}.{leaf}``
    * ``peft``  : ``{path}.lora_A.weight`` / ``.lora_B.weight`` (src/networks/lora.rs:193-194)
    * ``kohya`` : ``lora_unet_{path_with_underscores}.lora_down.weight`` / ``.lora_up.weight`` /
      ``.alpha`` (src/networks/lora_flame.rs:274-285, src/networks/sd_lora.rs:175-176)
    """
    if layout in ("phase4", "stable", "sdxl"):
        from .reference_keys import reference_state_dict
        if model is None:
            raise ValueError(f"the {layout} layout needs the model (block numbering, fused projections)")
        return reference_state_dict(adapters, model, layout, strict=strict)[0]
    sd = {}
    for path in sorted(adapters):
        ad = adapters[path]
        t = ad.export_tensors()
        for leaf, v in t.items():
            v = v.detach()
            if layout == "kohya":
                key = "lora_unet_" + path.replace(".", "_") + "." + leaf
            elif layout == "peft":
                leaf2 = {"lora_down.weight": "lora_A.weight", "lora_up.weight": "lora_B.weight"}.get(leaf, leaf)
                if leaf == "alpha":
                    continue
                key = f"{path}.{leaf2}"
            else:
                leaf2 = {"lora_down.weight": "lora.A", "lora_up.weight": "lora.B"}.get(leaf, leaf)
                if leaf == "alpha":
                    continue
                key = f"lora.{path}.{leaf2}"
            sd[key] = v
    return sd


def load_adapter_state_dict(adapters: dict, sd: dict, strict: bool = True):
    """Inverse of ``adapter_state_dict`` for all three layouts; with ``strict`` every key of the
    file must be consumed and every adapter tensor found (the reference's LyCORIS loader errors on
    unused keys: crates/adapters/src/loader/safetensors_lyco.rs:29-136)."""
    used = set()
    for path in sorted(adapters):
        ad = adapters[path]
        for leaf, p in ad.export_tensors().items():
            cands = [
                "lora_unet_" + path.replace(".", "_") + "." + leaf,
                f"{path}." + {"lora_down.weight": "lora_A.weight", "lora_up.weight": "lora_B.weight"}.get(leaf, leaf),
                f"lora.{path}." + {"lora_down.weight": "lora.A", "lora_up.weight": "lora.B"}.get(leaf, leaf),
            ]
            hit = next((c for c in cands if c in sd), None)
            if hit is None:
                if leaf == "alpha" or not strict:
                    continue
                raise KeyError(f"adapter tensor for {path}.{leaf} not in checkpoint")
            used.add(hit)
            if leaf == "alpha":
                continue
            with torch.no_grad():
                p.copy_(sd[hit].to(p.dtype).view_as(p))
    extra = set(sd) - used
    if strict and extra:
        raise KeyError(f"unused keys in adapter checkpoint: {sorted(extra)[:8]} ...")
    return used


def merge_adapters(model: nn.Module):
    """Fold every attached adapter into its base weight and detach it."""
    for mod in model.modules():
        if isinstance(mod, Linear) and mod.adapter is not None:
            with torch.no_grad():
                mod.weight.add_(mod.adapter.delta_weight(mod).to(mod.weight.dtype))
            mod.adapter = None
            mod.drop_transpose()


def load_adapters_into(model: nn.Module, path, alpha: float | None = None, strict: bool = True):
    """Attach LoRA adapters to ``model`` from a checkpoint file in any supported key layout: the
    rank is read from the first down-projection tensor, ``alpha`` from the file when it carries
    one (kohya layout), else it defaults to the rank. Returns the adapter dict."""
    from ..io import safetensors as st
    from .reference_keys import detect_layout, load_reference_lora
    sd = st.load_file(path)
    ref_layout = detect_layout(sd.keys())
    if ref_layout is not None:
        # a file written by the reference (per-site names): sites are stacked into the fused adapters
        if alpha is None:
            md = st.read_metadata(path) or {}
            alpha = float(md["alpha"]) if md.get("alpha") not in (None, "") else None
        return load_reference_lora(model, sd, ref_layout, alpha=alpha, strict=strict)
    down = next((v for k, v in sd.items() if k.endswith(("lora.A", "lora_A.weight", "lora_down.weight"))), None)
    if down is None:
        raise KeyError(f"{path}: no LoRA down-projection tensor found")
    rank = int(down.shape[0])
    if alpha is None:
        a = next((v for k, v in sd.items() if k.endswith(".alpha")), None)
        alpha = float(a) if a is not None else float(rank)
    dtype = next(model.parameters()).dtype
    adapters = inject_adapters(model, AdapterConfig(rank=rank, alpha=alpha, dtype=dtype))
    # only the adapted sites present in the file are kept (a checkpoint may cover a subset)
    present = {p for p in adapters
               if any(p in k or p.replace(".", "_") in k for k in sd)}
    for p in list(adapters):
        if p not in present:
            dict(model.named_modules())[p].adapter = None
            del adapters[p]
    load_adapter_state_dict(adapters, sd, strict=strict)
    return adapters
