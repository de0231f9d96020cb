"""LoRA files under the reference's tensor names, in both directions.

The reference enumerates one adapter per projection and names it by block number:

* ``phase4``  ``lora.block{NN}.attn.{q,k,v,o}.lora.{A,B}``, ``lora.block{NN}.mlp.{fc1,fc2}.lora.{A,B}``
  — what its FLUX LoRA trainer writes (crates/training/src/flux/lora.rs:86-120, 225-240;
  crates/training/src/flux_trainer.rs:633-666; image stream only);
* ``stable``  ``lora.blocks.{NN}.attn.{q,k,v,o}.{A,B}``, ``lora.blocks.{NN}.mlp.{fc1,fc2}.{A,B}``
  — the stable key enumeration (crates/training/src/lora_keys.rs:35-104);
* ``sdxl``    ``blocks.{NN}.{attn1,attn2}.{to_q,to_k,to_v,to_out.0}.{A,B}`` over the 70 transformer
  blocks in checkpoint order (crates/training/src/sdxl/registry.rs:1048-1066,
  crates/training/src/sdxl/keymap.rs:6-77).

This package adapts FUSED projections (``qkv``, the single-stream ``linear1`` = [q | k | v | mlp-in]
and ``linear2`` over [attention | mlp], SDXL ``to_qkv`` / ``to_kv``), so one module corresponds to
several reference sites. With A [r, in] the down- and B [out, r] the up-matrix of ``dW = s B A``:

* export — a site that is a ROW range of the fused output keeps the shared A and takes its rows of
  B; a site that is a COLUMN range of the fused input takes its columns of A and the shared B. The
  split is exact.
* import — the sites of one module are stacked into one adapter of rank ``sum r_i``: row sites give
  ``A = [A_1; A_2; ...]`` and a block-diagonal B, column sites a block-diagonal A and
  ``B = [B_1 | B_2 | ...]``. The rank is padded with zero rows up to 16 / 32 / 64 so that the
  adapter stays on the fused GEMM path. The adapted linear computes exactly what the separate
  adapters would.
"""
from __future__ import annotations

import re
from dataclasses import dataclass

import torch

from ..models.layers import Linear
from .lora import LoRA

LAYOUTS = ("phase4", "stable", "sdxl")
_FUSED_RANKS = (16, 32, 64)


@dataclass(frozen=True)
class Site:
    """One reference adapter site and where it lives in this package's model."""
    block: int | str          # reference block number (or "mid")
    name: str                 # "attn.q", "mlp.fc1", "attn1.to_out.0", ...
    module: str               # module path of the (possibly fused) Linear
    axis: str                 # "whole" | "rows" (range of the output dim) | "cols" (range of the input dim)
    lo: int = 0
    hi: int = 0


def _key(layout: str, site: Site, part: str) -> str:
    b = f"{site.block:02d}" if isinstance(site.block, int) else str(site.block)
    if layout == "phase4":
        return f"lora.block{b}.{site.name}.lora.{part}"
    if layout == "stable":
        return f"lora.blocks.{b}.{site.name}.{part}"
    if layout == "sdxl":
        return f"blocks.{b}.{site.name}.{part}"
    raise ValueError(f"unknown reference LoRA layout {layout!r}; known: {LAYOUTS}")


def detect_layout(keys) -> str | None:
    """Which reference layout a set of tensor names follows (None: none of them)."""
    for k in keys:
        if re.match(r"lora\.block\d+\.(attn|mlp)\.\w+\.lora\.[AB]$", k):
            return "phase4"
        if re.match(r"lora\.blocks\.(\d+|mid)\.(attn|mlp)\.\w+\.[AB]$", k):
            return "stable"
        if re.match(r"blocks\.\d+\.attn[12]\.to_(q|k|v|out\.0)\.[AB]$", k):
            return "sdxl"
    return None


# ------------------------------------------------------------------------------- site tables
def mmdit_sites(model) -> list[Site]:
    """FLUX-style MMDiT: reference block NN is double block NN (image stream) for NN < number of
    double blocks, then the single blocks follow. In a single block q / k / v / fc1 are row ranges
    of ``linear1`` and o / fc2 column ranges of ``linear2``."""
    D = model.cfg.hidden
    sites = []
    n_double = len(model.double_blocks)
    for i in range(n_double):
        p = f"double_blocks.{i}"
        for j, n in enumerate(("q", "k", "v")):
            sites.append(Site(i, f"attn.{n}", f"{p}.img_attn.qkv", "rows", j * D, (j + 1) * D))
        sites.append(Site(i, "attn.o", f"{p}.img_attn.proj", "whole"))
        sites.append(Site(i, "mlp.fc1", f"{p}.img_mlp_0", "whole"))
        sites.append(Site(i, "mlp.fc2", f"{p}.img_mlp_2", "whole"))
    for j, blk in enumerate(model.single_blocks):
        i, p = n_double + j, f"single_blocks.{j}"
        F_ = blk.mlp_dim
        for c, n in enumerate(("q", "k", "v")):
            sites.append(Site(i, f"attn.{n}", f"{p}.linear1", "rows", c * D, (c + 1) * D))
        sites.append(Site(i, "mlp.fc1", f"{p}.linear1", "rows", 3 * D, 3 * D + F_))
        sites.append(Site(i, "attn.o", f"{p}.linear2", "cols", 0, D))
        sites.append(Site(i, "mlp.fc2", f"{p}.linear2", "cols", D, D + F_))
    return sites


def sdxl_sites(model) -> list[Site]:
    """SDXL UNet: transformer blocks in checkpoint order (input blocks, middle block, output
    blocks); self-attention q / k / v are row ranges of ``attn1.to_qkv``, cross-attention k / v of
    ``attn2.to_kv``."""
    order = {"down": 0, "mid": 1, "up": 2}
    found = []
    for name, mod in model.named_modules():
        if type(mod).__name__ != "BasicTransformerBlock":
            continue
        parts = name.split(".")
        nums = [int(x) for x in parts if x.isdigit()]
        found.append(((order.get(parts[0], 3), *nums), name, mod))
    sites = []
    for i, (_, name, blk) in enumerate(sorted(found, key=lambda t: t[0])):
        D = blk.attn1.to_out.in_features
        for j, n in enumerate(("to_q", "to_k", "to_v")):
            sites.append(Site(i, f"attn1.{n}", f"{name}.attn1.to_qkv", "rows", j * D, (j + 1) * D))
        sites.append(Site(i, "attn1.to_out.0", f"{name}.attn1.to_out", "whole"))
        sites.append(Site(i, "attn2.to_q", f"{name}.attn2.to_q", "whole"))
        for j, n in enumerate(("to_k", "to_v")):
            sites.append(Site(i, f"attn2.{n}", f"{name}.attn2.to_kv", "rows", j * D, (j + 1) * D))
        sites.append(Site(i, "attn2.to_out.0", f"{name}.attn2.to_out", "whole"))
    return sites


def sites_for(model, layout: str) -> list[Site]:
    if layout == "sdxl":
        if not any(type(m).__name__ == "BasicTransformerBlock" for m in model.modules()):
            raise ValueError("the sdxl LoRA layout needs a UNet with transformer blocks")
        return sdxl_sites(model)
    if not (hasattr(model, "double_blocks") and hasattr(model, "single_blocks")):
        raise ValueError(f"the {layout} LoRA layout names the blocks of an MMDiT (double / single stream) model")
    return mmdit_sites(model)


# ------------------------------------------------------------------------------- export
def reference_state_dict(adapters: dict, model, layout: str = "phase4", strict: bool = True):
    """``{reference tensor name: tensor}`` for the plain-LoRA adapters in ``adapters``
    (``{module path: adapter}``). Adapters that have no reference name (the text stream of a double
    block, adapter kinds other than LoRA) raise with ``strict``; otherwise they are listed in the
    second return value and left out."""
    by_module = {}
    for s in sites_for(model, layout):
        by_module.setdefault(s.module, []).append(s)
    sd, skipped = {}, []
    for path in sorted(adapters):
        ad = adapters[path]
        if getattr(ad, "kind", "") != "lora" or path not in by_module:
            skipped.append(path)
            continue
        A, B = ad.lora_A.detach(), ad.lora_B.detach()
        for s in by_module[path]:
            if s.axis == "rows":
                a, b = A, B[s.lo:s.hi]
            elif s.axis == "cols":
                a, b = A[:, s.lo:s.hi], B
            else:
                a, b = A, B
            sd[_key(layout, s, "A")] = a.contiguous()
            sd[_key(layout, s, "B")] = b.contiguous()
    if strict and skipped:
        raise KeyError(f"adapters without a name in the {layout} layout (train the image stream / plain LoRA only, "
                       f"or export with strict=False): {skipped[:6]}{' ...' if len(skipped) > 6 else ''}")
    return sd, skipped


def adapter_alpha(adapters: dict) -> float | None:
    ad = next(iter(adapters.values()), None)
    return None if ad is None else float(getattr(ad, "alpha", 0.0)) or None


# ------------------------------------------------------------------------------- import
def _pad_rank(r: int) -> int:
    return next((x for x in _FUSED_RANKS if x >= r), r)


def load_reference_lora(model, sd: dict, layout: str | None = None, alpha: float | None = None,
                        strict: bool = True, dtype=None) -> dict:
    """Attach adapters to ``model`` from a file in one of the reference layouts. ``alpha`` is the
    per-site alpha (the files do not store it; default: the site rank, scale 1). Returns
    ``{module path: adapter}``; all other parameters are frozen."""
    layout = layout or detect_layout(sd.keys())
    if layout is None:
        raise KeyError("no tensor name of this file follows a reference LoRA layout")
    table = {}
    for s in sites_for(model, layout):
        table[_key(layout, s, "A")] = (s, "A")
        table[_key(layout, s, "B")] = (s, "B")
    unknown = [k for k in sd if k not in table]
    if strict and unknown:
        raise KeyError(f"tensor names without a site in this model ({layout} layout): {sorted(unknown)[:6]}")
    per_module = {}
    for k, t in sd.items():
        if k in table:
            s, part = table[k]
            per_module.setdefault(s.module, {}).setdefault(s, {})[part] = t
    mods = dict(model.named_modules())
    for p in model.parameters():
        p.requires_grad_(False)
    out = {}
    for path in sorted(per_module):
        base = mods[path]
        if not isinstance(base, Linear):
            raise TypeError(f"{path} is not an adaptable Linear")
        parts = sorted(per_module[path].items(), key=lambda kv: (kv[0].lo, kv[0].name))
        for s, ab in parts:
            if "A" not in ab or "B" not in ab:
                raise KeyError(f"site block {s.block} {s.name}: file has only one of A / B")
        ranks = [ab["A"].shape[0] for _, ab in parts]
        r_site = ranks[0]
        R = _pad_rank(sum(ranks))
        dt = dtype or base.weight.dtype
        dev = base.weight.device
        A = torch.zeros(R, base.in_features, dtype=torch.float32, device=dev)
        B = torch.zeros(base.out_features, R, dtype=torch.float32, device=dev)
        off = 0
        for (s, ab), r in zip(parts, ranks):
            a, b = ab["A"].float().to(dev), ab["B"].float().to(dev)
            if s.axis == "rows":
                want_a, want_b = (r, base.in_features), (s.hi - s.lo, r)
            elif s.axis == "cols":
                want_a, want_b = (r, s.hi - s.lo), (base.out_features, r)
            else:
                want_a, want_b = (r, base.in_features), (base.out_features, r)
            if tuple(a.shape) != want_a or tuple(b.shape) != want_b:
                raise ValueError(f"block {s.block} {s.name}: A {tuple(a.shape)} / B {tuple(b.shape)}, expected "
                                 f"{want_a} / {want_b}")
            if s.axis == "rows":
                A[off:off + r] = a
                B[s.lo:s.hi, off:off + r] = b
            elif s.axis == "cols":
                A[off:off + r, s.lo:s.hi] = a
                B[:, off:off + r] = b
            else:
                A[off:off + r] = a
                B[:, off:off + r] = b
            off += r
        site_alpha = float(alpha) if alpha is not None else float(r_site)
        scale = site_alpha / r_site
        ad = LoRA(base, rank=R, alpha=scale * R, dtype=dt)     # alpha / rank keeps the sites' scale
        with torch.no_grad():
            ad.lora_A.copy_(A.to(dt))
            ad.lora_B.copy_(B.to(dt))
        base.adapter = ad
        out[path] = ad
    return out


def fill_adapters_from_reference(adapters: dict, model, sd: dict, layout: str | None = None):
    """Copy a reference-named file back into EXISTING fused adapters of the same rank (resuming a run
    whose checkpoints were written with a reference layout). That is possible exactly when the sites
    of a module share their down matrix (row sites) or their up matrix (column sites) — true for
    files exported by this package; a file with independent per-site matrices needs
    ``load_reference_lora`` (stacked rank) instead and is refused here."""
    layout = layout or detect_layout(sd.keys())
    if layout is None:
        raise KeyError("no tensor name of this file follows a reference LoRA layout")
    by_module = {}
    for s in sites_for(model, layout):
        by_module.setdefault(s.module, []).append(s)
    used = set()
    for path, ad in adapters.items():
        sites = by_module.get(path)
        if sites is None:
            raise KeyError(f"adapter {path} has no site in the {layout} layout")
        A, B = ad.lora_A, ad.lora_B
        shared = None
        with torch.no_grad():
            for s in sites:
                ka, kb = _key(layout, s, "A"), _key(layout, s, "B")
                if ka not in sd or kb not in sd:
                    raise KeyError(f"{ka} / {kb} missing from the checkpoint")
                a, b = sd[ka].to(A.dtype), sd[kb].to(B.dtype)
                used.update((ka, kb))
                if s.axis == "rows":
                    if shared is not None and not torch.equal(shared, a):
                        raise ValueError(f"{path}: the sites have different down matrices; load this file with "
                                         "adapters.load_adapters_into (stacked rank) instead")
                    shared = a
                    A.copy_(a.view_as(A))
                    B[s.lo:s.hi].copy_(b)
                elif s.axis == "cols":
                    if shared is not None and not torch.equal(shared, b):
                        raise ValueError(f"{path}: the sites have different up matrices; load this file with "
                                         "adapters.load_adapters_into (stacked rank) instead")
                    shared = b
                    B.copy_(b.view_as(B))
                    A[:, s.lo:s.hi].copy_(a)
                else:
                    A.copy_(a.view_as(A))
                    B.copy_(b.view_as(B))
    extra = set(sd) - used
    if extra:
        raise KeyError(f"unused keys in adapter checkpoint: {sorted(extra)[:6]}")
    return used
