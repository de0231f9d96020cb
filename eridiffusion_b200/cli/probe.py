"""Registry probe: list every registered model kind, build it at reduced size and report its
parameter count and adapter sites; ``--full KIND`` builds one kind at full size on the meta
device and prints the exact parameter count.

    python -m eridiffusion_b200.cli.probe [--full flux]

Counterpart of the reference's ``sd35_probe`` binary and of its ``REGISTRY_ONLY=1`` mode
(crates/training/src/bin/sd35_probe.rs; crates/training/src/run.rs:62-104), which walk the model
registry and print what would be trained without running a step.
"""
from __future__ import annotations

import argparse
import re
import sys

import torch

from ..models import build_model, known_models
from ..models.layers import Linear

_SMALL = {
    "mmdit": dict(hidden=128, num_heads=2, depth_double=1, depth_single=1, context_dim=64, vec_dim=32, axes_dim=(16, 24, 24)),
    "nextdit": dict(dim=128, num_heads=2, depth=2, refiner_depth=1, mlp_hidden=256, caption_dim=64),
}


def count(m):
    return sum(p.numel() for p in m.parameters())


def adapter_sites(m):
    pats = m.lora_targets() if hasattr(m, "lora_targets") else [r".*"]
    names = [n for n, mod in m.named_modules() if isinstance(mod, Linear) and type(mod).__name__ != "SmallLinear"]
    return sum(1 for n in names if any(re.search(p, n) for p in pats))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--full", help="build this kind at full size on the meta device")
    a = ap.parse_args(argv)
    if a.full:
        m = build_model(a.full, device=torch.device("meta"))
        print(f"{a.full}: {count(m) / 1e9:.3f} B parameters, {adapter_sites(m)} adapter sites, "
              f"{sum(1 for _ in m.modules())} modules")
        return 0
    for kind in known_models():
        try:
            m = build_model(kind, device=torch.device("meta"))
            print(f"{kind:18s} {count(m) / 1e6:12.1f} M parameters  {adapter_sites(m):5d} adapter sites  {type(m).__name__}")
        except Exception as e:                          # a kind that cannot build on meta is reported, not fatal
            print(f"{kind:18s} build failed on the meta device: {type(e).__name__}: {e}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
