"""SDXL training smoke harness driven by environment variables, as the reference's
``sdxl_10steps`` binary is (crates/training/src/bin/sdxl_10steps.rs: ``STEPS BATCH HEIGHT WIDTH
CTX_DIM TOKENS HIDDEN DEVICE SYNTHETIC SEED BLOCK_INDEX SDXL_MMAP_PATH``); prints the per-step time
in milliseconds and the ``avg step time`` line the reference prints.

    STEPS=10 BATCH=1 HEIGHT=1024 WIDTH=1024 python -m eridiffusion_b200.cli.sdxl_10steps

``MODE=lora|full`` (default lora), ``LORA_RANK``, ``LR``. ``SDXL_MMAP_PATH`` points at a UNet
safetensors file to load; without it the weights are random. ``BLOCK_INDEX`` restricts the trainable
adapters to one transformer block (the reference trains a single block per run).
``SDXL_TIMING=1`` prints the device-timed phase breakdown at the end, ``SDXL_LOAD_TRACE=1`` the GiB/s
of the weight load, ``BACKWARD_DEBUG=1`` runs the first step under autograd anomaly detection and
prints per-parameter gradient statistics; ``ATTN_Q_CHUNK ATTN_KV_CHUNK ATTN_REUSE ATTN_MAX_WS_MB
ATTN_MIN_FREE_MB`` act on the library attention path (``utils/env_flags.py``).
"""
from __future__ import annotations

import os
import sys
import time

import torch

from ..adapters import AdapterConfig
from ..data import synthetic_batch
from ..models import build_model
from ..models.sdxl_unet import sdxl_forward
from ..train.trainer import Trainer, TrainerConfig


def _env(name, default, cast=int):
    v = os.environ.get(name)
    return cast(v) if v not in (None, "") else default


def main():
    steps, batch = _env("STEPS", 10), _env("BATCH", 1)
    height, width = _env("HEIGHT", 1024), _env("WIDTH", 1024)
    seed = _env("SEED", 0)
    device = os.environ.get("DEVICE", "cuda:0" if torch.cuda.is_available() else "cpu")
    dev = torch.device(device if not device.isdigit() else f"cuda:{device}")
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    overrides = {}
    if os.environ.get("CTX_DIM"):
        overrides["context_dim"] = int(os.environ["CTX_DIM"])
    if os.environ.get("HIDDEN"):
        h = int(os.environ["HIDDEN"])
        overrides["block_channels"] = (h // 4, h // 2, h)
    torch.manual_seed(seed)
    model = build_model("sdxl", device=dev, dtype=dt, **overrides)
    path = os.environ.get("SDXL_MMAP_PATH")
    if path:
        from ..io.weights import load_model_weights
        from ..utils.env_flags import load_trace
        with load_trace("sdxl unet", lambda: os.path.getsize(path) if os.path.isfile(path) else sum(
                os.path.getsize(os.path.join(path, f)) for f in os.listdir(path))):
            load_model_weights(model, path, "sdxl")
    mode = os.environ.get("MODE", "lora")
    acfg = AdapterConfig(rank=_env("LORA_RANK", 16), alpha=float(_env("LORA_RANK", 16)), dtype=dt) if mode == "lora" else None
    cfg = TrainerConfig(mode=mode, adapter=acfg, objective="eps", lr=_env("LR", 1e-4, float), seed=seed, patch=1,
                        stochastic_rounding=dev.type == "cuda")
    tr = Trainer(model, cfg, forward_fn=sdxl_forward)
    from ..utils.env_flags import backward_debug, flag
    if flag("SDXL_TIMING"):
        tr.phases.enabled = True
    blk = os.environ.get("BLOCK_INDEX")
    if blk is not None and mode == "lora":
        keep = f"blocks.{int(blk)}."
        for n, p in model.named_parameters():
            if p.requires_grad and keep not in n:
                p.requires_grad_(False)
    times = []
    for i in range(steps):
        b = synthetic_batch("sdxl", batch, dev, dt, seed + i, height, width, _env("TOKENS", 77))
        if model.cfg.context_dim != b["txt"].shape[-1]:       # CTX_DIM override: resize the synthetic text
            g = torch.Generator().manual_seed(seed + i)
            b["txt"] = torch.randn(batch, _env("TOKENS", 77), model.cfg.context_dim, generator=g).to(dt).to(dev)
        if dev.type == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        if i == 0:
            with backward_debug([(n, p) for n, p in model.named_parameters() if p.requires_grad]):
                loss = tr.train_step(b)
        else:
            loss = tr.train_step(b)
        if dev.type == "cuda":
            torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3
        times.append(ms)
        print(f"step {i + 1}/{steps} loss {float(loss):.5f} {ms:.1f} ms")
    warm = times[1:] or times
    print(f"avg step time: {sum(warm) / len(warm):.1f} ms ({len(warm)} steps after warm-up)")
    if flag("SDXL_TIMING"):
        for name, v in tr.phases.summary().items():
            print(f"  phase {name:<10s} {v['ms'] / max(1, v['calls']):9.3f} ms/call  {100 * v['share']:5.1f} %")
    return 0


if __name__ == "__main__":
    sys.exit(main())
