"""FLUX LoRA smoke harness with the reference's flags (crates/training/src/bin/flux_10steps.rs:20-118):
``--model --manifest --manifest-root --manifest-index --manifest-validate --manifest-repeat
--manifest-no-shuffle --synthetic --device --steps --batch --grad-accum --height --width --tokens
--seed --lr --lora-rank --lora-alpha``; prints ``step NN/NN loss grad_norm time`` per step."""
from __future__ import annotations

import argparse
import sys
import time

import torch

from ..adapters import AdapterConfig
from ..data import CachedEmbeddingLoader, synthetic_batch
from ..models import build_model
from ..train.trainer import Trainer, TrainerConfig


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model"); ap.add_argument("--vae"); ap.add_argument("--t5"); ap.add_argument("--clip")
    ap.add_argument("--t5-tokenizer"); ap.add_argument("--clip-tokenizer")
    ap.add_argument("--manifest"); ap.add_argument("--manifest-root"); ap.add_argument("--manifest-index")
    ap.add_argument("--manifest-validate", action="store_true"); ap.add_argument("--manifest-repeat", type=int, default=1)
    ap.add_argument("--manifest-no-shuffle", action="store_true"); ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--steps", type=int, default=10); ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--grad-accum", type=int, default=1)
    ap.add_argument("--height", type=int, default=1024); ap.add_argument("--width", type=int, default=1024)
    ap.add_argument("--tokens", type=int, default=512); ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--lr", type=float, default=1e-4); ap.add_argument("--lora-rank", type=int, default=16)
    ap.add_argument("--lora-alpha", type=float, default=16.0)
    ap.add_argument("--arch", default="flux", help="flux | tiny_mmdit")
    a = ap.parse_args(argv)
    dev = torch.device(a.device)
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    torch.manual_seed(a.seed)
    model = build_model(a.arch, device=dev, dtype=dt)
    if a.model:
        from ..io.weights import load_model_weights
        load_model_weights(model, a.model, "flux")
    cfg = TrainerConfig(mode="lora", adapter=AdapterConfig(rank=a.lora_rank, alpha=a.lora_alpha, dtype=dt),
                        lr=a.lr, grad_accum=a.grad_accum, seed=a.seed, guidance=1.0,
                        stochastic_rounding=dev.type == "cuda")
    tr = Trainer(model, cfg)
    loader = None
    if a.manifest and not a.synthetic:
        loader = CachedEmbeddingLoader(a.manifest, "flux", a.batch, a.manifest_root, a.manifest_index,
                                       shuffle=not a.manifest_no_shuffle, repeat=a.manifest_repeat, seed=a.seed,
                                       device=dev, validate=a.manifest_validate)
    kind = "tiny_mmdit" if a.arch == "tiny_mmdit" else "flux"
    i = 0
    while tr.step < a.steps:
        b = loader.next() if loader else synthetic_batch(kind, a.batch, dev, dt, a.seed + i, a.height, a.width, a.tokens)
        t0 = time.time()
        before = tr.step
        loss = tr.train_step(b)
        i += 1
        if tr.step != before:
            lv = float(loss)
            gn = tr.grad_norm()
            print(f"step {tr.step:02d}/{a.steps:02d} loss {lv:.5f} grad_norm {float(gn) if gn is not None else float('nan'):.4f} "
                  f"time {time.time() - t0:.3f}s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
