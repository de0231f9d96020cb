"""Unified trainer: ``python -m eridiffusion_b200.cli.train <config.yaml> [--steps N] [--resume]``.

Accepts both YAML schemas of the reference (``trainer <config.yaml>``, src/bin/trainer.rs:5-37, and
the flat ``model_kind`` files consumed by ``run_training``, crates/training/src/run.rs:35-42).
Multi-GPU: launch with ``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1
-m eridiffusion_b200.cli.train cfg.yaml``.
"""
from __future__ import annotations

import argparse
import sys

from ..config import load_config
from ..train.factory import build_job
from ..train.services import CSVLogger, SampleCallback, StepWatchdog, run_training


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("config")
    ap.add_argument("--steps", type=int)
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--log-every", type=int)
    ap.add_argument("--csv")
    a = ap.parse_args(argv)
    cfg = load_config(a.config)
    if a.steps:
        cfg.steps = a.steps
    trainer, batches, info = build_job(cfg)
    if a.resume and cfg.training_folder:
        r = trainer.load_latest_checkpoint()
        if r and info["rank"] == 0:
            print(f"resumed from step {r[0]} (seed {r[1]})")
    cbs = [CSVLogger(a.csv)] if a.csv and info["rank"] == 0 else []
    if cfg.sample.sample_every and cfg.training_folder and info["rank"] == 0:
        cbs.append(SampleCallback(cfg.sample, info["model"], cfg.training_folder, rank=info["rank"]))
    wd = StepWatchdog()
    run_training(trainer, batches, cfg.steps, callbacks=cbs, log_every=a.log_every or cfg.performance_log_every,
                 world=info["world"], batch_size=cfg.batch_size, watchdog=wd,
                 print_fn=print if info["rank"] == 0 else (lambda *_: None))
    if cfg.training_folder and info["rank"] == 0 or info["world"] > 1:
        trainer.save_checkpoint()
    wd.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
