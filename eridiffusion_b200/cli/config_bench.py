"""Training-step throughput of the multi-GPU configurations other than the headline one:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m eridiffusion_b200.cli.config_bench --config sdxl_zero2|qwen_zero3|ltx_ulysses|ltx_av|sd15|sd35_medium \
        [--steps 4 --warmup 2] [--scale 1.0]

* ``sdxl_zero2``   SDXL UNet (2.57 B parameters) full fine-tune, eps objective, 1024^2 (128 x 128
                   latents), gradients reduce-scattered and the 8-bit optimizer state sharded: the
                   fused reduce-scatter + AdamW8bit + all-gather kernel on the whole parameter arena.
* ``qwen_zero3``   Qwen-Image-architecture MMDiT (60 dual-stream blocks, 20.4 B parameters) full
                   fine-tune with parameters sharded (ZeRO-3): every large linear gathers its weight
                   inside the consuming GEMM launch.
* ``ltx_ulysses``  LTX-video-architecture DiT (48 blocks, hidden 4096) LoRA on a 19 008-token clip with
                   the sequence sharded over the ranks (Ulysses): both all-to-alls folded into the
                   QKV / output projections.

* ``ltx_av``       LTX audio + video DiT (48 block pairs with cross-modal attention) LoRA r16 on a 9-frame
                   16 x 16 clip (2304 video tokens) with 64 audio tokens; data parallel over the ranks.
* ``sd15``         SD1.5 UNet LoRA r16, eps objective, 512^2 (head sizes 40 / 80 / 160); data parallel.
* ``sd35_medium``  SD3.5-medium MMDiT (24 joint blocks, dual attention in the first 13) LoRA r16, 1024^2;
                   data parallel.

``--scale`` shrinks the depth (number of blocks) for quick checks; the printed line says so. Times are
CUDA events bracketed by barriers, max over ranks; synthetic N(0,1) inputs, random-init weights.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch
import torch.distributed as dist

from ..adapters import AdapterConfig
from ..data import synthetic_batch
from ..models import build_model
from ..ops import functional as F
from ..parallel.dist import GradSync, ProcessGroup, init_from_env
from ..train.trainer import Trainer, TrainerConfig, default_forward, ltx_av_forward, ltx_forward


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=["sdxl_zero2", "qwen_zero3", "ltx_ulysses", "ltx_av", "sd15", "sd35_medium"])
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--scale", type=float, default=1.0, help="fraction of the block count to build")
    ap.add_argument("--batch", type=int, default=1)
    a = ap.parse_args(argv)
    rank, world, local = init_from_env()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dt = torch.bfloat16
    torch.manual_seed(1234)
    pg = ProcessGroup()
    info = {}
    if a.config == "sdxl_zero2":
        from ..models.sdxl_unet import sdxl_forward
        ov = {}
        if a.scale < 1.0:
            ov["transformer_depth"] = (0, max(1, int(2 * a.scale)), max(1, int(10 * a.scale)))
        model = build_model("sdxl", device=dev, **ov)
        gs = GradSync("fused") if world > 1 else None
        cfg = TrainerConfig(mode="full", objective="eps", optimizer="adamw8bit", lr=1e-5, patch=1, seed=0)
        tr = Trainer(model, cfg, grad_sync=gs, forward_fn=sdxl_forward)
        batch = lambda i: synthetic_batch("sdxl", a.batch, dev, dt, 100 + i * world + rank)
        info = {"model": "SDXL UNet full fine-tune", "parallelism": f"zero2-dp{world} (fused RS + AdamW8bit + AG)",
                "tokens": 128 * 128}
    elif a.config == "qwen_zero3":
        depth = max(1, int(round(60 * a.scale)))
        model = build_model("qwen_image", device=dev, depth_double=depth)
        gs = None
        if world > 1:
            from ..parallel.zero3 import Zero3Context, Zero3Sync, shard_model
            n_params = sum(p.numel() for p in model.parameters())
            z3 = Zero3Context(pg, heap_bytes=int(n_params * 2 / world * 2.2) + (256 << 20))
            sharded, replicated = shard_model(model, z3)
            gs = Zero3Sync(z3, sharded, replicated)
            torch.cuda.empty_cache()
        cfg = TrainerConfig(mode="full", objective="flow", optimizer="adamw8bit", lr=1e-5, seed=0, guidance=None)
        tr = Trainer(model, cfg, grad_sync=gs, forward_fn=default_forward)
        batch = lambda i: synthetic_batch("qwen_image", a.batch, dev, dt, 100 + i * world + rank)
        info = {"model": f"Qwen-Image-arch MMDiT ({depth} dual-stream blocks) full fine-tune",
                "parallelism": f"zero3-{world} (gather-in-GEMM)", "tokens": 4096 + 256}
    elif a.config in ("ltx_av", "sd15", "sd35_medium"):
        lora = AdapterConfig(rank=16, alpha=16, dtype=dt)
        gs = GradSync("fused") if world > 1 else None
        if a.config == "ltx_av":
            depth = max(1, int(round(48 * a.scale)))
            model = build_model("ltx_av", device=dev, depth=depth)
            frames, hh, ww, la = 9, 16, 16, 64
            cfg = TrainerConfig(mode="lora", adapter=lora, objective="flow", optimizer="adamw8bit", lr=1e-4, patch=1,
                                seed=0, guidance=None)
            tr = Trainer(model, cfg, grad_sync=gs, forward_fn=ltx_av_forward)

            def batch(i):
                b = synthetic_batch("ltx", a.batch, dev, dt, 100 + i * world + rank, 512, 512, frames=frames)
                g = torch.Generator().manual_seed(7 + i * world + rank)
                audio = torch.randn(a.batch, 128, la, 1, generator=g).to(dt).to(dev)
                b["latents"] = torch.cat([b["latents"], audio], dim=2)          # [video tokens | audio tokens]
                b["grid_fhw"] = (frames, hh, ww)
                return b
            info = {"model": f"LTX audio+video DiT ({depth} block pairs) LoRA r16", "tokens": frames * hh * ww + la}
        elif a.config == "sd15":
            from ..models.sdxl_unet import sdxl_forward
            model = build_model("sd15", device=dev)
            cfg = TrainerConfig(mode="lora", adapter=lora, objective="eps", optimizer="adamw8bit", lr=1e-4, patch=1, seed=0)
            tr = Trainer(model, cfg, grad_sync=gs, forward_fn=sdxl_forward)
            batch = lambda i: synthetic_batch("sd15", a.batch, dev, dt, 100 + i * world + rank, 512, 512)
            info = {"model": "SD1.5 UNet LoRA r16, 512^2", "tokens": 64 * 64}
        else:
            model = build_model("sd35_medium", device=dev)
            cfg = TrainerConfig(mode="lora", adapter=lora, objective="flow", optimizer="adamw8bit", lr=1e-4, seed=0,
                                guidance=None)
            tr = Trainer(model, cfg, grad_sync=gs, forward_fn=default_forward)
            batch = lambda i: synthetic_batch("sd35", a.batch, dev, dt, 100 + i * world + rank)
            info = {"model": "SD3.5-medium MMDiT LoRA r16, 1024^2", "tokens": 4096 + 333}
        info["parallelism"] = f"dp{world}"
    else:
        depth = max(1, int(round(48 * a.scale)))
        model = build_model("ltx_video", device=dev, depth=depth)
        frames, hh, ww = 33, 24, 24                                   # 19 008 tokens
        L = frames * hh * ww
        Ll = L // world
        gs = GradSync("allreduce") if world > 1 else None
        cfg = TrainerConfig(mode="lora", adapter=AdapterConfig(rank=16, alpha=16, dtype=dt), objective="flow",
                            optimizer="adamw8bit", lr=1e-4, patch=1, seed=0, guidance=None,
                            seq_parallel=world)   # the ranks work on ONE sample: same timestep stream
        tr = Trainer(model, cfg, grad_sync=gs, forward_fn=ltx_forward)
        if world > 1:
            from ..parallel.ulysses import UlyssesContext
            if L % world or model.cfg.num_heads % world:
                raise SystemExit("token count and head count must divide by the world size")
            model.set_sequence_parallel(UlyssesContext(pg, batch=a.batch, l_local=Ll, hidden=model.cfg.hidden,
                                                       heads=model.cfg.num_heads, attn_slots=depth))

        def batch(i):
            # every rank sees the same clip and text (seeded by step only) and keeps its token slice
            b = synthetic_batch("ltx", a.batch, dev, dt, 100 + i, 768, 768, frames=frames)
            b["grid_fhw"] = (frames, hh, ww)
            b["latents"] = b["latents"][:, :, rank * Ll:(rank + 1) * Ll].contiguous()
            return b
        info = {"model": f"LTX-video-arch DiT ({depth} blocks, hidden {model.cfg.hidden}) LoRA r16",
                "parallelism": f"ulysses-{world}", "tokens": L}

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(a.warmup):
        tr.train_step(batch(i))
        if i == 0:
            # a bounded wait that ran out in any kernel of any rank ends the run here, on all ranks
            bad = torch.tensor([1.0 if F.kernel_error_check() else 0.0], device=dev)
            if world > 1:
                dist.all_reduce(bad, dist.ReduceOp.MAX)
            if bad.item():
                raise SystemExit(f"rank {rank}: a kernel reported an error in the first step; stopping")
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    loss = None
    for i in range(a.steps):
        loss = tr.train_step(batch(a.warmup + i))
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, dist.ReduceOp.MAX)
    ms = ms.item()
    errs = F.kernel_error_check()
    samples = a.batch * (1 if a.config == "ltx_ulysses" else world)       # Ulysses: one clip for the group
    if rank == 0:
        print(json.dumps({"config": a.config, **info, "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
                          "ms_per_step": round(ms / a.steps, 2),
                          "samples_per_s": round(samples * a.steps / (ms / 1e3), 4),
                          "loss": round(float(loss), 5), "depth_scale": a.scale, "dtype": "bf16",
                          "data": "synthetic", "kernel_errors": errs, "attention_forward_calls": dict(F.ATTENTION_CALLS),
                          "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
