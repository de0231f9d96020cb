"""Training loop for all model families.

One ``Trainer`` drives: timestep sampling -> fused noise-mix/patchify -> model forward ->
fused weighted-MSE (loss + gradient in one pass) -> backward -> gradient synchronisation
(``parallel.GradSync``: NCCL or the fused reduce-scatter + 8-bit AdamW + all-gather kernel) ->
device-side clip + optimizer -> EMA. Nothing in the step reads a scalar back to the host; the
loss tensor is returned and read only where the caller logs it.

Reference loop being covered: crates/training/src/flux_trainer.rs:286-414
(``train_step_precomputed``: noise, sigma, forward, MSE, accumulate, clip, step, EMA),
crates/training/src/run.rs:208-308 (per-step console/CSV line, periodic checkpoint),
crates/training/src/chroma/train.rs:1262-1378 (non-finite loss/grad -> skip + back-off),
crates/training/src/gradient_accumulator.rs:107-146.
"""
from __future__ import annotations

import json
import math
import os
import time
from dataclasses import dataclass, field
from pathlib import Path

import torch

from ..adapters import (AdapterConfig, adapter_parameters, adapter_state_dict, inject_adapters,
                        load_adapter_state_dict)
from ..io import safetensors as st
from ..objectives import DDPM, FlowMatching, SigmaEps, loss_fn
from ..ops import functional as F
from ..optim import EMA, GradScaler, LRSchedule, ParamArena, create_optimizer


@dataclass
class TrainerConfig:
    mode: str = "lora"                      # lora | full
    adapter: AdapterConfig | None = None
    objective: str = "flow"                 # flow | eps | v | sample | sigma_eps (x0 + sigma eps, target eps)
    sigma_min: float = 0.02                 # sigma_eps: sigma = sigma_min * (sigma_max / sigma_min)^(-t)
    sigma_max: float = 1.0
    timestep_sampler: str = "logit_normal"
    timestep_kw: dict = field(default_factory=dict)
    guidance: float | None = 3.5            # value fed to the guidance embedder (None: 1.0)
    optimizer: str = "adamw8bit"
    lr: float = 1e-4
    weight_decay: float = 0.01
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    lr_schedule: str = "constant"
    warmup_steps: int = 0
    total_steps: int = 0
    grad_accum: int = 1
    max_grad_norm: float = 1.0
    loss: str = "mse"
    min_snr_gamma: float | None = None
    ema_decay: float | None = None
    stochastic_rounding: bool = True
    patch: int = 2
    seed: int = 0
    out_dir: str | None = None
    ckpt_every: int = 0
    # After this many optimizer steps the objects alive so far (model, adapters, arena views, launch
    # plans) are moved out of the cyclic collector's generations (gc.freeze): a full collection in the
    # middle of a step costs tens of milliseconds of host time, which shows as soon as something reads a
    # result back every step. 0 leaves the collector alone.
    gc_freeze_after: int = 3
    keep_last: int = 0
    lr_if_contains: dict = field(default_factory=dict)   # {name substring: LR multiplier}
    rotate_window: int = 0                  # >0: train only this many consecutive blocks at a time
    rotate_period: int = 100                # optimizer steps between window moves
    seq_parallel: int = 1                   # ranks that share ONE sample (Ulysses); they draw the same timestep
    log_csv: str | None = None
    nan_policy: str = "skip"                # skip | raise
    lr_backoff: float = 0.5
    activation_checkpointing: bool = False
    # {"contains", "target_mult", "warmup_steps", "kind"}: the LR multiplier of parameters whose name
    # contains ``contains`` moves from its base value to ``target_mult`` over ``warmup_steps``
    # optimizer steps ("linear" or "cosine"; src/trainers/flux_layer_streaming.rs:362-392)
    lr_ramp: dict | None = None
    # tensor names of lora.safetensors in checkpoints: "eri" (module paths; every adapter kind) or
    # the reference's per-site names "phase4" / "stable" / "sdxl" (plain LoRA on sites that have one)
    lora_layout: str = "eri"


class Trainer:
    def __init__(self, model, cfg: TrainerConfig, grad_sync=None, forward_fn=None):
        self.model, self.cfg = model, cfg
        self.forward_fn = forward_fn or default_forward
        self.adapters = None
        if cfg.mode == "lora":
            acfg = cfg.adapter or AdapterConfig()
            if acfg.target == [r".*"] and hasattr(model, "lora_targets"):
                acfg.target = model.lora_targets()
            self.adapters = inject_adapters(model, acfg, seed=cfg.seed)
            params = adapter_parameters(self.adapters)
            self.param_names = [f"{path}.{n}" for path in sorted(self.adapters)
                                for n, _ in self.adapters[path].named_parameters()]
        else:
            named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
            if grad_sync is not None and hasattr(grad_sync, "ordered_params"):
                order = {id(p): i for i, p in enumerate(grad_sync.ordered_params())}
                named.sort(key=lambda kv: order.get(id(kv[1]), len(order)))
            params = [p for _, p in named]
            self.param_names = [n for n, _ in named]
        world = grad_sync.world_size if grad_sync is not None else 1
        self.arena = ParamArena(params, shard_multiple=world,
                                alloc=getattr(grad_sync, "arena_alloc", None))
        self.grad_sync = grad_sync
        shard = grad_sync.optimizer_shard() if grad_sync is not None else None
        kw = dict(lr=cfg.lr, weight_decay=cfg.weight_decay, betas=cfg.betas, eps=cfg.eps)
        if cfg.optimizer.lower().replace("_", "") in ("adamw8bit", "adam8bit", "adamw"):
            kw.update(stochastic_rounding=cfg.stochastic_rounding, seed=cfg.seed, shard=shard)
        self.optimizer = create_optimizer(cfg.optimizer, self.arena, **kw)
        if grad_sync is not None:
            grad_sync.attach(self.arena, self.optimizer)
        # per-layer learning rates and block rotation act through the 8-bit optimizer's per-block
        # multiplier (single-process and ZeRO-1 sharded optimizers; the fused DP kernel has none)
        self.rotator = None
        self._ramp_done = cfg.lr_ramp is None
        if cfg.lr_ramp is not None and (not hasattr(self.optimizer, "lr_scale") or (
                grad_sync is not None and grad_sync.fused_optimizer)):
            raise ValueError("lr_ramp needs an optimizer with per-block learning-rate multipliers (adamw8bit, "
                             "not the fused data-parallel step)")
        if (cfg.lr_if_contains or cfg.rotate_window or cfg.lr_ramp) and hasattr(self.optimizer, "lr_scale") and not (
                grad_sync is not None and grad_sync.fused_optimizer):
            from ..optim.arena import block_lr_scale
            self._lr_shard = shard
            if cfg.rotate_window:
                from .rotation import LayerRotator
                n_double = len(getattr(model, "double_blocks", []))
                self.rotator = LayerRotator(self.param_names, cfg.rotate_window, cfg.rotate_period, n_double)
                self.rotator.apply(self.optimizer, self.arena, 0, cfg.lr_if_contains, shard)
            else:
                self.optimizer.lr_scale = block_lr_scale(self.arena, self.param_names, self.lr_rules(0),
                                                         shard=shard)
        self.schedule = LRSchedule(cfg.lr, cfg.lr_schedule, cfg.warmup_steps, cfg.total_steps)
        self.scaler = GradScaler(enabled=False)
        self.ema = EMA(self.arena, cfg.ema_decay) if cfg.ema_decay else None
        if cfg.objective == "flow":
            self.objective = FlowMatching(cfg.timestep_sampler, cfg.timestep_kw)
        elif cfg.objective == "sigma_eps":
            self.objective = SigmaEps(cfg.sigma_min, cfg.sigma_max)
        else:
            pred = {"eps": "epsilon", "v": "v", "sample": "sample"}[cfg.objective]
            self.objective = DDPM(prediction=pred, min_snr_gamma=cfg.min_snr_gamma)
        self._lora_mats = [m for ad in (self.adapters or {}).values() if getattr(ad, "kind", "") == "lora"
                           for m in (ad.lora_A, ad.lora_B)]
        self._lora_t_stale = True
        self.step = 0
        self.micro = 0
        self.nan_skips = 0
        self._gen = None
        self._sumsq = None
        self._csv = None
        # per-phase device times (noise / forward / backward / optimizer), read with
        # ``trainer.phases.summary()``; off unless ERI_B200_PHASE_TIMING=1
        from ..utils.trace import PhaseTimer
        self.phases = PhaseTimer(enabled=os.environ.get("ERI_B200_PHASE_TIMING") == "1")

    def lr_rules(self, step):
        """``lr_if_contains`` with the ramp applied: during the warm-up the multiplier of the ramped
        parameters is ``base * (1 - f) + target * f`` with ``f`` the linear or half-cosine progress."""
        rules = dict(self.cfg.lr_if_contains or {})
        ramp = self.cfg.lr_ramp
        if ramp is None:
            return rules
        prog = min(1.0, step / max(1, ramp["warmup_steps"]))
        f = 0.5 * (1.0 - math.cos(prog * math.pi)) if ramp.get("kind") == "cosine" else prog
        key = ramp["contains"]
        base = next((float(m) for sub, m in rules.items() if sub in key or key in sub), 1.0)
        # the ramp rule goes first: block_lr_scale takes the first rule a name contains
        return {key: base * (1.0 - f) + float(ramp["target_mult"]) * f, **{k: v for k, v in rules.items() if k != key}}

    # ------------------------------------------------------------------ one micro-step
    def _generator(self, device):
        if self._gen is None or self._gen.device != torch.device(device):
            rank = self.grad_sync.rank if self.grad_sync is not None else 0
            # the ranks of a sequence-parallel group hold token slices of one sample: same timestep
            # stream for the group (the noise below stays per rank, as every rank owns other tokens)
            group = rank // max(1, self.cfg.seq_parallel)
            self._gen = torch.Generator(device=device).manual_seed(self.cfg.seed * 1000003 + group)
        return self._gen

    def train_step(self, batch: dict):
        """batch: ``latents`` [B, C, H, W] plus the conditioning tensors the model's forward
        function consumes. Returns the (device) loss tensor of this micro-batch."""
        mode = getattr(self, "strict_bf16", None)
        if mode:
            # STRICT_BF16: count (or refuse) clones, layout-fixing copies and fp32 up-casts of
            # activations during the step; the totals are in ``self.strict_events``
            from ..utils.strict import strict_scope
            with strict_scope(panic=mode == "panic", reset=False) as c:
                out = self._train_step(batch)
            self.strict_events = c.snapshot()
            return out
        if self.cfg.gc_freeze_after and self.step == self.cfg.gc_freeze_after and not getattr(self, "_gc_frozen", False):
            import gc
            gc.collect()
            gc.freeze()
            self._gc_frozen = True
        return self._train_step(batch)

    def _train_step(self, batch: dict):
        cfg = self.cfg
        x0 = batch["latents"]
        B = x0.shape[0]
        dev = x0.device
        ph = self.phases
        with ph.phase("noise"):
            t = self.objective.sample_t(B, self._generator(dev), dev)
            coef = self.objective.coefficients(t)
            rank = self.grad_sync.rank if self.grad_sync is not None else 0
            xt, target = F.noise_mix(x0, coef, seed=cfg.seed + 7919 * rank, offset=self.micro << 24,
                                     eps=batch.get("noise"), patch=cfg.patch)
        with ph.phase("forward"):
            pred = self.forward_fn(self.model, xt, self.objective.model_time(t), batch, cfg)
            loss = loss_fn(cfg.loss, pred, target, self.objective.loss_weight(t))
        with ph.phase("backward"):
            if self._lora_mats and self._lora_t_stale:
                # one launch transposes every adapter matrix for this step's backward
                F.prepare_lora_transposes(self._lora_mats)
                self._lora_t_stale = False
            (loss / cfg.grad_accum).backward()
        self.micro += 1
        if self.micro % cfg.grad_accum == 0:
            with ph.phase("optimizer"):
                self._optimizer_step()
        return loss.detach()

    def _optimizer_step(self):
        cfg = self.cfg
        lr = self.schedule.apply(self.optimizer, self.step)
        if self.rotator is not None:
            self.rotator.apply(self.optimizer, self.arena, self.step, cfg.lr_if_contains, self._lr_shard)
        elif not self._ramp_done:
            from ..optim.arena import block_lr_scale
            self.optimizer.lr_scale = block_lr_scale(self.arena, self.param_names, self.lr_rules(self.step),
                                                     shard=self._lr_shard)
            self._ramp_done = self.step >= cfg.lr_ramp["warmup_steps"]
        if self.grad_sync is not None and self.grad_sync.fused_optimizer:
            # reduce-scatter + clip + 8-bit AdamW + all-gather in the communication kernel
            self.grad_sync.reduce_and_step(lr=lr, max_grad_norm=cfg.max_grad_norm, step=self.step + 1)
        else:
            if self.grad_sync is not None:
                self.grad_sync.reduce_grads()
            if hasattr(self.optimizer, "arena"):
                sumsq = None
                if cfg.max_grad_norm > 0 or cfg.nan_policy == "skip":
                    if self.grad_sync is not None:
                        self._sumsq = self.grad_sync.grad_sumsq(self._sumsq)
                    else:
                        self._sumsq = F.sumsq(self.arena.grad, self._sumsq)
                    sumsq = self._sumsq
                self.optimizer.step(grad_sumsq=sumsq, max_grad_norm=cfg.max_grad_norm)
            else:
                if cfg.max_grad_norm > 0:
                    torch.nn.utils.clip_grad_norm_(self.arena.params, cfg.max_grad_norm)
                self.optimizer.step()
                self.arena.rebind_grads()
            if self.grad_sync is not None:
                self.grad_sync.gather_params()
        self.arena.zero_grad()
        if self._lora_mats:
            F.invalidate_lora_transposes()
            self._lora_t_stale = True
        if self.ema is not None:
            self.ema.update()
        self.step += 1
        if cfg.ckpt_every and cfg.out_dir and self.step % cfg.ckpt_every == 0:
            self.save_checkpoint()

    def grad_norm(self):
        """Last global gradient norm (device tensor) when clipping or NaN checks are on."""
        return None if self._sumsq is None else self._sumsq.sqrt()

    # ------------------------------------------------------------------ device health
    def status_sources(self):
        """Objects whose ``status()`` returns (and clears) a device status word set by a bounded
        peer wait that ran out: the fused data-parallel communicator, and the ZeRO-3 / sequence-
        parallel communicators when the job wired them (``extra_status_sources``)."""
        src = []
        fused = getattr(self.grad_sync, "_fused", None) if self.grad_sync is not None else None
        if fused is not None:
            src.append(("fused data-parallel step", fused))
        for name, obj in getattr(self, "extra_status_sources", []):
            src.append((name, obj))
        return src

    def check_device_status(self):
        """Read every device status word (this synchronises; call it where the loss is read anyway:
        log and checkpoint boundaries). A kernel whose bounded wait ran out has skipped its work
        (the fused optimizer step leaves parameters and moments untouched), so the step that set the
        word did not happen: raise instead of training on or saving from that state."""
        from ..utils.errors import CommTimeoutError, KernelError
        rank = self.grad_sync.rank if self.grad_sync is not None else 0
        for name, obj in self.status_sources():
            st = int(obj.status())
            if st:
                raise CommTimeoutError(st, rank=rank)
        if torch.cuda.is_available() and F.N.lib() is not None:
            words = F.kernel_error_check()
            if words:
                fam, code = next(iter(words.items()))
                raise KernelError(f"device error word of the {fam} kernels (all: {words})", code)

    # ------------------------------------------------------------------ logging
    def log_row(self, loss, sec_per_it, ckpt_path=""):
        """Append ``step,loss,grad_norm,sec_per_it,alloc_mb,ckpt_path`` (the reference's
        TRAIN_LOG_CSV columns, crates/training/src/run.rs:181-188). The device status words are
        read first: a logged step is a step that really ran."""
        self.check_device_status()
        path = self.cfg.log_csv or os.environ.get("TRAIN_LOG_CSV")
        if not path:
            return
        new = not os.path.exists(path)
        with open(path, "a") as f:
            if new:
                f.write("step,loss,grad_norm,sec_per_it,alloc_mb,ckpt_path\n")
            gn = self.grad_norm()
            alloc = torch.cuda.memory_allocated() / 2 ** 20 if torch.cuda.is_available() else 0.0
            f.write(f"{self.step},{float(loss):.6f},{float(gn) if gn is not None else float('nan'):.6f},"
                    f"{sec_per_it:.6f},{alloc:.1f},{ckpt_path}\n")

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, root=None):
        """LoRA: ``{root}/step_{step:06}/lora.safetensors`` (+ ``ema.safetensors``, ``meta.json``),
        the phase-4 layout (crates/training/src/flux_trainer.rs:416-439, 633-666). Full fine-tune:
        ``{root}/checkpoint-{step:06}/model.safetensors`` with ``model.`` key prefix plus
        ``optimizer.safetensors`` and ``metadata.json`` (src/trainers/checkpoint_saver.rs:63-118)."""
        from .checkpoint import save_training_checkpoint
        self.check_device_status()          # never write a checkpoint from a state a failed step left
        return save_training_checkpoint(self, root or self.cfg.out_dir)

    def load_latest_checkpoint(self, root=None):
        from .checkpoint import load_latest_training_checkpoint
        return load_latest_training_checkpoint(self, root or self.cfg.out_dir)


def default_forward(model, xt, t, batch, cfg):
    """MMDiT-style call: model(img_tokens, txt, t, pooled, guidance)."""
    g = None
    if getattr(getattr(model, "cfg", None), "guidance_embed", False):
        gv = 1.0 if cfg.guidance is None else cfg.guidance
        g = torch.full((xt.shape[0],), float(gv), device=xt.device)
    if cfg.activation_checkpointing:
        from .act_checkpoint import checkpointed_forward
        return checkpointed_forward(model, xt, batch["txt"], t, batch.get("pooled"), g)
    return model(xt, batch["txt"], t, batch.get("pooled"), g, grid_hw=batch.get("grid_hw"))


def ltx_forward(model, xt, t, batch, cfg):
    """LTX-style call: model(tokens, text, t, (frames, h, w))."""
    return model(xt, batch["txt"], t, batch["grid_fhw"])


def ltx_av_forward(model, xt, t, batch, cfg):
    """LTX audio + video: the training latent is the token sequence [video tokens | audio tokens]
    (both 128 channels), noised with one timestep; the prediction is the two streams' outputs in the
    same order, so the loss covers both (joint forward of ltx2_model.rs:53-151)."""
    f, h, w = batch["grid_fhw"]
    lv = f * h * w
    pv, pa = model(xt[:, :lv].contiguous(), xt[:, lv:].contiguous(), batch["txt"], t, batch["grid_fhw"])
    return torch.cat([pv, pa], dim=1)
