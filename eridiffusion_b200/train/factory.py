"""From a loaded ``TrainCfg`` to a running job: model, adapters / full fine-tune, parallel engine,
data source, trainer. This is the dispatch the reference's unified CLI advertises but leaves
disabled for every family (src/trainers/mod.rs:356-430 returns "temporarily disabled").
"""
from __future__ import annotations

import torch

from ..adapters import AdapterConfig
from ..config import TrainCfg
from ..data import CachedEmbeddingLoader, synthetic_batch
from ..models import build_model
from ..parallel.dist import GradSync, init_from_env
from .trainer import Trainer, TrainerConfig, default_forward, ltx_forward

_KIND_TO_MODEL = {"flux": "flux", "chroma": "chroma", "qwen_image": "qwen_image", "sdxl": "sdxl",
                  "sd3": "sd35", "sd35": "sd35", "ltx": "ltx_video", "wan22": "wan22", "klein": "klein",
                  "zimage": "zimage", "tiny_mmdit": "tiny_mmdit", "krea": "krea", "hunyuan": "hunyuan",
                  "lumina": "lumina", "hidream_i1": "hidream", "hidream": "hidream", "omnigen2": "omnigen2",
                  "qwen_edit_image": "qwen_edit_image", "sd15": "sd15"}
_UNIMPLEMENTED = set()


def build_job(cfg: TrainCfg, device=None):
    """Returns (trainer, batch_iterator, info)."""
    if cfg.model.kind in _UNIMPLEMENTED:
        raise NotImplementedError(
            f"model kind {cfg.model.kind!r}: the reference registers this family with a forward that "
            "returns zeros (crates/models/*/src/lib.rs); no architecture is defined to train")
    rank, world, local = init_from_env()
    cuda = torch.cuda.is_available() and not cfg.device.startswith("cpu")
    dev = torch.device(device) if device else (torch.device("cuda", local) if cuda else torch.device("cpu"))
    dtype = torch.bfloat16 if cuda else torch.float32
    model_id = _KIND_TO_MODEL[cfg.model.kind]
    model = build_model(model_id, device=dev, dtype=dtype, **cfg.model.overrides)
    if cfg.model.name_or_path:
        from ..io.weights import load_model_weights
        load_model_weights(model, cfg.model.name_or_path, cfg.model.kind)
    if cfg.model.quantize and cfg.train_mode == "lora":
        from ..memory import quantize_model
        quantize_model(model, "int8")

    par = cfg.parallel
    grad_sync = None
    seq_par = par.ulysses if world > 1 else 1
    ctx_par = par.context if world > 1 else 1
    if ctx_par > 1:
        # ring attention: every rank holds a token slice of the same sample; only self-attention
        # communicates, so the degree is not tied to the head count
        if seq_par > 1:
            raise ValueError("parallel.context and parallel.ulysses are mutually exclusive")
        if ctx_par != world:
            raise ValueError(f"parallel.context ({ctx_par}) must equal the number of ranks ({world})")
        if not hasattr(model, "set_context_parallel"):
            raise ValueError(f"model kind '{cfg.model.kind}' has no context-parallel attention path")
        model.set_context_parallel()
        grad_sync = GradSync("allreduce")
        seq_par = ctx_par                    # same batch / timestep handling as a sequence-parallel group
    elif seq_par > 1:
        # one sequence-parallel group spanning the job: every rank holds a token slice of the same
        # sample, the two all-to-alls run inside the QKV / output projections
        if seq_par != world:
            raise ValueError(f"parallel.ulysses ({seq_par}) must equal the number of ranks ({world})")
        if not hasattr(model, "set_sequence_parallel"):
            raise ValueError(f"model kind '{cfg.model.kind}' has no sequence-parallel attention path")
        if model.cfg.num_heads % world:
            raise ValueError("the head count must divide by parallel.ulysses")
        grad_sync = GradSync("allreduce")
    elif world > 1:
        if par.zero_stage == 3:
            from ..parallel.zero3 import Zero3Context, Zero3Sync, shard_model
            z3 = Zero3Context()
            sharded, replicated = shard_model(model, z3)
            grad_sync = Zero3Sync(z3, sharded, replicated)
        else:
            mode = "allreduce" if par.zero_stage == 0 and par.fused_comm != "on" else \
                ("fused" if par.fused_comm == "on" and cfg.train_mode == "lora" or
                 (par.fused_comm == "on" and cfg.optimizer.lower().startswith("adamw8")) else "zero1")
            grad_sync = GradSync(mode)

    objective = {"flowmatch": "flow", "flow": "flow", "ddpm": "eps", "eps": "eps", "v": "v"}.get(
        cfg.noise_scheduler, "flow" if cfg.model.kind not in ("sdxl", "sd15") else "eps")
    if cfg.model.kind in ("sdxl", "sd15"):
        objective = "eps" if objective == "flow" else objective
    acfg = None
    if cfg.train_mode == "lora":
        n = cfg.network
        acfg = AdapterConfig(kind=n.type if n.type in ("lora", "loha", "lokr", "dora", "ia3", "glora") else "lora",
                             rank=n.linear, alpha=n.linear_alpha, dropout=n.dropout, dtype=dtype)
    tcfg = TrainerConfig(
        mode=cfg.train_mode, adapter=acfg, objective=objective,
        timestep_sampler="uniform" if cfg.linear_timesteps else cfg.timestep_sampler,
        guidance=1.0 if cfg.bypass_guidance_embedding and cfg.guidance is None else (cfg.guidance or 3.5),
        optimizer=cfg.optimizer, lr=cfg.lr, weight_decay=cfg.weight_decay, lr_schedule=cfg.lr_schedule,
        warmup_steps=cfg.warmup_steps, total_steps=cfg.steps, grad_accum=cfg.grad_accum_steps,
        max_grad_norm=cfg.max_grad_norm, ema_decay=cfg.ema_decay, seed=cfg.seed, seq_parallel=seq_par,
        out_dir=cfg.training_folder, ckpt_every=cfg.ckpt_every, keep_last=cfg.save.max_step_saves_to_keep,
        activation_checkpointing=cfg.gradient_checkpointing and not cuda, stochastic_rounding=cuda,
        patch=1 if cfg.model.kind in ("sdxl", "sd15", "ltx", "wan22") else 2,
        lr_if_contains=dict(cfg.network.lr_if_contains or {}) if cfg.train_mode == "lora" else {})
    fwd = default_forward
    if cfg.model.kind == "ltx":
        fwd = ltx_forward
    elif cfg.model.kind in ("sdxl", "sd15"):
        from ..models.sdxl_unet import sdxl_forward
        fwd = sdxl_forward
    trainer = Trainer(model, tcfg, grad_sync=grad_sync, forward_fn=fwd)

    ds = cfg.datasets[0] if cfg.datasets else None
    if ds is not None and ds.manifest and not ds.synthetic:
        loader = CachedEmbeddingLoader(ds.manifest, kind="sdxl" if cfg.model.kind == "sdxl" else "flux",
                                       batch_size=cfg.batch_size, root_dir=ds.manifest_root,
                                       index_path=ds.manifest_index, shuffle=ds.manifest_shuffle,
                                       repeat=ds.manifest_repeat, seed=cfg.seed, device=dev,
                                       rank=0 if seq_par > 1 else rank, world=1 if seq_par > 1 else world,
                                       validate=ds.manifest_validate)
        batches = iter(loader)
    else:
        res = (ds.resolution[0] if ds and ds.resolution else 1024)

        def gen():
            i = 0
            while True:
                yield synthetic_batch(model_id if model_id != "ltx_video" else "ltx", cfg.batch_size, dev, dtype,
                                      seed=cfg.seed + (i if seq_par > 1 else i * world + rank), height=res,
                                      width=res)
                i += 1
        batches = gen()
    if ctx_par > 1:
        batches = _token_slices(batches, rank, world)
    elif seq_par > 1:
        batches = _sequence_parallel_batches(batches, model, rank, world)
    return trainer, batches, {"rank": rank, "world": world, "device": str(dev), "model": model_id}


def _token_slices(batches, rank, world):
    """Every rank keeps its contiguous token slice of the token-major latents ``[B, C, L, 1]``."""
    for b in batches:
        lat = b["latents"]
        L = lat.shape[2]
        if L % world:
            raise ValueError(f"token count {L} must divide by the context-parallel size {world}")
        Ll = L // world
        yield {**b, "latents": lat[:, :, rank * Ll:(rank + 1) * Ll].contiguous()}


def _sequence_parallel_batches(batches, model, rank, world):
    """Every rank of the group receives the same sample and keeps its contiguous token slice of the
    token-major latents ``[B, C, L, 1]``; the attention context is created from the first batch."""
    from ..parallel.dist import ProcessGroup
    from ..parallel.ulysses import UlyssesContext
    attached = False
    for b in batches:
        lat = b["latents"]
        L = lat.shape[2]
        if L % world:
            raise ValueError(f"token count {L} must divide by the sequence-parallel size {world}")
        Ll = L // world
        if not attached:
            model.set_sequence_parallel(UlyssesContext(ProcessGroup(), batch=lat.shape[0], l_local=Ll,
                                                       hidden=model.cfg.hidden, heads=model.cfg.num_heads,
                                                       attn_slots=len(model.blocks)))
            attached = True
        b = dict(b)
        b["latents"] = lat[:, :, rank * Ll:(rank + 1) * Ll].contiguous()
        yield b
