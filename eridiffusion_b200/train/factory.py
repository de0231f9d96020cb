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


def _reject_unsupported(cfg: TrainCfg, world: int):
    """Every accepted key either changes what runs or is refused here, by name: a configuration
    that asks for something this job cannot do must not train as if it had not asked."""
    from ..config import ConfigError
    n = cfg.network
    if cfg.train_mode == "lora" and n.conv:
        raise ConfigError("network.conv: convolution adapters (LoCon) are injected through adapters.LoConConv2d "
                          "by hand; the job factory only adapts linear layers — remove network.conv")
    if len(cfg.datasets) > 1:
        raise ConfigError(f"{len(cfg.datasets)} datasets configured: the job factory trains on one; merge the "
                          "folders (or their manifests) into one dataset entry")
    if cfg.mode == "srpo":
        raise ConfigError("mode srpo: the reference gates this mode off (model_registry.rs:327-347, "
                          "'baseline-only for now') and defines no objective for it; nothing to run")
    if cfg.use_layer_streaming and cfg.train_mode != "lora":
        raise ConfigError("use_layer_streaming needs train_mode lora: trainable weights live in the "
                          "optimizer's flat arena and cannot leave the device")
    if cfg.use_layer_streaming and world > 1:
        raise ConfigError("use_layer_streaming is a single-GPU memory measure; with several ranks use "
                          "parallel.zero_stage 3 instead")
    if (cfg.tread.enabled or cfg.mode == "tread") and cfg.model.kind not in _TREAD_KINDS:
        raise ConfigError(f"tread: token routing is wired into the single-stream stack of the MMDiT families "
                          f"{sorted(_TREAD_KINDS)}; model kind {cfg.model.kind!r} has none")
    if cfg.recipe:
        from .pipelines import StageName
        known = {s.value if hasattr(s, "value") else str(s) for s in StageName}
        bad = [r for r in cfg.recipe if str(r) not in known]
        if bad:
            raise ConfigError(f"recipe: unknown stages {bad}; known: {sorted(known)}")


_TREAD_KINDS = {"flux", "chroma", "krea", "tiny_mmdit", "hunyuan", "hidream", "hidream_i1"}


def _block_runner(cfg: TrainCfg, model, dev, cuda: bool):
    """Activation policy, layer streaming and TREAD routing for the MMDiT families (``model.runner``);
    other families get per-block recomputation through ``enable_block_recompute``."""
    from .act_checkpoint import BlockRunner, TreadRouter
    policy = "none"
    if cfg.gradient_checkpointing:
        # GRADIENT_CHECKPOINT_POLICY (recorded by config.apply_env) wins; low_vram parks block inputs on the host
        policy = cfg.meta.get("checkpoint_policy") or ("cpu_offload" if (cfg.model.low_vram and cuda) else "recompute")
    streamer = None
    if cfg.use_layer_streaming:
        from ..memory import BlockSwapConfig, BlockSwapManager
        blocks = model.block_list()
        budget = cfg.streaming_memory_limit_gb or BlockSwapConfig.gpu_budget_gb
        # the first and the last block stay resident (the reference pins the input / output layers,
        # src/trainers/flux_layer_streaming.rs:259-283)
        scfg = BlockSwapConfig(gpu_budget_gb=float(budget), persistent=(0, len(blocks) - 1))
        streamer = BlockSwapManager(blocks, scfg, device=dev, frozen_only=True)
    tread = None
    if cfg.tread.enabled or cfg.mode == "tread":
        t = cfg.tread
        n_single = len(getattr(model, "single_blocks", []))
        schedule = t.schedule or [{"out": 1, "in": max(2, n_single - 1)}]
        tread = TreadRouter(schedule, k=t.k, k_frac=t.k_frac if t.k is None else None or 0.5,
                            mask_type=t.mask_type, reinject=t.reinject)
    if policy == "none" and streamer is None and tread is None:
        return None
    return BlockRunner(policy=policy, streamer=streamer, tread=tread)


def enable_block_recompute(model):
    """Re-run every block of ``model.block_list()`` in backward instead of keeping its activations
    (families without a ``runner`` hook: UNets, video and single-stream DiTs)."""
    import torch.utils.checkpoint as ckpt
    n = 0
    for blk in model.block_list():
        if getattr(blk, "_eri_recompute", False):
            continue
        inner = blk.forward

        def fwd(*a, _inner=inner, **kw):
            if torch.is_grad_enabled() and any(torch.is_tensor(x) and x.requires_grad for x in a):
                return ckpt.checkpoint(_inner, *a, use_reentrant=False, **kw)
            return _inner(*a, **kw)
        blk.forward = fwd
        blk._eri_recompute = True
        n += 1
    return n


def _folder_manifest(cfg: TrainCfg, ds, dev, dtype):
    """A dataset given as a folder of images (+ ``.txt`` captions) and no manifest: encode all latents,
    free the VAE, encode all captions, free the text encoders, write the manifest — the order of the
    reference's sequential trainer (src/trainers/pipeline_flux_lora_sequential.rs:98-557). Cached
    samples are reused; a second start costs nothing."""
    from pathlib import Path
    from ..config import ConfigError
    from ..data.precache import precache_folder
    from ..models import build_model as build
    m = cfg.model
    sdxl = m.kind in ("sdxl", "sd15")
    rnd = bool(ds.random_init_encoders)
    if not rnd and not m.vae_path:
        raise ConfigError(f"dataset folder {ds.folder_path!r} has no manifest and model.vae_path is not set: give "
                          "the VAE and text-encoder weights (so that the folder can be cached), a prepared "
                          "manifest, or `synthetic: true` for synthetic batches")
    enc_w = (m.clip_l_path, m.clip_g_path) if sdxl else (m.t5_path or m.text_encoder_path, m.clip_l_path or m.text_encoder_2_path)
    if not rnd and not enc_w[0]:
        raise ConfigError(f"dataset folder {ds.folder_path!r} has no manifest and no text-encoder weights are set "
                          f"({'clip_l_path / clip_g_path' if sdxl else 't5_path / clip_l_path'})")
    enc_kw = dict(ds.encoder_overrides or {})

    def load(kind, weights):
        mod = build(kind, device=dev, dtype=dtype, **enc_kw.get(kind, {})).eval()
        if weights:
            from ..io.weights import load_model_weights
            load_model_weights(mod, weights, kind, strict=False)
        return mod

    def make_vae():
        return load("vae_sdxl" if sdxl else "vae_flux", m.vae_path)

    def make_text_encoder():
        from ..data.tokenizers import HashTokenizer, load_tokenizer
        first = load("clip_l" if sdxl else "t5_encoder", enc_w[0])
        second = load("open_clip_g" if sdxl else "clip_l", enc_w[1]) if (enc_w[1] or rnd) else None

        def tok(path, kind, enc, n):
            # no tokenizer files: the deterministic hash tokeniser, sized to the encoder's vocabulary
            if path:
                return load_tokenizer(path, kind, n)
            return HashTokenizer(enc.cfg.vocab_size, n, eos_id=1 if kind == "t5" else None,
                                 pad_id=0, first_id=min(1000, enc.cfg.vocab_size // 2))
        tok1 = tok(m.clip_l_tokenizer if sdxl else m.t5_tokenizer, "clip" if sdxl else "t5", first,
                   int(ds.max_text_tokens or (77 if sdxl else 512)))
        tok2 = None if second is None else tok(m.clip_g_tokenizer if sdxl else m.clip_l_tokenizer, "clip", second, 77)

        def encode(prompt):
            ids, mask = tok1(prompt)
            if sdxl:
                h1, _ = first(ids.to(dev), output_layer=-2)
                ids2, _ = tok2(prompt)
                h2, pooled = second(ids2.to(dev), output_layer=-2)
                return torch.cat([h1, h2], dim=-1), pooled, None
            h = first(ids.to(dev), mask.to(dev))
            pooled = None
            if second is not None:
                ids2, _ = tok2(prompt)
                _, pooled = second(ids2.to(dev))
            return h, pooled, mask
        return encode

    res = ds.resolution[0] if ds.resolution else 1024
    root = Path(cfg.training_folder) / cfg.name
    name = Path(ds.folder_path).name or "dataset"
    if ds.force_recache:
        import shutil
        shutil.rmtree(root / "cache" / "vae" / name, ignore_errors=True)
        shutil.rmtree(root / "cache" / "text" / name, ignore_errors=True)
    mpath, report = precache_folder(ds.folder_path, root, name, make_vae, make_text_encoder, size=res,
                                    trigger_word=cfg.trigger_word)
    return mpath, root, report


def build_job(cfg: TrainCfg, device=None):
    """Returns (trainer, batch_iterator, info)."""
    if cfg.model.kind in _UNIMPLEMENTED:
        raise NotImplementedError(
            f"model kind {cfg.model.kind!r}: the reference registers this family with a forward that "
            "returns zeros (crates/models/*/src/lib.rs); no architecture is defined to train")
    rank, world, local = init_from_env()
    _reject_unsupported(cfg, world)
    cuda = torch.cuda.is_available() and not cfg.device.startswith("cpu")
    dev = torch.device(device) if device else (torch.device("cuda", local) if cuda else torch.device("cpu"))
    dtype = torch.bfloat16 if cuda else torch.float32
    model_id = _KIND_TO_MODEL[cfg.model.kind]
    torch.manual_seed(cfg.seed)             # random-init weights (no checkpoint given) are a function of the seed
    model = build_model(model_id, device=dev, dtype=dtype, **cfg.model.overrides)
    if cfg.model.name_or_path:
        from ..io.weights import load_model_weights
        load_model_weights(model, cfg.model.name_or_path, cfg.model.kind)
    if cfg.model.quantize and cfg.train_mode == "lora":
        from ..memory import quantize_model
        quantize_model(model, "int8")
    elif cfg.model.quantize:
        from ..config import ConfigError
        raise ConfigError("model.quantize needs train_mode lora: a quantised base weight cannot be fine-tuned in full")

    par = cfg.parallel
    grad_sync = None
    status_sources = []
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
            status_sources.append(("ZeRO-3 communicator", z3.comm))
        else:
            mode = "allreduce" if par.zero_stage == 0 and par.fused_comm != "on" else \
                ("fused" if par.fused_comm == "on" and cfg.train_mode == "lora" or
                 (par.fused_comm == "on" and cfg.optimizer.lower().startswith("adamw8")) else "zero1")
            grad_sync = GradSync(mode)

    sigma_eps = cfg.schedule_name in ("sigma_eps", "eps_sigma", "bounded_sigma", "phase4_eps")
    objective = {"flowmatch": "flow", "flow": "flow", "ddpm": "eps", "eps": "eps", "v": "v"}.get(
        cfg.noise_scheduler, "flow" if cfg.model.kind not in ("sdxl", "sd15") else "eps")
    if cfg.model.kind in ("sdxl", "sd15"):
        objective = "eps" if objective == "flow" else objective
    if sigma_eps:
        objective = "sigma_eps"
    elif cfg.schedule_name and cfg.schedule_name not in ("flow", "flowmatch", "flow_matching", "ddpm", "eps", "v",
                                                         "linear", "cosine", "constant"):
        from ..config import ConfigError
        raise ConfigError(f"schedule_name {cfg.schedule_name!r}: known names are flow / flowmatch / ddpm / eps / v "
                          "(objective), linear / cosine / constant (learning-rate schedule) and sigma_eps")
    if (cfg.sigma_min is not None or cfg.sigma_max is not None) and not sigma_eps:
        from ..config import ConfigError
        raise ConfigError("sigma_min / sigma_max belong to the additive-noise eps objective: set "
                          "schedule_name: sigma_eps (schedule.name in the nested form)")
    lr_schedule = cfg.schedule_name if cfg.schedule_name in ("linear", "cosine", "constant") else cfg.lr_schedule
    acfg = None
    if cfg.train_mode == "lora":
        n = cfg.network
        acfg = AdapterConfig(kind=n.type if n.type in ("lora", "loha", "lokr", "dora", "ia3", "glora") else "lora",
                             rank=n.linear, alpha=n.linear_alpha, dropout=n.dropout, dtype=dtype,
                             init="kaiming" if n.zero_init else "nonzero")
    mmdit_runner = hasattr(model, "runner")
    tcfg = TrainerConfig(
        mode=cfg.train_mode, adapter=acfg, objective=objective,
        sigma_min=cfg.sigma_min if cfg.sigma_min is not None else 0.02,
        sigma_max=cfg.sigma_max if cfg.sigma_max is not None else 1.0,
        timestep_sampler="uniform" if cfg.linear_timesteps else cfg.timestep_sampler,
        guidance=1.0 if cfg.bypass_guidance_embedding and cfg.guidance is None else (cfg.guidance or 3.5),
        optimizer=cfg.optimizer, lr=cfg.lr, weight_decay=cfg.weight_decay, lr_schedule=lr_schedule,
        warmup_steps=cfg.warmup_steps, total_steps=cfg.schedule_steps or cfg.steps, grad_accum=cfg.grad_accum_steps,
        max_grad_norm=cfg.max_grad_norm, ema_decay=cfg.ema_decay, seed=cfg.seed, seq_parallel=seq_par,
        out_dir=cfg.training_folder, ckpt_every=cfg.ckpt_every, keep_last=cfg.save.max_step_saves_to_keep,
        activation_checkpointing=False, stochastic_rounding=cuda,
        patch=1 if cfg.model.kind in ("sdxl", "sd15", "ltx", "wan22") else 2,
        lr_if_contains=dict(cfg.network.lr_if_contains or {}) if cfg.train_mode == "lora" else {},
        lr_ramp=_lr_ramp(cfg))
    fwd = default_forward
    if cfg.model.kind == "ltx":
        fwd = ltx_forward
    elif cfg.model.kind in ("sdxl", "sd15"):
        from ..models.sdxl_unet import sdxl_forward
        fwd = sdxl_forward
    trainer = Trainer(model, tcfg, grad_sync=grad_sync, forward_fn=fwd)
    trainer.extra_status_sources = status_sources
    trainer.strict_bf16 = cfg.meta.get("strict_bf16")       # None | "count" | "panic" (STRICT_BF16)
    # activation policy / layer streaming / token routing are attached after the adapters exist, so
    # that the streamer sees which tensors are trainable
    recompute_blocks = 0
    if mmdit_runner:
        model.runner = _block_runner(cfg, model, dev, cuda)
    elif cfg.gradient_checkpointing and hasattr(model, "block_list"):
        recompute_blocks = enable_block_recompute(model)
    elif cfg.gradient_checkpointing:
        from ..config import ConfigError
        raise ConfigError(f"gradient_checkpointing: model kind {cfg.model.kind!r} exposes no block list to recompute")
    if cfg.use_layer_streaming and not mmdit_runner:
        from ..config import ConfigError
        raise ConfigError(f"use_layer_streaming: model kind {cfg.model.kind!r} has no streamed block stack")

    ds = cfg.datasets[0] if cfg.datasets else None
    data_info = {"source": "synthetic"}
    manifest, manifest_root = (ds.manifest, ds.manifest_root) if ds is not None else (None, None)
    if ds is not None and not ds.synthetic and not manifest and ds.folder_path:
        manifest, manifest_root, report = _folder_manifest(cfg, ds, dev, dtype)
        data_info = {"source": "folder", "cache": report}
    if ds is not None and manifest and not ds.synthetic:
        loader = CachedEmbeddingLoader(manifest, kind="sdxl" if cfg.model.kind == "sdxl" else "flux",
                                       batch_size=cfg.batch_size, root_dir=manifest_root,
                                       index_path=ds.manifest_index, shuffle=ds.manifest_shuffle,
                                       repeat=ds.manifest_repeat, seed=cfg.seed, device=dev,
                                       rank=0 if seq_par > 1 else rank, world=1 if seq_par > 1 else world,
                                       validate=ds.manifest_validate,
                                       prefetch=cfg.prefetch if cfg.prefetch else 2)
        batches = iter(loader)
        if dtype != torch.bfloat16:
            # cache files hold bf16; a CPU (fp32) job converts the floating tensors of every batch
            batches = ({k: (v.to(dtype) if torch.is_tensor(v) and v.is_floating_point() else v) for k, v in b.items()}
                       for b in batches)
        if data_info["source"] == "synthetic":
            data_info = {"source": "manifest"}
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
        batches = _sequence_parallel_batches(batches, model, rank, world, trainer)
    return trainer, batches, {"rank": rank, "world": world, "device": str(dev), "model": model_id,
                              "data": data_info, "objective": objective,
                              "runner": None if not getattr(model, "runner", None) else {
                                  "policy": model.runner.policy, "streaming": model.runner.streamer is not None,
                                  "tread": model.runner.tread is not None},
                              "recompute_blocks": recompute_blocks}


def _lr_ramp(cfg: TrainCfg):
    """``network.ramp_*``: the learning-rate multiplier of the double-stream blocks moves from its
    base value to ``ramp_target_lr / lr`` over ``ramp_warmup_steps`` optimizer steps, linearly or on
    a half cosine (src/trainers/flux_layer_streaming.rs:362-392)."""
    n = cfg.network
    if not n.ramp_double_blocks:
        return None
    if not n.ramp_target_lr or not n.ramp_warmup_steps:
        from ..config import ConfigError
        raise ConfigError("network.ramp_double_blocks needs ramp_target_lr and ramp_warmup_steps")
    return {"contains": "double_blocks", "target_mult": float(n.ramp_target_lr) / float(cfg.lr),
            "warmup_steps": int(n.ramp_warmup_steps), "kind": (n.ramp_type or "linear").lower()}


def _token_slices(batches, rank, world):
    """Every rank keeps its contiguous token slice of the token-major latents ``[B, C, L, 1]``."""
    for b in batches:
        lat = b["latents"]
        L = lat.shape[2]
        if L % world:
            raise ValueError(f"token count {L} must divide by the context-parallel size {world}")
        Ll = L // world
        yield {**b, "latents": lat[:, :, rank * Ll:(rank + 1) * Ll].contiguous()}


def _sequence_parallel_batches(batches, model, rank, world, trainer=None):
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
            u = UlyssesContext(ProcessGroup(), batch=lat.shape[0], l_local=Ll, hidden=model.cfg.hidden,
                               heads=model.cfg.num_heads, attn_slots=len(model.blocks))
            model.set_sequence_parallel(u)
            if trainer is not None:
                trainer.extra_status_sources = list(getattr(trainer, "extra_status_sources", [])) + [
                    ("sequence-parallel communicator", u.comm)]
            attached = True
        b = dict(b)
        b["latents"] = lat[:, :, rank * Ll:(rank + 1) * Ll].contiguous()
        yield b
