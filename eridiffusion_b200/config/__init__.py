"""Training configuration: loads the reference's two YAML schemas unchanged and maps them onto
one typed tree, plus a ``parallel:`` block and a single ``ERI_B200_*`` environment namespace.

Schema 1 — ai-toolkit style nested YAML (src/config/trainer_config.rs:9-236):
``job / config{name, process[{type, training_folder, device, network{type, linear, linear_alpha,
conv, conv_alpha, network_kwargs.lr_if_contains}, save{dtype, save_every,
max_step_saves_to_keep}, datasets[{folder_path, caption_ext, caption_dropout_rate, shuffle_tokens,
cache_latents_to_disk, resolution}], train{batch_size, steps, gradient_accumulation_steps,
gradient_checkpointing, noise_scheduler, optimizer, lr, ema_config, dtype, linear_timesteps,
bypass_guidance_embedding, use_layer_streaming, streaming_memory_limit_gb}, model{name_or_path,
arch, is_flux, is_v3, is_sdxl, quantize, low_vram, vae_path, ...}, sample{sampler, sample_every,
width, height, prompts, neg, seed, walk_seed, guidance_scale, sample_steps}, tread{...}}]} / meta``

Schema 2 — flat ``TrainCfg`` keyed by ``model_kind`` (crates/training/src/model_registry.rs:125-289;
templates crates/training/config/templates/train_*.yaml): ``model_kind, weights, bf16_params,
steps, batch_size, grad_accum_steps, lr, seed, ckpt_every, optimizer, mode, flux_manifest*, ...``

Validation follows crates/training/src/eridiffusion_config.rs:203-369 (batch > 0, steps > 0,
lr in [1e-7, 1e-2], bf16 only, device ``cuda:N``); unknown keys raise instead of being ignored.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field, fields, asdict
from pathlib import Path

import yaml

MODEL_KINDS = ("flux", "sdxl", "sd3", "sd35", "qwen_image", "wan22", "ltx", "hunyuan", "lumina",
               "hidream_i1", "hidream", "omnigen2", "chroma", "klein", "zimage", "krea", "qwen_edit_image",
               "tiny_mmdit", "sd15")


class ConfigError(ValueError):
    pass


@dataclass
class NetworkCfg:
    type: str = "lora"
    linear: int = 16
    linear_alpha: float = 16.0
    conv: int | None = None
    conv_alpha: float | None = None
    dropout: float = 0.0
    lr_if_contains: dict = field(default_factory=dict)
    ramp_double_blocks: bool | None = None
    ramp_target_lr: float | None = None
    ramp_warmup_steps: int | None = None
    ramp_type: str | None = None


@dataclass
class SaveCfg:
    dtype: str = "bf16"
    save_every: int = 0
    max_step_saves_to_keep: int = 0
    push_to_hub: bool = False
    hf_repo_id: str | None = None
    hf_private: bool | None = None


@dataclass
class DatasetCfg:
    folder_path: str = ""
    caption_ext: str = "txt"
    caption_dropout_rate: float = 0.0
    shuffle_tokens: bool = False
    cache_latents_to_disk: bool = True
    resolution: list = field(default_factory=lambda: [1024])
    force_recache: bool = False
    manifest: str | None = None
    manifest_root: str | None = None
    manifest_index: str | None = None
    manifest_validate: bool = False
    manifest_shuffle: bool = True
    manifest_repeat: int = 1
    synthetic: bool = False


@dataclass
class TreadCfg:
    enabled: bool = False
    mask_type: str = "topk_norm"        # attn_topk | topk_norm | random | uniform
    k: int | None = None
    k_frac: float | None = 0.5
    schedule: list = field(default_factory=list)     # [{out: i, in: j}]
    reinject: str = "scatter"
    route_lambda: float = 0.0


@dataclass
class SampleCfg:
    sampler: str = "flowmatch"
    sample_every: int = 0
    width: int = 1024
    height: int = 1024
    prompts: list = field(default_factory=list)
    neg: str = ""
    seed: int = 42
    walk_seed: bool = False
    guidance_scale: float = 3.5
    sample_steps: int = 20


@dataclass
class ModelCfg:
    kind: str = "flux"
    name_or_path: str | None = None
    arch: str | None = None
    quantize: bool = False
    low_vram: bool = False
    vae_path: str | None = None
    text_encoder_path: str | None = None
    text_encoder_2_path: str | None = None
    clip_l_path: str | None = None
    t5_path: str | None = None
    variant: str | None = None
    overrides: dict = field(default_factory=dict)


@dataclass
class ParallelCfg:
    dp: int = 1
    zero_stage: int = 0                 # 0 (DDP) | 1/2 (sharded optimizer + grads) | 3 (sharded params)
    ulysses: int = 1
    context: int = 1                    # ring-attention context parallelism degree (token slices per sample)
    fused_comm: str = "on"              # on | nccl


@dataclass
class TrainCfg:
    name: str = "run"
    training_folder: str = "output"
    device: str = "cuda:0"
    mode: str = "baseline"              # baseline | tread | srpo
    train_mode: str = "lora"            # lora | full
    batch_size: int = 1
    steps: int = 10
    grad_accum_steps: int = 1
    lr: float = 1e-4
    optimizer: str = "adamw8bit"
    weight_decay: float = 0.01
    lr_schedule: str = "constant"
    warmup_steps: int = 0
    max_grad_norm: float = 1.0
    noise_scheduler: str = "flowmatch"
    timestep_sampler: str = "logit_normal"
    linear_timesteps: bool = False
    bypass_guidance_embedding: bool = True
    guidance: float | None = None
    gradient_checkpointing: bool = False
    use_layer_streaming: bool = False
    streaming_memory_limit_gb: float | None = None
    dtype: str = "bf16"
    seed: int = 42
    ckpt_every: int = 0
    ema_decay: float | None = None
    performance_log_every: int = 10
    trigger_word: str | None = None
    offload_pinned_threshold_mb: int | None = None
    network: NetworkCfg = field(default_factory=NetworkCfg)
    save: SaveCfg = field(default_factory=SaveCfg)
    datasets: list = field(default_factory=list)
    model: ModelCfg = field(default_factory=ModelCfg)
    sample: SampleCfg = field(default_factory=SampleCfg)
    tread: TreadCfg = field(default_factory=TreadCfg)
    parallel: ParallelCfg = field(default_factory=ParallelCfg)
    meta: dict = field(default_factory=dict)

    def validate(self):
        if self.batch_size <= 0:
            raise ConfigError("batch_size must be > 0")
        if self.steps <= 0:
            raise ConfigError("steps must be > 0")
        if not (1e-7 <= self.lr <= 1e-2):
            raise ConfigError(f"lr {self.lr} outside [1e-7, 1e-2]")
        if self.dtype not in ("bf16", "bfloat16"):
            raise ConfigError("only bf16 training is supported")
        if not (self.device == "cpu" or self.device.startswith("cuda")):
            raise ConfigError(f"device {self.device!r} must be cuda:N")
        if self.model.kind not in MODEL_KINDS:
            raise ConfigError(f"unknown model kind {self.model.kind!r}")
        if self.parallel.zero_stage not in (0, 1, 2, 3):
            raise ConfigError("zero_stage must be 0..3")
        if self.mode not in ("baseline", "tread", "srpo"):
            raise ConfigError(f"unknown mode {self.mode!r}")
        return self

    def to_dict(self):
        return asdict(self)


def _take(cls, d: dict, where: str, rename: dict | None = None):
    """Build dataclass ``cls`` from ``d``; unknown keys are an error (the reference ignores many
    silently)."""
    d = dict(d or {})
    for a, b in (rename or {}).items():
        if a in d:
            d[b] = d.pop(a)
    names = {f.name for f in fields(cls)}
    unknown = set(d) - names
    if unknown:
        raise ConfigError(f"unknown keys in {where}: {sorted(unknown)}")
    # YAML 1.1 reads ``1e-05`` (no dot) as a string: numeric fields take such strings as numbers
    for f in fields(cls):
        v = d.get(f.name)
        if isinstance(v, str) and str(f.type) in ("float", "int"):
            try:
                d[f.name] = float(v) if str(f.type) == "float" else int(v)
            except ValueError:
                raise ConfigError(f"{where}.{f.name}: {v!r} is not a number") from None
    return cls(**d)


def detect_model_kind(model: dict) -> str:
    """arch string -> flags -> path substrings (src/trainers/mod.rs:161-221)."""
    arch = (model.get("arch") or "").lower()
    for k in MODEL_KINDS:
        if arch == k or (arch and k in arch):
            return k
    if model.get("is_flux"):
        return "flux"
    if model.get("is_v3"):
        return "sd35"
    if model.get("is_sdxl"):
        return "sdxl"
    p = str(model.get("name_or_path", "")).lower()
    for key, kind in (("flux", "flux"), ("sd3", "sd35"), ("xl", "sdxl"), ("qwen", "qwen_image"),
                      ("ltx", "ltx"), ("wan", "wan22"), ("chroma", "chroma")):
        if key in p:
            return kind
    return "flux"


def _from_ai_toolkit(doc: dict) -> TrainCfg:
    cfg = doc["config"]
    procs = cfg.get("process") or []
    proc = next((p for p in procs if p.get("type") in ("sd_trainer", "flux_trainer")), None)
    if proc is None:
        raise ConfigError("no process of type sd_trainer / flux_trainer")
    tr = dict(proc.get("train") or {})
    net = dict(proc.get("network") or {})
    kw = net.pop("network_kwargs", None) or {}
    net["lr_if_contains"] = kw.get("lr_if_contains") or {}
    model = dict(proc.get("model") or {})
    kind = detect_model_kind(model)
    for k in ("is_flux", "is_v3", "is_sdxl"):
        model.pop(k, None)
    ema = tr.pop("ema_config", None) or {}
    tread = dict(proc.get("tread") or {})
    mask = tread.pop("mask", None) or {}
    reinj = tread.pop("reinject", None) or {}
    tloss = tread.pop("loss", None) or {}
    out = TrainCfg(
        name=cfg.get("name", "run"), training_folder=proc.get("training_folder", "output"),
        device=proc.get("device", "cuda:0"), trigger_word=proc.get("trigger_word"),
        performance_log_every=proc.get("performance_log_every") or 10,
        batch_size=tr.pop("batch_size", 1), steps=tr.pop("steps", 10),
        grad_accum_steps=tr.pop("gradient_accumulation_steps", 1),
        gradient_checkpointing=tr.pop("gradient_checkpointing", True),
        noise_scheduler=tr.pop("noise_scheduler", "flowmatch"), optimizer=tr.pop("optimizer", "adamw8bit"),
        lr=float(tr.pop("lr", 1e-4)), dtype=tr.pop("dtype", "bf16"),
        linear_timesteps=bool(tr.pop("linear_timesteps", False)),
        bypass_guidance_embedding=tr.pop("bypass_guidance_embedding", True),
        use_layer_streaming=bool(tr.pop("use_layer_streaming", False)),
        streaming_memory_limit_gb=tr.pop("streaming_memory_limit_gb", None),
        ema_decay=ema.get("ema_decay") if ema.get("use_ema") else None,
        train_mode="lora" if net.get("type", "lora") != "full" else "full",
        network=_take(NetworkCfg, net, "network"),
        save=_take(SaveCfg, proc.get("save"), "save"),
        datasets=[_take(DatasetCfg, {**d, "folder_path": str(d.get("folder_path", ""))}, "datasets[]")
                  for d in (proc.get("datasets") or [])],
        model=_take(ModelCfg, {**model, "kind": kind, "name_or_path": str(model.get("name_or_path") or "") or None},
                    "model"),
        sample=_take(SampleCfg, proc.get("sample"), "sample"),
        tread=TreadCfg(enabled=bool(tread.get("enabled", False)), mask_type=mask.get("type") or "topk_norm",
                       k=mask.get("k"), k_frac=mask.get("k_frac", 0.5), schedule=tread.get("schedule") or [],
                       reinject=reinj.get("mode") or "scatter", route_lambda=tloss.get("route_lambda") or 0.0),
        parallel=_take(ParallelCfg, proc.get("parallel"), "parallel"),
        meta=dict(doc.get("meta") or {}),
    )
    for k in ("train_unet", "train_text_encoder", "skip_first_sample", "disable_sampling"):
        tr.pop(k, None)
    if tr:
        raise ConfigError(f"unknown keys in train: {sorted(tr)}")
    out.ckpt_every = out.save.save_every
    # 8-bit Adam is switched on automatically under a small streaming budget (src/trainers/mod.rs:499-500)
    if out.streaming_memory_limit_gb is not None and out.streaming_memory_limit_gb <= 24 and \
            out.optimizer.lower() in ("adamw", "adam"):
        out.optimizer = "adamw8bit"
    return out


_FLAT_DATASET_KEYS = {"flux_manifest": "manifest", "flux_manifest_root": "manifest_root",
                      "flux_manifest_index": "manifest_index", "flux_manifest_validate": "manifest_validate",
                      "flux_manifest_shuffle": "manifest_shuffle", "flux_manifest_repeat": "manifest_repeat",
                      "sdxl_manifest": "manifest", "sdxl_manifest_root": "manifest_root"}
_FLAT_MODEL_KEYS = {"weights": "name_or_path", "flux_model_path": "name_or_path", "flux_vae_path": "vae_path",
                    "flux_t5_path": "t5_path", "flux_clip_path": "clip_l_path", "flux_variant": "variant"}
_FLAT_IGNORED = {"flux_t5_tokenizer", "flux_clip_tokenizer", "recipe"}


def _from_flat(doc: dict) -> TrainCfg:
    d = dict(doc)
    kind = str(d.pop("model_kind")).lower()
    ds, model = {}, {"kind": kind}
    for k, v in list(d.items()):
        if k in _FLAT_DATASET_KEYS:
            ds[_FLAT_DATASET_KEYS[k]] = d.pop(k)
        elif k in _FLAT_MODEL_KEYS:
            model[_FLAT_MODEL_KEYS[k]] = d.pop(k)
        elif k in _FLAT_IGNORED:
            d.pop(k)
    d.pop("bf16_params", None)
    nested = {}
    for k, cls in (("network", NetworkCfg), ("save", SaveCfg), ("sample", SampleCfg), ("tread", TreadCfg),
                   ("parallel", ParallelCfg)):
        if k in d:
            nested[k] = _take(cls, d.pop(k), k)
    if "model" in d:
        model.update(d.pop("model"))
    if "datasets" in d:
        nested["datasets"] = [_take(DatasetCfg, x, "datasets[]") for x in d.pop("datasets")]
    elif ds:
        nested["datasets"] = [_take(DatasetCfg, ds, "dataset")]
    if "optimizer" in d and d["optimizer"] is None:
        d.pop("optimizer")
    cfg = _take(TrainCfg, {**d, **nested, "model": _take(ModelCfg, model, "model")}, "config")
    return cfg


def load_config(path_or_dict) -> TrainCfg:
    """Load either schema from a YAML file (or an already parsed dict) and validate it."""
    doc = path_or_dict
    if not isinstance(doc, dict):
        doc = yaml.safe_load(Path(path_or_dict).read_text())
    if not isinstance(doc, dict):
        raise ConfigError("configuration must be a mapping")
    if "config" in doc and isinstance(doc["config"], dict) and "process" in doc["config"]:
        cfg = _from_ai_toolkit(doc)
    elif "model_kind" in doc:
        cfg = _from_flat(doc)
    elif isinstance(doc.get("job"), dict) and isinstance(doc.get("model"), dict) and "architecture" in doc["model"]:
        from .universal import UniversalConfig, UniversalConfigError
        try:
            return UniversalConfig.from_dict(doc).to_train_cfg()
        except UniversalConfigError as e:
            raise ConfigError(str(e)) from e
    else:
        raise ConfigError("not an ai-toolkit style document (config.process), a flat model_kind document or a "
                          "universal job document (job + model.architecture)")
    apply_env(cfg)
    return cfg.validate()


# ------------------------------------------------------------------------- environment namespace
ENV_VARS = {
    "ERI_B200_BACKEND": "fused | eager: kernel path for CUDA bf16 tensors",
    "ERI_B200_GEMM": "native | library: GEMM implementation inside the fused path",
    "ERI_B200_ATTN": "native | library: attention implementation inside the fused path",
    "ERI_B200_NO_BUILD": "1: never try to build the native library on import",
    "ERI_B200_FROZEN_TRANSPOSE": "1: keep transposed copies of frozen weights for input-gradient GEMMs",
    "ERI_B200_WAIT_MS": "bound of in-kernel cross-GPU waits, milliseconds",
    "ERI_B200_GEMM2": "1 | 0: two-CTA (cta_group::2) GEMM tiles for large problems",
    "ERI_B200_GATHER_PAIR": "1 | 0: gather-fused GEMMs on the two-CTA kernel",
    "ERI_B200_GATHER_LOCAL": "1 | 0: read this rank's own slab in place instead of copying it",
    "ERI_B200_ZERO3_GATHER": "sm | ce: copy CTAs inside the GEMM launch, or copy engines on a side stream",
    "ERI_B200_RANK_STREAM": "1 | 0: streaming kernel for LoRA down-projections",
    "ERI_B200_SKINNY_MIN_K": "smallest K that uses the split-K tcgen05 kernel when the streaming kernel declines",
    "ERI_B200_PDL": "1 | 0: launch the LoRA-fused GEMM as a programmatic dependent of the down-projection",
    "ERI_B200_ACCUM_INTO_GRAD": "1 | 0: accumulate adapter gradients into the arena inside the GEMM call",
    "ERI_B200_FA_POLY / ERI_B200_FA_BWD_POLY": "0 | 4 | 8: exponentials per 16 pairs evaluated as a polynomial",
    "ERI_B200_NVTX": "1: NVTX ranges per block and phase",
    "ERI_B200_PHASE_TIMING": "1: device-timed noise / forward / backward / optimizer phases in the trainer",
    "ERI_B200_NATIVE_PREFETCH": "1 | 0: native read-ahead threads in the cached-embedding loader",
    "ERI_B200_PLUGINS": "colon-separated plug-in modules loaded at start-up",
    "ATTN_Q_CHUNK / ATTN_KV_CHUNK / ATTN_REUSE / ATTN_MAX_WS_MB / ATTN_MIN_FREE_MB":
        "block sizes, shared workspace and caps of the library (blockwise) attention path",
    "SDXL_TIMING / SDXL_LOAD_TRACE / BACKWARD_DEBUG": "1: phase breakdown, load GiB/s, anomaly mode + gradient report",
    "ERID_PINNED_CHECKPOINT_CACHE_MB": "pinned staging cache for checkpoint writes, MiB",
    "AI_TOOLKIT_<SECTION>__<KEY>": "override of a universal-schema document (config/universal.py)",
    "TRAIN_LOG_CSV": "per-step CSV path (step,loss,grad_norm,sec_per_it,alloc_mb,ckpt_path)",
    "CKPT_EVERY": "checkpoint interval override",
    "EXPECT_STEP_SEC": "fail the run when a step is slower than this many seconds",
    "WORLD_SIZE / RANK / LOCAL_RANK / MASTER_ADDR / MASTER_PORT": "rendezvous",
}


def apply_env(cfg: TrainCfg):
    if os.environ.get("CKPT_EVERY"):
        cfg.ckpt_every = int(os.environ["CKPT_EVERY"])
    return cfg


# ------------------------------------------------------------------------- modelPath.yaml
@dataclass
class VaeBlock:
    kind: str
    path: str
    latent_div: int
    latent_channels: int
    latent_scale: float


def load_model_paths(path) -> dict:
    """``modelPath.yaml``: ``{models, text_encoders, policies, vae{kind, path, latent_div,
    latent_channels, latent_scale}}``; ``latent_scale`` must be explicit
    (crates/common/config/src/lib.rs:5-110)."""
    doc = yaml.safe_load(Path(path).read_text()) or {}
    out = {"models": doc.get("models") or {}, "text_encoders": doc.get("text_encoders") or {},
           "policies": doc.get("policies") or {}, "vae": None}
    if doc.get("vae"):
        v = doc["vae"]
        for k in ("kind", "path", "latent_div", "latent_channels", "latent_scale"):
            if k not in v:
                raise ConfigError(f"vae.{k} must be given explicitly")
        out["vae"] = VaeBlock(v["kind"], v["path"], int(v["latent_div"]), int(v["latent_channels"]), float(v["latent_scale"]))
    return out


def assert_precomp_vae_compat(vae: VaeBlock, latent_channels: int, latent_div: int):
    if vae.latent_channels != latent_channels or vae.latent_div != latent_div:
        raise ConfigError(f"cached latents ({latent_channels} ch, /{latent_div}) do not match VAE "
                          f"{vae.kind} ({vae.latent_channels} ch, /{vae.latent_div})")


TEMPLATES = {k: f"model_kind: {k}\nweights: \"/path/to/weights\"\nbf16_params: true\nsteps: 10\n"
                f"batch_size: 1\ngrad_accum_steps: 1\nlr: 0.0001\noptimizer: adamw\n"
             for k in ("flux", "sdxl", "sd3", "qwen_image", "wan22", "ltx", "hunyuan", "lumina", "hidream_i1", "omnigen2")}
