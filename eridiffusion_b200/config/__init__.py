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
templates crates/training/config/templates/train_*.yaml). EVERY field of that struct is accepted:
``model_kind`` (``flux sdxl sd3 qwen_image_v1 wan22 hidream_i1 omnigen2 ltx hunyuan lumina``),
``recipe, weights, bf16_params, steps, batch_size, grad_accum_steps, lr, seed, ckpt_every, optimizer,
offload_pinned_threshold_mb``, the ``flux_* / sdxl_* / sd35_*`` model, tokenizer and manifest paths,
``lora_rank, lora_alpha, lora_zero_init, data_root, prefetch, schedule_name, schedule_steps,
sigma_min, sigma_max, clip_grad_norm``, the nested groups ``paths / data / lora / train / schedule``
(also under their struct names ``paths_nested`` ...; hydrated into the flat fields with the
reference's precedence: an explicit flat value wins, model_registry.rs:351-482) and the ``mode``
struct ``{baseline, tread, srpo}`` of which exactly one must be true (:327-347, :483-492; a plain
string is accepted too).

Validation follows crates/training/src/eridiffusion_config.rs:203-369 (batch > 0, steps > 0,
lr in [1e-7, 1e-2], bf16 only, device ``cuda:N``); unknown keys raise instead of being ignored.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field, fields, asdict
from pathlib import Path

import yaml

MODEL_KINDS = ("flux", "sdxl", "sd3", "sd35", "sd35_medium", "qwen_image", "wan22", "ltx", "hunyuan", "lumina",
               "hidream_i1", "hidream", "omnigen2", "chroma", "klein", "zimage", "krea", "qwen_edit_image",
               "tiny_mmdit", "sd15")
# spellings of the reference's ``ModelKind`` enum that differ from this package's registry names
MODEL_KIND_ALIASES = {"qwen_image_v1": "qwen_image", "qwenimagev1": "qwen_image", "s_d_x_l": "sdxl", "s_d3": "sd3",
                      "hi_dream_i1": "hidream_i1"}


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
    zero_init: bool = True              # up-projection starts at zero (flat schema: lora_zero_init)
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
    random_init_encoders: bool = False          # smoke runs: cache a folder with randomly initialised encoders
    encoder_overrides: dict = field(default_factory=dict)   # {encoder kind: constructor overrides}
    max_text_tokens: int | None = None          # text length when a folder is cached (default 512 / 77)


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
    clip_g_path: str | None = None
    t5_path: str | None = None
    t5_tokenizer: str | None = None
    clip_l_tokenizer: str | None = None
    clip_g_tokenizer: str | None = None
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
    bf16_params: bool = True
    recipe: list | None = None          # optional stage list for the pipeline orchestrator
    schedule_name: str = ""             # "" | flow names | "sigma_eps" / "eps_sigma" / "bounded_sigma" (phase-4 eps objective)
    schedule_steps: int = 0             # > 0: length of the LR schedule when it differs from ``steps``
    sigma_min: float | None = None
    sigma_max: float | None = None
    prefetch: int | None = None         # loader read-ahead depth (batches)
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
        if self.sigma_min is not None and self.sigma_min <= 0:
            raise ConfigError("sigma_min must be > 0")
        if self.sigma_min is not None and self.sigma_max is not None and self.sigma_max < self.sigma_min:
            raise ConfigError("sigma_max must be >= sigma_min")
        if self.prefetch is not None and self.prefetch < 0:
            raise ConfigError("prefetch must be >= 0")
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


# flat key -> ModelCfg field, per model family (the reference keeps one set of path fields per family)
_FLAT_MODEL_KEYS = {
    "weights": "name_or_path",
    "flux_model_path": "name_or_path", "flux_vae_path": "vae_path", "flux_t5_path": "t5_path",
    "flux_clip_path": "clip_l_path", "flux_t5_tokenizer": "t5_tokenizer", "flux_clip_tokenizer": "clip_l_tokenizer",
    "flux_variant": "variant",
    "sdxl_unet_path": "name_or_path", "sdxl_vae_path": "vae_path", "sdxl_clip_l_path": "clip_l_path",
    "sdxl_clip_g_path": "clip_g_path", "sdxl_clip_l_tokenizer": "clip_l_tokenizer",
    "sdxl_clip_g_tokenizer": "clip_g_tokenizer",
    "sd35_model_path": "name_or_path", "sd35_vae_path": "vae_path", "sd35_clip_l_path": "clip_l_path",
    "sd35_clip_g_path": "clip_g_path", "sd35_t5_path": "t5_path", "sd35_clip_l_tokenizer": "clip_l_tokenizer",
    "sd35_clip_g_tokenizer": "clip_g_tokenizer", "sd35_t5_tokenizer": "t5_tokenizer",
}
_MANIFEST_FIELDS = ("", "_root", "_index", "_validate", "_shuffle", "_repeat")
_MANIFEST_FAMILY = {"sdxl": "sdxl", "sd15": "sdxl", "sd3": "sd35", "sd35": "sd35", "sd35_medium": "sd35"}
# nested group -> {group key: flat key}; ``data`` is expanded below because of its three manifest sets
_NESTED = {
    "paths": {"flux_weights": "flux_model_path", "vae": "flux_vae_path", "t5": "flux_t5_path", "clip": "flux_clip_path",
              "t5_tokenizer": "flux_t5_tokenizer", "clip_tokenizer": "flux_clip_tokenizer"},
    "data": {"root": "data_root", "batch_size": "batch_size", "prefetch": "prefetch",
             **{f"manifest{f}": f"flux_manifest{f}" for f in _MANIFEST_FIELDS},
             **{f"manifest_sdxl{f}": f"sdxl_manifest{f}" for f in _MANIFEST_FIELDS},
             **{f"manifest_sd35{f}": f"sd35_manifest{f}" for f in _MANIFEST_FIELDS}},
    "lora": {"rank": "lora_rank", "alpha": "lora_alpha", "zero_init": "lora_zero_init"},
    "train": {"steps": "steps", "grad_accum_steps": "grad_accum_steps", "lr": "lr", "ckpt_every": "ckpt_every",
              "bf16": "bf16_params", "clip_grad_norm": "clip_grad_norm"},
    "schedule": {"name": "schedule_name", "steps": "schedule_steps", "sigma_min": "sigma_min", "sigma_max": "sigma_max"},
}
_SIGMA_EPS_NAMES = ("sigma_eps", "eps_sigma", "bounded_sigma", "phase4_eps")


def _hydrate_nested(d: dict) -> dict:
    """Fold the nested groups into the flat keys with the reference's precedence: a flat key that is
    present wins; zero / empty group values count as "not given" (model_registry.rs:351-482)."""
    d = dict(d)
    for group, mapping in _NESTED.items():
        for name in (group, f"{group}_nested"):
            if name not in d:
                continue
            g = d.pop(name) or {}
            if not isinstance(g, dict):
                raise ConfigError(f"{name} must be a mapping")
            unknown = set(g) - set(mapping)
            if unknown:
                raise ConfigError(f"unknown keys in {name}: {sorted(unknown)}")
            for k, flat in mapping.items():
                v = g.get(k)
                if v is None or v == "" or (isinstance(v, (int, float)) and not isinstance(v, bool) and v == 0):
                    continue
                d.setdefault(flat, v)
            if group == "lora" and "rank" in g:
                d.setdefault("lora_alpha", float(g["rank"]))       # alpha defaults to the rank
                d.setdefault("lora_zero_init", True)
    return d


def _mode_name(mode) -> str:
    """``mode`` is a struct of three booleans in the reference (exactly one true); a plain string names
    the mode directly."""
    if mode is None:
        return "baseline"
    if isinstance(mode, str):
        return mode
    if isinstance(mode, dict):
        unknown = set(mode) - {"baseline", "tread", "srpo"}
        if unknown:
            raise ConfigError(f"unknown keys in mode: {sorted(unknown)}")
        flags = {"baseline": bool(mode.get("baseline", not (mode.get("tread") or mode.get("srpo")))),
                 "tread": bool(mode.get("tread", False)), "srpo": bool(mode.get("srpo", False))}
        on = [k for k, v in flags.items() if v]
        if len(on) != 1:
            raise ConfigError("config.mode must set exactly one of baseline|tread|srpo to true")
        return on[0]
    raise ConfigError("mode must be a string or a {baseline, tread, srpo} mapping")


def _from_flat(doc: dict) -> TrainCfg:
    d = _hydrate_nested(doc)
    kind = str(d.pop("model_kind")).lower()
    kind = MODEL_KIND_ALIASES.get(kind, kind)
    model = {"kind": kind}
    # model / encoder / tokenizer paths: the family's own keys win over the generic ``weights``
    own_prefix = {"sdxl": "sdxl_", "sd15": "sdxl_", "sd3": "sd35_", "sd35": "sd35_", "sd35_medium": "sd35_"}.get(kind, "flux_")
    for k in list(d):
        if k in _FLAT_MODEL_KEYS:
            v = d.pop(k)
            if v in (None, ""):
                continue
            fld = _FLAT_MODEL_KEYS[k]
            if k.startswith(own_prefix) or fld not in model:
                model[fld] = v
    # manifests: the set that belongs to the model family feeds the dataset; the others are kept in meta
    fam = _MANIFEST_FAMILY.get(kind, "flux")
    ds, other = {}, {}
    for f in ("flux", "sdxl", "sd35"):
        for suf in _MANIFEST_FIELDS:
            k = f"{f}_manifest{suf}"
            if k in d:
                v = d.pop(k)
                if v is None:
                    continue
                (ds if f == fam else other)["manifest" + suf] = v
    data_root = d.pop("data_root", None)
    lora_rank, lora_alpha = d.pop("lora_rank", None), d.pop("lora_alpha", None)
    lora_zero = d.pop("lora_zero_init", None)
    clip = d.pop("clip_grad_norm", None)
    if clip is not None:
        d.setdefault("max_grad_norm", float(clip))
    d["mode"] = _mode_name(d.get("mode"))
    if "schedule_name" in d and d["schedule_name"] is None:
        d.pop("schedule_name")
    nested = {}
    for k, cls in (("network", NetworkCfg), ("save", SaveCfg), ("sample", SampleCfg), ("tread", TreadCfg),
                   ("parallel", ParallelCfg)):
        if k in d:
            nested[k] = _take(cls, d.pop(k), k)
    net = nested.get("network") or NetworkCfg()
    if lora_rank is not None:
        net.linear = int(lora_rank)
        net.linear_alpha = float(lora_alpha if lora_alpha is not None else lora_rank)
    elif lora_alpha is not None:
        net.linear_alpha = float(lora_alpha)
    if lora_zero is not None:
        net.zero_init = bool(lora_zero)
    nested["network"] = net
    if "model" in d:
        model.update(d.pop("model"))
    if "datasets" in d:
        nested["datasets"] = [_take(DatasetCfg, x, "datasets[]") for x in d.pop("datasets")]
    elif ds or data_root:
        if data_root and not ds.get("manifest"):
            ds["folder_path"] = str(data_root)           # a folder of images + captions, cached on the fly
        elif data_root:
            ds.setdefault("manifest_root", str(data_root))
        nested["datasets"] = [_take(DatasetCfg, ds, "dataset")]
    for k in ("optimizer", "ckpt_every", "offload_pinned_threshold_mb", "recipe", "sigma_min", "sigma_max", "prefetch"):
        if k in d and d[k] is None:
            d.pop(k)
    cfg = _take(TrainCfg, {**d, **nested, "model": _take(ModelCfg, model, "model")}, "config")
    if other:
        cfg.meta["other_manifests"] = other
    if cfg.mode == "tread":
        cfg.tread.enabled = True
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
    "FLUX_FORCE_DENSE_ATTENTION": "1: dense library attention instead of the flash kernels",
    "STREAMING_SDPA_CHUNK_MAX / ATTN_CHUNK_SIZE / ATTN_MAX_WORKSPACE_MB / ATTN_CHUNK_REUSE":
        "blockwise library attention: key-block size, workspace cap, shared workspace",
    "STREAM_ATTENTION_SELFTEST": "1: compare blockwise with dense attention once at start-up",
    "STREAM_ATTENTION_CAUSAL_TEXT": "refused (no causal text mask)",
    "ERID_FUSE": "1 fused kernels (default) | 0 unfused PyTorch statements",
    "STRICT_BF16": "1 | panic: strict-bf16 counters around every training step",
    "GRADIENT_CHECKPOINT_POLICY": "recompute | cpu_offload | adaptive (+ GRADIENT_CHECKPOINT_MEMORY_THRESHOLD_MB, "
                                  "GRADIENT_CHECKPOINT_PREFER_RECOMPUTE)",
    "DISABLE_LAYER_STREAMING": "1: ignore use_layer_streaming",
    "TREAD_ENABLED / TREAD_MASK_TYPE / TREAD_K / TREAD_K_FRAC / TREAD_SCHEDULE / TREAD_REINJECT_MODE / TREAD_LAMBDA":
        "override the tread block (schedule as out:in,out:in)",
    "ERI_B200_WGRAD": "native | library: weight-gradient GEMMs on tcgen05 or torch",
    "ERI_B200_SCATTER_PAIR": "1 | 0: peer-scatter epilogue on the two-CTA kernel",
    "ERI_B200_GLU_FUSED": "1 | 0: GEGLU / SwiGLU in the up-projection GEMM epilogue",
    "ERI_B200_DEBUG_BOUNDS": "1: build and load the bounds-checked debug variant of the kernel library",
    "ERI_B200_FA_PAIR": "1: attention forward for head size 128 on CTA pairs (measured slower; default 0)",
    "ERI_B200_ATTN_HEAD_PAD": "1 | 0: head sizes other than 64 / 128 (below 128) zero-padded onto the native attention kernels",
    "ERI_B200_PAIR_MIN_TILES": "GEMMs with at most this many 256 x 256 tiles use the one-CTA kernel's 128-column tiles (default 36)",
    "ERI_B200_NORM_SKIP": "1: the gradient of the residual branch around a norm is added inside the norm's backward kernel (no measurable gain; default 0)",
    "ERI_B200_NORM_SMEM": "1 | 0: norm + modulate rows resident in shared memory (32 warps per SM) or in registers",
    "ERI_B200_ADAMW8_PAIR": "1 | 0: 8-bit AdamW on packed fp32 pairs (default) or the element-wise kernel",
    "ERI_B200_MLP_FUSE": "1: dual-stream MLP pairs apply the activation derivative in the down-projection's input-gradient epilogue (measured slower; default 0)",
    "ERI_B200_ACT_EPILOGUE": "1: activation + stored pre-activation in the GEMM epilogue during training (default 0: the GEMM writes the pre-activation, a separate pass applies the activation)",
    "ERI_B200_SS_ACT_EPILOGUE": "1: single-stream blocks apply GELU in the first linear's epilogue (default 0: the GEMM writes the pre-activation, a row pass applies GELU)",
    "ERI_B200_SS_ACT_BWD_EPILOGUE": "1 | 0: single-stream blocks apply the GELU derivative in the second linear's input-gradient epilogue (default 1)",
    "ERI_B200_GEMM_EPI_WARPS": "8 | 4: epilogue warps of a plain two-CTA GEMM launch (gather / scatter launches always use 4)",
    "ERI_B200_GEMM_GROUP": "1 | 0: image and text projection of a dual-stream block in one grouped launch of the two-CTA GEMM",
    "ERI_B200_GATHER_JOIN": "1: copy clusters of a gather-fused GEMM take tiles after their last slab (default 0)",
    "ERI_B200_ZERO3_PREFETCH": "1 | 0: ZeRO-3 next-layer prefetch (copy engines pull layer i + 1's shards while GEMM i runs)",
    "ERI_B200_ZERO3_FUSED_RS": "1 | 0: ZeRO-3 weight-gradient reduce-scatter in the dW GEMM's epilogue",
    "ERI_B200_ZERO3_MOD": "native | nccl: collectives of the ZeRO-3 conditioning-vector linears",
    "TRAIN_LOG_CSV": "per-step CSV path (step,loss,grad_norm,sec_per_it,alloc_mb,ckpt_path)",
    "CKPT_EVERY": "checkpoint interval override",
    "EXPECT_STEP_SEC": "fail the run when a step is slower than this many seconds",
    "WORLD_SIZE / RANK / LOCAL_RANK / MASTER_ADDR / MASTER_PORT": "rendezvous",
}


def apply_env(cfg: TrainCfg):
    if os.environ.get("CKPT_EVERY"):
        cfg.ckpt_every = int(os.environ["CKPT_EVERY"])
    # the reference's behaviour switches (attention mode, fusion, checkpoint policy, TREAD_*, ...)
    from ..utils.env_flags import ReferenceEnvError, apply_reference_env
    try:
        applied = apply_reference_env(cfg, print_fn=lambda *_: None)
    except ReferenceEnvError as e:
        raise ConfigError(str(e)) from e
    if applied:
        cfg.meta["reference_env"] = applied
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


_TEMPLATE_TAIL = "bf16_params: true\nsteps: 10\nbatch_size: 1\ngrad_accum_steps: 1\nlr: 0.0001\noptimizer: adamw\n"
# the ten templates of crates/training/config/templates/, field for field
TEMPLATES = {k: f"model_kind: {k}\nweights: \"/path/to/weights\"\n" + _TEMPLATE_TAIL
             for k in ("flux", "qwen_image_v1", "wan22", "ltx", "hunyuan", "lumina", "hidream_i1", "omnigen2")}
TEMPLATES["sdxl"] = "model_kind: sdxl\n" + _TEMPLATE_TAIL + "".join(
    f"sdxl_{k}: \"/path/to/{v}\"\n" for k, v in (
        ("unet_path", "sdxl_unet.safetensors"), ("vae_path", "sdxl_vae.safetensors"), ("clip_l_path", "clip_l.safetensors"),
        ("clip_g_path", "clip_g.safetensors"), ("clip_l_tokenizer", "clip_l_tokenizer.json"),
        ("clip_g_tokenizer", "clip_g_tokenizer.json")))
TEMPLATES["sd3"] = "model_kind: sd3\n" + _TEMPLATE_TAIL + "".join(
    f"sd35_{k}: \"/path/to/{v}\"\n" for k, v in (
        ("model_path", "sd35_model.safetensors"), ("vae_path", "sd35_vae.safetensors"), ("clip_l_path", "clip_l.safetensors"),
        ("clip_g_path", "clip_g.safetensors"), ("t5_path", "t5.safetensors"), ("clip_l_tokenizer", "clip_l_tokenizer.json"),
        ("clip_g_tokenizer", "clip_g_tokenizer.json"), ("t5_tokenizer", "t5_tokenizer.json")))
