"""The "universal" job document and its loader.

Third configuration schema of the reference, besides the ai-toolkit and the flat one:
``UniversalConfig{job, model, network, training, dataset, inference, extensions, attention}`` with
tagged optimizer / scheduler / augmentation variants, and ``ConfigLoader`` with search paths, YAML /
JSON / TOML by file extension and environment overrides under the ``AI_TOOLKIT`` prefix
(crates/core/src/config.rs:25-155 loader, :157-400 schema).

``UniversalConfig.to_train_cfg()`` maps a training job onto the ``TrainCfg`` the job factory
consumes, so all three schemas drive the same trainer; ``load_config`` recognises the document by
its ``job`` + ``model.architecture`` keys.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field, fields
from pathlib import Path

import yaml

JOB_TYPES = ("training", "inference", "conversion", "evaluation", "custom")
JOB_PRIORITIES = ("low", "normal", "high", "critical")
INIT_STRATEGIES = ("normal", "xavier", "kaiming", "zero", "pissa")
MIXED_PRECISION = ("no", "fp16", "bf16", "fp8")
INFERENCE_SCHEDULERS = ("ddpm", "ddim", "dpm_solver_multistep", "dpm_solver_singlestep", "euler_discrete",
                        "euler_ancestral_discrete", "heun_discrete", "lcm", "flow_match_euler")
OPTIMIZER_DEFAULTS = {
    "adam": {"betas": (0.9, 0.999), "eps": 1e-8, "weight_decay": 0.01},
    "adam8bit": {"betas": (0.9, 0.999), "eps": 1e-8},
    "prodigy": {"betas": (0.9, 0.999), "beta3": 0.0, "weight_decay": 0.0, "eps": 1e-8, "decouple": True,
                "use_bias_correction": False, "safeguard_warmup": False},
    "adafactor": {"scale_parameter": True, "relative_step": True, "warmup_init": False, "weight_decay": 0.0},
}
SCHEDULER_DEFAULTS = {
    "constant": {}, "linear": {"num_warmup_steps": 0}, "cosine": {"num_warmup_steps": 0, "num_cycles": 0.5},
    "cosine_with_restarts": {"num_warmup_steps": 0, "num_cycles": 1}, "polynomial": {"num_warmup_steps": 0, "power": 1.0},
}
AUGMENTATION_KINDS = {"color_jitter": ("brightness", "contrast", "saturation", "hue"), "random_rotation": ("degrees",),
                      "random_crop": ("size",)}
# architecture names the reference's enum uses -> model kinds of this framework
ARCHITECTURES = {"flux": "flux", "flux_dev": "flux", "flux_schnell": "flux", "sdxl": "sdxl", "sd15": "sd15", "sd1_5": "sd15",
                 "sd3": "sd35", "sd35": "sd35", "sd3_5": "sd35", "chroma": "chroma", "qwen_image": "qwen_image",
                 "ltx": "ltx", "ltx_video": "ltx", "wan22": "wan22", "wan2_2": "wan22", "klein": "klein", "zimage": "zimage",
                 "hunyuan": "hunyuan", "lumina": "lumina", "hidream": "hidream", "omnigen2": "omnigen2", "krea": "krea"}


class UniversalConfigError(ValueError):
    pass


def _choice(value, allowed, what):
    v = str(value).lower()
    if v not in allowed:
        raise UniversalConfigError(f"{what}: {value!r} is not one of {list(allowed)}")
    return v


def _build(cls, d, where):
    if d is None:
        return None
    if not isinstance(d, dict):
        raise UniversalConfigError(f"{where} must be a mapping")
    known = {f.name for f in fields(cls)}
    extra = set(d) - known
    if extra:
        raise UniversalConfigError(f"{where}: unknown keys {sorted(extra)}")
    return cls(**d)


def _tagged(d, table, where):
    """{"type": name, ...fields} -> (name, fields merged over the variant's defaults)."""
    if isinstance(d, str):
        d = {"type": d}
    d = dict(d or {"type": next(iter(table))})
    name = _choice(d.pop("type", None), table, f"{where}.type")
    extra = set(d) - set(table[name])
    if extra:
        raise UniversalConfigError(f"{where} ({name}): unknown keys {sorted(extra)}")
    return {"type": name, **table[name], **d}


@dataclass
class JobConfig:
    name: str = "job"
    job_type: str = "training"
    description: str | None = None
    priority: str = "normal"
    tags: list = field(default_factory=list)

    def __post_init__(self):
        self.job_type = _choice(self.job_type, JOB_TYPES, "job.job_type")
        self.priority = _choice(self.priority, JOB_PRIORITIES, "job.priority")


@dataclass
class UModelConfig:
    architecture: str = "flux"
    pretrained_model_name_or_path: str = ""
    revision: str | None = None
    variant: str | None = None
    torch_dtype: str | None = None
    use_safetensors: bool = True

    def __post_init__(self):
        self.architecture = _choice(self.architecture, ARCHITECTURES, "model.architecture")


@dataclass
class UNetworkConfig:
    network_type: str = "lora"
    rank: int = 16
    alpha: float = 16.0
    dropout: float = 0.0
    target_modules: list = field(default_factory=list)
    use_bias: bool = False
    init_strategy: str = "normal"

    def __post_init__(self):
        self.network_type = str(self.network_type).lower()
        self.init_strategy = _choice(self.init_strategy, INIT_STRATEGIES, "network.init_strategy")


@dataclass
class UTrainingConfig:
    num_epochs: int = 1
    batch_size: int = 1
    learning_rate: float = 1e-4
    gradient_accumulation_steps: int = 1
    max_grad_norm: float = 1.0
    warmup_steps: int = 0
    save_steps: int = 0
    logging_steps: int = 10
    validation_steps: int | None = None
    checkpointing_steps: int | None = None
    resume_from_checkpoint: str | None = None
    output_dir: str = "output"
    mixed_precision: str = "bf16"
    optimizer: dict = field(default_factory=lambda: {"type": "adam8bit"})
    scheduler: dict = field(default_factory=lambda: {"type": "constant"})
    max_steps: int | None = None             # not in the reference: bounds a run without a dataset length

    def __post_init__(self):
        self.mixed_precision = _choice(self.mixed_precision, MIXED_PRECISION, "training.mixed_precision")
        self.optimizer = _tagged(self.optimizer, OPTIMIZER_DEFAULTS, "training.optimizer")
        self.scheduler = _tagged(self.scheduler, SCHEDULER_DEFAULTS, "training.scheduler")


@dataclass
class UDatasetConfig:
    dataset_name_or_path: str = ""
    caption_column: str = "text"
    image_column: str = "image"
    conditioning_image_column: str | None = None
    resolution: int = 1024
    random_flip: bool = False
    center_crop: bool = False
    augmentations: list = field(default_factory=list)
    cache_dir: str | None = None

    def __post_init__(self):
        self.augmentations = [self._aug({"type": a} if isinstance(a, str) else a) for a in self.augmentations]

    @staticmethod
    def _aug(a):
        name = _choice(a.get("type"), AUGMENTATION_KINDS, "dataset.augmentations[].type")
        extra = set(a) - {"type", *AUGMENTATION_KINDS[name]}
        if extra:
            raise UniversalConfigError(f"augmentation {name}: unknown keys {sorted(extra)}")
        return dict(a, type=name)


@dataclass
class UInferenceConfig:
    num_inference_steps: int = 20
    guidance_scale: float = 3.5
    negative_prompt: str | None = None
    num_images_per_prompt: int = 1
    seed: int | None = None
    scheduler: str = "flow_match_euler"

    def __post_init__(self):
        self.scheduler = _choice(self.scheduler, INFERENCE_SCHEDULERS, "inference.scheduler")


@dataclass
class AttentionRuntimeConfig:
    impl: str | None = None                  # "flash" (native kernels) | "sdpa" (library)
    packed_qkv: bool | None = None


@dataclass
class UniversalConfig:
    job: JobConfig = field(default_factory=JobConfig)
    model: UModelConfig = field(default_factory=UModelConfig)
    network: UNetworkConfig | None = None
    training: UTrainingConfig | None = None
    dataset: UDatasetConfig | None = None
    inference: UInferenceConfig | None = None
    extensions: dict = field(default_factory=dict)
    attention: AttentionRuntimeConfig | None = None

    @classmethod
    def from_dict(cls, doc: dict) -> "UniversalConfig":
        extra = set(doc) - {f.name for f in fields(cls)}
        if extra:
            raise UniversalConfigError(f"unknown top-level keys {sorted(extra)}")
        if "job" not in doc or "model" not in doc:
            raise UniversalConfigError("a universal document needs `job` and `model`")
        att = dict(doc.get("attention") or {})
        if "impl_sel" in att:
            att["impl"] = att.pop("impl_sel")
        return cls(job=_build(JobConfig, doc["job"], "job"), model=_build(UModelConfig, doc["model"], "model"),
                   network=_build(UNetworkConfig, doc.get("network"), "network"),
                   training=_build(UTrainingConfig, doc.get("training"), "training"),
                   dataset=_build(UDatasetConfig, doc.get("dataset"), "dataset"),
                   inference=_build(UInferenceConfig, doc.get("inference"), "inference"),
                   extensions=dict(doc.get("extensions") or {}),
                   attention=_build(AttentionRuntimeConfig, att, "attention") if att else None).validate()

    def validate(self):
        if self.job.job_type == "training" and self.training is None:
            raise UniversalConfigError("a training job needs a `training` section")
        if self.job.job_type == "inference" and self.inference is None:
            raise UniversalConfigError("an inference job needs an `inference` section")
        if self.network is not None and self.network.rank <= 0:
            raise UniversalConfigError("network.rank must be > 0")
        if self.training is not None and self.training.mixed_precision in ("fp16", "fp8"):
            raise UniversalConfigError("training computes in bf16; mixed_precision must be `bf16` (or `no` on CPU)")
        return self

    def to_dict(self):
        return asdict(self)

    def to_yaml(self) -> str:
        return yaml.safe_dump(json.loads(json.dumps(self.to_dict())), sort_keys=False)

    # ------------------------------------------------------------------ bridge to the job factory
    def to_train_cfg(self, steps_per_epoch: int | None = None):
        """The ``TrainCfg`` equivalent of a training job. Steps = ``max_steps`` or ``num_epochs *
        steps_per_epoch`` (the caller knows the dataset length), else ``num_epochs``."""
        from . import DatasetCfg, ModelCfg, NetworkCfg, SaveCfg, TrainCfg, apply_env
        if self.training is None:
            raise UniversalConfigError("no `training` section to convert")
        t, m, n = self.training, self.model, self.network
        steps = t.max_steps or (t.num_epochs * steps_per_epoch if steps_per_epoch else t.num_epochs)
        opt = {"adam": "adamw", "adam8bit": "adamw8bit"}.get(t.optimizer["type"], t.optimizer["type"])
        sched = {"cosine_with_restarts": "cosine_with_restarts"}.get(t.scheduler["type"], t.scheduler["type"])
        ds = []
        if self.dataset is not None and self.dataset.dataset_name_or_path:
            p = self.dataset.dataset_name_or_path
            is_manifest = p.endswith((".tsv", ".jsonl"))
            ds = [DatasetCfg(folder_path="" if is_manifest else p, manifest=p if is_manifest else None,
                             resolution=[self.dataset.resolution])]
        elif self.dataset is not None:
            ds = [DatasetCfg(synthetic=True, resolution=[self.dataset.resolution])]
        cfg = TrainCfg(
            name=self.job.name, training_folder=t.output_dir, train_mode="lora" if n is not None else "full",
            batch_size=t.batch_size, steps=steps, grad_accum_steps=t.gradient_accumulation_steps, lr=t.learning_rate,
            optimizer=opt, weight_decay=t.optimizer.get("weight_decay", 0.01), lr_schedule=sched,
            warmup_steps=t.scheduler.get("num_warmup_steps", t.warmup_steps) or t.warmup_steps,
            max_grad_norm=t.max_grad_norm, ckpt_every=t.checkpointing_steps or t.save_steps,
            performance_log_every=t.logging_steps,
            noise_scheduler="ddpm" if ARCHITECTURES[m.architecture] in ("sdxl", "sd15") else "flowmatch",
            model=ModelCfg(kind=ARCHITECTURES[m.architecture], name_or_path=m.pretrained_model_name_or_path or None,
                           variant=m.variant),
            network=NetworkCfg(type=n.network_type, linear=n.rank, linear_alpha=n.alpha, dropout=n.dropout)
            if n is not None else NetworkCfg(),
            save=SaveCfg(save_every=t.save_steps), datasets=ds,
            meta={"schema": "universal", "job": asdict(self.job), "extensions": self.extensions,
                  "resume_from_checkpoint": t.resume_from_checkpoint,
                  "attention": asdict(self.attention) if self.attention else None,
                  "optimizer_args": {k: v for k, v in t.optimizer.items() if k != "type"},
                  "target_modules": list(n.target_modules) if n is not None else []})
        apply_env(cfg)
        return cfg.validate()


def is_universal_document(doc) -> bool:
    return isinstance(doc, dict) and isinstance(doc.get("job"), dict) and isinstance(doc.get("model"), dict) \
        and "architecture" in doc["model"]


class ConfigLoader:
    """Finds a configuration file in a list of directories (``.``, ``config``, the user's
    configuration directory), parses it by extension (``.yaml`` / ``.yml`` / ``.json`` / ``.toml``)
    and applies environment overrides: ``AI_TOOLKIT_TRAINING__LEARNING_RATE=2e-4`` sets
    ``training.learning_rate`` (double underscore = one level down, values parsed as YAML scalars)."""

    def __init__(self, search_paths=None, environment_prefix: str = "AI_TOOLKIT", environ=None):
        home_cfg = Path(os.environ.get("XDG_CONFIG_HOME", Path.home() / ".config")) / "eridiffusion"
        self.search_paths = [Path(p) for p in (search_paths if search_paths is not None else (".", "config", home_cfg))]
        self.environment_prefix = environment_prefix
        self.environ = os.environ if environ is None else environ

    def add_search_path(self, path):
        self.search_paths.append(Path(path))

    def find_config_file(self, filename) -> Path:
        p = Path(filename)
        if p.is_absolute() and p.exists():
            return p
        for base in self.search_paths:
            for cand in (base / p, *(base / (str(p) + ext) for ext in (".yaml", ".yml", ".json", ".toml"))):
                if cand.is_file():
                    return cand
        raise FileNotFoundError(f"configuration {filename!r} not found in {[str(s) for s in self.search_paths]}")

    @staticmethod
    def parse(path: Path) -> dict:
        text = Path(path).read_text()
        ext = Path(path).suffix.lower()
        if ext == ".json":
            return json.loads(text)
        if ext == ".toml":
            import tomllib
            return tomllib.loads(text)
        if ext in (".yaml", ".yml"):
            return yaml.safe_load(text)
        raise UniversalConfigError(f"unsupported configuration format {ext!r}")

    def env_overrides(self) -> dict:
        out = {}
        pre = self.environment_prefix + "_"
        for k, v in self.environ.items():
            if not k.startswith(pre):
                continue
            path = [s.lower() for s in k[len(pre):].split("__") if s]
            if not path:
                continue
            node = out
            for s in path[:-1]:
                node = node.setdefault(s, {})
            node[path[-1]] = self._scalar(v)
        return out

    @staticmethod
    def _scalar(text: str):
        """``3e-4`` is a string to a YAML 1.1 parser (no dot): try the numeric readings first."""
        for cast in (int, float):
            try:
                return cast(text)
            except ValueError:
                pass
        return yaml.safe_load(text)

    @staticmethod
    def _merge(base, over):
        for k, v in over.items():
            if isinstance(v, dict) and isinstance(base.get(k), dict):
                ConfigLoader._merge(base[k], v)
            else:
                base[k] = v
        return base

    def load_document(self, filename) -> dict:
        doc = self.parse(self.find_config_file(filename))
        if not isinstance(doc, dict):
            raise UniversalConfigError("configuration must be a mapping")
        return self._merge(doc, self.env_overrides())

    def load(self, filename) -> UniversalConfig:
        return UniversalConfig.from_dict(self.load_document(filename))
