"""Universal job schema and its loader (search paths, formats, environment overrides)."""
import json
from pathlib import Path

import pytest

import eridiffusion_b200.config as C
from eridiffusion_b200.config.universal import ConfigLoader, UniversalConfig, UniversalConfigError

DOC = {"job": {"name": "j", "job_type": "training", "priority": "high", "tags": ["a"]},
       "model": {"architecture": "sdxl", "pretrained_model_name_or_path": "/w/sdxl.safetensors"},
       "network": {"network_type": "lora", "rank": 8, "alpha": 4.0, "target_modules": ["to_q"]},
       "training": {"num_epochs": 2, "batch_size": 4, "learning_rate": 2e-5, "gradient_accumulation_steps": 2,
                    "save_steps": 50, "output_dir": "out", "optimizer": {"type": "prodigy", "beta3": 0.5},
                    "scheduler": {"type": "cosine", "num_warmup_steps": 7}},
       "dataset": {"dataset_name_or_path": "data/m.jsonl", "resolution": 768,
                   "augmentations": [{"type": "color_jitter", "brightness": 0.1}, "random_rotation"]},
       "attention": {"impl_sel": "flash", "packed_qkv": True}, "extensions": {"x": 1}}


def test_universal_document_to_train_cfg():
    u = UniversalConfig.from_dict(json.loads(json.dumps(DOC)))
    assert u.training.optimizer["use_bias_correction"] is False and u.training.optimizer["beta3"] == 0.5
    assert u.training.scheduler == {"type": "cosine", "num_warmup_steps": 7, "num_cycles": 0.5}
    assert u.attention.impl == "flash" and u.dataset.augmentations[1] == {"type": "random_rotation"}
    cfg = u.to_train_cfg(steps_per_epoch=30)
    assert cfg.model.kind == "sdxl" and cfg.steps == 60 and cfg.batch_size == 4 and cfg.grad_accum_steps == 2
    assert cfg.optimizer == "prodigy" and cfg.lr_schedule == "cosine" and cfg.warmup_steps == 7
    assert cfg.network.linear == 8 and cfg.network.linear_alpha == 4.0 and cfg.train_mode == "lora"
    assert cfg.noise_scheduler == "ddpm" and cfg.datasets[0].manifest == "data/m.jsonl" and cfg.ckpt_every == 50
    assert cfg.meta["target_modules"] == ["to_q"] and cfg.meta["optimizer_args"]["beta3"] == 0.5
    same = C.load_config(json.loads(json.dumps(DOC)))             # the common entry point recognises the schema
    assert same.model.kind == "sdxl" and same.meta["schema"] == "universal"
    full = json.loads(json.dumps(DOC)); full.pop("network")
    assert UniversalConfig.from_dict(full).to_train_cfg().train_mode == "full"
    assert "architecture: sdxl" in u.to_yaml()


@pytest.mark.parametrize("mutate,msg", [
    (lambda d: d["job"].update(job_type="dance"), "job.job_type"),
    (lambda d: d["model"].update(architecture="vqgan"), "model.architecture"),
    (lambda d: d["training"].update(mixed_precision="fp16"), "bf16"),
    (lambda d: d["training"]["optimizer"].update(momentum=0.9), "unknown keys"),
    (lambda d: d.pop("training"), "needs a `training`"),
    (lambda d: d.update(extra=1), "unknown top-level"),
    (lambda d: d["network"].update(rank=0), "rank"),
    (lambda d: d["dataset"]["augmentations"].append({"type": "color_jitter", "zoom": 1}), "unknown keys"),
])
def test_universal_validation(mutate, msg):
    d = json.loads(json.dumps(DOC))
    mutate(d)
    with pytest.raises(UniversalConfigError, match=msg):
        UniversalConfig.from_dict(d)
    if "job" in d and "architecture" in d.get("model", {}) and d["model"]["architecture"] != "vqgan":
        with pytest.raises(C.ConfigError):
            C.load_config(d)


def test_loader_search_paths_formats_and_env(tmp_path):
    (tmp_path / "a").mkdir(); (tmp_path / "b").mkdir()
    (tmp_path / "b" / "job.json").write_text(json.dumps(DOC))
    toml = ('[job]\nname = "t"\njob_type = "inference"\n[model]\narchitecture = "flux"\n'
            '[inference]\nnum_inference_steps = 8\nscheduler = "euler_discrete"\n')
    (tmp_path / "a" / "inf.toml").write_text(toml)
    env = {"AI_TOOLKIT_TRAINING__LEARNING_RATE": "3e-4", "AI_TOOLKIT_JOB__NAME": "from_env",
           "AI_TOOLKIT_TRAINING__OPTIMIZER__TYPE": "adam8bit", "OTHER_X": "1"}
    ld = ConfigLoader(search_paths=[tmp_path / "a"], environ=env)
    with pytest.raises(FileNotFoundError):
        ld.find_config_file("job")
    ld.add_search_path(tmp_path / "b")
    assert ld.find_config_file("job") == tmp_path / "b" / "job.json"
    doc = ld.load_document("job")
    assert doc["training"]["learning_rate"] == 3e-4 and doc["job"]["name"] == "from_env"
    with pytest.raises(UniversalConfigError, match="unknown keys"):      # prodigy's beta3 is not an adam8bit key
        ld.load("job")
    inf = ConfigLoader(search_paths=[tmp_path / "a"], environ={}).load("inf.toml")
    assert inf.job.job_type == "inference" and inf.inference.num_inference_steps == 8 and inf.training is None
    with pytest.raises(UniversalConfigError):
        inf.to_train_cfg()


def test_universal_template_loads():
    cfg = C.load_config(Path(C.__file__).parent / "templates" / "universal_flux_lora.yaml")
    assert cfg.model.kind == "flux" and cfg.steps == 10 and cfg.optimizer == "adamw8bit"
    assert cfg.datasets and cfg.datasets[0].synthetic and cfg.meta["attention"]["impl"] == "flash"
