"""Every shipped configuration template loads, validates and names a buildable model family."""
from pathlib import Path

import pytest

import eridiffusion_b200.config as C
from eridiffusion_b200.train.factory import _KIND_TO_MODEL

TEMPLATES = sorted((Path(C.__file__).parent / "templates").glob("train_*.yaml"))


def test_templates_exist_for_every_family():
    names = {p.stem[len("train_"):] for p in TEMPLATES}
    assert {"flux", "sdxl", "sd3", "qwen_image", "wan22", "ltx", "hunyuan", "lumina", "hidream_i1", "omnigen2"} <= names


@pytest.mark.parametrize("path", TEMPLATES, ids=lambda p: p.stem)
def test_template_loads(path):
    cfg = C.load_config(path)
    assert cfg.model.kind in _KIND_TO_MODEL and cfg.steps == 10 and cfg.batch_size == 1 and isinstance(cfg.lr, float)
    if cfg.model.kind == "sdxl":
        assert cfg.parallel.zero_stage == 2 and cfg.train_mode == "full"
    if cfg.model.kind == "qwen_image":
        assert cfg.parallel.zero_stage == 3 and cfg.lr == 1e-5


def test_numeric_strings_and_bad_values():
    cfg = C.load_config({"model_kind": "flux", "lr": "1e-05", "steps": "7"})
    assert cfg.lr == 1e-5 and cfg.steps == 7
    with pytest.raises(C.ConfigError):
        C.load_config({"model_kind": "flux", "lr": "fast"})
    assert "ERI_B200_PDL" in C.ENV_VARS and "ERI_B200_ZERO3_GATHER" in C.ENV_VARS


def test_nested_template_loads():
    cfg = C.load_config(Path(C.__file__).parent / "templates" / "flux_lora_nested.yaml")
    assert cfg.model.kind == "flux" and cfg.network.linear == 16 and cfg.parallel.fused_comm == "on"
    assert cfg.sample.sample_every == 250 and cfg.network.lr_if_contains == {"single_blocks": 0.5}
