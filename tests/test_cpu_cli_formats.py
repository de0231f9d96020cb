"""Entry points (generate, cache_embeddings, probe, sdxl_10steps), adapter-file loading in all key
layouts, and the reference's secondary checkpoint layouts."""
import json
import os

import numpy as np
import pytest
import torch

from eridiffusion_b200.adapters import (AdapterConfig, adapter_state_dict, inject_adapters, load_adapters_into)
from eridiffusion_b200.io import safetensors as st
from eridiffusion_b200.models import build_model
from eridiffusion_b200.train import checkpoint_formats as CF


def _adapted_model(seed=0):
    torch.manual_seed(seed)
    m = build_model("tiny_mmdit")
    ads = inject_adapters(m, AdapterConfig(rank=8, alpha=8, dtype=torch.float32))
    for a in ads.values():
        for p in a.parameters():
            torch.nn.init.normal_(p, std=0.02)
    return m, ads


@pytest.mark.parametrize("layout", ["eri", "peft", "kohya"])
def test_load_adapters_into_reads_every_layout(layout, tmp_path):
    m, ads = _adapted_model()
    f = tmp_path / f"{layout}.safetensors"
    st.save_file(adapter_state_dict(ads, layout), f)
    m2 = build_model("tiny_mmdit")
    ads2 = load_adapters_into(m2, f)
    assert set(ads2) == set(ads)
    k = sorted(ads)[0]
    assert ads2[k].rank == 8 and torch.allclose(ads[k].lora_A, ads2[k].lora_A) and torch.allclose(ads[k].lora_B, ads2[k].lora_B)


def test_chroma_adapter_and_strict_layouts_roundtrip(tmp_path):
    m, ads = _adapted_model()
    # Chroma: positional keys + trainer_state.json
    CF.save_chroma_lora(ads, tmp_path / "chroma", 12)
    keys = st.SafeFile(tmp_path / "chroma" / "lora_step0012.safetensors").keys()
    assert "lora_param_0" in keys and st.read_metadata(tmp_path / "chroma" / "lora_step0012.safetensors")["param_count"] == str(len(keys))
    state = json.loads((tmp_path / "chroma" / "trainer_state.json").read_text())
    assert state["global_step"] == 12 and "grad_scaler" in state
    m2, ads2 = _adapted_model(seed=5)
    assert CF.load_chroma_lora(ads2, tmp_path / "chroma") == 12
    k = sorted(ads)[3]
    assert torch.allclose(ads[k].lora_B, ads2[k].lora_B, atol=1e-2)
    # adapter checkpoint: directory, symlink, metadata, keep-last
    for step in (10, 20, 30):
        CF.save_adapter_checkpoint(ads, tmp_path / "ad", step, rank=8, alpha=8.0, keep_last=2)
    names = sorted(p.name for p in (tmp_path / "ad").iterdir())
    assert names == ["checkpoint-20", "checkpoint-30", "checkpoint-latest"]
    m3, ads3 = _adapted_model(seed=7)
    meta = CF.load_adapter_checkpoint(ads3, tmp_path / "ad")
    assert meta["step"] == 30 and meta["format"] == "eridiffusion" and meta["rank"] == 8
    assert torch.allclose(ads[k].lora_A, ads3[k].lora_A, atol=1e-2)
    # strict: exact key set or an error
    tensors = {"a.w": torch.ones(2, 2), "b.w": torch.zeros(3)}
    CF.save_strict(tensors, tmp_path / "s.safetensors", lora_rank=8, lora_alpha=8.0, step=4)
    sd, md = CF.load_strict(tmp_path / "s.safetensors", ["a.w", "b.w"])
    assert md["step"] == "4" and torch.equal(sd["a.w"], tensors["a.w"])
    with pytest.raises(KeyError, match="missing"):
        CF.load_strict(tmp_path / "s.safetensors", ["a.w", "b.w", "c.w"])
    with pytest.raises(KeyError, match="unexpected"):
        CF.load_strict(tmp_path / "s.safetensors", ["a.w"])
    # EMA with a storage dtype
    CF.save_ema({"x": torch.full((4,), 0.3)}, tmp_path / "ema.safetensors", dtype=torch.bfloat16, decay=0.999, step=4)
    back = CF.load_ema(tmp_path / "ema.safetensors")
    assert back["x"].dtype == torch.float32 and abs(float(back["x"][0]) - 0.3) < 2e-3


def test_generate_probe_and_cache_clis(tmp_path, capsys):
    from eridiffusion_b200.cli import cache_embeddings, generate, probe
    out = tmp_path / "o"
    assert generate.main(["--family", "tiny_mmdit", "--steps", "2", "--height", "256", "--width", "256",
                          "--out", str(out), "--device", "cpu"]) == 0
    lat = st.load_file(str(out) + ".latents.safetensors")["latent"]
    assert lat.shape == (1, 16, 32, 32) and torch.isfinite(lat).all()
    assert probe.main(["--full", "tiny_mmdit"]) == 0
    assert "adapter sites" in capsys.readouterr().out
    img = tmp_path / "img"
    img.mkdir()
    for i in range(2):
        np.save(img / f"a{i}.npy", (np.random.rand(96, 80, 3) * 255).astype(np.uint8))
        (img / f"a{i}.txt").write_text(f"a photo number {i}")
    ov = ["vae_flux:base=32", "vae_flux:mult=(1,2)", "vae_flux:groups=8", "t5_encoder:hidden=64", "t5_encoder:layers=1",
          "t5_encoder:heads=4", "t5_encoder:head_dim=16", "t5_encoder:ff=128", "clip_l:hidden=64", "clip_l:layers=1",
          "clip_l:heads=4", "clip_l:proj_dim=32"]
    args = ["--family", "flux", "--images", str(img), "--out", str(tmp_path / "cache"), "--size", "64", "--random-init",
            "--device", "cpu", "--t5-tokens", "16"]
    for o in ov:
        args += ["--override", o]
    assert cache_embeddings.main(args) == 0
    rows = (tmp_path / "cache" / "manifest.tsv").read_text().strip().split("\n")
    assert rows[0].split("\t") == ["latents_path", "t5_path", "clip_path", "caption"] and len(rows) == 3
    from eridiffusion_b200.data import load_cached_tensor, parse_manifest
    z = load_cached_tensor(tmp_path / "cache" / "a0.latent.safetensors")
    assert z.shape == (16, 32, 32)            # 64 px / 2 (two-level tiny VAE)
    entries = parse_manifest(tmp_path / "cache" / "manifest.tsv")
    assert len(entries) == 2 and entries[1].caption == "a photo number 1"


def test_sdxl_10steps_env_interface(monkeypatch, capsys):
    from eridiffusion_b200.cli import sdxl_10steps
    for k, v in dict(STEPS="2", HEIGHT="64", WIDTH="64", HIDDEN="128", CTX_DIM="64", DEVICE="cpu", BLOCK_INDEX="0").items():
        monkeypatch.setenv(k, v)
    assert sdxl_10steps.main() == 0
    out = capsys.readouterr().out
    assert "avg step time" in out and "step 2/2" in out
