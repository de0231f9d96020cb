"""Prompt-hash text cache, dataset cache layout and the sequential pre-encoding pipeline."""
import json

import numpy as np
import pytest
import torch

from eridiffusion_b200.data import load_cached_tensor, parse_manifest
from eridiffusion_b200.data.precache import DatasetCache, TextEmbeddingCache, precache_folder
from eridiffusion_b200.models.vae import AutoencoderKL, VaeConfig

PIL = pytest.importorskip("PIL.Image")


def test_text_embedding_cache(tmp_path):
    c = TextEmbeddingCache(tmp_path / "t", "t5-xxl")
    assert c.get("a cat") is None and c.misses == 1
    calls = []

    def enc(prompt):
        calls.append(prompt)
        return torch.ones(1, 6, 4) * len(prompt), torch.arange(3.0), torch.tensor([1, 1, 1, 0, 0, 0])

    h, pooled = c.get_or_encode("a cat", enc)
    assert h.shape == (3, 4) and pooled.tolist() == [0.0, 1.0, 2.0]           # padding stripped by the mask
    h2, _ = c.get_or_encode("a cat", enc, dtype=torch.bfloat16)
    assert calls == ["a cat"] and h2.dtype == torch.bfloat16 and c.hits == 1
    assert TextEmbeddingCache(tmp_path / "t", "clip").key("a cat") != c.key("a cat")
    assert c.has("a cat") and not c.has("a dog")


def test_precache_folder_pipeline(tmp_path):
    rng = np.random.default_rng(0)
    ds = tmp_path / "ds"
    ds.mkdir()
    for i, cap in enumerate(["a [trigger] dog", None, "third"]):
        PIL.fromarray(rng.integers(0, 255, size=(40, 48, 3), dtype=np.uint8)).save(ds / f"im{i}.png")
        if cap is not None:
            (ds / f"im{i}.txt").write_text(cap)
    made = []

    def make_vae():
        made.append("vae")
        return AutoencoderKL(VaeConfig(latent_channels=4, base=32), dtype=torch.float32, device="cpu").eval()

    def make_te():
        made.append("te")
        return lambda prompt: (torch.full((1, 5, 8), float(len(prompt))), torch.zeros(4))

    mpath, rep = precache_folder(ds, tmp_path / "out", "pets", make_vae, make_te, size=32, microbatch=2, trigger_word="sks")
    assert rep == {"samples": 3, "latents_encoded": 3, "texts_encoded": 3} and made == ["vae", "te"]
    rows = [json.loads(l) for l in mpath.read_text().splitlines()]
    assert [r["caption"] for r in rows] == ["a sks dog", "", "third"]
    assert rows[0]["latents_path"].startswith("cache/vae/pets/") and rows[0]["t5_path"].startswith("cache/text/pets/")
    lat = load_cached_tensor(tmp_path / "out" / rows[0]["latents_path"], torch.float32)
    txt = load_cached_tensor(tmp_path / "out" / rows[0]["t5_path"], torch.float32)
    assert lat.shape == (4, 4, 4) and txt.shape == (5, 8) and float(txt[0, 0]) == len("a sks dog")
    entries = parse_manifest(mpath, root_dir=tmp_path / "out")
    assert len(entries) == 3
    # second run: everything is cached, no model is built
    _, rep2 = precache_folder(ds, tmp_path / "out", "pets", make_vae, make_te, size=32)
    assert rep2["latents_encoded"] == 0 and rep2["texts_encoded"] == 0 and made == ["vae", "te"]
    dc = DatasetCache(tmp_path / "out", "pets")
    assert dc.latent_path(ds / "im0.png").exists() and dc.latent_path(ds / "im0.png") != dc.latent_path(tmp_path / "im0.png")
