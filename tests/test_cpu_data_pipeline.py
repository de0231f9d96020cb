"""Two-level cache, bucketed datasets and the VAE preprocessing command, on CPU."""
import json

import numpy as np
import pytest
import torch

from eridiffusion_b200.data.buckets import (BucketDataConfig, BucketedImageDataset, BucketedVideoDataset,
                                            VideoDataConfig, nearest_bucket)
from eridiffusion_b200.data.cache import CacheManager
from eridiffusion_b200.data import vae_preprocess as vp

PIL = pytest.importorskip("PIL.Image")


def _mk_images(root, specs):
    root.mkdir(parents=True, exist_ok=True)
    rng = np.random.default_rng(0)
    for name, (w, h), cap in specs:
        arr = rng.integers(0, 255, size=(h, w, 3), dtype=np.uint8)
        PIL.fromarray(arr).save(root / name)
        if cap is not None:
            (root / name).with_suffix(".txt").write_text(cap)


def test_cache_levels_and_eviction(tmp_path):
    cm = CacheManager(tmp_path / "c", memory_limit_mb=1, pin=False)
    a = torch.randn(128, 1024).to(torch.bfloat16)          # 256 KiB
    for i in range(6):
        cm.put(f"/data/img{i}.png", a + i)
    assert cm.memory_bytes() <= 1 << 20 and len(cm) == 4 and cm.stats.evictions == 2
    # oldest entries fell out of memory but are on disk
    e = cm.get("/data/img0.png")
    assert e is not None and torch.equal(e.tensor, a + 0) and e.metadata.dtype == "BF16"
    assert cm.stats.disk_hits == 1 and cm.stats.memory_misses == 1
    e = cm.get("/data/img0.png")
    assert cm.stats.memory_hits == 1
    assert cm.get("/data/none.png") is None and cm.stats.disk_misses == 1
    # a fresh manager over the same directory finds everything on disk
    cm2 = CacheManager(tmp_path / "c", memory_limit_mb=8, pin=False)
    assert torch.equal(cm2.get("/data/img5.png").tensor, a + 5)
    calls = []
    e = cm2.get_or_compute("/data/new.png", lambda p: (calls.append(p), torch.ones(4))[1])
    assert calls == ["/data/new.png"] and e.tensor.sum() == 4
    with pytest.raises(ValueError):
        cm.put("/x", torch.zeros(2, dtype=torch.float64))


def test_cache_detects_shape_mismatch(tmp_path):
    cm = CacheManager(tmp_path, memory_limit_mb=1, pin=False)
    cm.put("k", torch.zeros(2, 3))
    cm.clear_memory()
    meta = tmp_path / (cm.cache_key("k") + ".meta")
    md = json.loads(meta.read_text())
    md["shape"] = [3, 2]
    meta.write_text(json.dumps(md))
    assert cm.get("k") is None


def test_bucketed_image_dataset(tmp_path):
    _mk_images(tmp_path / "ds" / "sub", [("a.png", (64, 64), "a [trigger] cat"), ("b.png", (128, 64), None),
                                         ("c.jpg", (60, 66), "x"), ("d.png", (130, 64), "wide")])
    cfg = BucketDataConfig(str(tmp_path / "ds"), buckets=[(32, 32), (32, 64)], caption_trigger_word="sks",
                           batch_size=2)
    ds = BucketedImageDataset(cfg)
    assert ds.num_files() == 4
    assert ds.buckets_summary() == [((32, 32), 2), ((32, 64), 2)]
    batches = list(ds)
    assert len(batches) == ds.batches_per_epoch() == 2
    for b in batches:
        assert b["images"].shape == (2, b["h"], b["w"], 3) and b["images"].dtype == torch.bfloat16
        assert float(b["images"].float().abs().max()) <= 1.0
    prompts = sorted(p for b in batches for p in b["prompts"])
    assert prompts == ["a photo", "a sks cat", "wide", "x"]
    assert nearest_bucket(100, 50, [(32, 32), (32, 64)]) == 1
    with pytest.raises(FileNotFoundError):
        BucketedImageDataset(BucketDataConfig(str(tmp_path / "nope")))


def test_bucketed_video_dataset(tmp_path):
    _mk_images(tmp_path / "v", [("a.png", (96, 48), None), ("b.png", (20, 20), "clip")])
    ds = BucketedVideoDataset(VideoDataConfig(str(tmp_path / "v"), buckets=[(32, 64), (32, 32)], time_buckets=[9, 17],
                                              downscale_only=True))
    assert ds.buckets_summary() == [(32, 32, 1), (32, 64, 1)]
    b = ds.next_batch(0)
    assert b["t"] == 9 and b["images"].shape == (1, 32, 64, 3) and b["prompts"] == ["a short video"]
    assert b["latent_shape"] == (1, 9, 4, 8)
    with pytest.raises(ValueError, match="upscaling forbidden"):
        ds.next_batch(1)


def test_vae_preprocess_command(tmp_path, capsys):
    _mk_images(tmp_path / "in", [(f"{i}.png", (40 + 8 * i, 48), None) for i in range(5)])
    rc = vp.main(["--input", str(tmp_path / "in"), "--out", str(tmp_path / "out"), "--vae-kind", "flux", "--cpu",
                  "--size", "32", "--microbatch", "2", "--shard-size", "3", "--base-channels", "32"])
    assert rc == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["samples"] == 5 and rep["shards"] == 2 and rep["latent_shape"] == [16, 4, 4]
    rows = [json.loads(l) for l in (tmp_path / "out" / "manifest.jsonl").read_text().splitlines()]
    assert len(rows) == 5 and rows[0]["shard"] == "latents_00000.safetensors" and rows[4]["shard"] == "latents_00001.safetensors"
    assert rows[1]["orig_hw"] == [48, 48] and rows[3]["crop_xy"] == [8, 0]
    from safetensors.torch import load_file
    sh = load_file(str(tmp_path / "out" / "latents_00001.safetensors"))
    assert sorted(sh) == ["sample_00000003", "sample_00000004"] and sh["sample_00000003"].shape == (16, 4, 4)


def test_vae_spec_from_model_paths(tmp_path):
    y = tmp_path / "mp.yaml"
    y.write_text("models:\n  flux_dev:\n    arch: flux\n    vae: {kind: flux, path: /w/ae.safetensors, latent_div: 8, "
                 "latent_channels: 16, latent_scale: 0.3611}\n  bad:\n    vae: {kind: nope, path: x, latent_div: 8, "
                 "latent_channels: 4, latent_scale: 1.0}\n")
    s = vp.load_vae_spec_from_model_paths(y, "flux_dev")
    assert (s.kind, s.latent_channels, s.latent_div) == ("flux", 16, 8) and abs(s.latent_shift - 0.1159) < 1e-9
    with pytest.raises(ValueError):
        vp.load_vae_spec_from_model_paths(y, "bad")
    with pytest.raises(KeyError):
        vp.load_vae_spec_from_model_paths(y, "missing")
