"""The reference's flat ``TrainCfg`` surface (crates/training/src/model_registry.rs:125-482): every
field, the nested groups with their precedence, the ``mode`` struct, and the ten templates of its
training crate (kept under tests/fixtures/reference_templates). Then one test per job switch showing
that the key changes what runs — or is refused by name."""
from pathlib import Path

import numpy as np
import pytest
import torch

import eridiffusion_b200.config as C
from eridiffusion_b200.train.factory import build_job

FIXTURES = sorted((Path(__file__).parent / "fixtures" / "reference_templates").glob("train_*.yaml"))


def test_all_ten_reference_templates_load():
    assert len(FIXTURES) == 10
    kinds = {}
    for p in FIXTURES:
        cfg = C.load_config(p)
        kinds[p.stem[len("train_"):]] = cfg.model.kind
        assert cfg.steps == 10 and cfg.batch_size == 1 and cfg.lr == 1e-4 and cfg.optimizer == "adamw" and cfg.bf16_params
    assert kinds["qwen_image_v1"] == "qwen_image" and kinds["sd3"] == "sd3" and kinds["sdxl"] == "sdxl"
    sdxl = C.load_config(next(p for p in FIXTURES if p.stem == "train_sdxl"))
    assert sdxl.model.name_or_path.endswith("sdxl_unet.safetensors") and sdxl.model.clip_g_path.endswith("clip_g.safetensors")
    assert sdxl.model.clip_l_tokenizer.endswith("clip_l_tokenizer.json") and sdxl.model.vae_path.endswith("sdxl_vae.safetensors")
    sd3 = C.load_config(next(p for p in FIXTURES if p.stem == "train_sd3"))
    assert sd3.model.t5_path.endswith("t5.safetensors") and sd3.model.t5_tokenizer.endswith("t5_tokenizer.json")


def test_every_flat_field_is_accepted():
    doc = {
        "model_kind": "flux", "recipe": None, "weights": "/w", "bf16_params": True, "steps": 20, "batch_size": 2,
        "grad_accum_steps": 2, "lr": 2e-4, "seed": 7, "ckpt_every": 5, "optimizer": "adamw8bit",
        "offload_pinned_threshold_mb": 64,
        "flux_model_path": "/flux.safetensors", "flux_vae_path": "/vae", "flux_t5_path": "/t5", "flux_clip_path": "/clip",
        "flux_t5_tokenizer": "/t5tok", "flux_clip_tokenizer": "/cliptok", "flux_variant": "dev",
        "flux_manifest": "/m.tsv", "flux_manifest_root": "/root", "flux_manifest_index": "/idx",
        "flux_manifest_validate": True, "flux_manifest_shuffle": False, "flux_manifest_repeat": 3,
        "sdxl_manifest": "/x.tsv", "sdxl_manifest_root": "/xr", "sdxl_manifest_index": "/xi",
        "sdxl_manifest_validate": False, "sdxl_manifest_shuffle": True, "sdxl_manifest_repeat": 2,
        "sd35_manifest": "/s.tsv", "sd35_manifest_root": "/sr", "sd35_manifest_index": "/si",
        "sd35_manifest_validate": False, "sd35_manifest_shuffle": True, "sd35_manifest_repeat": 2,
        "lora_rank": 32, "lora_alpha": 16.0, "lora_zero_init": False, "data_root": "/data", "prefetch": 4,
        "schedule_name": "sigma_eps", "schedule_steps": 100, "sigma_min": 0.02, "sigma_max": 0.9, "clip_grad_norm": 0.5,
        "sdxl_unet_path": "/unet", "sdxl_vae_path": "/xvae", "sdxl_clip_l_path": "/xl", "sdxl_clip_g_path": "/xg",
        "sdxl_clip_l_tokenizer": "/xlt", "sdxl_clip_g_tokenizer": "/xgt",
        "sd35_model_path": "/sd35", "sd35_vae_path": "/svae", "sd35_clip_l_path": "/sl", "sd35_clip_g_path": "/sg",
        "sd35_t5_path": "/st5", "sd35_clip_l_tokenizer": "/slt", "sd35_clip_g_tokenizer": "/sgt", "sd35_t5_tokenizer": "/st5t",
        "mode": {"baseline": True, "tread": False, "srpo": False},
    }
    cfg = C.load_config(doc)
    # the family's own paths win over the generic ones and over the other families'
    assert cfg.model.name_or_path == "/flux.safetensors" and cfg.model.vae_path == "/vae" and cfg.model.t5_path == "/t5"
    assert cfg.model.clip_l_path == "/clip" and cfg.model.t5_tokenizer == "/t5tok" and cfg.model.clip_g_path == "/xg"
    ds = cfg.datasets[0]
    assert (ds.manifest, ds.manifest_root, ds.manifest_index, ds.manifest_validate, ds.manifest_shuffle,
            ds.manifest_repeat) == ("/m.tsv", "/root", "/idx", True, False, 3)
    assert cfg.meta["other_manifests"]["manifest"] in ("/x.tsv", "/s.tsv")
    assert cfg.network.linear == 32 and cfg.network.linear_alpha == 16.0 and cfg.network.zero_init is False
    assert cfg.max_grad_norm == 0.5 and cfg.prefetch == 4 and cfg.schedule_steps == 100
    assert (cfg.sigma_min, cfg.sigma_max, cfg.schedule_name) == (0.02, 0.9, "sigma_eps") and cfg.mode == "baseline"
    sdxl = C.load_config({**doc, "model_kind": "sdxl"})
    assert sdxl.model.name_or_path == "/unet" and sdxl.datasets[0].manifest == "/x.tsv" and sdxl.model.clip_l_tokenizer == "/xlt"
    sd3 = C.load_config({**doc, "model_kind": "sd3"})
    assert sd3.model.name_or_path == "/sd35" and sd3.datasets[0].manifest == "/s.tsv" and sd3.model.t5_path == "/st5"


def test_nested_groups_hydrate_with_flat_precedence():
    doc = {"model_kind": "flux", "lr": 3e-4,
           "paths": {"flux_weights": "/w", "vae": "/v", "t5": "/t5", "clip": "/c", "t5_tokenizer": "/tt", "clip_tokenizer": "/ct"},
           "data": {"root": "/d", "batch_size": 4, "prefetch": 3, "manifest": "/m.jsonl", "manifest_shuffle": False,
                    "manifest_sdxl": "/x.tsv"},
           "lora": {"rank": 8},
           "train": {"steps": 50, "grad_accum_steps": 2, "lr": 5e-4, "ckpt_every": 10, "bf16": True, "clip_grad_norm": 2.0},
           "schedule": {"name": "cosine", "steps": 40}}
    cfg = C.load_config(doc)
    assert cfg.model.name_or_path == "/w" and cfg.model.clip_l_tokenizer == "/ct" and cfg.batch_size == 4 and cfg.prefetch == 3
    assert cfg.datasets[0].manifest == "/m.jsonl" and cfg.datasets[0].manifest_shuffle is False
    assert cfg.datasets[0].manifest_root == "/d"
    assert cfg.network.linear == 8 and cfg.network.linear_alpha == 8.0 and cfg.network.zero_init is True
    assert cfg.steps == 50 and cfg.grad_accum_steps == 2 and cfg.ckpt_every == 10 and cfg.max_grad_norm == 2.0
    assert cfg.lr == 3e-4                      # the flat value wins over train.lr
    assert cfg.schedule_name == "cosine" and cfg.schedule_steps == 40
    # the struct names of the reference are accepted as group names too
    same = C.load_config({"model_kind": "flux", "lora_nested": {"rank": 8, "alpha": 4.0, "zero_init": False}})
    assert same.network.linear == 8 and same.network.linear_alpha == 4.0 and same.network.zero_init is False
    with pytest.raises(C.ConfigError):
        C.load_config({"model_kind": "flux", "paths": {"unet": "/x"}})


def test_mode_struct_needs_exactly_one_true():
    assert C.load_config({"model_kind": "flux", "mode": {"baseline": False, "tread": True}}).mode == "tread"
    assert C.load_config({"model_kind": "flux", "mode": {"tread": True}}).tread.enabled
    assert C.load_config({"model_kind": "flux", "mode": "tread"}).mode == "tread"
    assert C.load_config({"model_kind": "flux"}).mode == "baseline"
    for bad in ({"baseline": True, "tread": True}, {"baseline": False}, {"baseline": True, "other": True}):
        with pytest.raises(C.ConfigError):
            C.load_config({"model_kind": "flux", "mode": bad})


# ---------------------------------------------------------------------------------- job switches
TINY = {"model_kind": "tiny_mmdit", "device": "cpu", "steps": 2, "seed": 0, "optimizer": "adamw8bit",
        "datasets": [{"synthetic": True, "resolution": [256]}]}


def _run(doc, steps=2, tmp=None):
    cfg = C.load_config({**TINY, **doc, **({"training_folder": str(tmp)} if tmp else {})})
    trainer, batches, info = build_job(cfg, device="cpu")
    losses = [float(trainer.train_step(next(batches))) for _ in range(steps)]
    return trainer, info, losses


def test_gradient_checkpointing_recomputes_blocks_and_keeps_the_numbers():
    base, info0, l0 = _run({})
    ck, info1, l1 = _run({"gradient_checkpointing": True})
    assert info0["runner"] is None and info1["runner"]["policy"] == "recompute"
    assert l0 == pytest.approx(l1, rel=1e-5)                      # same function, activations recomputed
    calls = {"n": 0}
    blk = ck.model.single_blocks[0]
    inner = blk.forward
    blk.forward = lambda *a, **k: (calls.__setitem__("n", calls["n"] + 1), inner(*a, **k))[1]
    ck.train_step({k: v for k, v in next(iter([_batch()])).items()})
    assert calls["n"] == 2                                        # once in forward, once again in backward


def _batch():
    from eridiffusion_b200.data import synthetic_batch
    return synthetic_batch("tiny_mmdit", 1, "cpu", torch.float32, seed=0, height=256, width=256)


def test_tread_mode_routes_tokens_through_the_single_stack():
    plain, _, l0 = _run({})
    routed, info, l1 = _run({"mode": {"baseline": False, "tread": True}, "tread": {"k_frac": 0.5, "schedule": [{"out": 0, "in": 2}]}})
    assert info["runner"]["tread"] and routed.model.runner.tread.kept_frac        # routing really happened
    kept = list(routed.model.runner.tread.kept_frac.values())[0]
    n_txt, n_img = 64, 256
    assert kept == pytest.approx((n_txt + n_img // 2) / (n_txt + n_img))            # all text + half of the image tokens
    assert l0[0] != l1[0]                                                           # a different function is trained
    with pytest.raises(C.ConfigError, match="tread"):
        build_job(C.load_config({**TINY, "model_kind": "sdxl", "mode": "tread"}), device="cpu")


def test_layer_streaming_runs_blocks_through_the_swap_window():
    base, _, l0 = _run({})
    st, info, l1 = _run({"train": None} if False else {"use_layer_streaming": True, "streaming_memory_limit_gb": 1})
    assert info["runner"]["streaming"]
    mgr = st.model.runner.streamer
    n_blocks = len(st.model.block_list())
    assert mgr.cfg.persistent == (0, n_blocks - 1) and mgr.frozen_only
    # every block goes through the window in forward and again in backward, each step
    assert mgr.stats["prefetch_hits"] + mgr.stats["loads"] >= 2 * 2 * n_blocks
    assert l0 == pytest.approx(l1, rel=1e-5)
    with pytest.raises(C.ConfigError, match="use_layer_streaming"):
        build_job(C.load_config({**TINY, "use_layer_streaming": True, "train_mode": "full"}), device="cpu")


def test_double_block_lr_ramp_moves_the_multiplier():
    tr, _, _ = _run({"network": {"ramp_double_blocks": True, "ramp_target_lr": 4e-4, "ramp_warmup_steps": 4,
                                 "ramp_type": "linear", "lr_if_contains": {"single_blocks": 0.5}}}, steps=0)
    assert tr.lr_rules(0)["double_blocks"] == pytest.approx(1.0) and tr.lr_rules(2)["double_blocks"] == pytest.approx(2.5)
    assert tr.lr_rules(4)["double_blocks"] == pytest.approx(4.0) and tr.lr_rules(9)["double_blocks"] == pytest.approx(4.0)
    assert tr.lr_rules(2)["single_blocks"] == 0.5
    names = tr.param_names
    dbl = next(i for i, n in enumerate(names) if "double_blocks" in n)
    blk = tr.arena.offsets[dbl] // 256
    before = float(tr.optimizer.lr_scale[blk])
    for _ in range(3):
        tr.train_step(_batch())
    after = float(tr.optimizer.lr_scale[blk])
    assert before == pytest.approx(1.0) and after == pytest.approx(2.5)             # multiplier of step 2 is in place
    cos = _run({"network": {"ramp_double_blocks": True, "ramp_target_lr": 4e-4, "ramp_warmup_steps": 4, "ramp_type": "cosine"}}, steps=0)[0]
    assert cos.lr_rules(2)["double_blocks"] == pytest.approx(2.5) and cos.lr_rules(1)["double_blocks"] < 1.75
    with pytest.raises(C.ConfigError, match="ramp"):
        build_job(C.load_config({**TINY, "network": {"ramp_double_blocks": True}}), device="cpu")


def test_sigma_eps_schedule_switches_the_objective():
    tr, info, _ = _run({"schedule": {"name": "sigma_eps", "sigma_min": 0.05, "sigma_max": 0.8}})
    assert info["objective"] == "sigma_eps"
    t = torch.tensor([0.0, 0.5, 1.0])
    coef = tr.objective.coefficients(t)
    r = 0.8 / 0.05
    want = torch.tensor([0.05, 0.05 * r ** -0.5, 0.05 / r]).clamp(1e-3, 1.0)
    assert torch.allclose(coef[1], want) and torch.equal(coef[0], torch.ones(3))     # x_t = x0 + sigma eps
    assert torch.equal(coef[2], torch.ones(3)) and torch.equal(coef[3], torch.zeros(3))   # target = eps
    with pytest.raises(C.ConfigError, match="sigma"):
        build_job(C.load_config({**TINY, "sigma_min": 0.1}), device="cpu")
    with pytest.raises(C.ConfigError, match="schedule_name"):
        build_job(C.load_config({**TINY, "schedule_name": "karras7"}), device="cpu")


def test_lora_zero_init_and_schedule_steps_reach_the_trainer():
    z, _, _ = _run({"lora_rank": 4}, steps=0)
    nz, _, _ = _run({"lora_rank": 4, "lora_zero_init": False}, steps=0)
    up = lambda tr: next(iter(tr.adapters.values())).lora_B
    assert float(up(z).abs().max()) == 0.0 and float(up(nz).abs().max()) > 0.0
    assert up(z).shape[1] == 4
    tr, _, _ = _run({"schedule": {"name": "cosine", "steps": 40}}, steps=0)
    assert tr.schedule.total == 40 and tr.schedule.kind == "cosine"


def test_folder_dataset_is_cached_then_trained_on(tmp_path):
    PIL = pytest.importorskip("PIL.Image")
    rng = np.random.default_rng(0)
    folder = tmp_path / "pets"
    folder.mkdir()
    for i, cap in enumerate(["a [trigger] dog", "a cat", "third"]):
        PIL.fromarray(rng.integers(0, 255, size=(40, 48, 3), dtype=np.uint8)).save(folder / f"im{i}.png")
        (folder / f"im{i}.txt").write_text(cap)
    enc = {"vae_flux": {"base": 32, "latent_channels": 16},
           "t5_encoder": {"vocab_size": 512, "hidden": 128, "layers": 1, "heads": 2, "head_dim": 64, "ff": 256},
           "clip_l": {"vocab_size": 512, "hidden": 64, "layers": 1, "heads": 2, "proj_dim": 64, "eos_token_id": 511}}
    doc = {"name": "job", "trigger_word": "sks", "data_root": str(folder),
           "datasets": [{"folder_path": str(folder), "resolution": [64], "random_init_encoders": True,
                         "encoder_overrides": enc, "max_text_tokens": 16}]}
    trainer, info, losses = _run(doc, steps=2, tmp=tmp_path / "out")
    assert info["data"]["source"] == "folder" and info["data"]["cache"]["latents_encoded"] == 3
    assert (tmp_path / "out" / "job" / "manifest.jsonl").exists() and all(np.isfinite(losses))
    # second start: everything comes from the cache
    _, info2, _ = _run(doc, steps=1, tmp=tmp_path / "out")
    assert info2["data"]["cache"] == {"samples": 3, "latents_encoded": 0, "texts_encoded": 0}
    # a folder without encoders, manifest or `synthetic` is refused, not replaced by noise
    with pytest.raises(C.ConfigError, match="vae_path"):
        build_job(C.load_config({**TINY, "datasets": [{"folder_path": str(folder)}]}), device="cpu")


def test_keys_that_cannot_be_honoured_are_refused_by_name():
    for doc, word in (({"network": {"conv": 8}}, "network.conv"),
                      ({"datasets": [{"synthetic": True}, {"synthetic": True}]}, "datasets"),
                      ({"mode": {"baseline": False, "srpo": True}}, "srpo"),
                      ({"recipe": ["warp_drive"]}, "recipe"),
                      ({"train_mode": "full", "model": {"quantize": True}}, "quantize")):
        with pytest.raises(C.ConfigError, match=word):
            build_job(C.load_config({**TINY, **doc}), device="cpu")
