"""Per-architecture training pipelines, the staged orchestrator, SD1.5 wiring (CPU)."""
import pytest
import torch

from eridiffusion_b200.models import build_model
from eridiffusion_b200.train.pipelines import (Ctx, Orchestrator, PipelineAdapter, PipelineConfig, PipelineFactory,
                                               PromptEmbeds, SD3Pipeline, SDXLPipeline, StageName)
from tests.test_cpu_training import batch


def test_prompt_embeds_concat_and_masks():
    a = PromptEmbeds.with_pooled(torch.zeros(1, 3, 4), torch.zeros(1, 2))
    b = PromptEmbeds(torch.ones(2, 3, 4), torch.ones(2, 2)).with_mask(torch.tensor([[1, 1, 0], [1, 0, 0]]))
    c = a.concat(b)
    assert c.encoder_hidden_states.shape == (3, 3, 4) and c.pooled_projections.shape == (3, 2)
    assert c.attention_mask.tolist() == [[1, 1, 1], [1, 1, 0], [1, 0, 0]]
    with pytest.raises(ValueError):
        a.concat(PromptEmbeds(torch.ones(1, 3, 4)))
    e = SD3Pipeline.combine_text(torch.ones(1, 77, 768), torch.ones(1, 77, 1280), torch.ones(1, 20, 4096),
                                 torch.ones(1, 768), torch.ones(1, 1280))
    assert e.encoder_hidden_states.shape == (1, 97, 4096) and e.pooled_projections.shape == (1, 2048)
    assert e.encoder_hidden_states[0, 0, 2047] == 1 and e.encoder_hidden_states[0, 0, 2048] == 0


def test_flux_pipeline_matches_fused_noise_and_trains():
    from eridiffusion_b200.ops import functional as F
    pipe = PipelineFactory.create("tiny_mmdit", PipelineConfig(dynamic_shift=True))
    x0 = torch.randn(2, 16, 32, 32)
    eps = torch.randn(2, 16, 32, 32)
    t = torch.tensor([0.25, 0.8])
    noisy, target = pipe.add_noise(x0, eps, t)
    xt_ref, tgt_ref = F.noise_mix(x0, pipe.objective.coefficients(t), seed=0, eps=eps, patch=2)
    assert torch.allclose(pipe.pack(noisy), xt_ref, atol=1e-6) and torch.allclose(pipe.pack(target), tgt_ref, atol=1e-6)
    # dynamic shift moves timesteps towards the noisy end, more for longer sequences
    g = lambda: torch.Generator().manual_seed(0)
    t0 = pipe.sample_timesteps(64, g(), seq_len=None)
    t_small, t_big = pipe.sample_timesteps(64, g(), seq_len=256), pipe.sample_timesteps(64, g(), seq_len=4096)
    assert (t_small >= t0).all() and (t_big >= t_small).all() and (t_big > t0).any()
    torch.manual_seed(0)
    model = build_model("tiny_mmdit")
    loss = pipe.training_loss(model, batch(), torch.Generator().manual_seed(1))
    loss.backward()
    assert torch.isfinite(loss) and any(p.grad is not None for p in model.parameters())
    assert pipe.compute_prior_loss(model, None) is None
    assert torch.isfinite(pipe.compute_prior_loss(model, batch(3), torch.Generator().manual_seed(2)))
    masked = {**batch(), "loss_mask": torch.zeros(2, 1, 32, 32)}
    assert float(pipe.training_loss(model, masked, torch.Generator().manual_seed(1)).detach()) == 0.0
    with pytest.raises(ValueError):
        PipelineFactory.create("nope")
    assert {"flux", "sdxl", "sd3", "sd15", "ltx"} <= set(PipelineFactory.known())


def _tiny_unet(kind):
    torch.manual_seed(0)
    kw = dict(dtype=torch.float32, groups=8, context_dim=24)
    if kind == "sdxl":
        return build_model("sdxl", block_channels=(32, 64), transformer_depth=(0, 1), head_dim=16, pooled_dim=20,
                           addition_time_embed_dim=8, **kw)
    return build_model("sd15", block_channels=(32, 64, 64, 64), num_heads=2, **kw)


@pytest.mark.parametrize("kind", ["sdxl", "sd15"])
def test_unet_pipelines(kind):
    pipe = PipelineFactory.create(kind, PipelineConfig(prediction_type="v", min_snr_gamma=5.0, noise_offset=0.05,
                                                       input_perturbation=0.1, loss="huber"))
    model = _tiny_unet(kind)
    b = {"latents": torch.randn(2, 4, 16, 16), "txt": torch.randn(2, 7, 24)}
    if kind == "sdxl":
        b["pooled"] = torch.randn(2, 20)
        assert SDXLPipeline.time_ids((1024, 768), (0, 8), (1024, 768), 2).tolist()[0] == [1024, 768, 0, 8, 1024, 768]
    loss = pipe.training_loss(model, b, torch.Generator().manual_seed(0))
    loss.backward()
    assert torch.isfinite(loss)
    cfg = pipe.get_scheduler_config()
    assert cfg["prediction"] == "v" and cfg["num_steps"] == 1000
    t = torch.tensor([10, 900])
    noisy, target = pipe.add_noise(b["latents"], torch.zeros_like(b["latents"]), t)
    ab = pipe.objective.alphas_cumprod[t].view(2, 1, 1, 1)
    assert torch.allclose(noisy, ab.sqrt() * b["latents"], atol=1e-6)
    assert torch.allclose(target, -(1 - ab).sqrt() * b["latents"], atol=1e-6)      # v-target with zero noise


def test_sd15_full_size_and_job_wiring():
    full = build_model("sd15", device="meta")
    n = sum(p.numel() for p in full.parameters())
    assert abs(n - 859_520_964) < 1000 and full.num_transformer_blocks() == 16
    from eridiffusion_b200.config import TrainCfg, load_config
    from pathlib import Path
    import eridiffusion_b200.config as C
    cfg = load_config(Path(C.__file__).parent / "templates" / "train_sd15.yaml")
    assert cfg.model.kind == "sd15" and cfg.train_mode == "lora"
    from eridiffusion_b200.data import synthetic_batch
    sb = synthetic_batch("sd15", 1, height=256, width=256)
    assert sb["latents"].shape == (1, 4, 32, 32) and sb["txt"].shape == (1, 77, 768) and "pooled" not in sb


def test_orchestrator_runs_recipe_and_learns():
    torch.manual_seed(0)
    model = build_model("tiny_mmdit")
    params = [p for n, p in model.named_parameters() if "final_layer" in n]
    for p in model.parameters():
        p.requires_grad_(False)
    for p in params:
        p.requires_grad_(True)
    opt = torch.optim.AdamW(params, lr=3e-3)
    saved, evals = [], []
    b = batch()
    ad = PipelineAdapter(model, PipelineFactory.create("tiny_mmdit", PipelineConfig(dynamic_shift=False)), opt,
                         iter([b] * 100), max_grad_norm=1.0, checkpoint_fn=saved.append, eval_fn=evals.append)
    orch = Orchestrator(ad, recipe=[*ad.default_recipe(), "checkpoint", "eval_step"])
    ctx = Ctx(rng_seed=7)
    losses = []
    for _ in range(12):
        ctx.step = 0                                   # same seed -> same timesteps and noise every step
        orch.run_step(ctx)
        losses.append(float(ctx.loss))
    assert losses[-1] < losses[0]
    assert ctx.log[:9] == list(ad.default_recipe()) and ctx.log[9:11] == [StageName.CHECKPOINT, StageName.EVAL_STEP]
    assert saved == [0] * 12 and evals == [0] * 12
    assert all(p.grad is None for p in params)         # zero_grad ran
