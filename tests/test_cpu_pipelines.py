"""Inference schedules and the unified pipeline on CPU with small random-weight models."""
import math

import pytest
import torch

from eridiffusion_b200.models import build_model
from eridiffusion_b200.sampling import pipelines as P


def test_flux_timesteps_and_flow_match_scheduler():
    t = P.flux_timesteps(8, shift=3.0)
    assert t.shape == (9,) and abs(float(t[0]) - 1.0) < 1e-6 and (t[1:] < t[:-1]).all()
    # t' = sigmoid(shift t) / sigmoid(shift); at t = 0 that is 0.5 / sigmoid(shift)
    assert abs(float(t[-1]) - 0.5 / (1 / (1 + math.exp(-3.0)))) < 1e-6
    s = P.FlowMatchScheduler(5, shift=3.0)
    assert s.timesteps == [1.0, 0.75, 0.5, 0.25, 0.0]
    assert abs(s.apply_shift(0.5) - 0.5) < 1e-9 and s.apply_shift(1.0) > 0.95
    x, v = torch.ones(2, 3), torch.full((2, 3), 2.0)
    assert torch.equal(s.step(v, 1.0, x), x + v * (s.apply_shift(0.8) - s.apply_shift(1.0)))
    big = P.FlowMatchScheduler(5, shift=20.0)
    assert torch.equal(big.step(v, 1.0, x), x)                       # t > 0.999: sample returned unchanged
    assert torch.allclose(s.add_noise(x, v, 0.5), 0.5 * x + 0.5 * v)
    sig = s.sigmas()
    assert sig.shape == (6,) and float(sig[-1]) == 0.0
    with pytest.raises(ValueError):
        P.FlowMatchScheduler(1)


def test_ltx_schedule_and_euler_loop():
    sig = P.ltx_sigma_schedule(6, 4096, terminal=0.1)
    assert len(sig) == 7 and sig[0] == 1.0 and sig[-1] == 0.0 and all(a > b for a, b in zip(sig, sig[1:]))
    assert min(s for s in sig if s > 0) >= 0.1
    # more tokens -> larger shift -> sigmas stay higher
    lo, hi = P.ltx_sigma_schedule(6, 1024, terminal=0.0), P.ltx_sigma_schedule(6, 4096, terminal=0.0)
    assert hi[3] > lo[3]
    es = math.exp(0.95)
    assert abs(lo[3] - es / (es + 1.0)) < 1e-6                        # t = 0.5 at the base shift
    # exact velocity field of a point target: x_t = (1 - s) x0 + s n, v = n - x0 -> the loop returns x0
    x0, n = torch.randn(4, 5), torch.randn(4, 5)
    out = P.euler_denoise_flow(lambda x, s: n - x0, n, P.LTX_DISTILLED_SIGMAS)
    assert torch.allclose(out, x0, atol=1e-5)


def test_model_type_detection_and_memory_policy():
    MT = P.ModelType
    assert MT.from_path("/m/sd_xl_base_1.0_SDXL.safetensors") is MT.SDXL
    assert MT.from_path("sd3.5_medium.safetensors") is MT.SD35_MEDIUM and MT.from_path("SD35-large") is MT.SD35_LARGE
    assert MT.from_path("flux1-schnell.sft") is MT.FLUX_SCHNELL and MT.from_path("FLUX.1-dev") is MT.FLUX_DEV
    assert MT.from_path("flux2-klein-9b") is MT.KLEIN and MT.from_path("ltx-video-2b") is MT.LTX
    assert MT.from_path("Wan2.2-T2V-A14B") is MT.WAN22 and MT.from_path("qwen-image.safetensors") is MT.QWEN_IMAGE
    with pytest.raises(ValueError):
        MT.from_path("mystery.ckpt")
    assert MT.SD35_LARGE.family == "sd35" and MT.FLUX_DEV.family == "flux" and MT.LTX.is_video
    big = MT.FLUX_DEV.memory_config(180.0)
    assert not big.cpu_offload and big.vae_tiling
    small = MT.FLUX_DEV.memory_config(24.0)
    assert small.cpu_offload and small.sequential_offload and small.attention_slicing and small.vae_tile_size == 32
    assert not MT.SDXL.memory_config(24.0).sequential_offload


def test_pipeline_image_flow_and_offload():
    torch.manual_seed(0)
    m = build_model("tiny_mmdit", device="cpu", dtype=torch.float32).eval()
    calls = []

    def encode(prompt):
        calls.append(prompt)
        g = torch.Generator().manual_seed(len(prompt))
        return torch.randn(1, 64, 128, generator=g), torch.randn(1, 64, generator=g)

    pipe = P.UnifiedInferencePipeline(m, P.ModelType.FLUX_DEV, text_encode=encode,
                                      memory=P.MemoryConfig(cpu_offload=True), device="cpu")
    lat = pipe.generate("a cat", width=128, height=128, steps=3, seed=1)
    assert lat.shape == (1, 16, 16, 16) and torch.isfinite(lat).all() and calls == ["a cat"]
    assert torch.equal(lat, pipe.generate("a cat", width=128, height=128, steps=3, seed=1))
    assert not torch.equal(lat, pipe.generate("a cat", width=128, height=128, steps=3, seed=2))
    lat_cfg = pipe.generate("a cat", negative_prompt="blurry", width=128, height=128, steps=3, seed=1, cfg_scale=2.0)
    assert not torch.equal(lat, lat_cfg) and "blurry" in calls
    assert "flux_dev" in pipe.model_info()
    with pytest.raises(ValueError):
        P.UnifiedInferencePipeline(m, P.ModelType.FLUX_DEV, device="cpu").generate("no encoder")
    with pytest.raises(ValueError):
        pipe.decode(lat)


def test_pipeline_sdxl_and_video():
    torch.manual_seed(0)
    unet = build_model("sdxl", device="cpu", dtype=torch.float32, block_channels=(32, 64, 64),
                       transformer_depth=(0, 1, 1), head_dim=16, context_dim=32, pooled_dim=16,
                       addition_time_embed_dim=8).eval()
    pipe = P.UnifiedInferencePipeline(unet, P.ModelType.SDXL, device="cpu")
    txt, pooled = torch.randn(1, 7, 32), torch.randn(1, 16)
    for sampler in ("euler", "euler_a", "dpmpp_2m", "ddim"):
        lat = pipe.generate(txt=txt, pooled=pooled, width=64, height=64, steps=3, guidance_scale=5.0, sampler=sampler)
        assert lat.shape == (1, 4, 8, 8) and torch.isfinite(lat).all()
    with pytest.raises(ValueError):
        pipe.generate(txt=txt, pooled=pooled, width=64, height=64, steps=2, sampler="nope")
    ltx = build_model("ltx_video", device="cpu", dtype=torch.float32, hidden=64, num_heads=2, depth=2, in_channels=8,
                      context_dim=32, caption_dim=32, time_embed_dim=16).eval()
    vp = P.UnifiedInferencePipeline(ltx, P.ModelType.LTX, device="cpu")
    vid = vp.generate(txt=torch.randn(1, 5, 32), width=128, height=64, frames=3, steps=8)
    assert vid.shape == (1, 8, 3, 2, 4) and torch.isfinite(vid).all()
