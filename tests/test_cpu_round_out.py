"""Accumulation service, parameter registry, SD3.5 block variants and projections (CPU)."""
import json
import types

import pytest
import torch

from eridiffusion_b200.io.param_registry import ParamRegistry, assert_vram_below, vram_used_gb
from eridiffusion_b200.train.accumulation import (AccumulationConfig, CheckpointSelection, DynamicAccumulator,
                                                  GradientAccumulator, ReductionMode, SyncMode,
                                                  create_accumulation_schedule, effective_batch_size,
                                                  estimate_memory_requirement)


# ----------------------------------------------------------------------------- accumulation
def test_accumulator_mean_sum_weighted():
    g1, g2 = torch.tensor([1.0, 2.0]), torch.tensor([3.0, 6.0])
    for red, want in ((ReductionMode.MEAN, [2.0, 4.0]), (ReductionMode.SUM, [4.0, 8.0]),
                      (ReductionMode.WEIGHTED_MEAN, [1.0, 2.0])):
        acc = GradientAccumulator(AccumulationConfig(steps=2, reduction=red, weight=0.5))
        acc.accumulate("w", g1); acc.step()
        assert not acc.should_sync()
        acc.accumulate("w", g2); acc.step()
        assert acc.should_sync()
        assert acc.memory_usage() == 8
        out = acc.get_gradients()
        assert torch.allclose(out["w"], torch.tensor(want))
        assert acc.current_step == 0 and acc.memory_usage() == 0
    # the accumulator owns its buffer: the caller's gradient is not modified
    assert torch.equal(g1, torch.tensor([1.0, 2.0]))


def test_accumulator_sync_modes_count_reductions():
    calls = []

    def reduce_fn(t):
        calls.append(t.clone())
        t.mul_(2.0)                      # stands for a SUM over two identical ranks

    for mode, n_sync in ((SyncMode.IMMEDIATE, 4), (SyncMode.DEFERRED, 1), (SyncMode.ADAPTIVE, 1)):
        calls.clear()
        acc = GradientAccumulator(AccumulationConfig(steps=4, sync_mode=mode), reduce_fn)
        for i in range(4):
            acc.accumulate("w", torch.full((3,), float(i)))
            acc.step()
        out = acc.get_gradients()["w"]
        assert acc.syncs == n_sync == len(calls)
        assert torch.allclose(out, torch.full((3,), 2.0 * (0 + 1 + 2 + 3) / 4))


def test_accumulator_stats_and_apply():
    p = torch.nn.Parameter(torch.zeros(2, 2, dtype=torch.bfloat16))
    acc = GradientAccumulator(AccumulationConfig(steps=1, dtype="float32"))
    acc.accumulate("p", torch.ones(2, 2), scale=0.5)
    acc.accumulate("bad", torch.tensor([float("nan")]))
    st = acc.stats()
    assert st.num_tensors == 2 and st.num_nonfinite == 1 and abs(st.total_norm - 1.0) < 1e-6
    acc.apply_to({"p": p})
    assert p.grad.dtype == torch.bfloat16 and torch.allclose(p.grad.float(), torch.full((2, 2), 0.5))
    with pytest.raises(ValueError):
        AccumulationConfig(dtype="int8")


def test_dynamic_accumulator_and_helpers():
    dyn = DynamicAccumulator(AccumulationConfig(steps=2), memory_threshold=1000)
    assert dyn.adjust_steps(2000, 0.1) == 4
    assert dyn.adjust_steps(2000, 0.1) == 8
    assert dyn.adjust_steps(700, 0.1) == 8
    assert dyn.adjust_steps(100, 0.1) == 4
    for _ in range(10):
        dyn.adjust_steps(700, 2.0)
    assert dyn.get_optimal_config().sync_mode == SyncMode.DEFERRED
    dyn2 = DynamicAccumulator(AccumulationConfig(steps=64), memory_threshold=1000)
    assert dyn2.adjust_steps(5000, 0.1) == 64                 # capped
    assert effective_batch_size(4, 8) == 32 and effective_batch_size(4, 8, 8) == 256
    assert estimate_memory_requirement(10, 2, 3, 2) == 3 * 20 + 10 * 4 * 2 * 3 * 2
    assert create_accumulation_schedule(6, 4, 5) == [1, 2, 3, 4, 5, 5]
    sel = CheckpointSelection(True, segment_size=2)
    sel.select_every([f"b{i}" for i in range(6)])
    assert sel.should_checkpoint("b0") and not sel.should_checkpoint("b1")
    assert abs(sel.estimate_memory_savings(6) - 0.5 * 0.33) < 1e-6
    assert CheckpointSelection(False).estimate_memory_savings(6) == 0.0


# ----------------------------------------------------------------------------- registry
def test_param_registry():
    reg = ParamRegistry()
    a = reg.insert("a", torch.zeros(2, 3))
    b = reg.insert("b", torch.zeros(4, dtype=torch.bfloat16))
    assert a != b and reg.id_of("a") == a and reg.name_of(b) == "b" and len(reg) == 2
    reg.set_requires_grad([b])
    assert reg.get("b").requires_grad and not reg.get("a").requires_grad
    reg.assign(a, torch.ones(5))
    assert reg.get_by_id(a).shape == (5,)
    s = json.loads(reg.emit_json_summary())
    assert s["count"] == 2 and s["bytes"] == 20 + 8 and s["trainable"] == 1
    assert reg.remove("a") and not reg.remove("a") and reg.get_by_id(a) is None
    with pytest.raises(KeyError):
        reg.assign(a, torch.zeros(1))
    lin = torch.nn.Linear(3, 2)
    assert {n for n, _, _ in ParamRegistry.from_module(lin, "m.")} == {"m.weight", "m.bias"}


def test_vram_guard_with_fake_nvml():
    fake = types.SimpleNamespace(
        nvmlInit=lambda: None, nvmlDeviceGetHandleByIndex=lambda i: i,
        nvmlDeviceGetMemoryInfo=lambda h: types.SimpleNamespace(used=3 * 2 ** 30))
    assert vram_used_gb(nvml=fake) == 3.0
    assert assert_vram_below(4.0, nvml=fake) == 3.0
    with pytest.raises(MemoryError):
        assert_vram_below(2.0, nvml=fake)


# ----------------------------------------------------------------------------- SD3.5
def _sd35(**kw):
    from eridiffusion_b200.models.sd35_klein import SD35MMDiT
    torch.manual_seed(0)
    m = SD35MMDiT(hidden=64, num_heads=2, depth=3, in_channels=8, context_dim=16, pooled_dim=12,
                  dtype=torch.float32, **kw)
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.05)
    return m


def test_sd35_context_pre_only_and_dual_attention():
    from eridiffusion_b200.models.sd35_klein import SD35JointBlock
    m = _sd35(context_pre_only_last=True, x_self_attn_layers=(0, 1))
    blocks = m.joint_blocks
    assert isinstance(blocks[0], SD35JointBlock) and blocks[0].x_self_attn and not blocks[0].context_pre_only
    assert blocks[2].context_pre_only and not hasattr(blocks[2], "txt_mlp_0") and blocks[2].txt_attn.proj is None
    assert blocks[0].img_mod.lin.weight.shape[0] == 9 * 64 and blocks[2].txt_mod.lin.weight.shape[0] == 2 * 64
    img, txt = torch.randn(2, 16, 8), torch.randn(2, 5, 16)
    t, y = torch.rand(2), torch.randn(2, 12)
    out = m(img, txt, t, y, grid_hw=(4, 4))
    assert out.shape == (2, 16, 8) and torch.isfinite(out).all()
    out.square().mean().backward()
    assert blocks[0].img_attn2.qkv.weight.grad.abs().sum() > 0
    assert blocks[2].txt_attn.qkv.weight.grad.abs().sum() > 0
    # the last block's text stream is a pure input: its result must not depend on text modulation gates
    x, c = torch.randn(2, 16, 64), torch.randn(2, 5, 64)
    vec = torch.randn(2, 64)
    _, c_out = blocks[2](x, c, vec)
    assert torch.equal(c_out, c)
    # zero gate on the second attention reproduces the plain joint block's image update
    plain = _sd35(context_pre_only_last=False)
    assert not any(isinstance(b, SD35JointBlock) for b in plain.joint_blocks)
    assert any("attn2" in n for n, _ in m.named_parameters())


def test_sd35_projections_match_fp32_statement():
    from eridiffusion_b200.models.sd35_projections import (Latent1x1Conv, TextLinearPad, VelocityHead,
                                                           trainable_projections)
    lat = Latent1x1Conv(32, dtype=torch.float32, seed=1)
    x = torch.randn(2, 16, 3, 5)
    want = torch.einsum("bchw,oc->bohw", x, lat.proj.weight) + lat.proj.bias[None, :, None, None]
    assert torch.allclose(lat(x), want, atol=1e-5)
    assert abs(float(lat.proj.weight.detach().std()) - 0.25) < 0.05 and float(lat.proj.bias.detach().abs().sum()) == 0
    with pytest.raises(ValueError):
        lat(torch.randn(2, 4, 3, 5))
    tp = TextLinearPad(8, dtype=torch.float32, seed=2, in_dim=12, tokens=7)
    short, long = torch.randn(1, 3, 12), torch.randn(1, 9, 12)
    o = tp(short)
    assert o.shape == (1, 7, 8)
    assert torch.allclose(o[:, :3], short @ tp.proj.weight.T + tp.proj.bias, atol=1e-5)
    assert torch.allclose(o[:, 3:], tp.proj.bias.expand(1, 4, 8), atol=1e-6)
    assert torch.allclose(tp(long), long[:, :7] @ tp.proj.weight.T + tp.proj.bias, atol=1e-5)
    vh = VelocityHead(32, dtype=torch.float32, seed=3)
    h = torch.randn(2, 32, 3, 5)
    assert torch.allclose(vh(h), torch.einsum("bchw,oc->bohw", h, vh.proj.weight), atol=1e-5)
    d = trainable_projections(32, dtype=torch.float32)
    assert set(d) == {"latent_in", "text_in", "velocity_out"}
    assert d["velocity_out"](d["latent_in"](x)).shape == x.shape


# ----------------------------------------------------------------------------- slices
def test_narrow_copy_and_backward_add_cpu_path():
    from eridiffusion_b200.ops.narrow import narrow_backward_add, narrow_copy, narrow_copy_raw
    x = torch.randn(3, 10, 4)
    assert torch.equal(narrow_copy_raw(x, -2, 2, 5), x[:, 2:7])
    xr = x.clone().requires_grad_()
    narrow_copy(xr, 1, 2, 5).sum().backward()
    want = torch.zeros_like(x); want[:, 2:7] = 1
    assert torch.equal(xr.grad, want)
    gin = torch.ones(3, 10, 4)
    narrow_backward_add(torch.full((3, 2, 4), 2.0), gin, 1, 8)
    assert gin[:, 8:].eq(3).all() and gin[:, :8].eq(1).all()
    with pytest.raises(IndexError):
        narrow_copy_raw(x, 1, 8, 5)
    with pytest.raises(ValueError):
        narrow_backward_add(torch.zeros(3, 2, 5), gin, 1, 0)
    with pytest.raises(ValueError):
        narrow_backward_add(torch.zeros(3, 2, 4), torch.zeros(1, 10, 4).expand(3, 10, 4), 1, 0)


# ----------------------------------------------------------------------------- LTX audio + video
def _ltx_av():
    from eridiffusion_b200.models import build_model
    torch.manual_seed(0)
    m = build_model("ltx_av", dtype=torch.float32, hidden=48, num_heads=2, depth=2, in_channels=8,
                    context_dim=24, caption_dim=12, audio=dict(audio_in_channels=6, audio_heads=2,
                                                               audio_head_dim=8, audio_context_dim=16))
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.08)
    return m


def test_ltx_audio_video_streams_exchange_information():
    m = _ltx_av()
    B, grid, La = 2, (2, 2, 3), 7
    xv, xa = torch.randn(B, 12, 8), torch.randn(B, La, 6)
    ctx, t = torch.randn(B, 5, 12), torch.tensor([0.2, 0.8])
    pv, pa = m(xv, xa, ctx, t, grid)
    assert pv.shape == xv.shape and pa.shape == xa.shape
    assert torch.isfinite(pv).all() and torch.isfinite(pa).all()
    # the audio stream changes the video prediction and the other way round
    pv2, pa2 = m(xv, xa + 1.0, ctx, t, grid)
    assert (pv2 - pv).abs().max() > 1e-6
    pv3, pa3 = m(xv + 1.0, xa, ctx, t, grid)
    assert (pa3 - pa).abs().max() > 1e-6
    (pv.square().mean() + pa.square().mean()).backward()
    assert all(p.grad is not None for n, p in m.named_parameters() if "a2v" in n or "v2a" in n)
    # closing the cross-modal gates (per-layer row 4 and the gate embedder) decouples the streams
    # and the video prediction equals the video-only path
    with torch.no_grad():
        for blk in m.blocks:
            blk.video_ca_table[4].zero_(); blk.audio_ca_table[4].zero_()
        for io in (m.video_io, m.audio_io):
            io.ca_gate.weight.zero_()
            if io.ca_gate.bias is not None:
                io.ca_gate.bias.zero_()
    pv4, pa4 = m(xv, xa, ctx, t, grid)
    pv5, _ = m(xv, xa * 3.0, ctx, t, grid)
    assert torch.allclose(pv4, pv5, atol=1e-6)
    assert torch.allclose(pv4, m.forward_video_only(xv, ctx, t, grid), atol=1e-5)
    import re
    pats = [re.compile(p) for p in m.lora_targets()]
    hit = [n for n, _ in m.named_modules() if any(p.search(n) for p in pats)]
    assert len(hit) == 2 * (7 * 2 + 3 * 2)


def test_rope_1d_table_aligns_instants():
    from eridiffusion_b200.models.ltx_av import rope_1d_table
    c1, s1 = rope_1d_table(torch.tensor([0.0, 1.0, 2.0]), 16)
    c2, s2 = rope_1d_table(torch.tensor([1.0]), 16)
    assert c1.shape == (3, 8) and torch.allclose(c1[1], c2[0]) and torch.allclose(s1[1], s2[0])
    assert torch.allclose(c1 ** 2 + s1 ** 2, torch.ones_like(c1), atol=1e-6)


# ----------------------------------------------------------------------------- SD3.5 checkpoint keys
def _sd3_reference_pos(hidden, max_size, gh, gw):
    """fp32 restatement of RoPE2D::embed (src/models/mmdit_blocks.rs:2107-2136): centre crop of the
    largest grid, integer positions, [sin | cos] per axis, the column axis FIRST."""
    axis = hidden // 2
    half = axis // 2
    inv = torch.tensor([1.0 / 10000.0 ** (i / half) for i in range(half)], dtype=torch.float32)
    top, left = (max_size - gh) // 2, (max_size - gw) // 2
    hp = torch.arange(top, top + gh, dtype=torch.float32)
    wp = torch.arange(left, left + gw, dtype=torch.float32)
    ha, wa = hp[:, None] * inv[None], wp[:, None] * inv[None]
    he = torch.cat([ha.sin(), ha.cos()], 1).view(gh, 1, axis).expand(gh, gw, axis)
    we = torch.cat([wa.sin(), wa.cos()], 1).view(1, gw, axis).expand(gh, gw, axis)
    return torch.cat([we, he], 2).reshape(gh * gw, hidden)


def _sd3_reference_unpatchify(tok, gh, gw, C, p=2):
    """fp32 restatement of the reference unpatchify (src/models/mmdit_blocks.rs:2280-2288): a token
    holds its patch as [p, p, C]."""
    B = tok.shape[0]
    return tok.reshape(B, gh, gw, p, p, C).permute(0, 5, 1, 3, 2, 4).reshape(B, C, gh * p, gw * p)


def test_sd35_original_layout_loads(tmp_path):
    """A checkpoint in the ORIGINAL SD3 conventions — (p, p, c) rows of the final projection, a real
    ``pos_embed`` table over the largest grid, convolution-shaped patch embedding — loads into the
    model so that the model computes the ORIGINAL function: the position rows equal the reference's
    centre-cropped embed and the predicted image equals the reference's unpatchify of the file-order
    projection."""
    from eridiffusion_b200.io import safetensors as st
    from eridiffusion_b200.io.weights import canonical_key, export_sd3_original, load_model_weights
    from eridiffusion_b200.models import build_model
    from eridiffusion_b200.ops import reference as R
    M = 10                                                   # largest patch grid of this toy table
    kw = dict(hidden=64, num_heads=2, depth=2, in_channels=64, context_dim=16, pooled_dim=12, dtype=torch.float32,
              x_self_attn_layers=(0,), pos_embed_max_size=M)
    torch.manual_seed(0)
    src = build_model("sd35", **kw)
    for p in src.parameters():
        torch.nn.init.normal_(p, std=0.1)
    assert src.joint_blocks[1].context_pre_only            # released layout: last block's text stream is pre-only
    # the closed-form table is the reference's embed for every crop
    for gh, gw in ((4, 4), (3, 6), (10, 10)):
        assert torch.allclose(src.pos_table(gh, gw, "cpu", torch.float32), _sd3_reference_pos(64, M, gh, gw), atol=1e-5)
    # a checkpoint in the original layout, with a table that is NOT the closed form
    sd = {"model.diffusion_model." + k: v for k, v in export_sd3_original(src).items()}
    table = torch.randn(1, M * M, 64)
    sd["model.diffusion_model.pos_embed"] = table
    assert sd["model.diffusion_model.x_embedder.proj.weight"].shape == (64, 16, 2, 2)
    assert "model.diffusion_model.joint_blocks.0.x_block.attn2.qkv.weight" in sd
    key = canonical_key("model.diffusion_model.joint_blocks.3.x_block.attn.ln_q.weight", "sd35")
    assert key == "joint_blocks.3.img_attn.q_norm.scale"
    f = tmp_path / "sd35.safetensors"
    st.save_file(sd, f)
    dst = build_model("sd35", **kw)
    used = load_model_weights(dst, f, "sd35", strict=True)
    assert len(used) == len(list(dst.named_parameters())) + 1          # + the position table
    for (n, a), (_, b) in zip(src.named_parameters(), dst.named_parameters()):
        assert torch.equal(a, b), n
    # the file's table is used, centre-cropped
    gh, gw = 4, 6
    top, left = (M - gh) // 2, (M - gw) // 2
    want = table.view(M, M, 64)[top:top + gh, left:left + gw].reshape(gh * gw, 64)
    assert torch.equal(dst.pos_table(gh, gw, "cpu", torch.float32), want)
    # the final projection: file-order rows + the reference's unpatchify == model rows + this package's
    fw = sd["model.diffusion_model.final_layer.linear.weight"]
    fb = sd["model.diffusion_model.final_layer.linear.bias"]
    h = torch.randn(2, gh * gw, 64)
    ref_img = _sd3_reference_unpatchify(h @ fw.t() + fb, gh, gw, 16)
    lin = dst.final_layer.linear
    our_img = R.unpatchify(h @ lin.weight.t() + lin.bias, 16, gh * 2, gw * 2)
    assert torch.allclose(ref_img, our_img, atol=1e-6)
    assert not torch.allclose(fw, lin.weight)              # the rows really were permuted
    # and the patch embedding: the file's convolution over an image == the linear over packed tokens
    img = torch.randn(2, 16, gh * 2, gw * 2)
    conv = torch.nn.functional.conv2d(img, sd["model.diffusion_model.x_embedder.proj.weight"],
                                      sd["model.diffusion_model.x_embedder.proj.bias"], stride=2)
    tok = R.patchify(img) @ dst.x_embedder.weight.t() + dst.x_embedder.bias
    assert torch.allclose(conv.flatten(2).transpose(1, 2), tok, atol=1e-5)
    txt = torch.randn(2, 5, 16)
    t, y = torch.rand(2), torch.randn(2, 12)
    # end to end: with the file's table loaded, the model differs from the closed-form one only
    # through the position rows
    src.pos_embed.copy_(table[0])
    assert torch.equal(src(R.patchify(img), txt, t, y, grid_hw=(gh, gw)), dst(R.patchify(img), txt, t, y, grid_hw=(gh, gw)))



def test_klein_checkpoint_layout_loads(tmp_path):
    from eridiffusion_b200.io import safetensors as st
    from eridiffusion_b200.io.weights import load_model_weights
    from eridiffusion_b200.models import build_model
    kw = dict(dtype=torch.float32, in_channels=8, dim=64, num_heads=2, depth_double=1, depth_single=2, context_dim=16,
              axes_dim=(8, 8, 8, 8))
    torch.manual_seed(0)
    src = build_model("klein", **kw)
    for n, p in src.named_parameters():
        torch.nn.init.zeros_(p) if n.endswith(".bias") else torch.nn.init.normal_(p, std=0.1)
    back = [(".img.q_norm.scale", ".img_attn.norm.query_norm.scale"), (".img.k_norm.scale", ".img_attn.norm.key_norm.scale"),
            (".txt.q_norm.scale", ".txt_attn.norm.query_norm.scale"), (".txt.k_norm.scale", ".txt_attn.norm.key_norm.scale"),
            (".img.qkv.", ".img_attn.qkv."), (".img.proj.", ".img_attn.proj."), (".txt.qkv.", ".txt_attn.qkv."),
            (".txt.proj.", ".txt_attn.proj."), (".img.mlp_in.", ".img_mlp.0."), (".img.mlp_out.", ".img_mlp.2."),
            (".txt.mlp_in.", ".txt_mlp.0."), (".txt.mlp_out.", ".txt_mlp.2."),
            ("double_mod_img.", "double_stream_modulation_img."), ("double_mod_txt.", "double_stream_modulation_txt."),
            ("single_mod.", "single_stream_modulation."), ("final_layer.adaLN.lin.", "final_layer.adaLN_modulation.1.")]
    sd = {}
    for n, p in src.named_parameters():
        if n.endswith(".bias"):
            continue                                           # the released files have no bias tensors
        k = n
        for a, b in back:
            k = k.replace(a, b)
        if k.startswith("single_blocks.") and k.endswith(("q_norm.scale", "k_norm.scale")):
            k = k.replace("q_norm.scale", "norm.query_norm.scale").replace("k_norm.scale", "norm.key_norm.scale")
        sd[k] = p.detach().clone()
    assert "double_blocks.0.img_attn.norm.query_norm.scale" in sd and "single_blocks.1.norm.key_norm.scale" in sd
    f = tmp_path / "klein.safetensors"
    st.save_file(sd, f)
    dst = build_model("klein", **kw)
    load_model_weights(dst, f, "klein", strict=True)
    for (n, a), (_, b) in zip(src.named_parameters(), dst.named_parameters()):
        assert torch.equal(a, b), n
    sd["extra.weight"] = torch.zeros(1)
    st.save_file(sd, f)
    with pytest.raises(KeyError, match="unused"):
        load_model_weights(build_model("klein", **kw), f, "klein", strict=True)


def test_ltx_diffusers_layout_round_trip(tmp_path):
    from eridiffusion_b200.io import safetensors as st
    from eridiffusion_b200.io.ltx_keys import export_ltx_state_dict, remap_ltx_state_dict
    from eridiffusion_b200.io.weights import load_model_weights
    from eridiffusion_b200.models import build_model
    kw = dict(dtype=torch.float32, hidden=48, num_heads=2, depth=2, in_channels=8, context_dim=24, caption_dim=12)
    torch.manual_seed(0)
    src = build_model("ltx_video", **kw)
    for p in src.parameters():
        torch.nn.init.normal_(p, std=0.1)
    ext = export_ltx_state_dict({n: p.detach().clone() for n, p in src.named_parameters()})
    assert "transformer_blocks.1.attn1.to_k.weight" in ext and ext["transformer_blocks.1.attn1.to_k.weight"].shape == (48, 48)
    assert "transformer_blocks.0.attn2.to_v.bias" in ext and "transformer_blocks.0.ff.net.0.proj.weight" in ext
    assert "time_embed.linear.weight" in ext and "caption_projection.linear_2.bias" in ext and "proj_in.weight" in ext
    assert not any(k.startswith("blocks.") for k in ext)
    # tensors a released file has and this model does not store
    ext["transformer_blocks.0.norm1.weight"] = torch.ones(48)
    ext["audio_proj_in.weight"] = torch.zeros(4, 4)
    ext["transformer_blocks.0.audio_attn1.to_q.weight"] = torch.zeros(4, 4)
    back = remap_ltx_state_dict(ext)
    assert set(back) == {n for n, _ in src.named_parameters()}
    f = tmp_path / "ltx.safetensors"
    st.save_file({"transformer." + k: v for k, v in ext.items()}, f)
    dst = build_model("ltx_video", **kw)
    load_model_weights(dst, f, "ltx", strict=True)
    for (n, a), (_, b) in zip(src.named_parameters(), dst.named_parameters()):
        assert torch.equal(a, b), n
    del ext["transformer_blocks.1.attn1.to_v.weight"]
    with pytest.raises(KeyError, match="expected"):
        remap_ltx_state_dict(ext)


def test_ltx_audio_video_trains_through_the_trainer():
    """[video tokens | audio tokens] as one noised latent sequence: the joint forward's two
    predictions come back in the same order and both streams' adapters receive gradient."""
    from eridiffusion_b200.adapters import AdapterConfig
    from eridiffusion_b200.train.trainer import Trainer, TrainerConfig, ltx_av_forward
    from eridiffusion_b200.models import build_model
    torch.manual_seed(0)
    m = build_model("ltx_av", dtype=torch.float32, hidden=48, num_heads=2, depth=2, in_channels=8,
                    context_dim=24, caption_dim=12, audio=dict(audio_in_channels=8, audio_heads=2,
                                                               audio_head_dim=8, audio_context_dim=16))
    cfg = TrainerConfig(mode="lora", adapter=AdapterConfig(rank=4, alpha=4, dtype=torch.float32), objective="flow",
                        optimizer="adamw", lr=1e-2, patch=1, seed=0, guidance=None)
    tr = Trainer(m, cfg, forward_fn=ltx_av_forward)
    grid, la = (2, 2, 3), 5
    batch = {"latents": torch.randn(2, 8, 12 + la, 1), "txt": torch.randn(2, 5, 12), "grid_fhw": grid}
    l0 = float(tr.train_step(batch))
    for _ in range(5):
        l1 = float(tr.train_step(batch))
    assert l0 == l0 and l1 < l0
    names = [n for n, p in m.named_parameters() if p.requires_grad]
    assert any(".audio." in n for n in names) and any(".video." in n for n in names) and any("a2v" in n for n in names)
