"""SDXL checkpoint key remapping: original layout <-> this package's UNet, with fused projections."""
import pytest
import torch

from eridiffusion_b200.io.sdxl_keys import export_sdxl_state_dict, map_sdxl_key, remap_sdxl_state_dict
from eridiffusion_b200.models import build_model

P = "model.diffusion_model."


def test_spot_keys():
    assert map_sdxl_key(P + "input_blocks.4.1.transformer_blocks.0.attn1.to_q.weight") == \
        ("down.3.1.blocks.0.attn1.to_qkv.weight", 0)
    assert map_sdxl_key(P + "input_blocks.8.1.transformer_blocks.9.attn2.to_v.weight") == \
        ("down.7.1.blocks.9.attn2.to_kv.weight", 1)
    assert map_sdxl_key(P + "middle_block.1.transformer_blocks.3.ff.net.0.proj.bias") == ("mid.1.blocks.3.ff_in.bias", None)
    assert map_sdxl_key(P + "output_blocks.5.1.transformer_blocks.1.attn1.to_out.0.weight") == \
        ("up.6.1.blocks.1.attn1.to_out.weight", None)
    assert map_sdxl_key(P + "output_blocks.2.2.conv.weight") == ("up.3.weight", None)
    assert map_sdxl_key(P + "output_blocks.5.2.conv.bias") == ("up.7.bias", None)
    assert map_sdxl_key(P + "input_blocks.3.0.op.weight") == ("down.2.weight", None)
    assert map_sdxl_key(P + "input_blocks.0.0.weight") == ("conv_in.weight", None)
    assert map_sdxl_key(P + "input_blocks.1.0.in_layers.2.weight") == ("down.0.0.conv1.weight", None)
    assert map_sdxl_key(P + "input_blocks.4.0.skip_connection.weight") == ("down.3.0.skip.weight", None)
    assert map_sdxl_key(P + "label_emb.0.2.bias") == ("add_embed.2.bias", None)
    assert map_sdxl_key(P + "out.0.weight") == ("norm_out.weight", None) and map_sdxl_key(P + "out.2.bias") == ("conv_out.bias", None)
    assert map_sdxl_key("first_stage_model.decoder.conv_in.weight") is None
    assert map_sdxl_key("conditioner.embedders.0.transformer.text_model.embeddings.position_ids") is None


def test_full_size_key_coverage():
    m = build_model("sdxl", device="meta")
    own = {n: p.shape for n, p in m.named_parameters()}
    exported = export_sdxl_state_dict({n: torch.empty(s, device="meta") for n, s in own.items()})
    # 70 transformer blocks: to_qkv -> 3 keys, to_kv -> 2 keys
    assert len(exported) == len(own) + 70 * 3
    back = remap_sdxl_state_dict(exported)
    assert set(back) == set(own) and all(tuple(back[n].shape) == tuple(own[n]) for n in own)
    # the reference's per-block table names exist in the exported layout
    for k in ("input_blocks.7.1.transformer_blocks.9.attn2.to_k.weight", "output_blocks.0.1.transformer_blocks.0.norm3.bias",
              "middle_block.1.proj_out.weight", "output_blocks.3.1.transformer_blocks.1.ff.net.2.weight",
              "middle_block.2.out_layers.3.weight", "output_blocks.8.0.skip_connection.weight"):
        assert P + k in exported, k


def test_round_trip_values_and_load():
    torch.manual_seed(0)
    kw = dict(block_channels=(32, 64, 64), transformer_depth=(0, 1, 2), head_dim=16, context_dim=32, pooled_dim=16,
              addition_time_embed_dim=8)
    a = build_model("sdxl", device="cpu", dtype=torch.float32, **kw)
    b = build_model("sdxl", device="cpu", dtype=torch.float32, **kw)
    orig = export_sdxl_state_dict(a.state_dict())
    orig["first_stage_model.encoder.conv_in.weight"] = torch.zeros(1)          # ignored: not the UNet
    b.load_state_dict(remap_sdxl_state_dict(orig))
    x, t = torch.randn(1, 4, 16, 16), torch.tensor([500.0])
    ctx, pooled, tid = torch.randn(1, 5, 32), torch.randn(1, 16), torch.tensor([[64., 64, 0, 0, 64, 64]])
    with torch.no_grad():
        assert torch.equal(a(x, t, ctx, pooled, tid), b(x, t, ctx, pooled, tid))
    del orig[P + "middle_block.1.transformer_blocks.0.attn1.to_k.weight"]
    with pytest.raises(KeyError, match="missing parts"):
        remap_sdxl_state_dict(orig)
    orig[P + "mystery.weight"] = torch.zeros(1)
    assert "mid.1.blocks.0.attn1.to_qkv.weight" not in remap_sdxl_state_dict(orig, strict=False)


def test_load_model_weights_from_original_layout(tmp_path):
    from eridiffusion_b200.io import safetensors as st
    from eridiffusion_b200.io.weights import load_model_weights
    torch.manual_seed(1)
    kw = dict(block_channels=(32, 64, 64), transformer_depth=(0, 1, 1), head_dim=16, context_dim=32, pooled_dim=16,
              addition_time_embed_dim=8)
    a = build_model("sdxl", device="cpu", dtype=torch.float32, **kw)
    b = build_model("sdxl", device="cpu", dtype=torch.float32, **kw)
    ckpt = {k: v.contiguous() for k, v in export_sdxl_state_dict(a.state_dict()).items()}
    ckpt["first_stage_model.decoder.conv_out.bias"] = torch.zeros(3)
    st.save_file(ckpt, tmp_path / "sd_xl.safetensors")
    used = load_model_weights(b, tmp_path / "sd_xl.safetensors", kind="sdxl")
    assert len(used) == len(dict(b.named_parameters()))
    for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
        assert torch.equal(p, q), n
