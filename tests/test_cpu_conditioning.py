"""ControlNet, T2I-Adapter, IP-Adapter and Flux control concatenation on a tiny SDXL UNet (CPU)."""
import torch

from eridiffusion_b200.adapters.conditioning import (ControlNet, ControlNetConfig, IPAdapter, IPAdapterConfig,
                                                     PerceiverResampler, T2IAdapter, T2IAdapterConfig,
                                                     flux_control_concat, multiscale_control,
                                                     preprocess_control_image, widen_input_projection)
from eridiffusion_b200.models import build_model
from eridiffusion_b200.models.layers import Linear


def _tiny_unet():
    torch.manual_seed(0)
    return build_model("sdxl", dtype=torch.float32, block_channels=(32, 64, 64), transformer_depth=(0, 1, 1),
                       head_dim=16, context_dim=32, pooled_dim=16, addition_time_embed_dim=8, groups=8)


def _inputs(B=2):
    g = torch.Generator().manual_seed(1)
    return (torch.randn(B, 4, 16, 16, generator=g), torch.tensor([10.0, 500.0]), torch.randn(B, 7, 32, generator=g),
            torch.randn(B, 16, generator=g), torch.rand(B, 6, generator=g) * 100)


def test_controlnet_starts_as_identity_then_steers_and_trains():
    unet = _tiny_unet()
    x, t, ctx, pooled, tid = _inputs()
    base = unet(x, t, ctx, pooled, tid)
    cn = ControlNet(unet, ControlNetConfig(conditioning_scale=0.5))
    hint = preprocess_control_image(torch.randint(0, 255, (2, 3, 64, 64), dtype=torch.uint8), 128, 128)
    assert hint.shape == (2, 3, 128, 128) and 0.0 <= float(hint.min()) and float(hint.max()) <= 1.0
    down, mid = cn(x, t, ctx, pooled, tid, hint)
    assert len(down) == 9
    assert torch.allclose(unet(x, t, ctx, pooled, tid, control=(down, mid)), base)      # zero convs
    for z in cn.zero_convs:
        torch.nn.init.normal_(z.weight, std=0.1)
    down, mid = cn(x, t, ctx, pooled, tid, hint)
    out = unet(x, t, ctx, pooled, tid, control=multiscale_control(down, mid, [1.0, 0.5, 0.25]))
    assert (out - base).abs().max() > 0
    out.sum().backward()
    assert cn.hint_out.weight.grad is not None and cn.down[0][0].conv1.weight.grad is not None
    pooled_cn = ControlNet(unet, ControlNetConfig(global_pool_conditions=True))
    d2, m2 = pooled_cn(x, t, ctx, pooled, tid, hint)
    assert d2[0].shape[-2:] == (1, 1) and m2.shape[-2:] == (1, 1)


def test_t2i_adapter_features_enter_each_level():
    unet = _tiny_unet()
    x, t, ctx, pooled, tid = _inputs()
    base = unet(x, t, ctx, pooled, tid)
    ad = T2IAdapter(T2IAdapterConfig(channels=(32, 64, 64)), dtype=torch.float32)
    feats = ad(torch.rand(2, 3, 128, 128))
    assert [tuple(f.shape[1:]) for f in feats] == [(32, 16, 16), (64, 8, 8), (64, 4, 4)]
    assert (unet(x, t, ctx, pooled, tid, adapter_features=feats) - base).abs().max() > 0
    light = T2IAdapter(T2IAdapterConfig.lightweight(), dtype=torch.float32)
    assert len(light(torch.rand(1, 3, 64, 64))) == 3
    assert T2IAdapter.for_condition_type("canny", dtype=torch.float32).conv_in.in_channels == 64


def test_ip_adapter_decoupled_cross_attention():
    unet = _tiny_unet()
    x, t, ctx, pooled, tid = _inputs()
    base = unet(x, t, ctx, pooled, tid)
    ip = IPAdapter(unet, IPAdapterConfig(image_embed_dim=24, cross_attention_dim=32, num_tokens=4))
    assert torch.allclose(unet(x, t, ctx, pooled, tid), base)                          # no image set
    tokens = ip.set_image(torch.randn(2, 24))
    assert tokens.shape == (2, 4, 32)
    with_img = unet(x, t, ctx, pooled, tid)
    assert (with_img - base).abs().max() > 0
    ip.scale = 0.0
    assert torch.allclose(unet(x, t, ctx, pooled, tid), base)
    ip.scale = 1.0
    unet(x, t, ctx, pooled, tid).sum().backward()
    assert all(p.grad is not None for p in ip.trainable_parameters())
    res = PerceiverResampler(IPAdapterConfig(image_embed_dim=24, cross_attention_dim=32, num_tokens=6,
                                             hidden_dim=32, depth=2, heads=4, plus=True), torch.float32, None)
    assert res(torch.randn(2, 9, 24)).shape == (2, 6, 32)


def test_flux_control_concat_and_widened_projection():
    lat, ctl = torch.randn(2, 16, 8, 8), torch.randn(2, 16, 8, 8)
    assert flux_control_concat(lat, ctl).shape == (2, 32, 8, 8)
    lin = Linear(64, 48, dtype=torch.float32)
    wide = widen_input_projection(lin, 64)
    x = torch.randn(3, 5, 64)
    assert torch.allclose(wide(torch.cat([x, torch.randn(3, 5, 64)], -1)), lin(x), atol=1e-5)
