"""Text encoders (CLIP, T5, decoder-style) and the KL autoencoder, on tiny CPU configurations."""
import torch

from eridiffusion_b200.models import build_model
from eridiffusion_b200.models.text_encoders import attn_mask_from_lengths

F32 = dict(dtype=torch.float32)


def test_clip_text_encoder_is_causal_and_pools_at_eos():
    torch.manual_seed(0)
    clip = build_model("clip_l", hidden=64, layers=2, heads=4, proj_dim=32, vocab_size=1000, eos_token_id=999, **F32)
    ids = torch.randint(0, 998, (2, 12))
    ids[:, 7] = 999
    h, pooled = clip(ids, output_layer=-2)
    assert h.shape == (2, 12, 64) and pooled.shape == (2, 32)
    ids2 = ids.clone()
    ids2[:, 10] = 5                                   # a later token must not change earlier states
    h2, pooled2 = clip(ids2, output_layer=-2)
    assert torch.allclose(h[:, :10], h2[:, :10], atol=1e-5)
    assert torch.allclose(pooled, pooled2, atol=1e-5)  # EOS sits before the edited position
    g = build_model("open_clip_g", hidden=64, layers=2, heads=4, proj_dim=48, vocab_size=1000, **F32)
    assert g.cfg.act == "gelu" and g(ids)[1].shape == (2, 48)


def test_t5_encoder_ignores_padding_keys():
    torch.manual_seed(0)
    t5 = build_model("t5_encoder", hidden=64, layers=2, heads=4, head_dim=16, ff=128, vocab_size=500, **F32)
    ids = torch.randint(0, 500, (2, 12))
    km = attn_mask_from_lengths([9, 12], 12)[:, 0, 0]
    a = t5(ids, km)
    ids_b = ids.clone()
    ids_b[0, 9:] = 7                                  # padding content of sample 0 must not matter
    b = t5(ids_b, km)
    assert torch.allclose(a[0, :9], b[0, :9], atol=1e-4) and torch.isfinite(a).all()
    # relative-position buckets: symmetric split, within range
    bk = t5._buckets(40, ids.device)
    assert int(bk.min()) >= 0 and int(bk.max()) < t5.cfg.rel_buckets and int(bk[0, 0]) == 0


def test_decoder_text_encoder_grouped_kv_and_hidden_layer():
    torch.manual_seed(0)
    qw = build_model("qwen3_encoder", hidden=64, layers=3, heads=4, kv_heads=2, head_dim=16, ff=128, vocab_size=500, **F32)
    ids = torch.randint(0, 500, (2, 10))
    out = qw(ids)
    assert out.shape == (2, 10, 64)
    ids2 = ids.clone()
    ids2[:, -1] = 3
    assert torch.allclose(out[:, :-1], qw(ids2)[:, :-1], atol=1e-5)   # causal
    out.mean().backward()
    assert qw.layers[0].q.weight.grad is not None and qw.layers[2].q.weight.grad is None  # layer -2 output


def test_vae_roundtrip_shapes_scaling_and_tiling():
    torch.manual_seed(0)
    vae = build_model("vae_sdxl", base=32, mult=(1, 2, 2, 2), groups=8, **F32)
    img = torch.rand(1, 3, 64, 64) * 2 - 1
    mean, logvar = vae.moments(img)
    z = vae.encode(img, sample=False)
    assert z.shape == (1, 4, 8, 8) and torch.allclose(z, mean * vae.cfg.scaling_factor)
    assert vae.decode(z).shape == img.shape
    zs = vae.encode(img, sample=True, generator=torch.Generator().manual_seed(1))
    assert not torch.allclose(zs, z)
    big = torch.randn(1, 4, 24, 20)
    full, tiled = vae.decode(big), vae.tiled_decode(big, tile=16, overlap=8)
    assert tiled.shape == full.shape == (1, 3, 192, 160)
    # tiles see less context than the full pass, so only closeness is expected
    assert (full - tiled).abs().mean() < 0.1 * full.abs().mean() + 0.05
    e = torch.rand(1, 3, 192, 160) * 2 - 1
    assert vae.tiled_encode(e, tile=128, overlap=64).shape == vae.encode(e, sample=False).shape
    flux = build_model("vae_flux", base=32, mult=(1, 2), groups=8, **F32)
    zf = flux.encode(img, sample=False)
    m2, _ = flux.moments(img)
    assert zf.shape[1] == 16 and torch.allclose(zf, (m2 - 0.1159) * 0.3611)
