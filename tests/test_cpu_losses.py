"""Named loss objects, the multi-scale LPIPS proxy and the clamped masked epsilon loss."""
import math

import pytest
import torch

from eridiffusion_b200.objectives import losses as L


def test_named_losses_and_weights():
    torch.manual_seed(0)
    p, t = torch.randn(2, 3, 8, 8), torch.randn(2, 3, 8, 8)
    mse = (p - t).pow(2).mean()
    for kind in ("mse", "perceptual", "flow_matching", "v"):
        assert torch.allclose(L.create_loss(kind, 2.0)(p, t), 2.0 * mse)
    assert torch.allclose(L.create_loss("mae")(p, t), (p - t).abs().mean())
    assert torch.allclose(L.create_loss("huber", delta=0.5)(p, t), torch.nn.functional.huber_loss(p, t, delta=0.5))
    for bad in (-1.0, float("nan"), float("inf")):
        with pytest.raises(ValueError):
            L.create_loss("mse", bad)
    with pytest.raises(ValueError):
        L.create_loss("nope")
    with pytest.raises(ValueError):
        L.create_loss("mse")(p, t[:, :2])


def test_lpips_proxy_features():
    torch.manual_seed(1)
    lp = L.create_loss("lpips")
    x = torch.rand(2, 3, 16, 16)
    f = lp.features(x)
    assert [tuple(t.shape) for t in f] == [(2, 1, 16, 16), (2, 1, 8, 8), (2, 1, 4, 4), (2, 3, 1, 1), (2, 3, 1, 1)]
    assert float(lp(x, x)) == 0.0
    # a constant image has no edge / texture response away from the zero-padded border
    c = torch.full((1, 3, 16, 16), 0.3)
    assert lp.features(c)[0][..., 2:-2, 2:-2].abs().max() < 1e-6
    # brightness shift: only the colour-mean term differs -> (0.1^2) / 5 features
    assert abs(float(lp(c + 0.1, c)) - sum([(f_a - f_b).pow(2).mean() for f_a, f_b in zip(lp.features(c + 0.1), lp.features(c))]) / 5) < 1e-7
    y = x.clone().requires_grad_()
    lp(y, torch.rand(2, 3, 16, 16)).backward()
    assert y.grad is not None and torch.isfinite(y.grad).all()
    lat = torch.rand(2, 4, 8, 8)                       # latent-like input: no colour statistics
    assert len(lp.features(lat)) == 3 and float(lp(lat, lat)) == 0.0


def test_masked_eps_loss_clamp_schedule():
    assert L.clamp_limit(0, 100, 1.0, 10.0) == pytest.approx(1.0)
    assert L.clamp_limit(50, 100, 1.0, 10.0) == pytest.approx(5.5)
    assert L.clamp_limit(100, 100, 1.0, 10.0) is None and L.clamp_limit(5, 0, 1.0, 10.0) is None
    pred = torch.tensor([[[0.0, 4.0], [1.0, -3.0]]], requires_grad=True)
    true = torch.zeros(1, 2, 2)
    full = L.masked_eps_loss_safe(pred, true)
    assert full.item() == pytest.approx((16 + 1 + 9) / 4)
    clamped = L.masked_eps_loss_safe(pred, true, global_step=0, clamp_warmup_steps=10, clamp_start=2.0, clamp_end=8.0)
    assert clamped.item() == pytest.approx((4 + 1 + 4) / 4)
    clamped.backward()
    assert pred.grad[0, 0, 1] == 0 and pred.grad[0, 1, 0] != 0           # clamped residuals pass no gradient
    mask = torch.tensor([[1.0, 0.0]])
    assert L.masked_eps_loss_safe(pred, true, mask).item() == pytest.approx(16 / 2)
    bf = L.masked_eps_loss_safe(pred.detach().bfloat16(), true)           # target follows the prediction's dtype
    assert bf.dtype == torch.float32 and math.isfinite(bf.item())
