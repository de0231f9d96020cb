"""Whole-model checks on the GPU: the fused kernels path (including the single-stream block node)
against the PyTorch/library path of the same model, forward and LoRA gradients."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(backend, depth_double, depth_single):
    from eridiffusion_b200.adapters import AdapterConfig, inject_adapters
    from eridiffusion_b200.models import build_model
    from eridiffusion_b200.ops import functional as F
    F.set_backend(backend)
    try:
        torch.manual_seed(0)
        dev = "cuda"
        m = build_model("flux", device=dev, hidden=512, num_heads=4, depth_double=depth_double,
                        depth_single=depth_single, context_dim=256, vec_dim=64)
        ads = inject_adapters(m, AdapterConfig(rank=16, alpha=16, target=m.lora_targets()), seed=1)
        g = torch.Generator(device=dev).manual_seed(5)
        for a in ads.values():            # non-zero B so that every gradient path is exercised
            a.lora_B.data.copy_(torch.randn(a.lora_B.shape, device=dev, generator=g).mul_(0.05))
        img = torch.randn(1, 256, 64, device=dev, generator=g).bfloat16()
        txt = torch.randn(1, 128, 256, device=dev, generator=g).bfloat16()
        t = torch.tensor([0.3], device=dev)
        y = torch.randn(1, 64, device=dev, generator=g).bfloat16()
        out = m(img, txt, t, y, torch.tensor([3.5], device=dev))
        w = torch.randn(out.shape, device=dev, generator=g).bfloat16()
        (out.float() * w.float()).mean().backward()
        grads = {}
        for path, a in sorted(ads.items()):
            for p_n, p in a.named_parameters():
                if p.grad is not None:
                    grads[f"{path}.{p_n}"] = p.grad.float().clone()
        return out.float(), grads
    finally:
        F.set_backend("fused")


@pytest.mark.parametrize("dd,ds", [(1, 0), (0, 1), (1, 2)])
def test_fused_model_matches_library_path(dd, ds):
    from eridiffusion_b200.ops import functional as F
    o1, g1 = _run("fused", dd, ds)
    assert F.gemm_error_check() == 0
    o2, g2 = _run("eager", dd, ds)
    err = (o1 - o2).abs().max().item()
    assert err < 0.05 * o2.abs().max().item() + 0.05, err
    for k in g2:
        a, b = g1[k], g2[k]
        e = (a - b).abs().max().item()
        assert e < 0.06 * b.abs().max().item() + 1e-5, (k, e, b.abs().max().item())
