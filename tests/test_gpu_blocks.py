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


def _double_block(group, full_ft=False, depth_single=1, mlp_fuse=False):
    from eridiffusion_b200.adapters import AdapterConfig, inject_adapters
    from eridiffusion_b200.models import build_model
    from eridiffusion_b200.ops import functional as F
    from eridiffusion_b200.models import layers as LY
    old, old_fuse = F._GEMM_GROUP, LY._MLP_FUSE
    F._GEMM_GROUP, LY._MLP_FUSE = group, mlp_fuse
    try:
        torch.manual_seed(0)
        dev = "cuda"
        m = build_model("flux", device=dev, hidden=512, num_heads=4, depth_double=2, depth_single=depth_single,
                        context_dim=256, vec_dim=64)
        params = {}
        if full_ft:
            params = {n: p for n, p in m.named_parameters() if "double_blocks" in n and p.dim() == 2}
        else:
            m.requires_grad_(False)
            ads = inject_adapters(m, AdapterConfig(rank=16, alpha=16, target=m.lora_targets()), seed=1)
            g = torch.Generator(device=dev).manual_seed(5)
            for path, a in sorted(ads.items()):
                a.lora_B.data.copy_(torch.randn(a.lora_B.shape, device=dev, generator=g).mul_(0.05))
                for p_n, p in a.named_parameters():
                    params[f"{path}.{p_n}"] = p
        g = torch.Generator(device=dev).manual_seed(6)
        img = torch.randn(2, 1024, 64, device=dev, generator=g).bfloat16()
        txt = torch.randn(2, 256, 256, device=dev, generator=g).bfloat16()
        t = torch.tensor([0.3, 0.6], device=dev)
        y = torch.randn(2, 64, device=dev, generator=g).bfloat16()
        c0 = F.N.launch_count()
        out = m(img, txt, t, y, torch.tensor([3.5, 3.5], device=dev))
        w = torch.randn(out.shape, device=dev, generator=g).bfloat16()
        (out.float() * w.float()).mean().backward()
        n = F.N.launch_count() - c0
        assert F.gemm_error_check() == 0
        return out.float(), {k: p.grad.float().clone() for k, p in params.items() if p.grad is not None}, n
    finally:
        F._GEMM_GROUP, LY._MLP_FUSE = old, old_fuse


@pytest.mark.parametrize("full_ft,depth_single,mlp_fuse", [(False, 1, False), (True, 1, False), (False, 0, False),
                                                           (False, 1, True), (False, 0, True)])
def test_grouped_stream_linears_match_separate_launches(full_ft, depth_single, mlp_fuse):
    """Dual-stream blocks with the image and the text projection of each pair in one grouped launch
    (forward GEMM and input-gradient GEMM) against the same blocks with one launch per projection.
    Without single-stream blocks the last block's text output is unused: its gradient is None and the
    paired backward runs the image stream alone."""
    o1, g1, n1 = _double_block(True, full_ft, depth_single, mlp_fuse)
    o0, g0, n0 = _double_block(False, full_ft, depth_single)
    # two blocks x four projection pairs. Per grouped pair one GEMM launch fewer in forward and one in backward
    # (input gradient), and with adapters one rank-r launch fewer each way as well (both streams' x A^T, and
    # both streams' dY B, in one launch).
    # LoRA: the first pair of the first block has no input gradient to compute (frozen input projections):
    # 16 + 8 + 7. Without single-stream blocks three text projections of the last block have no gradient at
    # all: 16 + (1 + 4) + (1 + 3). Full fine-tune (no adapters; trainable gates are applied outside the GEMM in
    # both paths): 8 + 8. ``mlp_fuse`` (opt-in): the MLP pairs also drop their activation-gradient launches (the
    # derivative is applied in the down-projections' input-gradient epilogue): 4, or 3 when the last block's
    # text MLP has no gradient.
    extra = (4 if depth_single else 3) if mlp_fuse else 0
    assert n0 - n1 == (16 if full_ft else 31 if depth_single else 25) + extra, (n0, n1)
    assert (o1 - o0).abs().max().item() <= 0.02 * o0.abs().max().item()
    assert g0.keys() == g1.keys() and len(g0) > 0
    for k in g0:
        e = (g1[k] - g0[k]).abs().max().item()
        assert e <= 0.03 * g0[k].abs().max().item() + 1e-6, (k, e)
