"""GroupNorm(+SiLU) channels-last kernels and device-side token routing against fp32 references."""
import pytest
import torch

from eridiffusion_b200.ops import functional as F
from eridiffusion_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def rnd(*shape, seed=0, scale=1.0, dtype=torch.bfloat16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(dtype)


def close(a, b, rel_to_max, atol=0.0):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    tol = atol + rel_to_max * b.abs().max().item()
    assert err <= tol, f"max err {err:.4g} > {tol:.4g}"


@pytest.mark.parametrize("silu", [True, False])
@pytest.mark.parametrize("N,H,W,C", [(2, 17, 13, 320), (1, 32, 32, 64), (2, 8, 8, 1920), (1, 64, 64, 640)])
def test_group_norm_silu_fwd_bwd(silu, N, H, W, C):
    x = (rnd(N, H * W, C) + 0.5).requires_grad_()
    w = (rnd(C, seed=1, scale=0.5) + 1.0).requires_grad_()
    b = rnd(C, seed=2, scale=0.3).requires_grad_()
    y = F.group_norm_silu(x, w, b, 32, 1e-5, silu)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = R.group_norm_silu(xr, wr, br, 32, 1e-5, silu)
    close(y, yr, 2e-2)
    g = rnd(N, H * W, C, seed=5)
    y.backward(g)
    yr.backward(g.float())
    close(x.grad, xr.grad, 3e-2)
    close(w.grad, wr.grad, 3e-2)
    close(b.grad, br.grad, 3e-2)


def test_group_norm_nchw_channels_last_roundtrip():
    x = rnd(2, 320, 12, 10).contiguous(memory_format=torch.channels_last)
    w, b = rnd(320, seed=1) + 1.0, rnd(320, seed=2)
    y = F.group_norm_silu(x, w, b, 32, 1e-5, True)
    ref = torch.nn.functional.silu(torch.nn.functional.group_norm(x.float(), 32, w.float(), b.float(), 1e-5))
    assert y.shape == x.shape and y.is_contiguous(memory_format=torch.channels_last)
    close(y, ref, 2e-2)


@pytest.mark.parametrize("B,L,D,k", [(2, 1000, 256, 300), (1, 4096, 3072, 2048), (3, 37, 64, 5)])
def test_token_route_topk_gather_reinject(B, L, D, k):
    x = rnd(B, L, D).requires_grad_()
    scores = F.token_scores(x)
    close(scores, x.detach().float().norm(dim=-1), 1e-3)
    idx = F.topk_indices(scores, k)
    ref_idx = scores.topk(k, dim=1).indices
    # same set (scores are distinct with overwhelming probability), same descending order
    assert torch.equal(idx, ref_idx)
    idx = idx.sort(dim=1).values
    routed = F.gather_rows(x, idx)
    ref_routed = torch.gather(x.detach(), 1, idx.unsqueeze(-1).expand(-1, -1, D))
    assert torch.equal(routed.detach(), ref_routed)
    processed = (routed * 2).detach().requires_grad_()
    full = rnd(B, L, D, seed=3).requires_grad_()
    out = F.reinject_rows(full, processed, idx)
    ref_out = full.detach().scatter(1, idx.unsqueeze(-1).expand(-1, -1, D), processed.detach())
    assert torch.equal(out.detach(), ref_out)
    # gradients: gather scatters, reinject splits
    g = rnd(B, L, D, seed=7)
    out.backward(g)
    mask = torch.zeros(B, L, dtype=torch.bool, device="cuda").scatter_(1, idx, True)
    assert torch.equal(full.grad, g * (~mask).unsqueeze(-1))
    assert torch.equal(processed.grad, torch.gather(g, 1, idx.unsqueeze(-1).expand(-1, -1, D)))
    gr = rnd(B, k, D, seed=9)
    routed.backward(gr)
    ref_dx = torch.zeros(B, L, D, device="cuda", dtype=torch.bfloat16).scatter(1, idx.unsqueeze(-1).expand(-1, -1, D), gr)
    assert torch.equal(x.grad, ref_dx)


def test_topk_ties_prefer_lower_index():
    s = torch.tensor([[1.0, 3.0, 3.0, 0.5, 3.0, 2.0]], device="cuda")
    assert F.topk_indices(s, 4).tolist() == [[1, 2, 4, 5]]


@pytest.mark.parametrize("kind", ["int8", "int4", "nf4"])
def test_dequant_kernels_match_the_torch_statement(kind):
    """Quantised base weights: the CUDA expansion equals the elementwise PyTorch de-quantisation
    bit for bit, and a quantised linear runs through the fused GEMM."""
    from eridiffusion_b200 import memory as M
    from eridiffusion_b200.models.layers import Linear
    w = rnd(384, 512, seed=4, scale=0.05)
    q = M.quantize(w, kind, block=64)
    F.set_backend("eager")
    ref = M.dequantize(q)
    F.set_backend("fused")
    got = M.dequantize(q)
    assert got.dtype == torch.bfloat16 and torch.equal(got, ref)
    lin = Linear(512, 384, device="cuda")
    lin.weight.requires_grad_(False)
    ql = M.QuantizedLinear(lin, kind)
    x = rnd(2, 200, 512, seed=6)
    y = ql(x)
    yr = x.float() @ M.dequantize(ql.q).float().t() + lin.bias.float()
    close(y, yr, 2e-2)
