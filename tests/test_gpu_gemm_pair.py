"""Two-CTA (cta_group::2) GEMM variant against fp32 references."""
import math

import pytest
import torch

from eridiffusion_b200.ops import functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*s, seed=0, scale=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed + sum(s))
    return (torch.randn(*s, device=DEV, generator=g) * scale).bfloat16()


def close(a, b, atol):
    err = (a.float() - b.float()).abs().max().item()
    assert err <= atol + 0.02 * b.float().abs().max().item(), err


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 320), (1024, 3072, 1024), (300, 520, 136)])
def test_pair_plain_and_mn(M, N, K):
    F.set_gemm_pair(True)
    a, b = rnd(M, K), rnd(N, K, seed=1)
    out = F.gemm_native(a, b)
    assert F.gemm_error_check() == 0
    close(out, a.float() @ b.float().t(), 0.05 * math.sqrt(K / 64))
    bt = b.t().contiguous()
    out2 = F.gemm_native(a, bt, b_mn=True)
    assert F.gemm_error_check() == 0
    close(out2, a.float() @ b.float().t(), 0.05 * math.sqrt(K / 64))


@pytest.mark.parametrize("r", [16, 64])
def test_pair_lora_epilogues(r):
    F.set_gemm_pair(True)
    B, L, K, N = 2, 256, 512, 768
    M = B * L
    x, w, bias = rnd(M, K), rnd(N, K, scale=K ** -0.5, seed=1), rnd(N, seed=2)
    A, Bm = rnd(r, K, scale=K ** -0.5, seed=3), rnd(N, r, scale=0.1, seed=4)
    res, gate = rnd(M, N, seed=5), rnd(B, N, seed=6)
    h = F.gemm_native(x, A, alpha=0.5)
    pre = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    y = F.gemm_native(x, w, bias=bias, lora_h=h, lora_b=Bm, act="gelu", pre_out=pre, residual=res,
                      gate=gate, rows_per_batch=L)
    assert F.gemm_error_check() == 0
    pre_ref = x.float() @ w.float().t() + bias.float() + h.float() @ Bm.float().t()
    close(pre, pre_ref, 0.05)
    y_ref = res.float() + gate.float().repeat_interleave(L, 0) * torch.nn.functional.gelu(pre_ref, approximate="tanh")
    close(y, y_ref, 0.06)
    dy = rnd(M, N, seed=8)
    wt = rnd(K, N, scale=N ** -0.5, seed=9)
    n_split = 256
    out1 = torch.empty(M, n_split, device=DEV, dtype=torch.bfloat16)
    out2 = torch.empty(M, K - n_split, device=DEV, dtype=torch.bfloat16)
    pre2 = rnd(M, K - n_split, seed=10)
    F.gemm_native(dy, wt, out=out1, out2=out2, n_split=n_split, act="gelu_bwd", pre_in=pre2)
    assert F.gemm_error_check() == 0
    full = dy.float() @ wt.float().t()
    close(out1, full[:, :n_split], 0.06)
    pf = pre2.float().requires_grad_()
    gd = torch.autograd.grad(torch.nn.functional.gelu(pf, approximate="tanh").sum(), pf)[0]
    close(out2, full[:, n_split:] * gd, 0.06)
