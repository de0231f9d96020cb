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


@pytest.mark.parametrize("M0,M1,N,K", [(4096, 512, 3072, 320), (1024, 256, 768, 512), (768, 300, 1024, 256)])
@pytest.mark.parametrize("mn", [False, True])
def test_grouped_launch_of_two_problems(M0, M1, N, K, mn):
    """Two products with the same N and K (image and text stream of a dual-stream block) in one launch:
    each with its own weight, bias, LoRA pair, residual and gate; results equal the separate launches."""
    F.set_gemm_pair(True)
    lib = F.N.require()
    r = 16
    outs = []
    kws = []
    for i, M in enumerate((M0, M1)):
        x = rnd(M, K, seed=10 * i)
        w = rnd(N, K, scale=K ** -0.5, seed=10 * i + 1)
        b_op = w.t().contiguous() if mn else w
        bias, res = rnd(N, seed=10 * i + 2), rnd(M, N, seed=10 * i + 3)
        gate = rnd(1, N, seed=10 * i + 4)
        A, Bm = rnd(r, K, scale=K ** -0.5, seed=10 * i + 5), rnd(N, r, scale=0.1, seed=10 * i + 6)
        h = F.gemm_native(x, A, alpha=0.5)
        kw = dict(a=x, b=b_op, bias=bias, lora_h=h, lora_b=Bm, residual=res, gate=gate, rows_per_batch=M, b_mn=mn)
        kws.append(kw)
        outs.append(F.gemm_native(**kw).clone())
        ref = res.float() + gate.float() * (x.float() @ w.float().t() + bias.float() + h.float() @ Bm.float().t())
        close(outs[-1], ref, 0.06)
    c0 = F.N.launch_count()
    y0, y1 = F.gemm_native_pair(kws[0], kws[1])
    assert F.N.launch_count() == c0 + 1, "the two products did not share one launch"
    assert F.gemm_error_check() == 0
    # the separate launches may have run on another kernel (few tiles: one-CTA route), so compare values
    for y, o in ((y0, outs[0]), (y1, outs[1])):
        assert (y.float() - o.float()).abs().max().item() <= 0.02 * o.float().abs().max().item()
    # a pair that does not qualify (different K) is launched one by one and still right
    x2, w2 = rnd(M1, K + 64, seed=77), rnd(N, K + 64, seed=78)
    z0, z1 = F.gemm_native_pair(dict(a=kws[0]["a"], b=kws[0]["b"], b_mn=mn),
                                dict(a=x2, b=w2.t().contiguous() if mn else w2, b_mn=mn))
    close(z1, x2.float() @ w2.float().t(), 0.06)
    assert F.gemm_error_check() == 0


@pytest.mark.parametrize("paired", [False, True])
def test_activation_outside_the_epilogue_matches_the_fused_form(paired):
    """A large linear + GELU with a short reduction writes its pre-activation from the GEMM and applies GELU in
    a pass of its own during training; outputs and gradients equal the form with everything in the epilogue."""
    M, N, K, r = 4096, 8192, 512, 16
    assert F._act_outside_epilogue(M, N, K)

    def run(fused):
        old = F._ACT_EPILOGUE
        F._ACT_EPILOGUE = fused
        try:
            outs = []
            xs = [rnd(1, M, K, seed=1).requires_grad_(), rnd(1, 512, K, seed=2).requires_grad_()]
            ws = [rnd(N, K, scale=K ** -0.5, seed=3), rnd(N, K, scale=K ** -0.5, seed=4)]
            As = [rnd(r, K, scale=K ** -0.5, seed=5).requires_grad_(), rnd(r, K, scale=K ** -0.5, seed=6).requires_grad_()]
            Bs = [rnd(N, r, scale=0.1, seed=7).requires_grad_(), rnd(N, r, scale=0.1, seed=8).requires_grad_()]
            bias = [rnd(N, seed=9), rnd(N, seed=10)]
            if paired:
                ys = F.linear_pair(xs[0], (ws[0], bias[0], (As[0], Bs[0], 0.5), None, None),
                                   xs[1], (ws[1], bias[1], (As[1], Bs[1], 0.5), None, None), act="gelu")
            else:
                ys = [F.linear(xs[i], ws[i], bias[i], lora=(As[i], Bs[i], 0.5), act="gelu") for i in range(2)]
            c0 = F.N.launch_count()
            sum((y.float() * 0.01).sum() for y in ys).backward()
            for i in range(2):
                outs += [ys[i].detach().float(), xs[i].grad.float(), As[i].grad.float(), Bs[i].grad.float()]
            return outs
        finally:
            F._ACT_EPILOGUE = old
    a, b = run(False), run(True)
    for u, v in zip(a, b):
        assert (u - v).abs().max().item() <= 0.02 * v.abs().max().item() + 1e-6
    assert F.gemm_error_check() == 0
    # against fp32 for the first stream's output
    x, w, bi = rnd(1, M, K, seed=1).float(), rnd(N, K, scale=K ** -0.5, seed=3).float(), rnd(N, seed=9).float()
    A, B = rnd(r, K, scale=K ** -0.5, seed=5).float(), rnd(N, r, scale=0.1, seed=7).float()
    ref = torch.nn.functional.gelu(x @ w.t() + bi + 0.5 * (x @ A.t()) @ B.t(), approximate="tanh")
    close(a[0], ref, 0.05)
