"""Weight-gradient products on tcgen05: the two-CTA GEMM with both operands token-major (full
fine-tune dW, with and without accumulation), the skinny token reduction for the LoRA gradients, and
the gated-linear-unit epilogue. Every case is compared with an fp32 PyTorch statement."""
import pytest
import torch

from eridiffusion_b200.ops import functional as F
from eridiffusion_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*s, seed=0, scale=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed + sum(s))
    return (torch.randn(*s, device=DEV, generator=g) * scale).bfloat16()


def rel_close(got, want, tol):
    err = (got.float() - want.float()).abs().max().item()
    ref = want.float().abs().max().item()
    assert err <= tol * ref, (err, ref)


@pytest.mark.parametrize("T,N,K", [(512, 256, 256), (1000, 768, 320), (4608, 1024, 3072), (136, 264, 520)])
def test_wgrad_matches_fp32(T, N, K):
    dy, x = rnd(T, N, scale=0.5), rnd(T, K, seed=1)
    c0 = F.N.launch_count()
    dw = F.wgrad(dy, x)
    assert F.N.launch_count() == c0 + 1, "the weight gradient did not run on the native kernel"
    assert F.kernel_error_check() == {}
    rel_close(dw, dy.float().t() @ x.float(), 8e-3)


def test_wgrad_accumulates_into_existing_gradient():
    T, N, K = 768, 512, 256
    dy, x = rnd(T, N, scale=0.5), rnd(T, K, seed=1)
    g0 = rnd(N, K, seed=2, scale=3.0)
    g = g0.clone()
    out = F.wgrad(dy, x, accum=g)
    assert out.data_ptr() == g.data_ptr() and F.kernel_error_check() == {}
    rel_close(g, g0.float() + dy.float().t() @ x.float(), 8e-3)


def test_wgrad_strided_operands():
    # column slices of wider buffers (the fused single-stream block hands these in)
    T, N, K = 512, 512, 384
    wide_dy, wide_x = rnd(T, N + 256, scale=0.5), rnd(T, K + 128, seed=1)
    dy, x = wide_dy[:, 256:], wide_x[:, :K]
    dw = F.wgrad(dy, x)
    assert F.kernel_error_check() == {}
    rel_close(dw, dy.float().t() @ x.float(), 8e-3)


@pytest.mark.parametrize("r", [16, 32, 64])
@pytest.mark.parametrize("T,Mg", [(4608, 3072), (1000, 328), (640, 9216)])
def test_lora_token_reduction(r, T, Mg):
    lib = F.N.require()
    a, b = rnd(T, Mg, scale=0.5), rnd(T, r, seed=1)
    want = a.float().t() @ b.float()
    c0 = F.N.launch_count()
    got = F.lora_wgrad(a, b)
    assert F.N.launch_count() == c0 + 1, "token reduction did not run on the native kernel"
    assert lib.eri_gemm_tokred_check_error() == 0
    assert got.shape == (Mg, r)
    rel_close(got, want, 8e-3)
    got_t = F.lora_wgrad(a, b, transpose_out=True)
    assert got_t.shape == (r, Mg)
    rel_close(got_t, want.t(), 8e-3)
    # accumulation into an existing gradient, twice in a row (the workspace must come back clean)
    for _ in range(2):
        g0 = rnd(r, Mg, seed=5, scale=2.0)
        g = g0.clone()
        F.lora_wgrad(a, b, out=g, transpose_out=True, accumulate=True)
        rel_close(g, g0.float() + want.t(), 8e-3)
    assert lib.eri_gemm_tokred_check_error() == 0


@pytest.mark.parametrize("mode,act_first", [("gelu", False), ("silu", True), ("silu", False), ("gelu", True)])
@pytest.mark.parametrize("M,K,Hd", [(512, 320, 1280), (300, 256, 200), (1024, 640, 2560)])
def test_glu_epilogue(mode, act_first, M, K, Hd):
    x = rnd(M, K)
    w = rnd(2 * Hd, K, seed=1, scale=K ** -0.5)
    bias = rnd(2 * Hd, seed=2)
    pre = torch.full((M, 2 * Hd), float("nan"), device=DEV, dtype=torch.bfloat16)
    code = F._GLU_CODE[(mode, act_first)]
    out = F.gemm_native(x, w, bias=bias, glu=code, pre_out=pre)
    assert F.kernel_error_check() == {}
    h = x.float() @ w.float().t() + bias.float()
    rel_close(pre, h, 8e-3)
    want = R.glu(pre, mode, act_first)          # from the kept halves, as backward sees them
    assert out.shape == (M, Hd)
    rel_close(out, want, 1e-2)


def test_linear_glu_forward_backward_against_unfused(monkeypatch):
    from eridiffusion_b200.models.layers import Linear
    torch.manual_seed(0)
    lin = Linear(320, 2 * 1280, device=DEV)
    with torch.no_grad():
        lin.bias.normal_(0, 0.1)
    x = rnd(2, 256, 320).requires_grad_(True)
    dy = rnd(2, 256, 1280, seed=9)

    def run(fused):
        monkeypatch.setattr(F, "_GLU_FUSED", fused)
        lin.weight.grad = None
        lin.bias.grad = None
        xx = x.detach().clone().requires_grad_(True)
        y = F.linear_glu(xx, lin, "gelu", act_first=False)
        y.backward(dy)
        return y.detach(), xx.grad, lin.weight.grad.clone(), lin.bias.grad.clone()

    yf, dxf, dwf, dbf = run(True)
    yu, dxu, dwu, dbu = run(False)
    assert F.kernel_error_check() == {}
    rel_close(yf, yu, 1e-2)
    rel_close(dxf, dxu, 2e-2)
    rel_close(dwf, dwu, 2e-2)
    rel_close(dbf, dbu, 2e-2)
