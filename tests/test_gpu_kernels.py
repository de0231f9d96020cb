"""Numerics of every CUDA kernel against the plain PyTorch fp32 statement of the same op."""
import math

import pytest
import torch

from eridiffusion_b200.ops import functional as F
from eridiffusion_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def rnd(*s, scale=1.0, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed + sum(s))
    return (torch.randn(*s, device=DEV, generator=g) * scale).to(BF)


def close(a, b, atol, rtol=2e-2, rel_to_max=0.0):
    """|a-b| <= atol + rel_to_max*max|b| + rtol*|b| elementwise (bf16 pipelines carry an absolute
    error proportional to the tensor's scale, not to each element)."""
    a, b = a.float(), b.float()
    assert a.shape == b.shape
    err = (a - b).abs()
    tol = atol + rel_to_max * b.abs().max() + rtol * b.abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4g} (allowed {tol.max().item():.4g})"


@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("D", [256, 3072, 4096 + 8])
def test_norm_modulate_fwd_bwd(rms, D):
    B, L = 2, 67
    x = rnd(B, L, D).requires_grad_()
    mod = rnd(B, 3 * D, scale=0.3).requires_grad_()
    w = rnd(D, scale=0.5).requires_grad_()
    sh, sc, _ = mod.split(D, dim=-1)
    y = F.norm_modulate(x, sc, sh, w, None, 1e-6, rms)
    xr, modr, wr = (t.detach().float().requires_grad_() for t in (x, mod, w))
    shr, scr, _ = modr.split(D, dim=-1)
    yr = R.norm_modulate(xr, scr, shr, wr, None, 1e-6, rms)
    close(y, yr, 3e-2)
    g = rnd(B, L, D, seed=5)
    y.backward(g)
    yr.backward(g.float())
    close(x.grad, xr.grad, 3e-2, 3e-2)
    # parameter gradients are sums over B * L rows: bounded relative to the fp32 reference's own
    # magnitude (measured: worst element 0.37 % of |ref| + 1 % of max|ref|)
    close(mod.grad, modr.grad, 0.0, 1e-2, rel_to_max=1e-2)
    close(w.grad, wr.grad, 0.0, 1e-2, rel_to_max=1e-2)


@pytest.mark.parametrize("variant", [1, 0])
@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("L,D", [(67, 256), (2500, 3072), (5000, 264), (700, 4096), (9000, 3072)])
def test_norm_modulate_row_kernels(rms, L, D, variant):
    """Input-gradient-only case (frozen modulation and weight): the persistent warp-per-row
    kernels fed by bulk copies, rows resident in shared memory (variant 1) or in registers (0); the
    long cases make every warp cycle its row buffers several times. The rows carry a mean of several
    standard deviations, which the shifted one-pass statistics of variant 1 must survive."""
    lib = F.N.require()
    prev = lib.eri_norm_set_smem_variant(variant)
    try:
        _norm_rows_case(rms, L, D)
    finally:
        lib.eri_norm_set_smem_variant(prev)


@pytest.mark.parametrize("rms", [False, True])
def test_norm_modulate_skip_adds_the_residual_gradient_in_the_kernel(rms, request):
    """``norm_modulate_skip`` returns the normalised tensor and its input for the residual branch; the backward
    kernel adds the gradient of that branch to dx. Same result as the two-branch formulation left to autograd."""
    B, L, D = 2, 700, 3072
    x0 = (rnd(B, L, D) + 1.5).bfloat16()
    mod = rnd(B, 2 * D, scale=0.3)
    sh, sc = mod.split(D, dim=-1)
    g1, g2 = rnd(B, L, D, seed=5), rnd(B, L, D, seed=6)

    F._NORM_SKIP, old_skip = True, F._NORM_SKIP            # opt-in switch (ERI_B200_NORM_SKIP)
    request.addfinalizer(lambda: setattr(F, "_NORM_SKIP", old_skip))

    def run(skip):
        x = x0.clone().requires_grad_()
        if skip:
            y, xr = F.norm_modulate_skip(x, sc, sh, None, None, 1e-6, rms)
            assert xr.data_ptr() == x.data_ptr()
        else:
            y, xr = F.norm_modulate(x, sc, sh, None, None, 1e-6, rms), x
        c0 = F.N.launch_count()
        ((y.float() * g1.float()).sum() + (xr.float() * g2.float()).sum()).backward()
        return y.detach().float(), x.grad.float(), F.N.launch_count() - c0
    y1, d1, n1 = run(True)
    y0, d0, n0 = run(False)
    assert torch.equal(y1, y0) and n1 == n0 == 1
    close(d1, d0, 2e-2, 2e-2)
    xr = x0.float().requires_grad_()
    yr = R.norm_modulate(xr, sc.float(), sh.float(), None, None, 1e-6, rms)
    ((yr * g1.float()).sum() + (xr * g2.float()).sum()).backward()
    close(d1, xr.grad, 3e-2, 3e-2)
    # only the residual branch has a gradient: it passes through untouched
    x = x0.clone().requires_grad_()
    y, xs = F.norm_modulate_skip(x, sc, sh, None, None, 1e-6, rms)
    (xs.float() * g2.float()).sum().backward()
    assert torch.equal(x.grad, g2)
    assert F.kernel_error_check() == {}


def _norm_rows_case(rms, L, D):
    B = 2
    x = (rnd(B, L, D) + 4.0).bfloat16().requires_grad_()
    mod = rnd(B, 2 * D, scale=0.3)
    w = rnd(D, scale=0.5)
    sh, sc = mod.split(D, dim=-1)
    y = F.norm_modulate(x, sc, sh, w, None, 1e-6, rms)
    xr = x.detach().float().requires_grad_()
    yr = R.norm_modulate(xr, sc.float(), sh.float(), w.float(), None, 1e-6, rms)
    close(y, yr, 3e-2)
    g = rnd(B, L, D, seed=5)
    y.backward(g)
    yr.backward(g.float())
    close(x.grad, xr.grad, 3e-2, 3e-2)
    assert F.kernel_error_check() == {}


@pytest.mark.parametrize("Dh", [64, 128])
def test_qknorm_rope_joint(Dh):
    B, H, Lt, Li = 2, 4, 24, 40
    D = H * Dh
    cos = torch.cos(torch.rand(Lt + Li, Dh // 2, device=DEV) * 6)
    sin = torch.sin(torch.rand(Lt + Li, Dh // 2, device=DEV) * 6)
    ins = [rnd(B, Lt, 3 * D).requires_grad_(), rnd(B, Li, 3 * D, seed=1).requires_grad_()]
    scales = [rnd(Dh, scale=0.5, seed=i).add(1).requires_grad_() for i in range(4)]
    q, k, v = F.qknorm_rope_joint([(ins[0], scales[0], scales[1]), (ins[1], scales[2], scales[3])], cos, sin, H)
    insr = [t.detach().float().requires_grad_() for t in ins]
    scr = [t.detach().float().requires_grad_() for t in scales]
    o0 = R.qknorm_rope(insr[0], scr[0], scr[1], cos[:Lt], sin[:Lt], H)
    o1 = R.qknorm_rope(insr[1], scr[2], scr[3], cos[Lt:], sin[Lt:], H)
    qr, kr, vr = (torch.cat([a, b], 1) for a, b in zip(o0, o1))
    close(q, qr, 3e-2); close(k, kr, 3e-2); close(v, vr, 1e-6)
    gq, gk, gv = rnd(*q.shape, seed=7), rnd(*q.shape, seed=8), rnd(*q.shape, seed=9)
    torch.autograd.backward([q, k, v], [gq, gk, gv])
    torch.autograd.backward([qr, kr, vr], [gq.float(), gk.float(), gv.float()])
    for a, b in zip(ins, insr):
        close(a.grad, b.grad, 4e-2, 3e-2)
    for a, b in zip(scales, scr):
        close(a.grad, b.grad, 0.0, 1e-2, rel_to_max=1e-2)


def test_gate_residual_and_acts():
    B, L, D = 2, 33, 512
    x, y = rnd(B, L, D).requires_grad_(), rnd(B, L, D, seed=1).requires_grad_()
    gate = rnd(B, D, scale=0.5).requires_grad_()
    out = F.gate_residual(x, y, gate)
    xr, yr, gr = (t.detach().float().requires_grad_() for t in (x, y, gate))
    outr = R.gate_residual(xr, yr, gr)
    close(out, outr, 2e-2)
    g = rnd(B, L, D, seed=3)
    out.backward(g); outr.backward(g.float())
    close(x.grad, xr.grad, 1e-2); close(y.grad, yr.grad, 2e-2); close(gate.grad, gr.grad, 0.0, 1e-2, rel_to_max=1e-2)
    for fn, rf in ((F.gelu_tanh, R.gelu_tanh), (F.silu, R.silu)):
        a = rnd(4, 1024).requires_grad_()
        ar = a.detach().float().requires_grad_()
        o, orf = fn(a), rf(ar)
        close(o, orf, 1e-2)
        o.backward(g.view(-1)[:4096].view(4, 1024)); orf.backward(g.view(-1)[:4096].view(4, 1024).float())
        close(a.grad, ar.grad, 2e-2)
    for mode in ("gelu", "silu"):
        for af in (True, False):
            h = rnd(5, 7, 256).requires_grad_()
            hr = h.detach().float().requires_grad_()
            o, orf = F.glu(h, mode, af), R.glu(hr, mode, af)
            close(o, orf, 2e-2)
            gg = rnd(5, 7, 128, seed=4)
            o.backward(gg); orf.backward(gg.float())
            close(h.grad, hr.grad, 3e-2)


def test_noise_mix_and_mse():
    B, C, H, W = 2, 16, 32, 32
    x0 = rnd(B, C, H, W)
    eps = rnd(B, C, H, W, seed=3)
    t = torch.tensor([0.3, 0.8], device=DEV)
    coef = torch.stack([1 - t, t, torch.ones_like(t), -torch.ones_like(t)])
    xt, tg = F.noise_mix(x0, coef, seed=1, eps=eps)
    xtr, tgr = R.noise_mix(x0, eps, coef)
    close(xt, xtr, 1e-2); close(tg, tgr, 1e-2)
    xt2, tg2, e2 = F.noise_mix(x0, coef, seed=11, offset=5, want_eps=True)
    e = e2.float()
    assert abs(e.mean().item()) < 0.02 and abs(e.std().item() - 1.0) < 0.02
    xt3, _, e3 = F.noise_mix(x0, coef, seed=11, offset=5, want_eps=True)
    assert torch.equal(e2, e3)
    pred = rnd(B, 256, 64).requires_grad_()
    w = torch.tensor([0.5, 2.0], device=DEV)
    loss = F.mse_loss(pred, tg, w)
    pr = pred.detach().float().requires_grad_()
    lr_ = R.mse(pr, tg, w)
    assert abs(loss.item() - lr_.item()) < 1e-3 * max(1.0, lr_.item())
    loss.backward(); lr_.backward()
    close(pred.grad, pr.grad, 1e-6, 2e-2)


def _gemm_ref(a, b, **kw):
    return a.float() @ b.float().t()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (512, 3072, 3072), (300, 384, 136),
                                   (4096, 256, 1024), (256, 64, 128), (384, 16, 512)])
def test_gemm_plain(M, N, K):
    a, b = rnd(M, K), rnd(N, K, seed=1)
    out = F.gemm_native(a, b)
    torch.cuda.synchronize()
    assert F.gemm_error_check() == 0
    close(out, _gemm_ref(a, b), 0.05 * math.sqrt(K / 64), 2e-2)


@pytest.mark.parametrize("bn", [256, 128, 64])
def test_gemm_tile_variants(bn):
    M, N, K = 640, 1024, 512
    a, b = rnd(M, K), rnd(N, K, seed=1)
    out = F.gemm_native(a, b, force_bn=bn)
    assert F.gemm_error_check() == 0
    close(out, _gemm_ref(a, b), 0.15, 2e-2)


@pytest.mark.parametrize("r", [16, 32, 64])
def test_gemm_lora_epilogues(r):
    B, L, K, N = 2, 192, 512, 768
    M = B * L
    x, w, bias = rnd(M, K), rnd(N, K, scale=K ** -0.5, seed=1), rnd(N, seed=2)
    A, Bm = rnd(r, K, scale=K ** -0.5, seed=3), rnd(N, r, scale=0.1, seed=4)
    res, gate = rnd(M, N, seed=5), rnd(B, N, seed=6)
    s = 0.5
    h = F.gemm_native(x, A, alpha=s)
    close(h, (x.float() @ A.float().t()) * s, 0.03)
    pre = torch.empty(M, N, device=DEV, dtype=BF)
    y = F.gemm_native(x, w, bias=bias, lora_h=h, lora_b=Bm, act="gelu", pre_out=pre, residual=res,
                      gate=gate, rows_per_batch=L)
    assert F.gemm_error_check() == 0
    pre_ref = x.float() @ w.float().t() + bias.float() + h.float() @ Bm.float().t()
    close(pre, pre_ref, 0.05)
    y_ref = res.float() + gate.float().repeat_interleave(L, 0) * torch.nn.functional.gelu(pre_ref, approximate="tanh")
    close(y, y_ref, 0.06)
    # activation backward epilogue + column split
    dy = rnd(M, N, seed=8)
    wt = rnd(K, N, scale=N ** -0.5, seed=9)
    n_split = 256
    out1 = torch.empty(M, n_split, device=DEV, dtype=BF)
    out2 = torch.empty(M, K - n_split, device=DEV, dtype=BF)
    pre2 = rnd(M, K - n_split, seed=10)
    F.gemm_native(dy, wt, out=out1, out2=out2, n_split=n_split, act="gelu_bwd", pre_in=pre2)
    assert F.gemm_error_check() == 0
    full = dy.float() @ wt.float().t()
    close(out1, full[:, :n_split], 0.06)
    pf = pre2.float().requires_grad_()
    gd = torch.autograd.grad(torch.nn.functional.gelu(pf, approximate="tanh").sum(), pf)[0]
    close(out2, full[:, n_split:] * gd, 0.06)


def test_fused_linear_autograd_matches_reference():
    B, L, K, N, r = 2, 128, 256, 384, 16
    x = rnd(B, L, K).requires_grad_()
    w, bias = rnd(N, K, scale=K ** -0.5, seed=1), rnd(N, seed=2)
    A = rnd(r, K, scale=K ** -0.5, seed=3).requires_grad_()
    Bm = rnd(N, r, scale=0.2, seed=4).requires_grad_()
    res, gate = rnd(B, L, N, seed=5).requires_grad_(), rnd(B, N, seed=6)
    y = F.linear(x, w, bias, lora=(A, Bm, 2.0), act="gelu", residual=res, gate=gate, wt=w.t().contiguous())
    xr, Ar, Br, rr = (t.detach().float().requires_grad_() for t in (x, A, Bm, res))
    yr = R.linear(xr, w.float(), bias.float(), (Ar, Br, 2.0), "gelu", rr, gate.float())
    close(y, yr, 0.06)
    g = rnd(B, L, N, seed=7)
    y.backward(g); yr.backward(g.float())
    assert F.gemm_error_check() == 0
    close(x.grad, xr.grad, 0.02, 3e-2, rel_to_max=0.02)
    close(res.grad, rr.grad, 1e-2)
    close(A.grad, Ar.grad, 0.05, 3e-2, rel_to_max=0.02)
    close(Bm.grad, Br.grad, 0.05, 3e-2, rel_to_max=0.02)


def test_small_linear():
    x, w, b = rnd(2, 3072), rnd(1024, 3072, scale=0.02, seed=1), rnd(1024, seed=2)
    y = F.small_linear(x, w, b, silu_in=True)
    yr = torch.nn.functional.linear(torch.nn.functional.silu(x.float()), w.float(), b.float())
    close(y, yr, 0.03)


@pytest.fixture(params=[1, 0], ids=["pair-kernel", "element-kernel"])
def adamw8_variant(request):
    """Both 8-bit AdamW kernels: packed pairs (the default) and the element-wise one."""
    lib = F.N.require()
    prev = lib.eri_adamw8bit_set_pair_variant(request.param)
    yield request.param
    lib.eri_adamw8bit_set_pair_variant(prev)


def test_adamw8bit_stochastic_rounding_is_unbiased(adamw8_variant):
    """One step from p = 1 with a constant gradient moves every element to 1 - 2^-10, a quarter of the
    way down to the next bf16 value (1 - 2^-8): round-to-nearest leaves all of them at 1, stochastic
    rounding puts a quarter of them on the lower value, so that the mean keeps the update."""
    from eridiffusion_b200.optim import AdamW8bit
    n = 256 * 1024
    for stochastic in (False, True):
        p = [torch.nn.Parameter(torch.ones(n, device="cuda", dtype=torch.bfloat16))]
        opt = AdamW8bit(p, lr=2.0 ** -10, weight_decay=0.0, stochastic_rounding=stochastic)
        opt.arena.grad.fill_(1.0)
        opt.step()
        got = opt.arena.data[:n].float()
        if not stochastic:
            assert (got == 1.0).all()
            continue
        lower = (got == 1.0 - 2.0 ** -8)
        assert ((got == 1.0) | lower).all()
        frac = lower.float().mean().item()
        assert abs(frac - 0.25) < 0.01, frac                       # sigma = 0.00085
        assert abs(got.mean().item() - (1.0 - 2.0 ** -10)) < 4e-5
        # neighbouring elements share one hash (its two halves): they must still be independent
        both = (lower[0::2] & lower[1::2]).float().mean().item()
        assert abs(both - 0.0625) < 0.005, both


def test_adamw8bit_kernel_matches_reference(adamw8_variant):
    from eridiffusion_b200.optim import AdamW8bit
    torch.manual_seed(0)
    p1 = [torch.nn.Parameter(rnd(1000, 33)), torch.nn.Parameter(rnd(4099, seed=1))]
    p2 = [torch.nn.Parameter(p.detach().clone()) for p in p1]
    o1 = AdamW8bit(p1, lr=1e-2, stochastic_rounding=False)
    o2 = AdamW8bit(p2, lr=1e-2, stochastic_rounding=False)
    for s in range(5):
        g = rnd(o1.arena.numel, seed=100 + s)
        o1.arena.grad.copy_(g); o2.arena.grad.copy_(g)
        ss = F.sumsq(o1.arena.grad)
        o1.step(grad_sumsq=ss, max_grad_norm=1.0)
        F.set_backend("eager")
        try:
            o2.step(grad_sumsq=ss, max_grad_norm=1.0)
        finally:
            F.set_backend("fused")
    close(o1.arena.data, o2.arena.data, 2e-2, 2e-2)
    m1, v1 = o1.export_moments(); m2, v2 = o2.export_moments()
    close(m1, m2, 1e-4, 5e-2); close(v1, v2, 1e-7, 0.1)
    assert abs(ss.sqrt().item() - o1.arena.grad.float().norm().item()) < 1e-2 * ss.sqrt().item()


def test_adamw8bit_moments_track_fp32_adamw_over_hundreds_of_steps(adamw8_variant):
    """The 8-bit kernel (fast-math build, shared square root, magic-number rounding) against a plain
    fp32 AdamW over 300 steps of a gradient stream with a persistent component: the moments stay
    within the quantisation error of their block and the parameter trajectory does not drift."""
    from eridiffusion_b200.optim import AdamW8bit
    torch.manual_seed(0)
    n = 64 * 1024
    p = [torch.nn.Parameter(torch.zeros(n, device="cuda", dtype=torch.bfloat16))]
    opt = AdamW8bit(p, lr=1e-3, weight_decay=0.0, stochastic_rounding=False)
    pf = torch.zeros(opt.arena.numel, device="cuda")
    m = torch.zeros_like(pf); v = torch.zeros_like(pf)
    g_gen = torch.Generator(device="cuda").manual_seed(1)
    drift = torch.randn(opt.arena.numel, device="cuda", generator=g_gen) * 0.5
    b1, b2, eps, lr = 0.9, 0.999, 1e-8, 1e-3
    for s in range(1, 301):
        g = (drift + torch.randn(opt.arena.numel, device="cuda", generator=g_gen)).bfloat16()
        opt.arena.grad.copy_(g)
        opt.step()
        gf = g.float()
        m = b1 * m + (1 - b1) * gf
        v = b2 * v + (1 - b2) * gf * gf
        pf = pf - lr * (m / (1 - b1 ** s)) / ((v / (1 - b2 ** s)).sqrt() + eps)
    m8, v8 = opt.export_moments()
    # per 256-element block the codes resolve (k/127)^2 and (k/255)^4 of the block maximum
    mb = m.view(-1, 256).abs().amax(1, keepdim=True)
    vb = v.view(-1, 256).amax(1, keepdim=True)
    em = ((m8.view(-1, 256) - m.view(-1, 256)).abs() / mb).max().item()
    ev = ((v8.view(-1, 256) - v.view(-1, 256)).abs() / vb).max().item()
    ev_mean = ((v8.view(-1, 256) - v.view(-1, 256)).abs() / vb).mean().item()
    got = opt.arena.data.float()
    rel = (got - pf).norm().item() / pf.norm().item()
    cos = torch.nn.functional.cosine_similarity(got, pf, dim=0).item()
    print(f"adamw8bit drift after 300 steps: m {em:.4f} v max {ev:.4f} mean {ev_mean:.4f} of the block maximum; "
          f"parameters rel {rel:.4f} cos {cos:.5f}")
    # The codes resolve 0.8 % (m) and 1.6 % (v) of the block maximum at the top of their range. The
    # block maximum itself is kept exactly in fp32, so a block follows its collective growth or decay;
    # what the 8-bit codes lose is a change of one element RELATIVE to its block that is smaller than
    # half a code step per update (beta2 = 0.999 moves v by 0.1 % of (g^2 - v) per step): such an
    # element waits for a larger gradient before its code moves. Measured on B200 after 300 steps:
    # m 0.031, v 0.123 worst element / 0.024 mean, of the block maximum.
    assert em < 0.04 and ev < 0.15 and ev_mean < 0.03, (em, ev, ev_mean)
    # the sticky codes of v lean high (a spike moves a code up at once, the slow decay is lost until it
    # adds up to half a step), so the 8-bit run's steps are a few per cent shorter than fp32 AdamW's:
    # measured 0.064 relative distance between the two parameter vectors after 300 steps, cosine 0.9985
    assert rel < 0.08 and cos > 0.998, (rel, cos)


@pytest.mark.parametrize("T,N,K", [(1, 18432, 3072), (2, 1536, 256), (8, 777, 264), (3, 100000, 64)])
def test_small_linear_backward_kernels(T, N, K):
    """Weight and input gradients of the conditioning-vector linears (T <= 8 rows) on their own
    kernels, against fp32; the linear's autograd path uses them."""
    dy, x, w = rnd(T, N, scale=0.5), rnd(T, K, seed=1), rnd(N, K, scale=0.05, seed=2)
    c0 = F.N.launch_count()
    dw = F.small_wgrad(dy, x, 0.5)
    dx = F.small_dgrad(dy, w)
    assert F.N.launch_count() == c0 + 2, "the small-M backward left the native path"
    close(dw, 0.5 * dy.float().t() @ x.float(), 0.0, 1e-2, rel_to_max=1e-2)
    close(dx, dy.float() @ w.float(), 0.0, 1e-2, rel_to_max=1e-2)
    # through autograd (SiLU on the input, bias)
    xg, wg, b = x.clone().requires_grad_(), w.clone().requires_grad_(), rnd(N, seed=3).requires_grad_()
    if T * K <= 50000:
        y = F.small_linear(xg, wg, b, silu_in=True)
        y.backward(dy)
        xr, wr, br = (t.detach().float().requires_grad_() for t in (xg, wg, b))
        torch.nn.functional.linear(torch.nn.functional.silu(xr), wr, br).backward(dy.float())
        close(xg.grad, xr.grad, 0.0, 2e-2, rel_to_max=1e-2)
        close(wg.grad, wr.grad, 0.0, 2e-2, rel_to_max=1e-2)
        close(b.grad, br.grad, 0.0, 2e-2, rel_to_max=1e-2)
