"""tcgen05 flash attention against explicit fp32 softmax(QK^T)V."""
import math

import pytest
import torch

from eridiffusion_b200.ops import flash_attn as FA
from eridiffusion_b200.ops import reference as R

pytestmark = pytest.mark.gpu


def mk(B, L, H, D, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(B, L, H, D, device="cuda", generator=g).bfloat16()


@pytest.mark.parametrize("B,H,Lq,Lk,D", [(1, 2, 128, 128, 128), (2, 3, 256, 384, 128), (1, 2, 320, 200, 128),
                                         (1, 4, 1152, 1152, 128), (2, 2, 256, 256, 64), (1, 3, 192, 333, 64)])
def test_flash_fwd(B, H, Lq, Lk, D):
    q, k, v = mk(B, Lq, H, D, 1), mk(B, Lk, H, D, 2), mk(B, Lk, H, D, 3)
    out, lse = FA.fwd(q, k, v)
    torch.cuda.synchronize()
    assert FA.check_error() == 0
    ref = R.attention_fp32(q, k, v)
    err = (out.float() - ref).abs().max().item()
    assert err < 2e-2, err
    s = torch.einsum("blhd,bmhd->bhlm", q.float(), k.float()) / math.sqrt(D)
    lse_ref = torch.logsumexp(s, -1)
    assert (lse - lse_ref).abs().max().item() < 2e-2


def test_flash_large_logits_rescale():
    # scores spread over a wide range so that the lazy rescale path runs
    B, H, L, D = 1, 2, 512, 128
    q, k, v = mk(B, L, H, D, 1) * 4, mk(B, L, H, D, 2) * 4, mk(B, L, H, D, 3)
    out, lse = FA.fwd(q, k, v)
    assert FA.check_error() == 0
    ref = R.attention_fp32(q, k, v)
    assert (out.float() - ref).abs().max().item() < 3e-2


@pytest.mark.parametrize("B,H,Lq,Lk,D", [(1, 2, 256, 256, 128), (2, 2, 384, 256, 128), (1, 2, 320, 200, 128),
                                         (1, 2, 256, 256, 64)])
def test_flash_bwd(B, H, Lq, Lk, D):
    if not FA.has_backward():
        pytest.skip("native backward not in this build")
    q, k, v = mk(B, Lq, H, D, 1), mk(B, Lk, H, D, 2), mk(B, Lk, H, D, 3)
    do = mk(B, Lq, H, D, 4)
    out, lse = FA.fwd(q, k, v)
    dq, dk, dv = FA.bwd(do, q, k, v, out, lse)
    torch.cuda.synchronize()
    assert FA.check_error() == 0
    qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
    ref = R.attention_fp32(qf, kf, vf)
    ref.backward(do.float())
    for a, b, n in ((dq, qf.grad, "dq"), (dk, kf.grad, "dk"), (dv, vf.grad, "dv")):
        err = (a.float() - b).abs().max().item()
        assert err < 0.02 * b.abs().max().item() + 2e-2, (n, err, b.abs().max().item())


def test_flash_attention_into_caller_buffer():
    """``out=``: the forward writes into the caller's buffer (a peer-readable slot under sequence
    parallelism), autograd keeps that buffer for the backward, gradients match the default path."""
    from eridiffusion_b200.ops import functional as F
    q, k, v = (mk(1, 384, 2, 128, s).requires_grad_() for s in (11, 12, 13))
    go = mk(1, 384, 2, 128, 14)
    ref = F.attention(q, k, v)
    gref = torch.autograd.grad(ref, (q, k, v), go)
    buf = torch.full_like(q, float("nan")).detach()
    out = F.attention(q, k, v, out=buf)
    assert out.data_ptr() == buf.data_ptr() and torch.equal(out, ref)
    got = torch.autograd.grad(out, (q, k, v), go)
    for a, b in zip(gref, got):
        assert torch.equal(a, b)
    with pytest.raises(ValueError):
        F.attention(q, k, v, out=buf[:, :128])
    assert FA.check_error() == 0


@pytest.mark.parametrize("B,L,H,D", [(1, 384, 2, 128), (2, 300, 4, 64)])
def test_flash_output_as_column_block_of_a_wider_matrix(B, L, H, D):
    """The forward writes its output into the left column block of a wider row-major matrix (the input of
    a single-stream block's second linear) and the backward reads it there: bit-equal to the contiguous
    path, and the columns to the right stay untouched."""
    q, k, v = (mk(B, L, H, D, s) for s in (21, 22, 23))
    go = mk(B, L, H, D, 24)
    o_ref, lse_ref = FA.fwd(q, k, v)
    wide = torch.full((B * L, H * D + 136), 7.0, device="cuda", dtype=torch.bfloat16)
    view = wide.view(B, L, H * D + 136)[:, :, : H * D].unflatten(-1, (H, D))
    o, lse = FA.fwd(q, k, v, out=view)
    assert o.data_ptr() == wide.data_ptr() and torch.equal(o, o_ref) and torch.equal(lse, lse_ref)
    assert (wide[:, H * D:] == 7.0).all()
    for a, b in zip(FA.bwd(go, q, k, v, o_ref, lse_ref), FA.bwd(go, q, k, v, o, lse)):
        assert torch.equal(a, b)
    with pytest.raises(ValueError):                       # heads not packed inside a token
        FA.fwd(q, k, v, out=torch.empty(B, H, L, D, device="cuda", dtype=torch.bfloat16).transpose(1, 2))
    assert FA.check_error() == 0


def _ref_masked(q, k, v, bias):
    """fp32 softmax(QK^T / sqrt(D) + bias[b, key]) V with autograd, bias [B, Lk] additive."""
    D = q.shape[-1]
    s = torch.einsum("blhd,bmhd->bhlm", q, k) / math.sqrt(D) + bias[:, None, None, :]
    return torch.einsum("bhlm,bmhd->blhd", torch.softmax(s, -1), v)


@pytest.mark.parametrize("B,H,Lq,Lk,D", [(2, 2, 256, 384, 128), (2, 3, 200, 333, 64), (1, 2, 640, 640, 128)])
@pytest.mark.parametrize("kind", ["bool", "additive"])
def test_flash_key_padding_mask_fwd_bwd(B, H, Lq, Lk, D, kind):
    """Text-padding style key masks ([B, 1, 1, Lk]): per-sample valid prefixes in the middle of a joint
    sequence, forward and all three gradients against fp32; masked keys get zero gradient."""
    from eridiffusion_b200.ops import functional as F
    q, k, v = (mk(B, L, H, D, s).requires_grad_() for L, s in ((Lq, 1), (Lk, 2), (Lk, 3)))
    do = mk(B, Lq, H, D, 4)
    # keys [lo_b, 96) are padding (a whole first tile stays partly visible; for the last sample a
    # 128-key tile is masked completely when Lk allows it)
    visible = torch.ones(B, Lk, dtype=torch.bool, device="cuda")
    for b in range(B):
        visible[b, 17 + 31 * b:96] = False
    if Lk >= 384:
        visible[B - 1, 128:256] = False
    if kind == "bool":
        mask = visible[:, None, None, :]
    else:
        mask = torch.where(visible, 0.0, float("-inf"))[:, None, None, :]
        mask = mask + 0.25 * torch.randn(B, 1, 1, Lk, device="cuda") * visible[:, None, None, :]
    out = F.attention(q, k, v, mask=mask)
    gq, gk, gv = torch.autograd.grad(out, (q, k, v), do)
    assert FA.check_error() == 0
    bias = torch.where(visible, 0.0, -1e30) if kind == "bool" else mask.reshape(B, Lk).clamp_min(-1e30)
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = _ref_masked(qf, kf, vf, bias.float())
    ref.backward(do.float())
    assert (out.float() - ref).abs().max().item() < 2e-2
    for a, b_, n in ((gq, qf.grad, "dq"), (gk, kf.grad, "dk"), (gv, vf.grad, "dv")):
        err = (a.float() - b_).abs().max().item()
        assert err < 0.02 * b_.abs().max().item() + 2e-2, (n, err)
    hidden = ~visible
    assert gk.float()[hidden].abs().max().item() == 0.0 and gv.float()[hidden].abs().max().item() == 0.0


@pytest.mark.parametrize("B,H,Lq,Lk,D", [(2, 10, 1024, 77, 64), (1, 20, 256, 77, 64), (1, 2, 200, 1, 128),
                                         (1, 4, 130, 127, 128)])
def test_flash_short_keys_cross_attention(B, H, Lq, Lk, D):
    """Fewer than 128 keys (SDXL cross-attention over 77 text tokens) stay on the native kernels."""
    from eridiffusion_b200.ops import functional as F
    q, k, v = (mk(B, L, H, D, s).requires_grad_() for L, s in ((Lq, 1), (Lk, 2), (Lk, 3)))
    do = mk(B, Lq, H, D, 4)
    c0 = F.N.launch_count()
    out = F.attention(q, k, v)
    assert F.N.launch_count() > c0, "short-key attention left the native path"
    gq, gk, gv = torch.autograd.grad(out, (q, k, v), do)
    assert FA.check_error() == 0
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = R.attention_fp32(qf, kf, vf)
    ref.backward(do.float())
    assert (out.float() - ref).abs().max().item() < 2e-2
    for a, b_, n in ((gq, qf.grad, "dq"), (gk, kf.grad, "dk"), (gv, vf.grad, "dv")):
        err = (a.float() - b_).abs().max().item()
        assert err < 0.02 * b_.abs().max().item() + 2e-2, (n, err)


def test_flash_headline_shape_against_fp32():
    """The benchmark's attention call (B1, 4608 tokens, 24 heads of 128): 36 key tiles per query tile,
    forward and backward against fp32, head by head to bound the reference's memory."""
    B, L, H, D = 1, 4608, 24, 128
    q, k, v, do = (mk(B, L, H, D, s) for s in (1, 2, 3, 4))
    out, lse = FA.fwd(q, k, v)
    dq, dk, dv = FA.bwd(do, q, k, v, out, lse)
    assert FA.check_error() == 0
    worst = {}
    for h in range(0, H, 5):
        qf, kf, vf = (t[:, :, h:h + 1].float().requires_grad_() for t in (q, k, v))
        ref = R.attention_fp32(qf, kf, vf)
        ref.backward(do[:, :, h:h + 1].float())
        for name, got, want in (("out", out, ref.detach()), ("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad)):
            rel = (got[:, :, h:h + 1].float() - want).abs().max().item() / want.abs().max().item()
            worst[name] = max(worst.get(name, 0.0), rel)
    assert worst["out"] < 1.5e-2 and worst["dq"] < 2.5e-2 and worst["dk"] < 2.5e-2 and worst["dv"] < 2.5e-2, worst


@pytest.mark.parametrize("B,H,Lq,Lk", [(1, 2, 256, 128), (2, 3, 512, 384), (1, 2, 640, 333), (1, 4, 1152, 1152), (1, 2, 300, 256)])
def test_flash_fwd_cta_pair_kernel(B, H, Lq, Lk):
    """The CTA-pair forward (two CTAs share every K / V tile) against fp32 and against the one-CTA
    kernel, including query counts that leave the pair's second tile partly or wholly empty."""
    assert FA.pair_forward_ok(torch.device("cuda", 0), force=True), "the CTA-pair forward failed its self-check"
    lib = FA.N.require()
    q, k, v = mk(B, Lq, H, 128, 1), mk(B, Lk, H, 128, 2), mk(B, Lk, H, 128, 3)
    out = torch.full_like(q, float("nan"))
    lse = torch.empty(B, H, Lq, dtype=torch.float32, device="cuda")
    code = FA._pair_call(lib, q, k, v, out, lse, 1.0 / math.sqrt(128))
    assert code == 0
    torch.cuda.synchronize()
    assert FA.check_error() == 0
    ref = R.attention_fp32(q, k, v)
    assert (out.float() - ref).abs().max().item() < 2e-2
    s = torch.einsum("blhd,bmhd->bhlm", q.float(), k.float()) / math.sqrt(128)
    assert (lse - torch.logsumexp(s, -1)).abs().max().item() < 2e-2


@pytest.mark.parametrize("Dh,Lq,Lk", [(40, 1024, 1024), (80, 256, 256), (40, 1024, 77), (80, 320, 77)])
def test_other_head_sizes_ride_on_the_native_kernels(Dh, Lq, Lk):
    """SD1.5 head sizes (40 at 64 x 64, 80 at 32 x 32; self- and 77-key cross-attention): zero-padded to
    64 / 128 columns for the tcgen05 kernels; output and gradients equal fp32 attention at the true size."""
    from eridiffusion_b200.ops import functional as F
    B, H = 2, 8
    q, k, v = mk(B, Lq, H, Dh, 1), mk(B, Lk, H, Dh, 2), mk(B, Lk, H, Dh, 3)
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    n0 = F.ATTENTION_CALLS["native"]
    o = F.attention(q, k, v)
    assert F.ATTENTION_CALLS["native"] == n0 + 1 and o.shape == q.shape and o.is_contiguous()
    do = mk(B, Lq, H, Dh, 4)
    o.backward(do)
    assert FA.check_error() == 0
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = R.attention_fp32(qr, kr, vr)
    ref.backward(do.float())
    rel = lambda a, b: (a.float() - b).abs().max().item() / b.abs().max().item()
    assert rel(o, ref) < 1.5e-2
    assert rel(q.grad, qr.grad) < 2.5e-2 and rel(k.grad, kr.grad) < 2.5e-2 and rel(v.grad, vr.grad) < 2.5e-2
