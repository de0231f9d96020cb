"""Slice gather / slice-gradient kernels and the ring-attention slice products on the GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16, torch.uint8, torch.float64])
def test_narrow_copy_contiguous_and_strided(dtype):
    from eridiffusion_b200.ops.narrow import narrow_copy_raw
    dev = _cuda()
    x = (torch.randn(3, 37, 5, 24, device=dev) * 50).to(dtype)
    for dim, start, length in ((1, 5, 11), (0, 1, 2), (3, 8, 16), (3, 3, 7), (2, 0, 5), (1, 36, 1), (1, 4, 0)):
        got = narrow_copy_raw(x, dim, start, length)
        assert got.is_contiguous() and torch.equal(got, x.narrow(dim, start, length))
    xt = x.permute(2, 0, 3, 1)[:, :, ::2]                        # non-contiguous source, rank 4
    for dim, start, length in ((0, 1, 3), (2, 2, 9), (3, 30, 7)):
        assert torch.equal(narrow_copy_raw(xt, dim, start, length), xt.narrow(dim, start, length))
    y = torch.arange(2 ** 8, device=dev, dtype=torch.float32).view(2, 2, 2, 2, 2, 2, 2, 2).transpose(0, 7)
    assert torch.equal(narrow_copy_raw(y, 4, 1, 1), y.narrow(4, 1, 1))   # rank 8


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_narrow_backward_add_matches_fp32(dtype):
    from eridiffusion_b200.ops.narrow import narrow_backward_add, narrow_copy
    dev = _cuda()
    torch.manual_seed(0)
    for shape, dim, start, length in (((4, 33, 64), 1, 7, 20), ((4, 33, 63), 1, 0, 33), ((6, 40), 0, 2, 3),
                                      ((2, 5, 9, 16), 2, 4, 5)):
        gin = torch.randn(shape, device=dev).to(dtype)
        gshape = list(shape); gshape[dim] = length
        gout = torch.randn(gshape, device=dev).to(dtype)
        want = gin.float().clone()
        want.narrow(dim, start, length).add_(gout.float())
        got = narrow_backward_add(gout, gin.clone(), dim, start)
        assert torch.allclose(got.float(), want.to(dtype).float(), atol=0, rtol=0), (shape, dim)
    # strided destination
    base = torch.randn(8, 20, 12, device=dev).to(dtype)
    view = base.transpose(0, 2)                                   # [12, 20, 8]
    gout = torch.randn(12, 6, 8, device=dev).to(dtype)
    want = base.float().clone()
    want.transpose(0, 2).narrow(1, 3, 6).add_(gout.float())
    narrow_backward_add(gout, view, 1, 3)
    assert torch.equal(base.float(), want.to(dtype).float())
    # autograd: gradient of the dense slice is the padded upstream gradient
    x = torch.randn(4, 32, 16, device=dev, dtype=dtype, requires_grad=True)
    narrow_copy(x, 1, 8, 8).float().square().sum().backward()
    ref = torch.zeros_like(x)
    ref[:, 8:16] = (2 * x.detach()[:, 8:16].float()).to(dtype)
    assert torch.equal(x.grad, ref)


def test_ring_attention_slices_on_flash_kernels():
    """The slice products behind ring attention run on the native flash kernels; merged over two
    key slices they equal fp32 attention over the whole sequence, forward and gradients."""
    from eridiffusion_b200.ops import flash_attn as FA
    from eridiffusion_b200.ops.reference import attention_fp32
    from eridiffusion_b200.parallel import ring_attention as RA
    dev = _cuda()
    torch.manual_seed(1)
    B, L, H, D = 1, 512, 2, 128
    q, k, v, do = (torch.randn(B, L, H, D, device=dev, dtype=torch.bfloat16) for _ in range(4))
    ks, vs = k.split(256, dim=1), v.split(256, dim=1)
    ks, vs = [t.contiguous() for t in ks], [t.contiguous() for t in vs]
    assert RA._use_native(q, ks[0], vs[0])
    scale = D ** -0.5
    out, lse = RA.block_forward(q, ks[0], vs[0], scale)
    out, lse = RA.merge(out, lse, *RA.block_forward(q, ks[1], vs[1], scale))
    qq, kk, vv = (t.float().requires_grad_() for t in (q, k, v))
    ref = attention_fp32(qq, kk, vv, scale)
    ref.backward(do.float())
    assert (out - ref).abs().max() < 2e-2
    dq = torch.zeros_like(out)
    dks, dvs = [], []
    for i in range(2):
        a, b, c = RA.block_backward(do, q, ks[i], vs[i], out.to(torch.bfloat16), lse, scale)
        dq += a; dks.append(b); dvs.append(c)
    for have, want in ((dq, qq.grad), (torch.cat(dks, 1), kk.grad), (torch.cat(dvs, 1), vv.grad)):
        err = (have - want).abs().max().item()
        assert err < 0.02 * want.abs().max().item() + 2e-2, err
    assert FA.check_error() == 0
