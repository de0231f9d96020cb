"""Streaming rank-N GEMM (LoRA down-projection: [M, K] x [N, K]^T, N = 16 / 32 / 64) against an fp32
matmul: row tails, K ranges that do not divide by the eight warps, strided rows, and the fallback for
shapes outside the kernel's range."""
import pytest
import torch

from eridiffusion_b200.ops import _native as NAT
from eridiffusion_b200.ops import functional as F

pytestmark = pytest.mark.gpu


def _call(a, b, alpha):
    lib = NAT.require()
    M, K = a.shape
    n = b.shape[0]
    out = torch.full((M, n), float("nan"), dtype=torch.bfloat16, device=a.device)
    code = lib.eri_gemm_rank_stream(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), n, M, n, K,
                                    float(alpha), NAT.stream_ptr())
    return code, out


@pytest.mark.parametrize("M,N,K", [(4608, 16, 3072), (4608, 16, 21504), (512, 16, 3072), (301, 32, 1056),
                                   (16, 64, 256), (5000, 64, 12288), (7, 16, 288), (4608, 32, 15360)])
def test_rank_stream_matches_fp32(M, N, K):
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    ref = (a.float() @ b.float().t()) * 0.5
    code, out = _call(a, b, 0.5)
    assert code == 0
    assert torch.isfinite(out.float()).all()                      # every element was written
    err = (out.float() - ref).abs().max().item()
    assert err <= 1e-2 * ref.abs().max().item() + 1e-3, err


def test_rank_stream_strided_rows_and_fallback():
    g = torch.Generator(device="cuda").manual_seed(5)
    wide = torch.randn(2048, 4096 + 64, device="cuda", generator=g).bfloat16()
    a = wide[:, :4096]
    b = (torch.randn(16, 4096, device="cuda", generator=g) / 64).bfloat16()
    code, out = _call(a, b, 1.0)
    ref = a.float() @ b.float().t()
    assert code == 0 and (out.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-3
    # K not a multiple of 32 and an unsupported rank are declined, and the public op still answers
    a2 = torch.randn(256, 1000, device="cuda", generator=g).bfloat16()
    b2 = (torch.randn(16, 1000, device="cuda", generator=g) / 32).bfloat16()
    assert _call(a2, b2, 1.0)[0] == -100
    assert _call(a, b[:8], 1.0)[0] == -100
    out2 = F.skinny_gemm(a2, b2)
    ref2 = a2.float() @ b2.float().t()
    assert (out2.float() - ref2).abs().max().item() <= 2e-2 * ref2.abs().max().item() + 1e-3


@pytest.mark.parametrize("M0,M1,N,K", [(4096, 512, 16, 3072), (301, 77, 32, 1056), (4096, 512, 64, 12288), (16, 5000, 16, 288)])
def test_rank_stream_two_problems_in_one_launch(M0, M1, N, K):
    """The adapters of the image and the text projection in one launch: each problem with its own operands,
    scale and row tail; equal to the single-problem launches bit for bit."""
    g = torch.Generator(device="cuda").manual_seed(M0 + M1 + N + K)
    mk = lambda m: torch.randn(m, K, device="cuda", generator=g).bfloat16()
    a0, a1 = mk(M0), mk(M1)
    b0, b1 = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16(), \
        (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    c0 = NAT.launch_count()
    o0, o1 = F.skinny_gemm_pair(a0, b0, 0.5, a1, b1, 2.0)
    assert NAT.launch_count() == c0 + 1
    _, r0 = _call(a0, b0, 0.5)
    _, r1 = _call(a1, b1, 2.0)
    assert torch.equal(o0, r0) and torch.equal(o1, r1)
    ref1 = (a1.float() @ b1.float().t()) * 2.0
    assert (o1.float() - ref1).abs().max().item() <= 1e-2 * ref1.abs().max().item() + 1e-3
    # different K: two launches, same results
    a2 = torch.randn(M1, K + 32, device="cuda", generator=g).bfloat16()
    b2 = (torch.randn(N, K + 32, device="cuda", generator=g) / K ** 0.5).bfloat16()
    p0, p2 = F.skinny_gemm_pair(a0, b0, 0.5, a2, b2, 1.0)
    assert torch.equal(p0, r0)
    ref2 = a2.float() @ b2.float().t()
    assert (p2.float() - ref2).abs().max().item() <= 1e-2 * ref2.abs().max().item() + 1e-3
