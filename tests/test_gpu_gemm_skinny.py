"""Split-K skinny GEMM (LoRA down-projection shapes) against fp32 matmul; repeated calls check that
the shared fp32 workspace and arrival counters are left clean."""
import os

import pytest
import torch

os.environ.setdefault("ERI_B200_SKINNY_MIN_K", "512")     # exercise the split-K kernel on short K too

from eridiffusion_b200.ops import functional as F  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _split_k_kernel_only(monkeypatch):
    """These cases cover the split-K tcgen05 kernel; the streaming kernel has its own file."""
    monkeypatch.setattr(F, "_RANK_STREAM", False)


@pytest.mark.parametrize("M,N,K", [(4608, 16, 3072), (4096, 16, 21504), (512, 16, 3072), (300, 32, 1000),
                                   (128, 64, 512), (5000, 64, 12288), (4608, 16, 15360)])
def test_skinny_gemm_matches_fp32(M, N, K):
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    ref = (a.float() @ b.float().t()) * 0.5
    for _ in range(3):                       # the workspace must be zero again after every call
        out = F.skinny_gemm(a, b, alpha=0.5)
        err = (out.float() - ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item() + 1e-3, err
    assert F.kernel_error_check() == {}


def test_skinny_gemm_strided_rows_and_mixed_ranks():
    g = torch.Generator(device="cuda").manual_seed(3)
    wide = torch.randn(2048, 4096 + 64, device="cuda", generator=g).bfloat16()
    a = wide[:, :4096]                       # row stride 4160 elements
    for N in (16, 64, 32, 16):
        b = (torch.randn(N, 4096, device="cuda", generator=g) / 64).bfloat16()
        out = F.skinny_gemm(a, b)
        ref = a.float() @ b.float().t()
        assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-3
