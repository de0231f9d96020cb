"""LoRA-fused linear with the GEMM launched as a programmatic dependent of the down-projection
kernel: results must be bit-identical to the serialized launch order, forward and backward, over
many repetitions (a GEMM that read the rank-r operand too early would differ)."""
import pytest
import torch

from eridiffusion_b200.ops import functional as F

pytestmark = pytest.mark.gpu


def _run(x, w, la, lb, act, go):
    xg = x.clone().requires_grad_()
    a = la.clone().requires_grad_()
    b = lb.clone().requires_grad_()
    F.prepare_lora_transposes([a, b])
    y = F.linear(xg, w, lora=(a, b, 0.5), act=act)
    y.backward(go)
    F.invalidate_lora_transposes()
    return y.detach(), xg.grad, a.grad, b.grad


@pytest.mark.parametrize("M,N,K,act", [(4608, 3072, 3072, None), (512, 9216, 3072, "gelu"), (4096, 1024, 12288, None)])
def test_pdl_matches_serialized(M, N, K, act, monkeypatch):
    g = torch.Generator(device="cuda").manual_seed(M + N)
    x = torch.randn(1, M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    la = (torch.randn(16, K, device="cuda", generator=g) / K ** 0.5).bfloat16()
    lb = torch.randn(N, 16, device="cuda", generator=g).bfloat16()
    go = torch.randn(1, M, N, device="cuda", generator=g).bfloat16()
    monkeypatch.setattr(F, "_PDL", False)
    ref = _run(x, w, la, lb, act, go)
    monkeypatch.setattr(F, "_PDL", True)
    for _ in range(5):
        got = _run(x, w, la, lb, act, go)
        for r, t in zip(ref, got):
            assert torch.equal(r, t)
    assert F.kernel_error_check() == {}
