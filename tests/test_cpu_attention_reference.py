"""Blockwise online-softmax attention against the full softmax, its gradients against finite
differences, and the profiler export helper."""
import json

import torch

from eridiffusion_b200.ops import reference as R
from eridiffusion_b200.utils import trace


def test_chunked_attention_matches_full():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(2, L, 3, 16, generator=g) for L in (37, 53, 53))
    full = R.attention_fp32(q, k, v)
    for qc, kc in ((8, 16), (37, 53), (100, 7), (1, 1)):
        assert torch.allclose(R.attention_chunked(q, k, v, q_chunk=qc, kv_chunk=kc), full, atol=2e-5), (qc, kc)
    # large logits: the running maximum keeps the exponentials finite
    big = R.attention_chunked(q * 60, k * 60, v, q_chunk=8, kv_chunk=8)
    assert torch.isfinite(big).all() and torch.allclose(big, R.attention_fp32(q * 60, k * 60, v), atol=1e-4)
    assert R.attention_chunked(q.bfloat16(), k.bfloat16(), v.bfloat16()).dtype == torch.bfloat16


def test_attention_gradients_against_finite_differences():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(1, L, 2, 4, generator=g, dtype=torch.float64).requires_grad_() for L in (5, 6, 6))
    f = lambda a, b, c: R.attention_chunked(a, b, c, q_chunk=2, kv_chunk=4).double()
    w = torch.randn(1, 5, 2, 4, generator=g, dtype=torch.float64)
    (f(q, k, v) * w).sum().backward()
    eps = 1e-3
    for t in (q, k, v):
        flat, grad = t.detach().view(-1), t.grad.view(-1)
        for i in (0, 7, flat.numel() - 1):
            old = flat[i].item()
            with torch.no_grad():
                flat[i] = old + eps
                up = (f(q, k, v) * w).sum().item()
                flat[i] = old - eps
                dn = (f(q, k, v) * w).sum().item()
                flat[i] = old
            # the chunked path computes in fp32: central differences agree to ~1e-3 relative
            assert abs((up - dn) / (2 * eps) - grad[i].item()) < 2e-2 * max(1.0, abs(grad[i].item()))


def test_profile_steps_writes_a_trace(tmp_path):
    x = torch.randn(64, 64)
    table = trace.profile_steps(lambda: (x @ x).relu().sum(), 2, tmp_path / "trace.json", warmup=1)
    assert "aten::mm" in table or "aten::matmul" in table
    doc = json.loads((tmp_path / "trace.json").read_text())
    assert "traceEvents" in doc and len(doc["traceEvents"]) > 0
