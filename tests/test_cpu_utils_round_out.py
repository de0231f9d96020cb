"""Accuracy suite, tensor helpers, expert bank, model offloader / memory optimizer, EMA context (CPU)."""
import json

import pytest
import torch


def test_accuracy_reports(tmp_path):
    from eridiffusion_b200.utils.accuracy import AccuracyReport, AccuracyTestSuite, DifferenceStats, compare_shapes
    e = torch.linspace(-2, 2, 1000)
    a = e.clone(); a[10] += 1e-2; a[20] += 1e-5
    r = AccuracyReport.from_tensors("op", a, e, tolerance=1e-3)
    assert not r.passed and abs(r.max_absolute_error - 1e-2) < 1e-6 and r.num_elements == 1000
    assert AccuracyReport.from_tensors("op", a, e, tolerance=1e-2).passed
    bad = e.clone(); bad[0] = float("nan")
    rn = AccuracyReport.from_tensors("nan", bad, e, tolerance=1.0)
    assert not rn.passed and rn.num_nonfinite == 1
    both = AccuracyReport.from_tensors("both", bad, bad, tolerance=1e-6)
    assert both.passed                                        # NaN at the same place on both sides
    with pytest.raises(ValueError):
        compare_shapes("x", (1, 2), (2, 1))
    st = DifferenceStats.from_differences(a - e)
    assert st.num_zeros == 998 and st.num_large == 1 and st.num_medium == 1 and st.num_small == 0
    assert "p99" in st.format_report()
    suite = AccuracyTestSuite()
    suite.add_comparison("good", e, e)
    suite.add_comparison("bad", a, e)
    assert suite.num_passed() == 1 and suite.num_failed() == 1 and not suite.all_passed()
    assert "[FAIL] bad" in suite.generate_summary() and "1/2 passed" in suite.generate_summary()
    d = json.load(open(suite.save_to_file(tmp_path / "r.json")))
    assert d["passed"] is False and len(d["reports"]) == 2
    assert "[PASS] good" in open(suite.save_to_file(tmp_path / "r.txt")).read()


def test_tensor_helpers():
    from eridiffusion_b200.utils import tensor_utils as U
    x = torch.tensor([[1.0, 2.0, 3.0], [float("-inf")] * 3, [1e4, 1e4 - 1, -1e4]])
    p = U.stable_softmax(x)
    assert torch.allclose(p[0], torch.softmax(x[0], -1)) and p[1].eq(0).all() and torch.isfinite(p).all()
    assert torch.allclose(U.stable_log_softmax(x[[0, 2]]), torch.log_softmax(x[[0, 2]], -1), atol=1e-5)
    assert U.stable_softmax(x.to(torch.bfloat16)).dtype == torch.bfloat16
    assert U.safe_div(torch.tensor([1.0, 1.0, 1.0]), torch.tensor([0.0, -0.0, -2.0])).tolist() == [1e8, 1e8, -0.5]
    assert torch.isfinite(U.safe_log(torch.tensor([0.0]))).all() and U.safe_sqrt(torch.tensor([-1.0])).item() == 0
    assert U.nan_to_zero(torch.tensor([float("nan"), float("inf"), 2.0])).tolist() == [0, 0, 2]
    assert U.has_nonfinite(torch.tensor([float("inf")])) and not U.has_nonfinite(torch.ones(2))
    v = torch.arange(2.0)
    assert U.broadcast_to_rank(v, torch.zeros(2, 3, 4, 5)).shape == (2, 1, 1, 1)
    assert U.broadcast_over_tokens(torch.zeros(2, 8), 5).shape == (2, 5, 8)
    big = torch.full((4096,), 1.0, dtype=torch.bfloat16)
    assert U.mean_fp32(big).item() == 1.0 and U.sum_as(big.view(1, -1), 1, torch.bfloat16).item() == 4096
    assert U.clamp_finite(torch.tensor([float("nan"), 20.0, -20.0]), -10, 10).tolist() == [0, 10, -10]


def test_expert_bank_and_routing():
    from eridiffusion_b200.models.moe import (ExpertBank, QuantKind, dequantize_to_bf16, moe_linear, quantize_weight,
                                              route_tokens, select_topk_global)
    torch.manual_seed(0)
    W = [torch.randn(16, 64) * 0.1 for _ in range(4)]
    for kind, tol in ((QuantKind.NONE, 1e-2), (QuantKind.Q8, 1e-2), (QuantKind.NF4, 8e-2)):
        bank = ExpertBank(kind)
        for i, w in enumerate(W):
            bank.insert(i, w)
        got = dict(bank.fetch_topk_bf16([2, 0, 9]))
        assert list(got) == [2, 0] and got[2].dtype == torch.bfloat16
        assert (got[2].float() - W[2]).abs().max() < tol * W[2].abs().max() * 4
    assert ExpertBank(QuantKind.NF4).kind == "nf4" and bank.nbytes() < sum(w.numel() * 2 for w in W)
    assert select_topk_global(8, 3) == [0, 1, 2] and select_topk_global(2, 3) == [0, 1]
    scores = torch.tensor([[5.0, 0, 0, 1], [4.0, 0, 0, 2], [0, 0, 6.0, 0]])
    assert set(select_topk_global(scores, 2)) == {0, 2}
    idx, w = route_tokens(scores, 2)
    assert idx[:, 0].tolist() == [0, 0, 2] and torch.allclose(w.sum(-1), torch.ones(3))
    idx_r, _ = route_tokens(scores, 1, allowed=[1, 3])
    assert idx_r.flatten().tolist() == [3, 3, 1] or idx_r.flatten().tolist()[:2] == [3, 3]
    bank = ExpertBank(QuantKind.NONE)
    for i, wt in enumerate(W):
        bank.insert(i, wt)
    x = torch.randn(3, 64)
    y = moe_linear(x, scores, bank, k=2)
    ref = torch.stack([sum(w[t, j] * (x[t] @ W[int(idx[t, j])].T) for j in range(2)) for t in range(3)])
    assert torch.allclose(y, ref, atol=2e-2)
    assert isinstance(quantize_weight(W[0], "none"), torch.Tensor) and dequantize_to_bf16(W[0]).dtype == torch.bfloat16


def test_model_offloader_keeps_identity():
    from eridiffusion_b200.memory.offload import ModelOffloader
    off = ModelOffloader(device="cpu", pin=False)
    m = torch.nn.Linear(4, 3)
    w_id, ref = id(m.weight), m.weight.detach().clone()
    off.register_model("te", 60)
    assert off.is_loaded("te") and off.get_stats() == (1, 0)
    off.offload_model("te", m)
    assert off.is_offloaded("te") and not off.is_loaded("te") and off.offloaded_bytes() == (12 + 3) * 4
    off.prefetch("te")
    dev = off.load_model("te", m)
    assert id(m.weight) == w_id and torch.equal(m.weight, ref) and set(dev) == {"weight", "bias"}
    assert off.get_stats() == (1, 0)
    with pytest.raises(KeyError):
        off.load_model("te")
    off.offload_model("raw", {"a": torch.ones(2)})
    assert torch.equal(off.load_model("raw")["a"], torch.ones(2))
    off.offload_model("x", {"a": torch.ones(2)})
    off.clear_offloaded()
    assert off.get_stats()[1] == 0


def test_memory_optimizer_policy():
    from eridiffusion_b200.memory.offload import (MemoryOptimizer, MemoryPressure, MemoryStrategy,
                                                  get_optimization_tips)
    mo = MemoryOptimizer("aggressive", memory_limit_gb=1.0, batch_size=8)
    mo.set_batch_size_limits(1, 8)
    plan = mo.apply_strategy()
    assert plan["activation_checkpointing"] and plan["quantize_base"] and not plan["block_swap"]
    assert MemoryOptimizer(MemoryStrategy.EXTREME).apply_strategy()["block_swap"]
    assert not any(v for v in MemoryOptimizer().apply_strategy().values())
    mo.update_memory_usage(1000.0)
    assert mo.get_memory_pressure() == MemoryPressure.CRITICAL and mo.adjust_batch_size() == 4
    mo.update_memory_usage(900.0)
    assert mo.get_memory_pressure() == MemoryPressure.HIGH and mo.adjust_batch_size() == 3
    mo.update_memory_usage(100.0)
    for _ in range(9):
        assert mo.adjust_batch_size() == 3
    assert mo.adjust_batch_size() == 4
    st = mo.get_stats()
    assert st.peak_mb == 1000.0 and abs(st.usage_percent() - 100 * 100 / 1024) < 1e-6 and st.remaining_mb() == 924.0
    assert any("larger batch" in t for t in get_optimization_tips(st))
    mo.update_memory_usage(1010.0); mo.record_oom()
    tips = get_optimization_tips(mo.get_stats())
    assert any("zero_stage" in t for t in tips) and any("checkpointing" in t for t in tips)
    assert mo.optimize_tensor(torch.zeros(2), "blocks.0.attn.weight").dtype == torch.bfloat16
    assert mo.optimize_tensor(torch.zeros(2), "blocks.0.norm.weight").dtype == torch.float32


def test_ema_context_restores_on_error():
    from eridiffusion_b200.optim import EMA
    p = torch.nn.Parameter(torch.ones(3))
    ema = EMA([p], decay=0.5, warmup=False)
    with torch.no_grad():
        p.fill_(3.0)
    ema.update()                                              # shadow = 2
    with ema.applied():
        assert p.detach().tolist() == [2.0] * 3
    assert p.detach().tolist() == [3.0] * 3
    with pytest.raises(RuntimeError):
        with ema.applied():
            raise RuntimeError("sampling failed")
    assert p.detach().tolist() == [3.0] * 3
