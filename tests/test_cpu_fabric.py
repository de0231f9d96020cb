"""Protocol tests of the peer-memory communication layer on the CPU fake fabric: collectives
against their definitions, the fused data-parallel step against a single-process optimizer, host-
side fault injection (dropped flag write, late rank, absent rank), and the barrier model checker."""
import torch

from eridiffusion_b200.optim.adamw8bit import BLOCK, dequantize_m, dequantize_v, quantize_m, quantize_v
from eridiffusion_b200.parallel.fabric import (CommTimeout, FakeFabric, check_flag_barrier,
                                               decode_status)


def test_collectives_match_definitions():
    W, n = 4, 64
    fab = FakeFabric(W)
    src = fab.alloc((W * n,), torch.float32)
    g = torch.Generator().manual_seed(0)
    for r in range(W):
        src[r].copy_(torch.randn(W * n, generator=g))
    stacked = torch.stack([s.clone() for s in src])

    def body(rk):
        out = {}
        out["ag"] = rk.all_gather([s[:n] for s in src], torch.empty(W * n))
        out["rs"] = rk.reduce_scatter(src, torch.empty(n), avg=True)
        out["ar"] = rk.all_reduce(src, torch.empty(W * n))
        out["a2a"] = rk.all_to_all(src, torch.empty(W * n))
        out["bc"] = rk.broadcast(src, torch.empty(W * n), root=2)
        rk.barrier()
        return out

    res = fab.run(body)
    for r, o in enumerate(res):
        assert not isinstance(o, BaseException), o
        assert torch.equal(o["ag"], stacked[:, :n].reshape(-1))
        assert torch.allclose(o["rs"], stacked[:, r * n:(r + 1) * n].mean(0), atol=1e-6)
        assert torch.allclose(o["ar"], stacked.sum(0), atol=1e-5)
        assert torch.equal(o["a2a"], stacked[:, r * n:(r + 1) * n].reshape(-1))
        assert torch.equal(o["bc"], stacked[2])
    assert all(s == 0 for s in fab.status)


def _single_process_step(params, grad_mean, state, lr, wd, max_norm, step, b1=0.9, b2=0.999, eps=1e-8):
    norm = float((grad_mean.float() ** 2).sum()) ** 0.5
    gs = min(1.0, max_norm / (norm + 1e-6)) if max_norm > 0 else 1.0
    g = grad_mean.float() * gs
    m = b1 * dequantize_m(state["m_q"], state["m_absmax"]) + (1 - b1) * g
    v = b2 * dequantize_v(state["v_q"], state["v_absmax"]) + (1 - b2) * g * g
    upd = (m / (1 - b1 ** step)) / ((v / (1 - b2 ** step)).sqrt() + eps)
    new = (params.float() * (1 - lr * wd) - lr * upd).to(params.dtype)
    state["m_q"], state["m_absmax"] = quantize_m(m)
    state["v_q"], state["v_absmax"] = quantize_v(v)
    return new, norm


def test_fused_dp_step_matches_single_process():
    W, n = 2, 4 * BLOCK
    fab = FakeFabric(W)
    grads = fab.alloc((W * n,), torch.bfloat16)
    params = fab.alloc((W * n,), torch.bfloat16)
    slots = fab.alloc((16,), torch.float32)
    g = torch.Generator().manual_seed(1)
    p0 = torch.randn(W * n, generator=g).bfloat16()
    for r in range(W):
        params[r].copy_(p0)
    states = [dict(m_q=torch.zeros(n, dtype=torch.int8), v_q=torch.zeros(n, dtype=torch.uint8),
                   m_absmax=torch.zeros(n // BLOCK), v_absmax=torch.zeros(n // BLOCK)) for _ in range(W)]
    ref_state = dict(m_q=torch.zeros(W * n, dtype=torch.int8), v_q=torch.zeros(W * n, dtype=torch.uint8),
                     m_absmax=torch.zeros(W * n // BLOCK), v_absmax=torch.zeros(W * n // BLOCK))
    ref_p = p0.clone()
    for step in (1, 2, 3):
        for r in range(W):
            grads[r].copy_((torch.randn(W * n, generator=g) * 0.1).bfloat16())
        mean = torch.stack([x.float() for x in grads]).mean(0)
        ref_p, ref_norm = _single_process_step(ref_p, mean, ref_state, 1e-2, 0.01, 1.0, step)
        norms = fab.run(lambda rk: rk.fused_dp_step(grads, params, slots, states[rk.rank], lr=1e-2,
                                                    max_grad_norm=1.0, step=step))
        for r in range(W):
            assert abs(norms[r] - ref_norm) < 1e-4 * max(1.0, ref_norm)
            assert torch.equal(params[r], ref_p), f"rank {r} parameters diverge at step {step}"
    assert torch.equal(params[0], params[1])


def test_non_finite_gradient_skips_update_on_every_rank():
    W, n = 2, BLOCK
    fab = FakeFabric(W)
    grads, params = fab.alloc((W * n,), torch.bfloat16), fab.alloc((W * n,), torch.bfloat16)
    slots = fab.alloc((16,), torch.float32)
    for r in range(W):
        params[r].fill_(1.0)
        grads[r].fill_(0.5)
    grads[1][3] = float("nan")           # lands in rank 0's shard only
    states = [dict(m_q=torch.zeros(n, dtype=torch.int8), v_q=torch.zeros(n, dtype=torch.uint8),
                   m_absmax=torch.zeros(n // BLOCK), v_absmax=torch.zeros(n // BLOCK)) for _ in range(W)]
    norms = fab.run(lambda rk: rk.fused_dp_step(grads, params, slots, states[rk.rank], lr=1e-2))
    assert all(x != x for x in norms)
    for r in range(W):
        assert torch.all(params[r] == 1.0)
        assert int(states[r]["m_q"].abs().sum()) == 0


def test_dropped_flag_write_surfaces_as_timeout_and_job_recovers():
    W, n = 2, 32
    fab = FakeFabric(W, wait_s=0.2)
    src = fab.alloc((W * n,), torch.float32)
    for r in range(W):
        src[r].fill_(r + 1.0)
    fab.drop_flag(src=1, dst=0, channel=0, epoch=1)       # rank 0 never sees rank 1 arrive
    res = fab.run(lambda rk: rk.all_reduce(src, torch.empty(W * n)))
    assert isinstance(res[0], CommTimeout) and (res[0].channel, res[0].peer) == (0, 1)
    # rank 1 passed phase 0 but waits for rank 0 at phase 1, which never comes
    assert isinstance(res[1], CommTimeout) and (res[1].channel, res[1].peer) == (1, 0)
    assert decode_status(res[0].status) == (0, 1)
    # the status words were cleared by the read; the next collective (a new epoch) works
    res = fab.run(lambda rk: rk.all_reduce(src, torch.empty(W * n)))
    for o in res:
        assert torch.allclose(o, torch.full((W * n,), 3.0))


def test_late_rank_is_tolerated_and_absent_rank_times_out():
    W = 3
    fab = FakeFabric(W, wait_s=0.5)
    fab.delay_rank(2, 0.1)
    assert all(o is None for o in fab.run(lambda rk: rk.barrier()))
    fab.delay_rank(2, 0.0)
    res = fab.run(lambda rk: rk.barrier(), ranks=[0, 1])  # rank 2 never joins
    assert all(isinstance(res[r], CommTimeout) and res[r].peer == 2 for r in (0, 1))


def test_epoch_comparison_survives_wraparound():
    fab = FakeFabric(2, wait_s=0.2)
    for r in range(2):
        fab.epoch[r] = 0xFFFFFFFE
        for c in range(2):
            fab.flags[r][c][0] = fab.flags[r][c][1] = 0xFFFFFFFE
    for _ in range(4):                                    # epochs ...FF, 0 (wrapped, masked below), 1, 2
        fab.epoch = [e & 0xFFFFFFFF for e in fab.epoch]
        assert all(o is None for o in fab.run(lambda rk: rk.barrier()))


def test_model_checker_barrier_safe_and_live():
    for world, epochs in ((2, 3), (3, 2)):
        rep = check_flag_barrier(world=world, epochs=epochs, channels=2)
        assert rep["violations"] == [] and rep["stuck"] == [] and rep["finals"] == 1, rep
    rep = check_flag_barrier(world=2, epochs=2, channels=2, drop={(1, 0, 1, 1)})
    assert rep["violations"] == [] and rep["stuck"], rep   # a lost store can only stall, never let a rank through
