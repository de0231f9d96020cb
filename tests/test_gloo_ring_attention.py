"""Ring attention among CPU ranks (gloo): forward and gradients equal full attention over the
gathered sequence."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _full(seed=3, B=2, L=24, H=2, D=8):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(B, L, H, D, generator=g) for _ in range(4)]       # q, k, v, dO


def _worker(rank, world, port, q_out):
    os.environ.update(WORLD_SIZE=str(world), RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    import torch.distributed as dist
    from eridiffusion_b200.parallel.ring_attention import ring_attention, shard_sequence
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
    q, k, v, do = _full()
    ql, kl, vl, dol = (shard_sequence(t) for t in (q, k, v, do))
    ql.requires_grad_(); kl.requires_grad_(); vl.requires_grad_()
    out = ring_attention(ql, kl, vl)
    out.backward(dol)
    q_out.put((rank, out.detach(), ql.grad, kl.grad, vl.grad))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_ring_attention_matches_full(world):
    from eridiffusion_b200.ops.reference import attention_fp32
    ctx = mp.get_context("spawn")
    qu = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, qu)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted((qu.get(timeout=180) for _ in range(world)), key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    q, k, v, do = _full()
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    ref = attention_fp32(q, k, v)
    ref.backward(do)
    for i, want in enumerate((ref.detach(), q.grad, k.grad, v.grad)):
        have = torch.cat([g[i + 1] for g in got], dim=1)
        assert torch.allclose(have, want, atol=2e-5, rtol=1e-4), (i, (have - want).abs().max())


def test_merge_is_associative_and_matches_softmax():
    from eridiffusion_b200.ops.reference import attention_fp32
    from eridiffusion_b200.parallel.ring_attention import block_backward, block_forward, merge
    q, k, v, do = _full(seed=5, L=12)
    parts = [block_forward(q, k[:, a:a + 4], v[:, a:a + 4], 0.3) for a in (0, 4, 8)]
    o1, l1 = merge(*merge(*parts[0], *parts[1]), *parts[2])
    o2, l2 = merge(*parts[0], *merge(*parts[1], *parts[2]))
    ref = attention_fp32(q, k, v, 0.3)
    assert torch.allclose(o1, ref, atol=1e-5) and torch.allclose(o2, ref, atol=1e-5) and torch.allclose(l1, l2)
    # slice gradients from the final out / lse add up to the full gradient
    qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
    attention_fp32(qq, kk, vv, 0.3).backward(do)
    dq = torch.zeros_like(q)
    for a in (0, 4, 8):
        dq_s, dk_s, dv_s = block_backward(do, q, k[:, a:a + 4], v[:, a:a + 4], o1, l1, 0.3)
        dq += dq_s
        assert torch.allclose(dk_s, kk.grad[:, a:a + 4], atol=1e-5)
        assert torch.allclose(dv_s, vv.grad[:, a:a + 4], atol=1e-5)
    assert torch.allclose(dq, qq.grad, atol=1e-5)


def _ltx(seed=0):
    from eridiffusion_b200.models import build_model
    torch.manual_seed(seed)
    m = build_model("ltx_video", dtype=torch.float32, hidden=48, num_heads=2, depth=2, in_channels=8,
                    context_dim=24, caption_dim=12)
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.08)
    return m


def _ltx_inputs():
    g = torch.Generator().manual_seed(4)
    return (torch.randn(1, 24, 8, generator=g), torch.randn(1, 5, 12, generator=g), torch.tensor([0.4]),
            torch.randn(1, 24, 8, generator=g))


def _ltx_worker(rank, world, port, q_out):
    os.environ.update(WORLD_SIZE=str(world), RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    import torch.distributed as dist
    from eridiffusion_b200.parallel.ring_attention import shard_sequence
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
    m = _ltx()
    m.set_context_parallel()
    x, ctx, t, go = _ltx_inputs()
    out = m(shard_sequence(x), ctx, t, (2, 3, 4))
    out.backward(shard_sequence(go))
    grads = torch.cat([p.grad.flatten() for p in m.parameters()])
    dist.all_reduce(grads)                                  # per-token work is split: gradients add up
    q_out.put((rank, out.detach(), grads if rank == 0 else None))
    dist.barrier()
    dist.destroy_process_group()


def test_ltx_context_parallel_matches_single_process():
    world = 2
    ctx_mp = mp.get_context("spawn")
    qu = ctx_mp.Queue()
    port = _free_port()
    procs = [ctx_mp.Process(target=_ltx_worker, args=(r, world, port, qu)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted((qu.get(timeout=180) for _ in range(world)), key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    m = _ltx()
    x, ctx, t, go = _ltx_inputs()
    ref = m(x, ctx, t, (2, 3, 4))
    ref.backward(go)
    assert torch.allclose(torch.cat([g[1] for g in got], dim=1), ref.detach(), atol=1e-5)
    ref_g = torch.cat([p.grad.flatten() for p in m.parameters()])
    assert torch.allclose(got[0][2], ref_g, atol=1e-4, rtol=1e-3), (got[0][2] - ref_g).abs().max()
