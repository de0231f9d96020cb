"""Peer-memory communication kernels: bounded waits, fused data-parallel step, collectives.

Single-GPU cases run the kernels with world size 1 or with a fabricated two-rank context whose peer
never signals (the wait must run out and report, leaving the context usable). Two-GPU cases spawn
one process per GPU and compare against NCCL.
"""
import ctypes as C
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_barrier_wait_runs_out_and_reports():
    from eridiffusion_b200.ops import _native as N
    from eridiffusion_b200.parallel import symm
    lib = N.require()
    symm._bind(lib)
    flags = torch.zeros(symm.FLAG_CHANNELS * symm.MAX_WORLD, dtype=torch.int32, device="cuda")
    peer_flags = torch.zeros_like(flags)          # stands in for a peer that never signals us
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    c = symm.CommCtx()
    c.flags_local = flags.data_ptr()
    c.flags_peer[0], c.flags_peer[1] = flags.data_ptr(), peer_flags.data_ptr()
    c.rank, c.world, c.epoch, c.wait_ns, c.err = 0, 2, 1, 30_000_000, err.data_ptr()
    a = symm.CollArgs()
    a.op, a.count, a.dtype = 5, 0, 0
    rc = lib.eri_collective(C.byref(c), C.byref(a), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    code = int(err.item())
    assert code != 0 and (code & 0xFF) == 1 and (code >> 8) == 4      # channel 3 (+1), peer 1
    # the context is still usable
    assert torch.ones(4, device="cuda").sum().item() == 4.0


def test_fused_dp_step_skips_the_update_when_a_peer_never_arrives():
    """Fabricated two-rank context on one GPU whose peer never signals: every barrier of the fused
    data-parallel kernel runs out (30 ms each), the status word names the silent peer, and the
    kernel must NOT have touched parameters or optimizer state (nor pushed anything to the peer)."""
    from eridiffusion_b200.ops import _native as N
    from eridiffusion_b200.parallel import symm
    lib = N.require()
    symm._bind(lib)
    dev = "cuda"
    shard = 4096
    n = 2 * shard
    g = torch.Generator(device=dev).manual_seed(3)
    grads = [torch.randn(n, device=dev, generator=g).bfloat16() for _ in range(2)]
    params = [torch.randn(n, device=dev, generator=g).bfloat16() for _ in range(2)]
    before = [p.clone() for p in params]
    slots = [torch.zeros(16, device=dev) for _ in range(2)]
    mq = torch.randint(-100, 100, (shard,), device=dev, dtype=torch.int8)
    vq = torch.randint(0, 255, (shard,), device=dev, dtype=torch.uint8)
    mab, vab = torch.rand(shard // 256, device=dev), torch.rand(shard // 256, device=dev)
    state_before = [t.clone() for t in (mq, vq, mab, vab)]
    flags = torch.zeros(symm.FLAG_CHANNELS * symm.MAX_WORLD, dtype=torch.int32, device=dev)
    peer_flags = torch.zeros_like(flags)          # the peer's flag words: written, never answered
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    c = symm.CommCtx()
    c.flags_local = flags.data_ptr()
    c.flags_peer[0], c.flags_peer[1] = flags.data_ptr(), peer_flags.data_ptr()
    c.rank, c.world, c.epoch, c.wait_ns, c.err = 0, 2, 1, 30_000_000, err.data_ptr()
    a = symm.FusedDpArgs()
    for i in range(2):
        a.grads[i], a.params[i], a.sumsq_slots[i] = grads[i].data_ptr(), params[i].data_ptr(), slots[i].data_ptr()
    reduced = torch.zeros(shard, device=dev)
    sumsq_local = torch.zeros(1, device=dev)
    a.reduced, a.sumsq_local = reduced.data_ptr(), sumsq_local.data_ptr()
    a.mq, a.vq, a.m_absmax, a.v_absmax = mq.data_ptr(), vq.data_ptr(), mab.data_ptr(), vab.data_ptr()
    a.shard_elems = shard
    a.lr, a.beta1, a.beta2, a.eps, a.weight_decay, a.max_grad_norm = 1e-2, 0.9, 0.999, 1e-8, 0.01, 1.0
    a.step, a.seed, a.stochastic = 1, 7, 0
    rc = lib.eri_fused_dp_step(C.byref(c), C.byref(a), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    code = int(err.item())
    assert code != 0 and (code & 0xFF) == 1 and (code >> 8) == 1      # first barrier (channel 0 + 1), peer 1
    for p, b in zip(params, before):
        assert torch.equal(p, b), "parameters changed although the reduce was incomplete"
    for t, b in zip((mq, vq, mab, vab), state_before):
        assert torch.equal(t, b), "optimizer state changed although the reduce was incomplete"
    assert torch.ones(4, device=dev).sum().item() == 4.0               # the context is still usable


def test_fused_dp_world1_matches_plain_optimizer():
    from eridiffusion_b200.ops import functional as F
    from eridiffusion_b200.optim import AdamW8bit, ParamArena
    from eridiffusion_b200.parallel.dist import ProcessGroup
    from eridiffusion_b200.parallel.fused_dp import FusedDataParallel
    torch.manual_seed(0)
    mk = lambda: [torch.nn.Parameter(torch.randn(1000, 16, device="cuda").bfloat16()),
                  torch.nn.Parameter(torch.randn(777, device="cuda").bfloat16())]
    p1, p2 = mk(), None
    p2 = [torch.nn.Parameter(p.detach().clone()) for p in p1]
    a1, a2 = ParamArena(p1), ParamArena(p2)
    o1 = AdamW8bit(a1, lr=1e-2, stochastic_rounding=False, shard=(0, 1))
    o2 = AdamW8bit(a2, lr=1e-2, stochastic_rounding=False)
    fdp = FusedDataParallel(ProcessGroup(), a1, o1)
    for s in range(1, 4):
        g = torch.randn(a1.numel, device="cuda").bfloat16()
        a1.grad.copy_(g); a2.grad.copy_(g)
        fdp.step(lr=1e-2, max_grad_norm=1.0, step=s)
        ss = F.sumsq(a2.grad)
        o2.step(grad_sumsq=ss, max_grad_norm=1.0)
        torch.cuda.synchronize()
        assert fdp.status() == 0
        assert abs(fdp.grad_norm.item() - ss.sqrt().item()) < 1e-2 * ss.sqrt().item()
    assert (a1.data.float() - a2.data.float()).abs().max().item() < 2e-2
    assert p1[0].data_ptr() == a1.data.data_ptr()      # parameters now live in the symmetric arena


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, q):
    os.environ.update(WORLD_SIZE=str(world), RANK=str(rank), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    from eridiffusion_b200.adapters import AdapterConfig
    from eridiffusion_b200.models import build_model
    from eridiffusion_b200.parallel.dist import GradSync, init_from_env
    from eridiffusion_b200.parallel.symm import Communicator, SymmetricHeap
    from eridiffusion_b200.train.trainer import Trainer, TrainerConfig
    init_from_env("nccl", timeout_s=120)
    dev = torch.device("cuda", rank)
    out = {}
    # collectives against NCCL
    heap = SymmetricHeap(8 << 20)
    comm = Communicator(heap)
    n = 4096 * world
    src = heap.tensor((n,), torch.bfloat16)
    dstg = heap.tensor((n,), torch.bfloat16)
    torch.manual_seed(100 + rank)
    src.local.copy_(torch.randn(n, device=dev).bfloat16())
    ref = src.local.float().clone()
    dist.all_reduce(ref)
    comm.collective("all_reduce", src, dst_sym=dstg)
    torch.cuda.synchronize()
    out["allreduce_err"] = (dstg.local.float() - ref).abs().max().item()
    rs = torch.empty(n // world, dtype=torch.bfloat16, device=dev)
    comm.collective("reduce_scatter", src, dst=rs, avg=True)
    ref_rs = torch.empty(n // world, dtype=torch.float32, device=dev)
    dist.reduce_scatter_tensor(ref_rs, src.local.float(), dist.ReduceOp.AVG)
    torch.cuda.synchronize()
    out["rs_err"] = (rs.float() - ref_rs).abs().max().item()
    ag = torch.empty(n * world, dtype=torch.bfloat16, device=dev)
    comm.collective("all_gather", src, dst=ag, count=n)
    ref_ag = torch.empty_like(ag)
    dist.all_gather_into_tensor(ref_ag, src.local)
    torch.cuda.synchronize()
    out["ag_equal"] = bool(torch.equal(ag, ref_ag))
    a2a = torch.empty(n, dtype=torch.bfloat16, device=dev)
    comm.collective("all_to_all", src, dst=a2a)
    ref_a2a = torch.empty_like(a2a)
    dist.all_to_all_single(ref_a2a, src.local)
    torch.cuda.synchronize()
    out["a2a_equal"] = bool(torch.equal(a2a, ref_a2a))
    out["comm_status"] = comm.status()
    # fused data-parallel step against the NCCL sharded path
    res = {}
    for mode in ("zero1", "fused"):
        torch.manual_seed(0)
        model = build_model("flux", device=dev, hidden=256, num_heads=2, depth_double=1, depth_single=1,
                            context_dim=128, vec_dim=64)
        cfg = TrainerConfig(mode="lora", adapter=AdapterConfig(rank=16, alpha=16), seed=0,
                            stochastic_rounding=False, lr=1e-3)
        tr = Trainer(model, cfg, grad_sync=GradSync(mode))
        for step in range(2):
            g = torch.Generator(device=dev).manual_seed(7 + step * world + rank)
            mk = lambda *s: torch.randn(*s, device=dev, generator=g).bfloat16()
            batch = {"latents": mk(1, 16, 32, 32), "txt": mk(1, 128, 128), "pooled": mk(1, 64),
                     "noise": mk(1, 16, 32, 32)}
            tr._gen = torch.Generator(device=dev).manual_seed(3 + step)
            tr.train_step(batch)
        torch.cuda.synchronize()
        res[mode] = tr.arena.data.float().clone()
        if mode == "fused":
            out["fused_status"] = tr.grad_sync._fused.status()
    out["fused_vs_nccl"] = (res["fused"] - res["zero1"]).abs().max().item()
    out["param_scale"] = res["zero1"].abs().max().item()
    gathered = [None] * world
    dist.all_gather_object(gathered, res["fused"].cpu())
    out["ranks_agree"] = all(torch.equal(gathered[0], t) for t in gathered)
    if rank == 0:
        q.put(out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_collectives_and_fused_dp():
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert out["comm_status"] == 0 and out["fused_status"] == 0, out
    assert out["allreduce_err"] < 0.1 and out["rs_err"] < 0.05, out
    assert out["ag_equal"] and out["a2a_equal"], out
    assert out["ranks_agree"], out
    assert out["fused_vs_nccl"] < 2e-2 * max(1.0, out["param_scale"]), out
