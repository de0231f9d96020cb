"""Two-GPU checks of the fused ZeRO-3 (gather-in-GEMM) and Ulysses (scatter / gather in the
projections) paths against single-GPU math on the same data."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / max(1e-6, b.float().abs().max().item())


def _worker(rank, world, port, q):
    try:
        _worker_body(rank, world, port, q)
    except BaseException as e:                      # report instead of leaving the parent waiting
        import traceback
        q.put({"error": f"rank {rank}: {e!r}\n{traceback.format_exc()}"})
        raise


def _worker_body(rank, world, port, q):
    os.environ.update(WORLD_SIZE=str(world), RANK=str(rank), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    from eridiffusion_b200.models.layers import Linear, SmallLinear
    from eridiffusion_b200.models import build_model
    from eridiffusion_b200.ops import functional as F
    from eridiffusion_b200.parallel.dist import ProcessGroup, init_from_env
    from eridiffusion_b200.parallel.ulysses import UlyssesContext
    from eridiffusion_b200.parallel.zero3 import Zero3Context, Zero3Linear, Zero3SmallLinear
    init_from_env("nccl", timeout_s=120)
    dev = torch.device("cuda", rank)
    out = {}
    pg = ProcessGroup()

    # ---------------- ZeRO-3 linear: forward, input grad, reduce-scattered weight grad
    torch.manual_seed(0)
    lin = Linear(256, 512, device=dev)
    small = SmallLinear(256, 6 * 256, device=dev)
    z3 = Zero3Context(pg, heap_bytes=8 << 20, max_weight_elems=2 << 20, n_copy=4)
    zl, zs = Zero3Linear(lin, z3), Zero3SmallLinear(small, z3)
    # move the shards into the symmetric heap, as the trainer's arena does
    from eridiffusion_b200.optim import ParamArena
    arena = ParamArena([zl.weight, zs.weight, zs.bias], alloc=z3.arena_alloc)
    z3.barrier()
    xs = [torch.randn(2, 128, 256, device=dev, generator=torch.Generator(device=dev).manual_seed(5 + r)).bfloat16()
          for r in range(world)]
    vs = [torch.randn(2, 256, device=dev, generator=torch.Generator(device=dev).manual_seed(9 + r)).bfloat16()
          for r in range(world)]
    x = xs[rank].clone().requires_grad_()
    v = vs[rank].clone().requires_grad_()
    y = zl(x, act="gelu")
    m = zs(v, silu_in=True)
    (y.float().pow(2).mean() + m.float().pow(2).mean()).backward()
    torch.cuda.synchronize()
    # reference: full weights, every rank's data
    xr = [t.clone().float().requires_grad_() for t in xs]
    vr = [t.clone().float().requires_grad_() for t in vs]
    wf, bf = lin.weight.detach().float().requires_grad_(), lin.bias.detach().float()
    sw = small.weight.detach().float().requires_grad_()
    sb = small.bias.detach().float().requires_grad_()
    tot = 0
    for r in range(world):
        yr = torch.nn.functional.gelu(torch.nn.functional.linear(xr[r], wf, bf), approximate="tanh")
        mr = torch.nn.functional.linear(torch.nn.functional.silu(vr[r]), sw, sb)
        if r == rank:
            out["z3_fwd"] = _rel(y, yr)
            out["z3_small_fwd"] = _rel(m, mr)
        tot = tot + (yr.pow(2).mean() + mr.pow(2).mean()) / world
    tot.backward()
    per = 512 // world
    out["z3_dx"] = _rel(x.grad, xr[rank].grad * world)
    out["z3_dw"] = _rel(zl.weight.grad, wf.grad[rank * per:(rank + 1) * per])
    pers = 6 * 256 // world
    out["z3_small_dw"] = _rel(zs.weight.grad, sw.grad[rank * pers:(rank + 1) * pers])
    out["z3_small_dx"] = _rel(v.grad, vr[rank].grad * world)
    # a second layer whose slabs (384 rows per rank) are not multiples of the 256-row pair tile:
    # forward gather, input gradient (gather along K) and the fused weight-gradient reduce-scatter
    torch.manual_seed(2)
    lin2 = Linear(512, 384 * world, bias=False, device=dev)
    zl2 = Zero3Linear(lin2, z3)
    arena2 = ParamArena([zl2.weight], alloc=z3.arena_alloc)
    z3.barrier()
    x2s = [torch.randn(2, 192, 512, device=dev, generator=torch.Generator(device=dev).manual_seed(21 + r)).bfloat16()
           for r in range(world)]
    x2 = x2s[rank].clone().requires_grad_()
    lib = F.N.require()
    c0 = lib.eri_gemm2_gather_count()
    y2 = zl2(x2)
    y2.float().pow(2).mean().backward()
    torch.cuda.synchronize()
    out["z3_pair_launches"] = lib.eri_gemm2_gather_count() - c0          # forward + input-gradient gathers
    w2 = lin2.weight.detach().float().requires_grad_()
    x2r = [t.clone().float().requires_grad_() for t in x2s]
    tot2 = 0
    for r in range(world):
        y2r = torch.nn.functional.linear(x2r[r], w2)
        if r == rank:
            out["z3u_fwd"] = _rel(y2, y2r)
        tot2 = tot2 + y2r.pow(2).mean() / world
    tot2.backward()
    out["z3u_dx"] = _rel(x2.grad, x2r[rank].grad * world)
    out["z3u_dw"] = _rel(zl2.weight.grad, w2.grad[rank * 384:(rank + 1) * 384])
    # next-layer prefetch: the same two layers as a repeated step (forward of both, backward of both). The
    # first step records the order of the gathers, later steps have every gather but the step's first one
    # delivered by the copy engines while the GEMM before it runs; results equal the unprefetched step's.
    def step():
        z3.begin_step()
        xa = xs[rank].clone().requires_grad_()
        ya = zl(xa, act="gelu")                       # [2, 128, 512]
        yb = zl2(ya)                                  # [2, 128, 384 * world]
        yb.float().pow(2).mean().backward()
        return yb.detach().clone(), xa.grad.clone(), zl.weight.grad.clone(), zl2.weight.grad.clone()
    zl.weight.grad = zl2.weight.grad = None
    base = step()                                     # records the order; nothing prefetched yet
    n0 = z3.prefetched_launches
    got = None
    for _ in range(3):
        zl.weight.grad = zl2.weight.grad = None
        got = step()
    z3.begin_step()
    torch.cuda.synchronize()
    out["z3_prefetched"] = z3.prefetched_launches - n0   # 3 steps x (4 gathers - the first of the step)
    out["z3_prefetch_diff"] = max(_rel(a, b) for a, b in zip(got, base))
    out["z3_status"] = z3.comm.status()
    out["gemm_err"] = F.gemm_error_check()

    # ---------------- Ulysses: LTX-style model, sequence sharded over ranks vs full sequence
    torch.manual_seed(1)
    # one rank's head group stays 128 columns wide and its sequence shard 128 tokens at every world size
    hid, nh = (256, 4) if world == 2 else (128 * world, world)
    kw = dict(hidden=hid, num_heads=nh, depth=2, context_dim=256, caption_dim=128, in_channels=64)
    model = build_model("ltx_video", device=dev, **kw)
    frames, hh, ww = 2, 8, 8 * world                # 128 tokens per rank
    L = frames * hh * ww
    Ll = L // world
    g = torch.Generator(device=dev).manual_seed(3)
    tok = torch.randn(1, L, 64, device=dev, generator=g).bfloat16()
    txt = torch.randn(1, 128, 128, device=dev, generator=g).bfloat16()
    t = torch.tensor([0.4], device=dev)
    full_in = tok.clone().requires_grad_()
    ref = model(full_in, txt, t, (frames, hh, ww))
    wgt = torch.randn_like(ref)
    (ref * wgt).sum().backward()
    ref_dx = full_in.grad.clone()
    ref_gw = model.blocks[0].attn1_qkv.weight.grad
    u = UlyssesContext(pg, batch=1, l_local=Ll, hidden=hid, heads=nh, n_copy=4)
    model.set_sequence_parallel(u)
    loc_in = tok[:, rank * Ll:(rank + 1) * Ll].clone().requires_grad_()
    for p in model.parameters():
        p.requires_grad_(False)
    model.blocks[0].attn1_qkv.weight.requires_grad_(True)
    model.blocks[0].attn1_qkv.weight.grad = None
    y = model(loc_in, txt, t, (frames, hh, ww))
    (y * wgt[:, rank * Ll:(rank + 1) * Ll]).sum().backward()
    torch.cuda.synchronize()
    out["ul_fwd"] = _rel(y, ref[:, rank * Ll:(rank + 1) * Ll])
    out["ul_dx"] = _rel(loc_in.grad, ref_dx[:, rank * Ll:(rank + 1) * Ll])
    gw = model.blocks[0].attn1_qkv.weight.grad.float().clone()
    dist.all_reduce(gw)
    out["ul_dw"] = _rel(gw, ref_gw) if ref_gw is not None else -1.0
    out["ul_status"] = u.comm.status()
    out["gemm_err2"] = F.gemm_error_check()
    if rank == 0:
        q.put(out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_zero3_and_ulysses_multi_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = q.get(timeout=300)
    if "error" in out:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
        pytest.fail(out["error"])
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert out["z3_status"] == 0 and out["ul_status"] == 0 and out["gemm_err"] == 0 and out["gemm_err2"] == 0, out
    for k in ("z3_fwd", "z3_small_fwd", "z3_dx", "z3_dw", "z3_small_dw", "z3_small_dx", "z3u_fwd", "z3u_dx", "z3u_dw",
              "ul_fwd", "ul_dx", "ul_dw"):
        assert out[k] < 4e-2, (k, out)
    assert out["z3_pair_launches"] == 2, out          # unaligned slabs stay on the two-CTA kernel
    # three steps, four gathers each, all but the first of a step delivered ahead by the copy engines
    assert out["z3_prefetched"] == 9 and out["z3_prefetch_diff"] < 1e-3, out
