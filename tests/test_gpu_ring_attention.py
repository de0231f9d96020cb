"""Ring attention over NCCL on real GPUs: forward and gradients of the sharded sequence equal fp32
attention over the whole sequence, with the slice products on the native flash kernels."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, q):
    try:
        os.environ.update(WORLD_SIZE=str(world), RANK=str(rank), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                          MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        import torch.distributed as dist
        from eridiffusion_b200.ops import flash_attn as FA
        from eridiffusion_b200.ops.reference import attention_fp32
        from eridiffusion_b200.parallel.dist import init_from_env
        from eridiffusion_b200.parallel.ring_attention import ring_attention, shard_sequence
        init_from_env("nccl", timeout_s=120)
        dev = torch.device("cuda", rank)
        out = {}
        for B, L, H, D in ((1, 256 * world, 4, 128), (2, 384 * world, 2, 64)):
            g = torch.Generator(device=dev).manual_seed(5)
            qf, kf, vf, dof = (torch.randn(B, L, H, D, device=dev, generator=g).bfloat16() for _ in range(4))
            ql, kl, vl, dol = (shard_sequence(t) for t in (qf, kf, vf, dof))
            ql.requires_grad_(); kl.requires_grad_(); vl.requires_grad_()
            o = ring_attention(ql, kl, vl)
            o.backward(dol)
            qr, kr, vr = (t.float().requires_grad_() for t in (qf, kf, vf))
            ref = attention_fp32(qr, kr, vr)
            ref.backward(dof.float())
            n = L // world
            sl = slice(rank * n, (rank + 1) * n)
            rel = lambda a, b: float((a.float() - b).abs().max() / b.abs().max())
            errs = torch.tensor([rel(o, ref[:, sl]), rel(ql.grad, qr.grad[:, sl]), rel(kl.grad, kr.grad[:, sl]),
                                 rel(vl.grad, vr.grad[:, sl])], device=dev)
            dist.all_reduce(errs, dist.ReduceOp.MAX)
            out[f"{L}x{H}x{D}"] = errs.tolist()
        out["fa_err"] = FA.check_error()
        if rank == 0:
            q.put(out)
        dist.barrier()
        dist.destroy_process_group()
    except BaseException as e:                      # report instead of leaving the parent waiting
        import traceback
        q.put({"error": f"rank {rank}: {e!r}\n{traceback.format_exc()}"})
        raise


@pytest.mark.parametrize("world", [2, 4])
def test_ring_attention_over_nccl(world):
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
    for p in procs:
        p.join(timeout=120)
    if "error" in out:
        pytest.fail(out["error"])
    assert all(p.exitcode == 0 for p in procs)
    assert out.pop("fa_err") == 0
    for shape, errs in out.items():
        assert max(errs) < 2e-2, (shape, errs)
