"""world_size=2 gloo runs on CPU: data-parallel gradient sync (all-reduce and sharded
reduce-scatter/all-gather) reproduces the single-process full-batch update."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, mode, q):
    os.environ.update(WORLD_SIZE=str(world), RANK=str(rank), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch
    import torch.distributed as dist
    from tests.test_cpu_training import batch, make_trainer
    from eridiffusion_b200.parallel.dist import GradSync, init_from_env, split_batch
    torch.set_num_threads(2)
    init_from_env("gloo", timeout_s=120)
    from eridiffusion_b200.adapters import AdapterConfig
    from eridiffusion_b200.models import build_model
    from eridiffusion_b200.train.trainer import Trainer, TrainerConfig
    torch.manual_seed(0)
    model = build_model("tiny_mmdit")
    cfg = TrainerConfig(mode="lora", adapter=AdapterConfig(rank=4, alpha=4, dtype=torch.float32),
                        guidance=None, optimizer="adamw8bit", lr=1e-3, seed=0, max_grad_norm=1.0,
                        stochastic_rounding=False)
    tr = Trainer(model, cfg, grad_sync=GradSync(mode))
    full = batch(1, B=2)
    noise = torch.randn(2, 16, 32, 32, generator=torch.Generator().manual_seed(9))
    ts = torch.tensor([0.3, 0.7])
    for step in range(2):
        mine = split_batch({**full, "noise": noise}, world, rank)
        tr.objective.sample_t = lambda n, gen=None, device="cpu", r=rank: ts[r:r + n]
        tr.train_step(mine)
    if rank == 0:
        q.put(tr.arena.data.clone())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["allreduce", "zero1"])
def test_dp2_matches_single_process(mode):
    from tests.test_cpu_training import batch, make_trainer
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    tr = make_trainer()
    tr.cfg.max_grad_norm = 1.0
    full = batch(1, B=2)
    noise = torch.randn(2, 16, 32, 32, generator=torch.Generator().manual_seed(9))
    ts = torch.tensor([0.3, 0.7])
    for step in range(2):
        tr.objective.sample_t = lambda n, gen=None, device="cpu": ts[:n]
        tr.train_step({**full, "noise": noise})
    assert torch.allclose(got, tr.arena.data, atol=3e-4), (got - tr.arena.data).abs().max()
