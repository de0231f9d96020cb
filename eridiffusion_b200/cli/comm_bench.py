"""Multi-GPU timing of the fused communication paths against their rooflines and against NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m eridiffusion_b200.cli.comm_bench [--params 56000000]

Times are CUDA-event device times, max over ranks, median of the timed launches after warm-up.
Roofline of the fused data-parallel step: bytes that must cross NVLink per direction,
``2 * (W-1)/W * arena_bytes``, over the measured 770 GB/s per direction (900 nominal).
"""
from __future__ import annotations

import argparse
import json
import statistics

import torch
import torch.distributed as dist

from ..ops import functional as F
from ..optim import AdamW8bit, ParamArena
from ..parallel.dist import GradSync, ProcessGroup, init_from_env
from ..parallel.fused_dp import FusedDataParallel

LINK_GBS = 770.0


def timed(fn, iters=10, warm=3):
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    t = torch.tensor([statistics.median(ts)], device="cuda")
    dist.all_reduce(t, dist.ReduceOp.MAX)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--params", type=int, default=56_000_000)
    a = ap.parse_args()
    rank, world, local = init_from_env()
    dev = torch.device("cuda", local)
    pg = ProcessGroup()
    n = a.params // (256 * world) * (256 * world)
    p = [torch.nn.Parameter(torch.randn(n, device=dev).bfloat16() * 0.02)]
    arena = ParamArena(p, shard_multiple=world)
    opt = AdamW8bit(arena, lr=1e-4, shard=(rank, world) if world > 1 else (0, 1))
    fdp = FusedDataParallel(pg, arena, opt)
    arena.grad.normal_()
    step = [0]

    def fused():
        step[0] += 1
        fdp.step(lr=1e-4, max_grad_norm=1.0, step=step[0])

    t_f = timed(fused)
    st = fdp.status()
    fdp.enable_phase_timing()
    dist.barrier()
    torch.cuda.synchronize()
    fused()
    torch.cuda.synchronize()
    phases = fdp.phase_times_us()
    fdp.stamps = None
    # NCCL + separate kernels: reduce-scatter, norm all-reduce, optimizer on shard, all-gather
    p2 = [torch.nn.Parameter(torch.randn(n, device=dev).bfloat16() * 0.02)]
    arena2 = ParamArena(p2, shard_multiple=world)
    opt2 = AdamW8bit(arena2, lr=1e-4, shard=(rank, world) if world > 1 else None)
    gs = GradSync("zero1")
    gs.attach(arena2, opt2)
    arena2.grad.normal_()

    def nccl():
        gs.reduce_grads()
        ss = gs.grad_sumsq()
        opt2.step(grad_sumsq=ss, max_grad_norm=1.0)
        gs.gather_params()

    t_n = timed(nccl)
    if rank == 0:
        nbytes = fdp.bytes_over_nvlink_per_direction()
        roof_ms = nbytes / (LINK_GBS * 1e9) * 1e3
        hbm_ms = 0.0
        print(json.dumps({"what": "fused_dp_step (reduce-scatter + clip + adamw8bit + all-gather)",
                          "world": world, "params": n, "fused_ms": round(t_f, 4), "nccl_path_ms": round(t_n, 4),
                          "nvlink_bytes_per_direction": nbytes, "roofline_ms": round(roof_ms, 4),
                          "fraction_of_roofline": round(roof_ms / t_f, 3) if world > 1 else None,
                          "link_gbs_used": LINK_GBS, "status": st,
                          "phases_us_rank0": {k: round(v, 1) for k, v in phases.items()}}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
