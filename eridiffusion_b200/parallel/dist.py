"""Process-group bootstrap and the library (NCCL / gloo) gradient-synchronisation paths.

One process per GPU; rendezvous through the usual environment contract
(``WORLD_SIZE, RANK, LOCAL_RANK, MASTER_ADDR, MASTER_PORT`` — the same variables the reference's
stub parses, crates/training/src/distributed.rs:351-374). The reference's collectives are
placeholders (``all_reduce`` divides by world size, ``all_gather`` clones, ``reduce_scatter``
returns the local slice: distributed.rs:155-183); here they are real, and the API vocabulary
(``ProcessGroup``, ``ReduceOp``, ``split_batch``, ``bucket_cap_bytes``) is kept.

``GradSync`` modes over the flat parameter arena:
  * ``allreduce`` — DDP semantics: average the whole gradient arena, every rank runs the optimizer.
  * ``zero1``     — reduce-scatter the gradient arena, optimizer state and update on this rank's
                    shard only, all-gather the updated parameters (ZeRO-1/2 style).
  * ``fused``     — the same dataflow as ``zero1`` in ONE kernel over NVLink peer memory
                    (``parallel.fused_dp``): reduce-scatter + clip + 8-bit AdamW + all-gather.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from enum import Enum

import torch
import torch.distributed as dist


class ReduceOp(Enum):
    SUM = "sum"
    AVG = "avg"
    MAX = "max"
    MIN = "min"


@dataclass
class DistributedConfig:
    backend: str = "nccl"                 # nccl | gloo
    bucket_cap_bytes: int = 25 * 1024 * 1024
    gradient_as_bucket_view: bool = True
    find_unused_parameters: bool = False
    broadcast_buffers: bool = True
    timeout_s: float = 600.0


def init_from_env(backend: str | None = None, timeout_s: float = 600.0):
    """Initialise ``torch.distributed`` from the environment. Returns (rank, world, local_rank).
    A single-process run (no WORLD_SIZE) returns (0, 1, 0) without creating a group."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1:
        return 0, 1, local
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if not dist.is_initialized():
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return rank, world, local


def split_batch(batch, world: int, rank: int):
    """Slice every tensor of a batch along dim 0 for this rank (distributed.rs:335-343)."""
    def cut(t):
        n = t.shape[0]
        per = (n + world - 1) // world
        return t[rank * per:min(n, (rank + 1) * per)]
    if torch.is_tensor(batch):
        return cut(batch)
    return {k: (cut(v) if torch.is_tensor(v) and v.dim() > 0 else v) for k, v in batch.items()}


class ProcessGroup:
    """Thin collective facade used by the trainer, metrics aggregation and tests."""

    def __init__(self, group=None):
        self.group = group
        self.initialized = dist.is_initialized()
        self.rank = dist.get_rank(group) if self.initialized else 0
        self.world_size = dist.get_world_size(group) if self.initialized else 1

    def all_reduce(self, t, op: ReduceOp = ReduceOp.SUM):
        if self.world_size == 1:
            return t
        if op == ReduceOp.AVG:
            if t.is_cuda:
                dist.all_reduce(t, dist.ReduceOp.AVG, group=self.group)
            else:
                dist.all_reduce(t, dist.ReduceOp.SUM, group=self.group)
                t.div_(self.world_size)
            return t
        m = {ReduceOp.SUM: dist.ReduceOp.SUM, ReduceOp.MAX: dist.ReduceOp.MAX, ReduceOp.MIN: dist.ReduceOp.MIN}
        dist.all_reduce(t, m[op], group=self.group)
        return t

    def broadcast(self, t, src=0):
        if self.world_size > 1:
            dist.broadcast(t, src, group=self.group)
        return t

    def all_gather(self, t):
        if self.world_size == 1:
            return [t]
        out = [torch.empty_like(t) for _ in range(self.world_size)]
        dist.all_gather(out, t, group=self.group)
        return out

    def all_gather_into(self, out, t):
        if self.world_size == 1:
            out.copy_(t)
            return out
        if t.is_cuda:
            dist.all_gather_into_tensor(out, t, group=self.group)
        else:
            parts = list(out.chunk(self.world_size))
            dist.all_gather(parts, t, group=self.group)
        return out

    def reduce_scatter_into(self, out, t, avg=True):
        if self.world_size == 1:
            out.copy_(t)
            return out
        if t.is_cuda:
            dist.reduce_scatter_tensor(out, t, dist.ReduceOp.AVG if avg else dist.ReduceOp.SUM, group=self.group)
        else:
            tmp = t.clone()
            dist.all_reduce(tmp, dist.ReduceOp.SUM, group=self.group)
            n = out.numel()
            out.copy_(tmp[self.rank * n:(self.rank + 1) * n])
            if avg:
                out.div_(self.world_size)
        return out

    def all_to_all_single(self, out, t):
        if self.world_size == 1:
            out.copy_(t)
            return out
        if t.is_cuda:
            dist.all_to_all_single(out, t, group=self.group)
        else:
            ins = list(t.chunk(self.world_size))
            outs = list(out.chunk(self.world_size))
            gathered = [None] * self.world_size
            for r in range(self.world_size):          # gloo lacks all_to_all: emulate with gathers
                parts = [torch.empty_like(ins[r]) for _ in range(self.world_size)]
                dist.all_gather(parts, ins[r], group=self.group)
                if r == self.rank:
                    gathered = parts
            for r in range(self.world_size):
                outs[r].copy_(gathered[r])
        return out

    def barrier(self):
        if self.world_size > 1:
            dist.barrier(group=self.group)


class GradSync:
    def __init__(self, mode: str = "allreduce", group=None):
        self.pg = ProcessGroup(group)
        self.rank, self.world_size = self.pg.rank, self.pg.world_size
        if mode not in ("allreduce", "zero1", "fused"):
            raise ValueError(mode)
        self.mode = mode
        self.fused_optimizer = False
        self.arena = self.optimizer = None
        self._fused = None

    def optimizer_shard(self):
        return None if self.mode == "allreduce" or self.world_size == 1 else (self.rank, self.world_size)

    def attach(self, arena, optimizer):
        self.arena, self.optimizer = arena, optimizer
        # all ranks start from rank 0's parameters (distributed.rs:322-327 broadcast_parameters)
        self.pg.broadcast(arena.data, 0)
        if self.mode == "fused" and self.world_size > 1:
            from .fused_dp import FusedDataParallel
            self._fused = FusedDataParallel(self.pg, arena, optimizer)
            self.fused_optimizer = True

    @property
    def sharded(self):
        return self.mode != "allreduce" and self.world_size > 1

    def reduce_grads(self):
        if self.world_size == 1:
            return
        if self.mode == "allreduce":
            self.pg.all_reduce(self.arena.grad, ReduceOp.AVG)
        else:
            _, gshard = self.arena.shard(self.rank, self.world_size)
            self.pg.reduce_scatter_into(gshard, self.arena.grad, avg=True)

    def grad_sumsq(self, out=None):
        """Squared global gradient norm as a device scalar (after ``reduce_grads``)."""
        from ..ops import functional as F
        if not self.sharded:
            return F.sumsq(self.arena.grad, out)
        _, gshard = self.arena.shard(self.rank, self.world_size)
        ss = F.sumsq(gshard, out)
        self.pg.all_reduce(ss, ReduceOp.SUM)
        return ss

    def gather_params(self):
        if not self.sharded:
            return
        pshard, _ = self.arena.shard(self.rank, self.world_size)
        self.pg.all_gather_into(self.arena.data, pshard)

    def reduce_and_step(self, lr, max_grad_norm, step):
        self._fused.step(lr=lr, max_grad_norm=max_grad_norm, step=step)


class MetricsAggregator:
    """Average scalar metrics over ranks (the reference's ``MetricsAggregator`` "would use
    all-reduce": crates/training/src/metrics.rs:199-230)."""

    def __init__(self, pg: ProcessGroup | None = None):
        self.pg = pg or ProcessGroup()

    def aggregate(self, metrics: dict, device="cpu"):
        keys = sorted(metrics)
        t = torch.tensor([float(metrics[k]) for k in keys], dtype=torch.float64 if device == "cpu" else torch.float32,
                         device=device)
        self.pg.all_reduce(t, ReduceOp.AVG)
        return {k: float(v) for k, v in zip(keys, t.tolist())}
