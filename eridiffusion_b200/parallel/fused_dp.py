"""Data parallelism with the communication fused into the optimizer kernel.

The gradient and parameter arenas live in symmetric (peer-mapped) memory. After backward, ONE
cooperative kernel per rank (``csrc/comm.cu: fused_dp_step_kernel``) does

    reduce-scatter (pull peers' gradient shards, fp32 sum, average)
    -> squared-norm exchange -> clip coefficient
    -> block-wise 8-bit AdamW on this rank's shard
    -> all-gather (push the new bf16 parameters into every rank's arena)

so gradients cross NVLink once, parameters cross it once, and no NCCL call, flatten copy or
separate optimizer launch remains. This is the product path for the data-parallel gradient site
the reference leaves as a stub (``DistributedDataParallel::sync_gradients``,
crates/training/src/distributed.rs:284-319); ``GradSync("zero1")`` is the same dataflow through
NCCL and serves as its oracle.

Roofline: each rank receives (W-1)/W of the gradient arena and of the parameter arena and sends
the same, i.e. ``2 * (W-1)/W * arena_bytes`` per direction; at the measured 770 GB/s per direction
that is the floor this step is reported against.
"""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import _native as N
from ..optim.adamw8bit import BLOCK, AdamW8bit
from .symm import Communicator, FusedDpArgs, SymmetricHeap


class FusedDataParallel:
    def __init__(self, pg, arena, optimizer, wait_ms: float = 2000.0):
        if not isinstance(optimizer, AdamW8bit):
            raise TypeError("the fused data-parallel step implements block-wise 8-bit AdamW")
        if arena.data.dtype != torch.bfloat16 or not arena.data.is_cuda:
            raise TypeError("fused data parallelism needs a CUDA bf16 arena")
        self.pg, self.arena, self.opt = pg, arena, optimizer
        self.rank, self.world = pg.rank, pg.world_size
        if arena.numel % (self.world * BLOCK):
            raise ValueError("arena size must be a multiple of world * 256")
        nb = arena.numel * 2
        self.heap = SymmetricHeap(2 * nb + 64 * 1024, group=pg.group)
        self.comm = Communicator(self.heap, wait_ms)
        self.sym_grad = self.heap.tensor((arena.numel,), torch.bfloat16)
        self.sym_param = self.heap.tensor((arena.numel,), torch.bfloat16)
        self.sumsq_slots = self.heap.tensor((16,), torch.float32)
        arena.rebase(self.sym_param.local, self.sym_grad.local)
        self.shard_elems = arena.numel // self.world
        dev = arena.data.device
        self.reduced = torch.empty(self.shard_elems, dtype=torch.float32, device=dev)
        self.sumsq_local = torch.zeros(1, dtype=torch.float32, device=dev)
        self.grad_norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.stamps = None     # set by enable_phase_timing()
        assert optimizer.m_q.numel() == self.shard_elems, "optimizer state must cover this rank's shard"
        torch.cuda.synchronize()
        pg.barrier()

    def step(self, lr, max_grad_norm, step):
        o = self.opt
        a = FusedDpArgs()
        for i in range(self.world):
            a.grads[i] = self.sym_grad.peer_ptrs[i]
            a.params[i] = self.sym_param.peer_ptrs[i]
            a.sumsq_slots[i] = self.sumsq_slots.peer_ptrs[i]
        a.reduced, a.sumsq_local = self.reduced.data_ptr(), self.sumsq_local.data_ptr()
        a.mq, a.vq = o.m_q.data_ptr(), o.v_q.data_ptr()
        a.m_absmax, a.v_absmax = o.m_absmax.data_ptr(), o.v_absmax.data_ptr()
        a.grad_norm_out = self.grad_norm.data_ptr()
        a.shard_elems = self.shard_elems
        a.lr, (a.beta1, a.beta2), a.eps, a.weight_decay = lr, o.betas, o.eps, o.weight_decay
        a.max_grad_norm = max_grad_norm
        a.step, a.seed, a.stochastic = step, o.seed, int(o.stochastic_rounding)
        a.stamps = self.stamps.data_ptr() if self.stamps is not None else None
        o.step_count = step
        c = self.comm.ctx()
        N.check(self.comm.lib.eri_fused_dp_step(C.byref(c), C.byref(a), N.stream_ptr()), "fused_dp_step")

    def status(self) -> int:
        return self.comm.status()

    def enable_phase_timing(self):
        """Record the device timer at the kernel's phase boundaries (thread 0 of CTA 0)."""
        self.stamps = torch.zeros(8, dtype=torch.int64, device=self.arena.data.device)

    def phase_times_us(self) -> dict:
        """Durations of the last step's phases on this rank, in microseconds."""
        t = self.stamps.cpu().tolist()
        names = ["entry_barrier", "reduce_scatter", "norm_exchange", "adamw_and_push", "exit_barrier"]
        return {n: (t[i + 1] - t[i]) / 1e3 for i, n in enumerate(names)}

    def bytes_over_nvlink_per_direction(self) -> int:
        return int(2 * (self.world - 1) / self.world * self.arena.numel * 2)
