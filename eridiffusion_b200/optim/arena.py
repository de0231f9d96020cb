"""Flat parameter arena.

All trainable parameters of a run live in ONE contiguous buffer (and their gradients in a second
one); each ``nn.Parameter`` is re-pointed to a view. Every per-tensor loop of the reference
(global-norm clipping with one device->host copy per tensor, crates/training/src/optimizer.rs:88-123;
per-parameter optimizer updates, src/trainers/pipeline_flux_lora_sequential.rs:749-794; DDP bucket
flattening, crates/training/src/distributed.rs:284-319) becomes a single launch over the arena,
and the data-parallel reduce-scatter operates on the same buffer without a flatten copy.

Each parameter is padded to a multiple of ``align`` elements (256 = the optimizer's quantisation
block), so quantisation blocks never straddle two tensors and shards can be cut on block edges.
"""
from __future__ import annotations

import torch


class ParamArena:
    def __init__(self, params, align: int = 256, shard_multiple: int = 1, alloc=None):
        """``alloc(numel, dtype, device) -> 1-D tensor`` lets the caller place the two buffers
        (e.g. in symmetric peer-mapped memory); default is ``torch.zeros``."""
        params = [p for p in params if p.requires_grad]
        if not params:
            raise ValueError("no trainable parameters")
        dt, dev = params[0].dtype, params[0].device
        for p in params:
            if p.dtype != dt or p.device != dev:
                raise ValueError("arena parameters must share dtype and device")
        self.params = params
        self.align = align
        self.offsets, off = [], 0
        for p in params:
            self.offsets.append(off)
            off += (p.numel() + align - 1) // align * align
        unit = align * max(1, shard_multiple)
        self.numel = (off + unit - 1) // unit * unit
        mk = alloc or (lambda n, dtype, device: torch.zeros(n, dtype=dtype, device=device))
        self.data = mk(self.numel, dt, dev)
        self.grad = mk(self.numel, dt, dev)
        self.data.zero_()
        self.grad.zero_()
        with torch.no_grad():
            for p, o in zip(params, self.offsets):
                n = p.numel()
                self.data[o:o + n].copy_(p.detach().reshape(-1))
                p.data = self.data[o:o + n].view(p.shape)
                p.grad = self.grad[o:o + n].view(p.shape)

    def rebase(self, new_data: torch.Tensor, new_grad: torch.Tensor):
        """Move the arena into caller-provided buffers (e.g. symmetric peer-mapped memory) and
        re-point every parameter and gradient view."""
        assert new_data.numel() == self.numel and new_grad.numel() == self.numel
        with torch.no_grad():
            new_data.copy_(self.data)
            new_grad.copy_(self.grad)
            self.data, self.grad = new_data, new_grad
            for p, o in zip(self.params, self.offsets):
                n = p.numel()
                p.data = self.data[o:o + n].view(p.shape)
                p.grad = self.grad[o:o + n].view(p.shape)

    def zero_grad(self):
        self.grad.zero_()

    def rebind_grads(self):
        """Re-attach ``.grad`` views (after something set them to None)."""
        for p, o in zip(self.params, self.offsets):
            if p.grad is None or p.grad.data_ptr() != self.grad[o:].data_ptr():
                p.grad = self.grad[o:o + p.numel()].view(p.shape)

    def shard(self, rank: int, world: int):
        n = self.numel // world
        return self.data[rank * n:(rank + 1) * n], self.grad[rank * n:(rank + 1) * n]

    def named_slices(self, names):
        return {n: (o, p.numel(), tuple(p.shape)) for n, p, o in zip(names, self.params, self.offsets)}


def block_lr_scale(arena: ParamArena, names, rules: dict | None = None, frozen=None, block: int = 256,
                   shard=None):
    """Per-block learning-rate multipliers for an arena-based optimizer (fp32 [numel / block]).

    ``rules``: ``{substring: multiplier}`` — a parameter takes the multiplier of the first rule its
    name contains (the reference's ``lr_if_contains``, crates/training/src/chroma/train.rs:98).
    ``frozen``: a predicate ``name -> bool``; frozen parameters get multiplier 0 (their values and
    optimizer moments stay untouched). ``shard = (rank, world)`` returns this rank's slice."""
    scale = torch.ones(arena.numel // block, dtype=torch.float32)
    for name, p, off in zip(names, arena.params, arena.offsets):
        mult = 1.0
        for sub, m in (rules or {}).items():
            if sub in name:
                mult = float(m)
                break
        if frozen is not None and frozen(name):
            mult = 0.0
        n_blocks = (p.numel() + block - 1) // block
        scale[off // block: off // block + n_blocks] = mult
    if shard is not None:
        rank, world = shard
        per = scale.numel() // world
        scale = scale[rank * per:(rank + 1) * per]
    return scale.to(arena.data.device)
