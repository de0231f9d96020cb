"""Activation checkpointing policies and TREAD token routing.

Checkpointing (crates/training/src/gradient_checkpointing.rs:12-140,
src/trainers/gpu_gradient_checkpoint.rs:165-188): ``recompute`` re-runs a block in backward,
``cpu_offload`` parks the block input in pinned host memory on a side stream and fetches it back
before backward, ``adaptive`` chooses per block from the free device memory. On a 180 GB device
the flagship configurations run with checkpointing off; the policies exist for larger batches.

TREAD (crates/training/src/tread.rs:140-248; config ``tread.mask / schedule / reinject``): between
layer ``out`` and layer ``in`` only a subset of the image tokens is carried (top-k by L2 norm,
random or uniform stride); at ``in`` the routed tokens are scattered back into the full sequence.
Selection runs on the device (the reference computes its top-k on the host).
"""
from __future__ import annotations

import torch
import torch.utils.checkpoint as ckpt

from ..ops import functional as F


class _OffloadStore:
    """Pinned-host parking lot for block inputs (one buffer per slot, reused every step)."""

    def __init__(self):
        self.bufs = {}
        self.stream = torch.cuda.Stream() if torch.cuda.is_available() else None

    def park(self, slot, t):
        if not t.is_cuda:
            return t, None
        buf = self.bufs.get(slot)
        if buf is None or buf.shape != t.shape or buf.dtype != t.dtype:
            buf = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
            self.bufs[slot] = buf
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            buf.copy_(t, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        return buf, ev

    def fetch(self, buf, ev, device):
        if ev is None:
            return buf
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ev)
            out = buf.to(device, non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.stream)
        torch.cuda.current_stream().wait_event(done)
        return out


_STORE = _OffloadStore()


class _OffloadedBlock(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, slot, x, *rest):
        ctx.fn, ctx.rest, ctx.device = fn, rest, x.device
        ctx.host, ctx.ev = _STORE.park(slot, x.detach())
        with torch.no_grad():
            return fn(x, *rest)

    @staticmethod
    def backward(ctx, dy):
        x = _STORE.fetch(ctx.host, ctx.ev, ctx.device).detach().requires_grad_()
        with torch.enable_grad():
            y = ctx.fn(x, *ctx.rest)
        torch.autograd.backward(y, dy)
        return (None, None, x.grad) + (None,) * len(ctx.rest)


def run_block(fn, x, *rest, policy="none", slot=0):
    """policy: none | recompute | cpu_offload | adaptive."""
    if policy == "adaptive":
        if x.is_cuda:
            free, total = torch.cuda.mem_get_info(x.device)
            policy = "none" if free > 0.3 * total else ("recompute" if free > 0.1 * total else "cpu_offload")
        else:
            policy = "none"
    if policy == "none" or not torch.is_grad_enabled():
        return fn(x, *rest)
    if policy == "recompute":
        return ckpt.checkpoint(fn, x, *rest, use_reentrant=False)
    if policy == "cpu_offload":
        return _OffloadedBlock.apply(fn, slot, x, *rest)
    raise ValueError(policy)


def checkpointed_forward(model, img, txt, t, y, guidance, policy="recompute"):
    """MMDiT forward with every block under ``policy`` (used by ``TrainerConfig.activation_checkpointing``)."""
    from ..models.layers import timestep_embedding
    from ..ops import functional as F
    cfg = model.cfg
    dt = model.img_in.weight.dtype
    B, Li, _ = img.shape
    Lt = txt.shape[1]
    s = int(round(Li ** 0.5))
    vec = model.time_in(timestep_embedding(t, cfg.time_embed_dim).to(dt))
    if model.guidance_in is not None:
        g = guidance if guidance is not None else torch.ones_like(t)
        vec = vec + model.guidance_in(timestep_embedding(g, cfg.time_embed_dim).to(dt))
    if model.vector_in is not None:
        vec = vec + model.vector_in(y.to(dt))
    cos, sin = model.rope(Lt, s, Li // s, img.device)
    x = model.img_in(img)
    if model.txt_norm is not None:
        txt = F.norm_modulate(txt, weight=model.txt_norm.scale, rms=True)
    c = model.txt_in(txt)
    for i, blk in enumerate(model.double_blocks):
        x, c = ckpt.checkpoint(blk, x, c, vec, cos, sin, use_reentrant=False) if policy == "recompute" \
            else blk(x, c, vec, cos, sin)
    if len(model.single_blocks) == 0:
        return model.final_layer(x, vec)
    h = torch.cat((c, x), dim=1)
    for i, blk in enumerate(model.single_blocks):
        h = run_block(blk, h, vec, cos, sin, policy=policy, slot=i)
    return model.final_layer(h[:, Lt:], vec)


# ------------------------------------------------------------------------------ TREAD routing
def tread_select(x, k=None, k_frac=0.5, mask_type="topk_norm", gen=None):
    """x [B, L, D] -> indices [B, k] (sorted) of the tokens to keep."""
    B, L, _ = x.shape
    k = k or max(1, int(L * k_frac))
    if mask_type in ("topk_norm", "attn_topk"):
        # scoring and selection stay on the device (row-norm kernel + in-kernel bitonic top-k)
        idx = F.topk_indices(F.token_scores(x), k)
    elif mask_type == "random":
        idx = torch.rand(B, L, device=x.device, generator=gen).topk(k, dim=1).indices
    elif mask_type == "uniform":
        idx = torch.linspace(0, L - 1, k, device=x.device).round().long().unsqueeze(0).expand(B, k)
    else:
        raise ValueError(mask_type)
    return idx.sort(dim=1).values


def tread_gather(x, idx):
    return F.gather_rows(x, idx)


def tread_reinject(full, routed, idx, mode="scatter"):
    """Put the routed tokens back at their positions; the other positions keep the value they had
    when routing started (``scatter``) or are zeroed (``zero``)."""
    base = full if mode == "scatter" else torch.zeros_like(full)
    return F.reinject_rows(base, routed, idx)


class TreadRouter:
    """Applies a ``schedule`` [{out: i, in: j}, ...] to a list of blocks that map x -> x."""

    def __init__(self, schedule, k=None, k_frac=0.5, mask_type="topk_norm", reinject="scatter"):
        self.schedule = {int(p["out"]): int(p["in"]) for p in schedule}
        self.k, self.k_frac, self.mask_type, self.reinject = k, k_frac, mask_type, reinject
        self.kept_frac = {}

    def run(self, blocks, x, step, rope=None):
        """``step(block, x, cos, sin) -> x``; ``rope`` = (cos, sin) rows follow the routed tokens."""
        active = None          # (resume_layer, idx, saved_full)
        for i, blk in enumerate(blocks):
            if active is not None and i == active[0]:
                x = tread_reinject(active[2], x, active[1], self.reinject)
                active = None
            if active is None and i in self.schedule and self.schedule[i] > i:
                idx = tread_select(x, self.k, self.k_frac, self.mask_type)
                active = (self.schedule[i], idx, x)
                x = tread_gather(x, idx)
                self.kept_frac[i] = idx.shape[1] / active[2].shape[1]
            if rope is not None and active is not None:
                c = rope[0][active[1][0]]
                s = rope[1][active[1][0]]
                x = step(blk, x, c, s)
            else:
                x = step(blk, x, *(rope or (None, None)))
        if active is not None:
            x = tread_reinject(active[2], x, active[1], self.reinject)
        return x
