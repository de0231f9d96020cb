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
    """Applies a ``schedule`` [{out: i, in: j}, ...] to a list of blocks that map x -> x.

    ``keep_prefix``: the first tokens of the sequence (the text tokens of a joint [text | image]
    stream) are never routed out; the selection runs over the remaining tokens only. When a rotary
    table accompanies the tokens, every sample of the micro-batch routes the SAME positions (scores
    are averaged over the batch) so that one table slice serves the whole batch."""

    def __init__(self, schedule, k=None, k_frac=0.5, mask_type="topk_norm", reinject="scatter"):
        self.schedule = {int(p["out"]): int(p["in"]) for p in schedule}
        self.k, self.k_frac, self.mask_type, self.reinject = k, k_frac, mask_type, reinject
        self.kept_frac = {}

    def _select(self, x, keep_prefix, shared):
        body = x[:, keep_prefix:]
        if shared and body.shape[0] > 1 and self.mask_type in ("topk_norm", "attn_topk"):
            L = body.shape[1]
            k = self.k or max(1, int(L * self.k_frac))
            score = body.float().pow(2).sum(-1).mean(0, keepdim=True)
            idx = score.topk(k, dim=1).indices.sort(dim=1).values.expand(body.shape[0], k)
        else:
            idx = tread_select(body, self.k, self.k_frac, self.mask_type)
            if shared and body.shape[0] > 1:
                idx = idx[:1].expand(body.shape[0], idx.shape[1])
        if keep_prefix:
            pre = torch.arange(keep_prefix, device=x.device).unsqueeze(0).expand(x.shape[0], keep_prefix)
            idx = torch.cat([pre, idx + keep_prefix], dim=1)
        return idx.contiguous()

    def run(self, blocks, x, step, rope=None, keep_prefix=0):
        """``step(block, x, cos, sin) -> x``; ``rope`` = (cos, sin) rows follow the routed tokens."""
        active = None          # (resume_layer, idx, saved_full)
        for i, blk in enumerate(blocks):
            if active is not None and i == active[0]:
                x = tread_reinject(active[2], x, active[1], self.reinject)
                active = None
            if active is None and i in self.schedule and self.schedule[i] > i:
                idx = self._select(x, keep_prefix, shared=rope is not None)
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


# ------------------------------------------------------------------------------ layer streaming
class _StreamedBlock(torch.autograd.Function):
    """One block of a streamed stack: forward runs without an autograd graph while the block's
    frozen weights are resident (``BlockSwapManager`` window), backward makes them resident again,
    re-runs the block with a graph and back-propagates through it. Streaming therefore implies
    recomputation; the trainable adapter tensors are ordinary leaves and receive their gradients
    from the inner backward (src/trainers/flux_layer_streaming.rs:395-771 streams per layer in both
    directions the same way)."""

    @staticmethod
    def forward(ctx, mgr, idx, fn, n_args, *rest):
        # rest = the block's call arguments followed by its trainable tensors. The latter are not
        # used here; they are inputs so that autograd knows the output depends on them even when no
        # activation requires a gradient yet (first block behind a frozen input projection).
        args = rest[:n_args]
        ctx.mgr, ctx.idx, ctx.fn, ctx.n_args, ctx.n_rest = mgr, idx, fn, n_args, len(rest)
        ctx.is_tensor = [torch.is_tensor(a) for a in args]
        ctx.consts = [None if torch.is_tensor(a) else a for a in args]
        ctx.save_for_backward(*[a for a in args if torch.is_tensor(a)])
        with torch.no_grad():
            out = mgr.run(idx, lambda b: fn(b, *args))
        ctx.tuple_out = isinstance(out, tuple)
        return out

    @staticmethod
    def backward(ctx, *douts):
        it = iter(ctx.saved_tensors)
        args = []
        for flag, const, need in zip(ctx.is_tensor, ctx.consts, ctx.needs_input_grad[4:4 + ctx.n_args]):
            if flag:
                t = next(it).detach()
                if need and t.is_floating_point():
                    t.requires_grad_()
                args.append(t)
            else:
                args.append(const)
        with torch.enable_grad():
            out = ctx.mgr.run(ctx.idx, lambda b: ctx.fn(b, *args), direction=-1)
        outs = out if ctx.tuple_out else (out,)
        pairs = [(o, g) for o, g in zip(outs, douts) if g is not None and o.requires_grad]
        # the trainable tensors are leaves: this inner backward adds to their .grad directly
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        grads = [a.grad if (torch.is_tensor(a) and a.requires_grad) else None for a in args]
        return (None, None, None, None, *grads, *([None] * (ctx.n_rest - ctx.n_args)))


def _streamed(mgr, idx, blk, *args):
    params = [p for p in blk.parameters() if p.requires_grad]
    return _StreamedBlock.apply(mgr, idx, lambda b, *a: b(*a), len(args), *args, *params)


class BlockRunner:
    """How the blocks of an MMDiT-style stack execute during training. A model consults its
    ``runner`` (when one is attached) instead of calling the blocks directly:

    * ``policy``: activation handling per block — ``none``, ``recompute``, ``cpu_offload`` (block
      inputs parked in pinned host memory), ``adaptive`` (crates/training/src/gradient_checkpointing.rs:
      76-140, src/trainers/gpu_gradient_checkpoint.rs:165-188);
    * ``streamer``: a ``memory.BlockSwapManager`` over ALL blocks (double first, then single): frozen
      weights live in pinned host memory and a window of blocks is resident (layer streaming with
      persistent blocks, src/trainers/flux_layer_streaming.rs:65-131);
    * ``tread``: a ``TreadRouter`` applied to the single-stream stack, text tokens always kept
      (crates/training/src/tread.rs:140-248).
    """

    def __init__(self, policy="none", streamer=None, tread=None):
        self.policy, self.streamer, self.tread = policy, streamer, tread

    def double(self, i, blk, img, txt, vec, cos, sin):
        if self.streamer is not None and torch.is_grad_enabled():
            return _streamed(self.streamer, i, blk, img, txt, vec, cos, sin)
        if self.streamer is not None:
            return self.streamer.run(i, lambda b: b(img, txt, vec, cos, sin))
        if self.policy != "none" and torch.is_grad_enabled():
            return ckpt.checkpoint(blk, img, txt, vec, cos, sin, use_reentrant=False)
        return blk(img, txt, vec, cos, sin)

    def _single(self, i, blk, x, vec, cos, sin):
        if self.streamer is not None and torch.is_grad_enabled():
            return _streamed(self.streamer, i, blk, x, vec, cos, sin)
        if self.streamer is not None:
            return self.streamer.run(i, lambda b: b(x, vec, cos, sin))
        return run_block(blk, x, vec, cos, sin, policy=self.policy, slot=i)

    def single_stack(self, blocks, x, vec, cos, sin, txt_len, first_index=0):
        index = {id(b): first_index + j for j, b in enumerate(blocks)}
        step = lambda blk, h, c, s: self._single(index[id(blk)], blk, h, vec, c, s)
        if self.tread is not None and torch.is_grad_enabled():
            return self.tread.run(list(blocks), x, step, rope=(cos, sin) if cos is not None else None,
                                  keep_prefix=txt_len)
        for blk in blocks:
            x = step(blk, x, cos, sin)
        return x
