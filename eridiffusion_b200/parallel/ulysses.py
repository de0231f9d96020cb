"""Ulysses sequence parallelism with both all-to-alls folded into the projections.

Tokens are sharded over W ranks (L_local each); attention needs every token of a head, so heads are
re-sharded around it:

* ``ulysses_qkv``: the QKV projection's epilogue stores each head group's output tile directly into
  the owning rank's receive buffer over NVLink (``scatter`` epilogue of ``csrc/gemm.cu``) — the
  forward all-to-all costs no extra pass and no staging buffer. With QK-norm across heads the
  epilogue also accumulates each row's sum of squares, and the receiver applies the norm
  (``dist_rmsnorm``).
* attention runs on [B, W*L_local, H/W, Dh] with the tcgen05 flash kernel.
* ``ulysses_out_proj``: the out-projection launch gathers its A operand — column block p of
  [L_local, H*Dh] comes from peer p's attention output — with copy CTAs inside the same launch;
  K blocks are consumed as they land, starting with the local block.

Backward mirrors this: the gradient of the gathered operand is produced by a GEMM with the scatter
epilogue, and the gradient of the scattered output is consumed by a GEMM with the column gather.
LoRA adapters on either projection ride along as the rank-r K step of the same launches.
The reference has no sequence parallelism; its long-sequence mechanism is single-GPU chunked
attention (crates/training/src/sdxl/runtime.rs:2814-3025).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import functional as F
from .dist import ProcessGroup
from .gather_gemm import GatherPlan
from .symm import Communicator, SymmetricHeap


class UlyssesContext:
    def __init__(self, pg: ProcessGroup | None, batch: int, l_local: int, hidden: int, heads: int,
                 n_copy: int = 16, wait_ms: float = 2000.0, attn_slots: int = 1):
        self.pg = pg or ProcessGroup()
        self.rank, self.world = self.pg.rank, self.pg.world_size
        W = self.world
        assert heads % W == 0
        self.B, self.Ll, self.D, self.H = batch, l_local, hidden, heads
        self.G = hidden // W                       # columns of one rank's head group
        self.Lt = W * l_local
        nb = batch * self.Lt * 3 * self.G * 2
        self.heap = SymmetricHeap(4 * nb + max(0, attn_slots - 1) * (nb // 3 + 4096) + (4 << 20),
                                  group=self.pg.group)
        self.comm = Communicator(self.heap, wait_ms)
        self.n_copy = n_copy
        # receive buffers (symmetric): qkv forward, attention output, and their gradients
        self.recv_qkv = self.heap.tensor((batch * self.Lt, 3 * self.G), torch.bfloat16)
        # Attention outputs that peers read. One slot per layer lets the attention kernel write its
        # output where the peers fetch it (no publish copy) while autograd keeps it for backward.
        self.attn_outs = [self.heap.tensor((batch * self.Lt, self.G), torch.bfloat16)
                          for _ in range(max(1, attn_slots))]
        self.attn_out = self.attn_outs[0]
        self._slot_of = {t.local.data_ptr(): t for t in self.attn_outs}
        self.d_recv_qkv = self.heap.tensor((batch * self.Lt, 3 * self.G), torch.bfloat16)
        self.d_attn_out = self.heap.tensor((batch * self.Lt, self.G), torch.bfloat16)
        self._plans = {}
        self.nvlink_bytes = 0

    def barrier(self):
        if self.world > 1:
            self.comm.collective("barrier", self.recv_qkv, count=0)

    def attn_buffer(self, slot: int, heads_local: int):
        """[B, W*L_local, H/W, Dh] view of attention-output slot ``slot`` (None when the context
        has fewer slots): pass it as ``out=`` to the attention call of layer ``slot``."""
        if len(self.attn_outs) < 2 or slot >= len(self.attn_outs):
            return None                  # a single slot is the staging buffer of the publish copy
        # Not a view of the heap tensor: views share one version counter, and autograd would see
        # layer i's saved output "modified" when layer i+1 writes its own slot. ``set_`` gives a
        # tensor over the same memory with a version counter of its own; a fresh one per call, so
        # that no autograd history of an earlier step hangs on it.
        base = self.attn_outs[slot].local
        t = torch.empty(0, dtype=base.dtype, device=base.device)
        t.set_(base.untyped_storage(), base.storage_offset(),
               (self.B, self.Lt, heads_local, self.G // heads_local))
        return t

    def cols_plan(self, key, src_sym, parts, landing):
        """landing [B*Ll, parts*W*G]: for each part, column block p comes from peer p's rows of
        this rank's tokens in ``src_sym`` ([B*Lt, parts*G])."""
        k = (key, landing.data_ptr())
        pl = self._plans.get(k)
        if pl is None:
            W, G = self.world, self.G
            # counters per 128-row group need the jobs' rows to line up with the GEMM's M tiles
            fine = self.B == 1 or self.Ll % 128 == 0
            groups = (self.B * self.Ll + 127) // 128 if fine else 1
            pl = GatherPlan(self.rank, W, self.n_copy, landing.device, n_flags=parts * W * groups)
            es = 2
            src_stride = parts * G * es
            order = [(self.rank + i) % W for i in range(W)]
            for b in range(self.B):
                for r0 in range(0, self.Ll, 128):
                    nr = min(128, self.Ll - r0)
                    for p in order:
                        for part in range(parts):
                            src = src_sym.peer_ptrs[p] + ((b * self.Lt + self.rank * self.Ll + r0) * parts * G + part * G) * es
                            dst = landing.data_ptr() + ((b * self.Ll + r0) * landing.stride(0) + part * W * G + p * G) * es
                            pl._add(src, dst, nr, G * es, src_stride, landing.stride(0) * es,
                                    (part * W + p) * groups + ((b * self.Ll + r0) // 128 if fine else 0),
                                    remote=p != self.rank)
            # K blocks are ordered [part][peer]; one counter per (part, peer, 128-row group)
            pl.kw = dict(a_flag_cols=G, rot_k_cols=self.rank * G, a_flag_rows=128 if fine else 0)
            if parts == 1 and self.B == 1:
                # this rank's own column block is read from its home buffer, not copied
                pl.local = dict(ptr=src_sym.peer_ptrs[self.rank] + self.rank * self.Ll * G * es, ld=G, mode=3,
                                lo=self.rank * G, hi=(self.rank + 1) * G)
            pl._finish()
            self._plans[k] = pl
        return pl

    def scatter_args(self, sym, rowsq=None):
        return dict(world=self.world, rank=self.rank, part_cols=self.D, group_cols=self.G,
                    local_rows=self.Ll, ptrs=sym.peer_ptrs, rowsq=rowsq)


def _t(x):
    return x.t().contiguous()


class _UlyssesQKV(torch.autograd.Function):
    """x [B, Ll, D] -> recv [B, W*Ll, 3, G] on every rank (this rank's head group, all tokens)."""

    @staticmethod
    def forward(ctx, x, w, bias, la, lb, ls, u, want_rowsq):
        B, Ll, D = x.shape
        x2 = x.contiguous().view(B * Ll, D)
        W = u.world
        rowsq = torch.zeros(2, B * Ll, dtype=torch.float32, device=x.device) if want_rowsq else None
        h = F.gemm_native(x2, la, alpha=ls) if la is not None else None
        u.barrier()           # receivers are done with the previous contents of recv_qkv
        F.gemm_native(x2, w, bias=bias, out=u.recv_qkv.local, lora_h=h, lora_b=lb,
                      scatter=u.scatter_args(u.recv_qkv, rowsq))
        u.barrier()           # every rank's tiles have landed
        u.nvlink_bytes += x2.shape[0] * 3 * D * 2 * (W - 1) // W
        ctx.save_for_backward(x2, w, la, lb, h)
        ctx.u, ctx.shape, ctx.has_bias, ctx.ls = u, (B, Ll, D), bias is not None, ls
        out = u.recv_qkv.local.view(B, u.Lt, 3, u.G).clone()
        if want_rowsq:
            ctx.mark_non_differentiable(rowsq)
            return out, rowsq
        return out, None

    @staticmethod
    def backward(ctx, d_recv, _):
        x2, w, la, lb, h = ctx.saved_tensors
        u = ctx.u
        B, Ll, D = ctx.shape
        # publish the gradient of what this rank received, then gather dY[:, part, peer-block]
        u.barrier()
        u.d_recv_qkv.local.copy_(d_recv.reshape(B * u.Lt, 3 * u.G))
        u.barrier()
        dY = torch.empty(B * Ll, 3 * D, dtype=x2.dtype, device=x2.device)
        pl = u.cols_plan("dqkv", u.d_recv_qkv, 3, dY)
        da = db_ = None
        if la is not None:
            ts = F.gemm_native(dY, _t(lb), alpha=ctx.ls, gather=pl.launch_args())   # lands dY
            dx = F.gemm_native(dY, w, b_mn=True, lora_h=ts, lora_b=_t(la))
            da = F.lora_wgrad(x2, ts, transpose_out=True) if ctx.needs_input_grad[3] else None
            db_ = F.lora_wgrad(dY, h) if ctx.needs_input_grad[4] else None
        else:
            dx = F.gemm_native(dY, w, b_mn=True, gather=pl.launch_args())           # lands dY
        dw = F.wgrad(dY, x2) if ctx.needs_input_grad[1] else None
        db = dY.sum(0) if (ctx.has_bias and ctx.needs_input_grad[2]) else None
        return dx.view(B, Ll, D), dw, db, da, db_, None, None, None


class _UlyssesOutProj(torch.autograd.Function):
    """attn [B, W*Ll, G] (this rank's heads, all tokens) -> y [B, Ll, D] = A Wo^T (+b, gate, res),
    A[:, p-block] taken from peer p."""

    @staticmethod
    def forward(ctx, attn, w, bias, la, lb, ls, u, residual, gate, keep_a=True):
        B, Ll, D = u.B, u.Ll, u.D
        W = u.world
        sym = u._slot_of.get(attn.data_ptr()) if len(u.attn_outs) > 1 else None
        if sym is None:
            sym = u.attn_out
            u.barrier()           # peers are done reading the previous contents
            sym.local.copy_(attn.reshape(B * u.Lt, u.G))
        # with a slot per layer the attention kernel wrote straight into ``sym``; peers finished
        # reading this slot's previous contents (last step) many barriers ago
        u.barrier()               # every rank has published
        A = torch.empty(B * Ll, D, dtype=attn.dtype, device=attn.device)
        pl = u.cols_plan(("attn", sym.local.data_ptr()), sym, 1, A)
        res2 = None if residual is None else residual.contiguous().view(B * Ll, D)
        gate_v = None
        if gate is not None:
            gate_v, _ = F._mod_view(gate, D)
        h = None
        ga = pl.launch_args()
        # A is kept for the weight / adapter gradients (and read again by the second GEMM of the
        # LoRA path), so it must land completely; only when nothing reads it afterwards may the
        # kernel take this rank's own column block from where it lives instead of copying it
        if la is not None or (keep_a and any(ctx.needs_input_grad[i] for i in (1, 3, 4))):
            ga.pop("local", None)
        if la is not None:
            h = F.gemm_native(A, la, alpha=ls, gather=ga)                            # lands A
            y = F.gemm_native(A, w, bias=bias, lora_h=h, lora_b=lb, residual=res2, gate=gate_v,
                              rows_per_batch=Ll)
        else:
            y = F.gemm_native(A, w, bias=bias, residual=res2, gate=gate_v, rows_per_batch=Ll, gather=ga)
        u.nvlink_bytes += B * Ll * D * 2 * (W - 1) // W
        ctx.save_for_backward(A, w, gate_v, la, lb, h)
        ctx.u, ctx.has_res, ctx.has_bias, ctx.ls = u, residual is not None, bias is not None, ls
        return y.view(B, Ll, D)

    @staticmethod
    def backward(ctx, dy):
        A, w, gate_v, la, lb, h = ctx.saved_tensors
        u = ctx.u
        B, Ll, D = u.B, u.Ll, u.D
        dy2 = dy.contiguous().view(B * Ll, D)
        d_res = dy if ctx.has_res else None
        if gate_v is not None:
            dy2 = F.gate_residual(None, dy2.view(B, Ll, D), gate_v).view(B * Ll, D)
        ts = F.gemm_native(dy2, _t(lb), alpha=ctx.ls) if la is not None else None
        # dA = dY Wo (+ ts La), scattered: column block p goes to peer p's rows of my tokens
        u.barrier()
        F.gemm_native(dy2, w, b_mn=True, out=u.d_attn_out.local, lora_h=ts,
                      lora_b=_t(la) if la is not None else None, scatter=u.scatter_args(u.d_attn_out))
        u.barrier()
        d_attn = u.d_attn_out.local.view(B, u.Lt, u.G).clone()
        dw = F.wgrad(dy2, A) if ctx.needs_input_grad[1] else None
        db = dy2.sum(0) if (ctx.has_bias and ctx.needs_input_grad[2]) else None
        da = F.lora_wgrad(A, ts, transpose_out=True) if (la is not None and ctx.needs_input_grad[3]) else None
        db_ = F.lora_wgrad(dy2, h) if (la is not None and ctx.needs_input_grad[4]) else None
        return d_attn, dw, db, da, db_, None, None, d_res, None, None


def _lora_of(linear):
    ad = getattr(linear, "adapter", None)
    if ad is None:
        return None, None, 1.0
    if getattr(ad, "kind", "") != "lora" or ad.rank not in (16, 32, 64):
        raise NotImplementedError("sequence-parallel projections support LoRA adapters of rank 16/32/64")
    return ad.lora_A, ad.lora_B, float(ad.scale)


def ulysses_qkv(x, linear, u: UlyssesContext, want_rowsq=False):
    la, lb, ls = _lora_of(linear)
    return _UlyssesQKV.apply(x, linear.weight, linear.bias, la, lb, ls, u, want_rowsq)


def ulysses_out_proj(attn, linear, u: UlyssesContext, residual=None, gate=None):
    la, lb, ls = _lora_of(linear)
    # grad mode is read here: inside an autograd Function's forward it is always off
    return _UlyssesOutProj.apply(attn, linear.weight, linear.bias, la, lb, ls, u, residual, gate,
                                 torch.is_grad_enabled())


class _DistRowNorm(torch.autograd.Function):
    """RMSNorm over a feature dimension that is sharded across ranks (QK-norm across heads after
    the head exchange): y = x * rstd[token] * w, with rstd computed from the full row elsewhere.
    Backward needs each token's sum over ALL columns of dy*w*x, an all-reduce of one scalar per
    token."""

    @staticmethod
    def forward(ctx, x, rstd, w, d_total, pg):
        y = (x.float() * rstd.unsqueeze(-1) * w.float()).to(x.dtype)
        ctx.save_for_backward(x, rstd, w)
        ctx.d_total, ctx.pg = d_total, pg
        return y

    @staticmethod
    def backward(ctx, dy):
        x, rstd, w = ctx.saved_tensors
        g = dy.float() * w.float()
        xf = x.float()
        part = (g * xf).sum(-1)
        if ctx.pg.world_size > 1:
            dist.all_reduce(part, group=ctx.pg.group)
        r = rstd.unsqueeze(-1)
        dx = (r * g - xf * (r ** 3) * (part / ctx.d_total).unsqueeze(-1)).to(x.dtype)
        dw = (dy.float() * xf * r).flatten(0, -2).sum(0).to(w.dtype)
        return dx, None, dw, None, None


def dist_rmsnorm(x, rstd, w_slice, d_total, pg):
    return _DistRowNorm.apply(x, rstd, w_slice, d_total, pg)
