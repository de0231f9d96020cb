"""Public op surface. CUDA bf16 tensors run the hand-written sm_100a kernels (through autograd
Functions that call the in-tree library); everything else runs the PyTorch statements in
``reference``. ``set_backend("eager")`` forces the PyTorch path on CUDA too — that is the
library baseline the fused path is measured against.
"""
from __future__ import annotations

import math
import os

import torch

from . import _native as N
from . import reference as R

_BACKEND = os.environ.get("ERI_B200_BACKEND", "fused")  # "fused" | "eager"
_GEMM_NATIVE = os.environ.get("ERI_B200_GEMM", "native")  # "native" | "library"
_ATTN_NATIVE = os.environ.get("ERI_B200_ATTN", "native")  # "native" | "library"
_GEMM_PAIR = os.environ.get("ERI_B200_GEMM2", "1") == "1"  # two-CTA tiles for large problems
_PAIR_MIN_TILES = int(os.environ.get("ERI_B200_PAIR_MIN_TILES", "36"))  # at most this many 256 x 256 tiles: one-CTA kernel
_GATHER_JOIN = os.environ.get("ERI_B200_GATHER_JOIN", "0") == "1"  # copy clusters compute tiles after copying
_GATHER_PAIR = os.environ.get("ERI_B200_GATHER_PAIR", "1") == "1"  # gather-fused GEMMs on the two-CTA kernel
_GATHER_LOCAL = os.environ.get("ERI_B200_GATHER_LOCAL", "1") == "1"  # own slab read in place, not copied
_SCATTER_PAIR = os.environ.get("ERI_B200_SCATTER_PAIR", "1") == "1"  # peer-scatter epilogue on the two-CTA kernel
_WGRAD_NATIVE = os.environ.get("ERI_B200_WGRAD", "native") == "native"  # weight gradients on tcgen05 (else torch.mm)
_RANK_STREAM = os.environ.get("ERI_B200_RANK_STREAM", "1") == "1"  # streaming kernel for [M,K] x [r,K]^T
# Launch the LoRA-fused GEMM as a programmatic dependent of the down-projection kernel that precedes
# it on the stream: its main K loop overlaps that kernel and only the rank-r step waits for it.
_PDL = os.environ.get("ERI_B200_PDL", "1") == "1"


def _pdl_ok() -> bool:
    # the overlap is only sound when the down-projection is the launch right before the GEMM;
    # deterministic mode makes torch.empty launch a fill kernel in between
    return _PDL and not torch.are_deterministic_algorithms_enabled()


def set_backend(name: str) -> None:
    global _BACKEND
    if name not in ("fused", "eager"):
        raise ValueError(name)
    _BACKEND = name


def get_backend() -> str:
    return _BACKEND


def set_gemm_impl(name: str) -> None:
    global _GEMM_NATIVE
    _GEMM_NATIVE = name


def set_attention_impl(name: str) -> None:
    global _ATTN_NATIVE
    _ATTN_NATIVE = name


def _native_ok(*ts) -> bool:
    if _BACKEND != "fused":
        return False
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda or t.dtype != torch.bfloat16:
            return False
    N.require()
    return True


def _c(t):
    return None if t is None else (t if t.is_contiguous() else t.contiguous())


def _tokmajor(t):
    """[B, L, W] whose tokens may be row-strided (a column slice of a wider buffer)."""
    if t.stride(2) == 1 and t.stride(0) == t.shape[1] * t.stride(1) and t.stride(1) % 8 == 0 \
            and t.data_ptr() % 16 == 0:
        return t
    return t.contiguous()


def _mod_view(t, D):
    """A [B, D] modulation tensor whose rows may be strided (a chunk of a wider tensor)."""
    if t is None:
        return None, 0
    assert t.dim() == 2 and t.shape[1] == D
    if t.stride(1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t, t.stride(0)


# ---------------------------------------------------------------------------- norm + modulation
class _NormModulate(torch.autograd.Function):
    """``skip``: also returns x itself as a second output for the residual branch that bypasses the norm; the
    gradient that comes back through it is added to dx inside the backward kernel instead of by a separate
    autograd sum (one launch and a pass over two tensors per norm)."""

    @staticmethod
    def forward(ctx, x, scale, shift, weight, bias, eps, rms, skip=False):
        B, L, D = x.shape
        x = _c(x)
        scale_v, s1 = _mod_view(scale, D)
        shift_v, s2 = _mod_view(shift, D)
        if scale_v is not None and shift_v is not None and s1 != s2:
            scale_v, shift_v = scale_v.contiguous(), shift_v.contiguous()
            s1 = s2 = D
        stride = s1 or s2 or D
        y = torch.empty_like(x)
        mean = torch.empty(B * L, dtype=torch.float32, device=x.device)
        rstd = torch.empty(B * L, dtype=torch.float32, device=x.device)
        lib = N.require()
        args = (x.data_ptr(), N.ptr(scale_v), N.ptr(shift_v), N.ptr(weight), N.ptr(bias),
                y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), B * L, D, L, stride, eps,
                1 if rms else 0, N.stream_ptr())
        code = lib.eri_norm_modulate_fwd_warp(*args) if hasattr(lib, "eri_norm_modulate_fwd_warp") else -100
        if code == -100:
            code = lib.eri_norm_modulate_fwd(*args)
        N.check(code, "norm_modulate_fwd")
        ctx.save_for_backward(x, scale_v, weight, bias, mean, rstd)
        ctx.meta = (B, L, D, stride, rms, scale is not None, shift is not None)
        ctx.set_materialize_grads(False)
        if skip:
            return y, x.view_as(x)
        return y

    @staticmethod
    def backward(ctx, dy, dskip=None):
        if dy is None:          # the consumer had no gradient for this input (an unused stream)
            return dskip, None, None, None, None, None, None, None
        x, scale_v, weight, bias, mean, rstd = ctx.saved_tensors
        B, L, D, stride, rms, has_scale, has_shift = ctx.meta
        dy = _c(dy)
        dx = torch.empty_like(x)
        need = ctx.needs_input_grad
        f32 = dict(dtype=torch.float32, device=x.device)
        dscale = torch.zeros(B, D, **f32) if (has_scale and need[1]) else None
        dshift = torch.zeros(B, D, **f32) if (has_shift and need[2]) else None
        dweight = torch.zeros(D, **f32) if (weight is not None and need[3]) else None
        dbias = torch.zeros(D, **f32) if (bias is not None and need[4]) else None
        lib = N.require()
        code = -100
        added = False
        if dscale is None and dshift is None and dweight is None and dbias is None \
                and hasattr(lib, "eri_norm_modulate_bwd_warp"):
            if dskip is not None and hasattr(lib, "eri_norm_modulate_bwd_warp_add") and dskip.dtype == dx.dtype:
                dsk = _c(dskip)
                code = lib.eri_norm_modulate_bwd_warp_add(
                    dy.data_ptr(), x.data_ptr(), N.ptr(scale_v), N.ptr(weight), mean.data_ptr(),
                    rstd.data_ptr(), dx.data_ptr(), dsk.data_ptr(), B * L, D, L, stride, 1 if rms else 0,
                    N.stream_ptr())
                added = code != -100
            if not added:
                code = lib.eri_norm_modulate_bwd_warp(
                    dy.data_ptr(), x.data_ptr(), N.ptr(scale_v), N.ptr(weight), mean.data_ptr(),
                    rstd.data_ptr(), dx.data_ptr(), B * L, D, L, stride, 1 if rms else 0, N.stream_ptr())
        if code == -100:
            code = lib.eri_norm_modulate_bwd(
                dy.data_ptr(), x.data_ptr(), N.ptr(scale_v), N.ptr(weight), N.ptr(bias),
                mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), N.ptr(dscale), N.ptr(dshift),
                N.ptr(dweight), N.ptr(dbias), B * L, D, L, stride, 1 if rms else 0, N.stream_ptr())
        N.check(code, "norm_modulate_bwd")
        cv = lambda t: None if t is None else t.to(torch.bfloat16)
        if dskip is not None and not added:
            dx = dx + dskip.view_as(dx)
        return dx, cv(dscale), cv(dshift), cv(dweight), cv(dbias), None, None, None


def norm_modulate_skip(x, scale=None, shift=None, weight=None, bias=None, eps=1e-6, rms=False):
    """``(norm_modulate(x, ...), x)``: the second value is x for the residual branch around the norm. On the
    native path the gradients of both branches are summed inside the norm's backward kernel."""
    if _NORM_SKIP and _native_ok(x, scale, shift, weight, bias) and x.dim() == 3 and x.shape[-1] % 8 == 0 \
            and torch.is_grad_enabled() and x.requires_grad:
        return _NormModulate.apply(x, scale, shift, weight, bias, eps, rms, True)
    return norm_modulate(x, scale, shift, weight, bias, eps, rms), x


# Off by default: the FLUX LoRA step measured 190.0 / 192.8 ms with it and 190.5 / 191.0 ms without (alternating runs).
_NORM_SKIP = os.environ.get("ERI_B200_NORM_SKIP", "0") == "1"


def norm_modulate(x, scale=None, shift=None, weight=None, bias=None, eps=1e-6, rms=False):
    if _native_ok(x, scale, shift, weight, bias) and x.dim() == 3 and x.shape[-1] % 8 == 0 \
            and x.shape[-1] <= 8192:
        return _NormModulate.apply(x, scale, shift, weight, bias, eps, rms)
    return R.norm_modulate(x, scale, shift, weight, bias, eps, rms)


# ---------------------------------------------------------------------------- QK-norm + RoPE
def qknorm_rope(qkv, q_scale, k_scale, cos, sin, num_heads, eps=1e-6):
    """qkv [B, L, 3*H*Dh] -> q, k, v [B, L, H, Dh] (norm + rotary on q, k)."""
    return qknorm_rope_joint([(qkv, q_scale, k_scale)], cos, sin, num_heads, eps)


class _QKNormRopeJoint(torch.autograd.Function):
    """Several token streams (e.g. text and image) -> one joint q, k, v of shape
    [B, sum(L_i), H, Dh]; each stream has its own QK-norm scales, the rotary table covers the
    joint sequence. One kernel launch per stream writes straight into the joint tensors, so no
    concatenation copy exists in forward, and backward splits the gradient the same way."""

    @staticmethod
    def forward(ctx, cos, sin, H, eps, width, *flat):
        n = len(flat) // 3
        qkvs = [_tokmajor(flat[3 * i]) for i in range(n)]
        B = qkvs[0].shape[0]
        Dh = width // (3 * H)
        Ls = [t.shape[1] for t in qkvs]
        Ltot = sum(Ls)
        q = torch.empty(B, Ltot, H, Dh, dtype=qkvs[0].dtype, device=qkvs[0].device)
        k, v = torch.empty_like(q), torch.empty_like(q)
        lib = N.require()
        off = 0
        for i in range(n):
            qs, ks = flat[3 * i + 1], flat[3 * i + 2]
            tok_stride = qkvs[i].stride(1)
            N.check(lib.eri_qknorm_rope_fwd(
                qkvs[i].data_ptr(), N.ptr(qs), N.ptr(ks), N.ptr(cos), N.ptr(sin), q.data_ptr(),
                k.data_ptr(), v.data_ptr(), B, Ls[i], H, Dh, Ltot, off, eps, tok_stride, H * Dh,
                N.stream_ptr()), "qknorm_rope_fwd")
            off += Ls[i]
        ctx.save_for_backward(cos, sin, *qkvs, *[flat[3 * i + 1] for i in range(n)],
                              *[flat[3 * i + 2] for i in range(n)])
        ctx.meta = (n, B, H, Dh, Ls, Ltot, eps)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        n, B, H, Dh, Ls, Ltot, eps = ctx.meta
        sv = ctx.saved_tensors
        cos, sin = sv[0], sv[1]
        qkvs, qss, kss = sv[2:2 + n], sv[2 + n:2 + 2 * n], sv[2 + 2 * n:2 + 3 * n]
        dq, dk, dv = _c(dq), _c(dk), _c(dv)
        lib = N.require()
        grads = []
        off = 0
        f32 = dict(dtype=torch.float32, device=dq.device)
        for i in range(n):
            dqkv = torch.empty(qkvs[i].shape, dtype=qkvs[i].dtype, device=qkvs[i].device)
            need_q = qss[i] is not None and ctx.needs_input_grad[5 + 3 * i + 1]
            need_k = kss[i] is not None and ctx.needs_input_grad[5 + 3 * i + 2]
            dqs = torch.zeros(Dh, **f32) if need_q else None
            dks = torch.zeros(Dh, **f32) if need_k else None
            N.check(lib.eri_qknorm_rope_bwd(
                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), qkvs[i].data_ptr(), N.ptr(qss[i]),
                N.ptr(kss[i]), N.ptr(cos), N.ptr(sin), dqkv.data_ptr(), N.ptr(dqs), N.ptr(dks),
                B, Ls[i], H, Dh, Ltot, off, eps, qkvs[i].stride(1), H * Dh, dqkv.stride(1),
                N.stream_ptr()), "qknorm_rope_bwd")
            off += Ls[i]
            cv = lambda t: None if t is None else t.to(torch.bfloat16)
            grads += [dqkv, cv(dqs), cv(dks)]
        return (None, None, None, None, None, *grads)


def qknorm_rope_joint(streams, cos, sin, num_heads, eps=1e-6):
    """streams: list of (qkv [B, L_i, 3*H*Dh], q_scale [Dh] | None, k_scale [Dh] | None).
    Returns joint q, k, v [B, sum L_i, H, Dh]; cos/sin [sum L_i, Dh/2] or None."""
    W = streams[0][0].shape[-1]
    Dh = W // (3 * num_heads)
    tens = [t for s in streams for t in s]
    if _native_ok(*tens) and Dh in (64, 128) and (cos is None or cos.is_cuda):
        cosf = None if cos is None else cos.float().contiguous()
        sinf = None if sin is None else sin.float().contiguous()
        return _QKNormRopeJoint.apply(cosf, sinf, num_heads, eps, W, *tens)
    outs, off = [], 0
    for qkv, qs, ks in streams:
        L = qkv.shape[1]
        c = None if cos is None else cos[off:off + L]
        s_ = None if sin is None else sin[off:off + L]
        outs.append(R.qknorm_rope(qkv, qs, ks, c, s_, num_heads, eps))
        off += L
    if len(outs) == 1:
        return outs[0]
    return tuple(torch.cat([o[j] for o in outs], dim=1) for j in range(3))


# ---------------------------------------------------------------------------- gate + residual
class _GateResidual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, y, gate):
        B, L, D = y.shape
        y = _c(y)
        x = _c(x)
        gate_v, gs = _mod_view(gate, D)
        out = torch.empty_like(y)
        lib = N.require()
        N.check(lib.eri_gate_residual(N.ptr(x), y.data_ptr(), N.ptr(gate_v), out.data_ptr(),
                                      B * L, D, L, gs, N.stream_ptr()), "gate_residual")
        ctx.save_for_backward(y if (gate is not None and ctx.needs_input_grad[2]) else None, gate_v)
        ctx.meta = (B, L, D, gs, x is not None)
        return out

    @staticmethod
    def backward(ctx, dout):
        y, gate_v = ctx.saved_tensors
        B, L, D, gs, has_x = ctx.meta
        dout = _c(dout)
        lib = N.require()
        dx = dout if has_x else None
        if gate_v is None:
            return dx, dout, None
        dy = torch.empty_like(dout)
        N.check(lib.eri_gate_residual(None, dout.data_ptr(), gate_v.data_ptr(), dy.data_ptr(),
                                      B * L, D, L, gs, N.stream_ptr()), "gate_residual_bwd")
        dgate = None
        if ctx.needs_input_grad[2]:
            dg = torch.zeros(B, D, dtype=torch.float32, device=dout.device)
            N.check(lib.eri_gate_grad(dout.data_ptr(), y.data_ptr(), dg.data_ptr(), B * L, D, L,
                                      N.stream_ptr()), "gate_grad")
            dgate = dg.to(torch.bfloat16)
        return dx, dy, dgate


def gate_residual(x, y, gate=None):
    if _native_ok(x, y, gate) and y.dim() == 3 and y.shape[-1] % 8 == 0:
        return _GateResidual.apply(x, y, gate)
    return R.gate_residual(x, y, gate)


class _SplitTokens(torch.autograd.Function):
    """(x[:, :n], x[:, n:]) as views. Autograd's own slice backward allocates a zero tensor of x's size per
    slice, copies the slice's gradient into it and sums the two (two fills, two copies and an add per
    dual-stream block); here the backward is one concatenation."""

    @staticmethod
    def forward(ctx, x, n):
        ctx.n, ctx.shape = n, x.shape
        ctx.set_materialize_grads(False)
        return x[:, :n], x[:, n:]

    @staticmethod
    def backward(ctx, d0, d1):
        if d0 is None and d1 is None:
            return None, None
        B, L = ctx.shape[0], ctx.shape[1]
        ref = d0 if d0 is not None else d1
        if d0 is None:
            d0 = ref.new_zeros((B, ctx.n, *ctx.shape[2:]))
        if d1 is None:
            d1 = ref.new_zeros((B, L - ctx.n, *ctx.shape[2:]))
        return torch.cat((d0, d1), dim=1), None


def split_tokens(x, n):
    """``(x[:, :n], x[:, n:])`` whose backward is a single concatenation."""
    if x.requires_grad and torch.is_grad_enabled():
        return _SplitTokens.apply(x, n)
    return x[:, :n], x[:, n:]


# ---------------------------------------------------------------------------- activations
class _Act(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mode):
        x = _c(x)
        y = torch.empty_like(x)
        N.check(N.require().eri_act_fwd(x.data_ptr(), y.data_ptr(), x.numel(), mode,
                                        N.stream_ptr()), "act_fwd")
        ctx.save_for_backward(x)
        ctx.mode = mode
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dy = _c(dy)
        dx = torch.empty_like(x)
        N.check(N.require().eri_act_bwd(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), x.numel(),
                                        ctx.mode, N.stream_ptr()), "act_bwd")
        return dx, None


def gelu_tanh(x):
    if _native_ok(x) and x.numel() % 8 == 0:
        return _Act.apply(x, 0)
    return R.gelu_tanh(x)


def silu(x):
    if _native_ok(x) and x.numel() % 8 == 0:
        return _Act.apply(x, 1)
    return R.silu(x)


class _Glu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, mode, act_first):
        h = _c(h)
        F2 = h.shape[-1]
        rows = h.numel() // F2
        out = torch.empty(*h.shape[:-1], F2 // 2, dtype=h.dtype, device=h.device)
        N.check(N.require().eri_glu_fwd(h.data_ptr(), out.data_ptr(), rows, F2 // 2, mode,
                                        1 if act_first else 0, N.stream_ptr()), "glu_fwd")
        ctx.save_for_backward(h)
        ctx.meta = (rows, F2 // 2, mode, act_first)
        return out

    @staticmethod
    def backward(ctx, dout):
        (h,) = ctx.saved_tensors
        rows, Fh, mode, act_first = ctx.meta
        dout = _c(dout)
        dh = torch.empty_like(h)
        N.check(N.require().eri_glu_bwd(dout.data_ptr(), h.data_ptr(), dh.data_ptr(), rows, Fh,
                                        mode, 1 if act_first else 0, N.stream_ptr()), "glu_bwd")
        return dh, None, None


def glu(h, mode="gelu", act_first=True):
    if _native_ok(h) and h.shape[-1] % 16 == 0:
        return _Glu.apply(h, 0 if mode == "gelu" else 1, act_first)
    return R.glu(h, mode, act_first)


# ---------------------------------------------------------------------------- GEMM family
_ACT_CODE = {None: 0, "gelu": 1, "silu": 2, "gelu_bwd": 3, "silu_bwd": 4}


def gemm_native(a, b, *, out=None, alpha=1.0, bias=None, lora_h=None, lora_b=None, act=None,
                pre_out=None, pre_in=None, residual=None, gate=None, rows_per_batch=0,
                n_split=0, out2=None, force_bn=0, b_mn=False, gather=None, scatter=None, pdl=False,
                a_mn=False, glu=0, _prepare_only=False):
    """out[M,N] = epilogue(a[M,K] @ op(b) (+ lora_h[M,r] @ lora_b[N,r]^T)) on the tcgen05 kernel.

    ``b`` is [N, K] (``op`` = transpose) or, with ``b_mn=True``, [K, N] used as is. ``a``/``b``/
    ``out`` may be row-strided views (last dim contiguous). ``gather``: dict built by
    ``parallel.gather_gemm`` (copy jobs + slab counters, fuses an operand gather into the launch).
    ``scatter``: dict(world, rank, part_cols, group_cols, local_rows, ptrs) routing column groups
    to peer buffers (``out`` is then only used for its row stride); with ``mode=1`` output ROW r goes to
    rank ``r // local_rows`` into slot ``rank`` of that rank's receive buffer ``[world][local_rows, N]``. ``a_mn=True``: ``a`` is [K, M]
    used as is (with ``b_mn`` this is the weight-gradient product over token-major activations).
    ``glu`` 1-4: ``b`` is an up-projection [2*hidden, K] and the output is the gated product of its
    halves, [M, hidden] (1 a*gelu(g), 2 a*silu(g), 3 gelu(a)*g, 4 silu(a)*g); ``pre_out``
    [M, 2*hidden] keeps the halves for backward. Returns ``out``.
    """
    lib = N.require()
    K, M = a.shape if a_mn else a.shape[::-1]
    Nn = b.shape[1] if b_mn else b.shape[0]
    assert (b.shape[0] if b_mn else b.shape[1]) == K and a.stride(1) == 1 and b.stride(1) == 1
    if out is None:
        cols = Nn // 2 if glu else (Nn if not n_split else n_split)
        out = torch.empty(M, cols, dtype=torch.bfloat16, device=a.device)
    g = N.GemmArgs()
    g.a, g.b = a.data_ptr(), b.data_ptr()
    g.lda, g.ldb = a.stride(0), b.stride(0)
    g.M, g.N, g.K = M, Nn, K
    g.alpha = alpha
    g.out, g.ldc = out.data_ptr(), out.stride(0)
    g.bias = N.ptr(bias)
    if lora_h is not None:
        g.lora_h, g.lora_b = lora_h.data_ptr(), lora_b.data_ptr()
        g.ld_h, g.ld_lb = lora_h.stride(0), lora_b.stride(0)
        g.lora_r = lora_h.shape[1]
    g.act = _ACT_CODE[act]
    if pre_out is not None:
        g.pre_out, g.ld_pre = pre_out.data_ptr(), pre_out.stride(0)
    if pre_in is not None:
        g.pre_in, g.ld_pre = pre_in.data_ptr(), pre_in.stride(0)
    if residual is not None:
        g.residual, g.ldr = residual.data_ptr(), residual.stride(0)
    if gate is not None:
        g.gate, g.gate_stride = gate.data_ptr(), gate.stride(0)
    g.rows_per_batch = rows_per_batch
    g.n_split = n_split
    if out2 is not None:
        g.out2, g.ldc2 = out2.data_ptr(), out2.stride(0)
    g.force_bn = force_bn
    if N.DEBUG_BOUNDS:
        g.dbg_out_bytes = N.extent_bytes(out) if scatter is None else 0
        g.dbg_out2_bytes, g.dbg_pre_bytes = N.extent_bytes(out2), N.extent_bytes(pre_out)
        g.dbg_res_bytes = N.extent_bytes(residual)
    g.b_mn = 1 if b_mn else 0
    g.a_mn = 1 if a_mn else 0
    g.glu = int(glu)
    g.pdl = 1 if (pdl and lora_h is not None and gather is None) else 0
    if gather is not None:
        g.n_copy, g.n_jobs = gather["n_copy"], gather["n_jobs"]
        g.jobs, g.flags, g.flag_target = gather["jobs"], gather["flags"], gather["flag_target"]
        g.b_flag_rows, g.a_flag_cols = gather.get("b_flag_rows", 0), gather.get("a_flag_cols", 0)
        g.rot_n_rows, g.rot_k_cols = gather.get("rot_n_rows", 0), gather.get("rot_k_cols", 0)
        g.a_flag_rows = gather.get("a_flag_rows", 0)
        g.all_flag = int(gather.get("all_flag", 0))
        st = gather.get("stamps")                 # optional uint64[8] phase record (see gemm_args.h)
        g.stamps = st.data_ptr() if st is not None else None
        # Copy clusters join the tile loop when their slabs have landed. The round from which the tile
        # schedule counts them in is the number of tiles a compute cluster finishes meanwhile: a copy
        # CTA moves ~35 GB/s (measured, bulk-copy ring), a K step of a pair tile is ~0.33 us.
        # Off unless asked for (``join_round`` in the plan's arguments, or ERI_B200_GATHER_JOIN=1): with
        # eight ranks emulated on one GPU it shortened the compute phase by one round of 13 but not the
        # launch as a whole.
        if gather.get("join_round") is not None:
            g.join_round = int(gather["join_round"])
        elif _GATHER_JOIN and g.n_copy > 0 and gather.get("copy_bytes"):
            copy_us = gather["copy_bytes"] / g.n_copy / 35e3
            tile_us = ((K + 63) // 64) * 0.33 + 2.0
            g.join_round = max(1, int(math.ceil(copy_us / tile_us)))
        loc = gather.get("local") if _GATHER_LOCAL else None
        if loc is not None:
            g.b_local, g.ldb_local = loc["ptr"], loc["ld"]
            g.loc_mode, g.loc_lo, g.loc_hi = loc["mode"], loc["lo"], loc["hi"]
            g.n_jobs_nl, g.jobs_nl, g.flag_target_nl = loc["n_jobs"], loc["jobs"], loc["flag_target"]
    if scatter is not None:
        g.scatter_world, g.scatter_rank = scatter["world"], scatter["rank"]
        g.scatter_part_cols, g.scatter_group_cols = scatter["part_cols"], scatter["group_cols"]
        g.scatter_local_rows = scatter["local_rows"]
        g.scatter_mode = int(scatter.get("mode", 0))
        for i, ptr_ in enumerate(scatter["ptrs"]):
            g.scatter_out[i] = ptr_
        if scatter.get("rowsq") is not None:
            g.rowsq, g.rowsq_parts = scatter["rowsq"].data_ptr(), scatter["rowsq"].shape[0]
    route = (M, Nn, K, a_mn, glu, gather, scatter, force_bn)
    if _prepare_only:
        return g, out, route          # ``gemm_native_pair`` launches it, alone or grouped
    return _launch_gemm(lib, g, out, route)


def _launch_gemm(lib, g, out, route):
    M, Nn, K, a_mn, glu, gather, scatter, force_bn = route
    # Few pair tiles (the 512-token text stream against a 3072-wide weight: 24 tiles for 74 CTA pairs)
    # leave most SMs idle; the one-CTA kernel's 128-column tiles spread the same work over four times
    # as many CTAs (measured 22.5 against 30.7 us at 512 x 3072 x 3072, 61 against 78 us at K = 12288).
    few_tiles = (force_bn == 0 and not (a_mn or glu) and gather is None and scatter is None
                 and ((M + 255) // 256) * ((Nn + 255) // 256) <= _PAIR_MIN_TILES)
    if (_GEMM_PAIR or a_mn or glu) and (gather is None or _GATHER_PAIR) and (scatter is None or _SCATTER_PAIR) \
            and force_bn in (0, 256) and M >= 256 and Nn >= 256 and not few_tiles:
        # two-CTA 256x256 tiles; in gather mode with whole copy clusters in front (answers -30 when
        # the gather plan does not line up with pair tiles, and the one-CTA kernel takes over)
        code = lib.eri_gemm2_bf16(g, N.stream_ptr())
        if code != -30:
            N.check(code, "gemm2_bf16")
            return out
    if a_mn or glu:
        raise ValueError(f"gemm_native: a_mn / glu need the two-CTA kernel's shape range (M={M}, N={Nn}, K={K})")
    code = lib.eri_gemm_bf16(g, N.stream_ptr())
    N.check(code, "gemm_bf16")
    return out


_GEMM_GROUP = os.environ.get("ERI_B200_GEMM_GROUP", "1") == "1"
_ACT_EPILOGUE = os.environ.get("ERI_B200_ACT_EPILOGUE", "0") == "1"   # activation + stored pre-activation in the GEMM epilogue


def _act_outside_epilogue(M, Nn, K) -> bool:
    """Whether a training-time linear + activation writes its pre-activation from the GEMM and applies the
    activation in a pass of its own. With a short reduction (K <= 4096) the epilogue of a pair tile is on the
    critical path and storing both tensors from it costs a large GEMM more than the separate pass
    ([4096 x 12288 x 3072]: 282 against 225 + 39 us); with a long reduction the epilogue is hidden, and a small
    problem is bound by its launches, so both keep the fused form."""
    return not _ACT_EPILOGUE and K <= 4096 and M * Nn >= (1 << 25)


def gemm_native_pair(kw0: dict, kw1: dict):
    """Two independent products (keyword arguments of ``gemm_native`` each) in ONE launch of the two-CTA
    kernel when they qualify: same N, K, operand majors, LoRA rank and epilogue kind, plain modes. The
    second problem's tiles follow the first's in the persistent schedule, so a small second problem
    (the text stream of a dual-stream block) runs in the first one's last, partly empty round instead of
    as a launch that leaves most SMs idle. Otherwise the two are launched one after the other.
    Returns (out0, out1)."""
    lib = N.require()
    g0, out0, r0 = gemm_native(**kw0, _prepare_only=True)
    g1, out1, r1 = gemm_native(**kw1, _prepare_only=True)
    plain = all(not (r[3] or r[4]) and r[5] is None and r[6] is None and r[7] == 0 and r[0] >= 256 and r[1] >= 256
                for r in (r0, r1))
    if _GEMM_GROUP and _GEMM_PAIR and plain and hasattr(lib, "eri_gemm2_bf16_group2"):
        code = lib.eri_gemm2_bf16_group2(g0, g1, N.stream_ptr())
        if code != -30:
            N.check(code, "gemm2_bf16_group2")
            return out0, out1
    return _launch_gemm(lib, g0, out0, r0), _launch_gemm(lib, g1, out1, r1)


def skinny_gemm(a, b, alpha=1.0):
    """alpha * a[M, K] @ b[N, K]^T for N in {16, 32, 64} (LoRA rank): split-K tcgen05 kernel that
    keeps every SM busy on a bandwidth-bound problem; other shapes use the general GEMM."""
    M, K = a.shape
    Nn = b.shape[0]
    lib = N.require()
    if _RANK_STREAM and hasattr(lib, "eri_gemm_rank_stream") and a.stride(1) == 1 and b.stride(1) == 1:
        # streaming kernel: bound by reading a once, no operand staging
        out = torch.empty(M, Nn, dtype=torch.bfloat16, device=a.device)
        code = lib.eri_gemm_rank_stream(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(),
                                        Nn, M, Nn, K, float(alpha), N.stream_ptr())
        if code != -100:
            N.check(code, "gemm_rank_stream")
            return out
    if hasattr(lib, "eri_gemm_skinny") and a.stride(1) == 1 and b.stride(1) == 1 and M >= 128:
        out = torch.empty(M, Nn, dtype=torch.bfloat16, device=a.device)
        code = lib.eri_gemm_skinny(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(),
                                   Nn, M, Nn, K, float(alpha), N.stream_ptr())
        if code != -100:
            N.check(code, "gemm_skinny")
            return out
    return gemm_native(a, b, alpha=alpha)


def skinny_gemm_pair(a0, b0, alpha0, a1, b1, alpha1):
    """(alpha0 * a0 b0^T, alpha1 * a1 b1^T) for two rank-r products with the same K and r (the adapters of the
    image and the text projection of a dual-stream block) in one launch of the streaming kernel; two
    launches when the shapes do not allow it."""
    lib = N.require()
    if (_RANK_STREAM and _GEMM_GROUP and hasattr(lib, "eri_gemm_rank_stream2") and a0.shape[1] == a1.shape[1]
            and b0.shape[0] == b1.shape[0] and all(t.stride(1) == 1 for t in (a0, b0, a1, b1))):
        r, K = b0.shape[0], a0.shape[1]
        o0 = torch.empty(a0.shape[0], r, dtype=torch.bfloat16, device=a0.device)
        o1 = torch.empty(a1.shape[0], r, dtype=torch.bfloat16, device=a1.device)
        code = lib.eri_gemm_rank_stream2(a0.data_ptr(), a0.stride(0), b0.data_ptr(), b0.stride(0), o0.data_ptr(), r,
                                         a0.shape[0], float(alpha0), a1.data_ptr(), a1.stride(0), b1.data_ptr(),
                                         b1.stride(0), o1.data_ptr(), r, a1.shape[0], float(alpha1), r, K,
                                         N.stream_ptr())
        if code != -100:
            N.check(code, "gemm_rank_stream2")
            return o0, o1
    return skinny_gemm(a0, b0, alpha=alpha0), skinny_gemm(a1, b1, alpha=alpha1)


def gemm_supported(M, Nn, K) -> bool:
    return M >= 128 and Nn >= 16 and K >= 8 and K % 8 == 0 and Nn % 8 == 0


def set_gemm_pair(on: bool) -> None:
    global _GEMM_PAIR
    _GEMM_PAIR = bool(on)


def gemm_error_check() -> int:
    """Synchronise and return the device error word of the GEMM kernels (0 = clean)."""
    lib = N.require()
    e = lib.eri_gemm_check_error()
    if not e and hasattr(lib, "eri_gemm2_check_error"):
        e = lib.eri_gemm2_check_error()
    return e


def kernel_error_check() -> dict:
    """Synchronise and read every kernel family's device error word (each is set when one of that
    family's bounded waits ran out, and cleared by the read). Empty dict = clean."""
    lib = N.require()
    out = {}
    for name in ("gemm", "gemm2", "gemm_skinny", "gemm_tokred", "fa", "fa2", "fa_bwd", "norm"):
        fn = getattr(lib, f"eri_{name}_check_error", None)
        if fn is not None:
            v = fn()
            if v:
                out[name] = v
    return out


def _mm(a, b_nk, **kw):
    """a[M,K] @ b_nk[N,K]^T with the native kernel when the shape qualifies."""
    if _GEMM_NATIVE == "native" and gemm_supported(a.shape[0], b_nk.shape[0], a.shape[1]) \
            and a.stride(0) % 8 == 0 and b_nk.stride(0) % 8 == 0 \
            and a.data_ptr() % 16 == 0 and b_nk.data_ptr() % 16 == 0:
        return gemm_native(a, b_nk, **kw)
    y = torch.matmul(a, b_nk.t())
    if kw.get("alpha", 1.0) != 1.0:
        y = y * kw["alpha"]
    return y


def _wgrad_ok(*ts) -> bool:
    return _WGRAD_NATIVE and _BACKEND == "fused" and _GEMM_NATIVE == "native" and all(
        t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1
        and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0 for t in ts)


def wgrad(dy2, x2, accum=None, out=None):
    """Weight gradient dW[N_out, K_in] = dy2[T, N_out]^T @ x2[T, K_in] on the two-CTA tcgen05 kernel:
    both activations are read token-major as MN-major operands, so no transposed copy is made.
    ``accum``: an existing bf16 gradient of that shape; the product is added into it (beta = 1 in the
    GEMM epilogue) and ``accum`` is returned. ``out``: destination for the plain product. Shapes
    outside the kernel's range use ``torch``."""
    T, Nn = dy2.shape
    K = x2.shape[1]
    dst = accum if accum is not None else out
    if _wgrad_ok(dy2, x2) and Nn >= 256 and K >= 256 and T >= 64 and Nn % 8 == 0 and K % 8 == 0 \
            and (dst is None or _wgrad_ok(dst)):
        return gemm_native(dy2, x2, a_mn=True, b_mn=True, out=dst, residual=accum)
    if accum is not None:
        return accum.addmm_(dy2.t(), x2)
    if out is not None:
        return torch.mm(dy2.t(), x2, out=out)
    return dy2.t() @ x2


def lora_wgrad(a_tok, b_tok, out=None, transpose_out=False, accumulate=False):
    """Skinny token reduction ``a_tok[T, Mg]^T @ b_tok[T, r]`` (r = adapter rank) for the LoRA
    gradients: dB[N_out, r] = dY^T H, and with ``transpose_out`` dA[r, K_in] = (X^T Ts)^T. Split over
    the tokens across CTAs on tcgen05; ``accumulate`` adds into ``out``."""
    T, Mg = a_tok.shape
    r = b_tok.shape[1]
    shape = (r, Mg) if transpose_out else (Mg, r)
    lib = N.lib() if a_tok.is_cuda else None
    if lib is not None and hasattr(lib, "eri_gemm_tokred") and _wgrad_ok(a_tok) and r in (16, 32, 64) \
            and b_tok.is_cuda and b_tok.dtype == torch.bfloat16 and b_tok.stride(1) == 1 and b_tok.stride(0) % 8 == 0 \
            and b_tok.data_ptr() % 16 == 0 and T >= 64 and Mg >= 128 and Mg % 8 == 0 \
            and (out is None or (out.dtype == torch.bfloat16 and out.stride(1) == 1 and tuple(out.shape) == shape)):
        if out is None:
            out, accumulate = torch.empty(shape, dtype=torch.bfloat16, device=a_tok.device), False
        code = lib.eri_gemm_tokred(a_tok.data_ptr(), a_tok.stride(0), b_tok.data_ptr(), b_tok.stride(0),
                                   out.data_ptr(), out.stride(0), T, Mg, r, 1.0, 1 if transpose_out else 0,
                                   1 if accumulate else 0, N.extent_bytes(out) if N.DEBUG_BOUNDS else 0,
                                   N.stream_ptr())
        if code != -100:
            N.check(code, "gemm_tokred")
            return out
    prod = b_tok.t() @ a_tok if transpose_out else a_tok.t() @ b_tok
    if out is None:
        return prod
    return out.add_(prod) if accumulate else out.copy_(prod)


_ACCUM_INTO_GRAD = os.environ.get("ERI_B200_ACCUM_INTO_GRAD", "1") == "1"
_LORA_T = {}        # data_ptr of an adapter matrix -> (epoch, transposed copy)
_LORA_T_EPOCH = 0
_LORA_T_PLAN = None


class _TransposeJob(__import__("ctypes").Structure):
    _fields_ = [("src", __import__("ctypes").c_void_p), ("dst", __import__("ctypes").c_void_p),
                ("rows", __import__("ctypes").c_int), ("cols", __import__("ctypes").c_int)]


def prepare_lora_transposes(matrices):
    """Transpose every adapter matrix of a model in ONE launch and publish the copies for this
    step's backward (which needs B^T for ``dY B`` and A^T as the rank-r K-step operand). Without
    this each adapted linear transposes its two small matrices itself: two extra launches per
    site per step. Call once per step after the optimizer update, before backward."""
    global _LORA_T_EPOCH, _LORA_T_PLAN
    import ctypes as C
    mats = [m for m in matrices if m.is_cuda and m.dtype == torch.bfloat16 and m.dim() == 2 and m.is_contiguous()]
    if not mats or _BACKEND != "fused":
        return 0
    key = tuple(m.data_ptr() for m in mats)
    if _LORA_T_PLAN is None or _LORA_T_PLAN[0] != key:
        total = sum(m.numel() for m in mats)
        buf = torch.empty(total, dtype=torch.bfloat16, device=mats[0].device)
        jobs = (_TransposeJob * len(mats))()
        outs, off = [], 0
        for i, m in enumerate(mats):
            o = buf[off:off + m.numel()].view(m.shape[1], m.shape[0])
            jobs[i].src, jobs[i].dst, jobs[i].rows, jobs[i].cols = m.data_ptr(), o.data_ptr(), m.shape[0], m.shape[1]
            outs.append(o)
            off += m.numel()
        dev_jobs = torch.frombuffer(bytearray(bytes(jobs)), dtype=torch.uint8).to(mats[0].device)
        _LORA_T_PLAN = (key, buf, outs, dev_jobs, max(m.numel() for m in mats))
    _, buf, outs, dev_jobs, max_elems = _LORA_T_PLAN
    lib = N.require()
    lib.eri_batched_transpose.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    lib.eri_batched_transpose.restype = C.c_int
    N.check(lib.eri_batched_transpose(dev_jobs.data_ptr(), len(mats), max_elems, N.stream_ptr()), "batched_transpose")
    _LORA_T_EPOCH += 1
    for m, o in zip(mats, outs):
        _LORA_T[m.data_ptr()] = (_LORA_T_EPOCH, o)
    return len(mats)


def invalidate_lora_transposes():
    """The adapter matrices changed (optimizer step): published transposes are stale."""
    global _LORA_T_EPOCH
    _LORA_T_EPOCH += 1


def _lora_transposed(m):
    hit = _LORA_T.get(m.data_ptr())
    if hit is not None and hit[0] == _LORA_T_EPOCH and hit[1].shape == (m.shape[1], m.shape[0]):
        return hit[1]
    return m.t().contiguous()


def _linear_grads(dy2, x2, w, lora_a, lora_b, h, s, wt, need, shp, has_bias, lib):
    """Gradients of y = x W^T + b + s (x A^T) B^T given dy2 = dL/dy [M, N]: (dx, dw, dbias, da, db).
    ``need``: five flags in that order. Adapter and weight gradients accumulate straight into the
    parameters' gradient views when those exist (the returned entry is then None)."""
    M, K = x2.shape
    Nn = dy2.shape[1]
    dx = dw = dbias = da = db = None
    r = 0 if lora_a is None else lora_a.shape[0]
    native = lib is not None and _GEMM_NATIVE == "native" and gemm_supported(M, K, Nn)
    ts = None
    la_t = None
    if r:
        # Ts = s * dY B  [M, r]
        if native and r in (16, 32, 64):
            # both transposes are looked up first: nothing may launch between Ts and the dX GEMM
            lb_t, la_t = _lora_transposed(lora_b), _lora_transposed(lora_a)
            ts = skinny_gemm(dy2, lb_t, alpha=s)
        else:
            ts = (dy2 @ lora_b) * s
    if need[0]:
        if native:
            # dX = dY W: with a cached transpose W^T is a K-major operand, otherwise W itself
            # is read as the MN-major operand (no copy).
            b_op, mn = (wt, False) if wt is not None else (w, True)
            copied = mn and K < 64
            if copied:
                b_op, mn = w.t().contiguous(), False       # a launch between Ts and the GEMM
            if r in (16, 32, 64):
                dx = gemm_native(dy2, b_op, b_mn=mn, lora_h=ts, lora_b=la_t,
                                 pdl=_pdl_ok() and not copied)
            else:
                dx = gemm_native(dy2, b_op, b_mn=mn)
                if r:
                    dx = dx + ts @ lora_a
        else:
            dx = dy2 @ w
            if r:
                dx = dx + ts @ lora_a
        dx = dx.view(shp)
    if need[1]:
        if _ACCUM_INTO_GRAD and w.grad is not None and w.grad.dtype == x2.dtype and w.grad.is_contiguous():
            wgrad(dy2, x2, accum=w.grad)       # beta = 1 into the (arena) gradient view
        else:
            dw = wgrad(dy2, x2)
    if has_bias and need[2]:
        dbias = dy2.sum(0)
    # Adapter gradients accumulate straight into the parameters' (arena) gradient views with
    # the GEMM's beta = 1, instead of returning a tensor that autograd adds with one more
    # launch per parameter.
    if r and need[3]:
        if _ACCUM_INTO_GRAD and lora_a.grad is not None and lora_a.grad.dtype == x2.dtype:
            lora_wgrad(x2, ts, out=lora_a.grad, transpose_out=True, accumulate=True)
        else:
            da = lora_wgrad(x2, ts, transpose_out=True)
    if r and need[4]:
        if _ACCUM_INTO_GRAD and lora_b.grad is not None and lora_b.grad.dtype == h.dtype:
            lora_wgrad(dy2, h, out=lora_b.grad, accumulate=True)
        else:
            db = lora_wgrad(dy2, h)
    return dx, dw, dbias, da, db


class _FusedLinear(torch.autograd.Function):
    """y = [residual + gate *] act(x W^T + b + s (x A^T) B^T), M = B*L rows.

    Saved for backward: x, the rank-r product H, the pre-activation (when act) — never a
    materialised LoRA delta. ``wt`` is an optional cached transpose of a frozen W ([K, N]) that
    lets the input-gradient GEMM read a K-major operand.
    """

    @staticmethod
    def forward(ctx, x, w, bias, lora_a, lora_b, lora_scale, act, residual, gate, wt):
        shp = x.shape
        K = shp[-1]
        x2 = _c(x).view(-1, K)
        M, Nn = x2.shape[0], w.shape[0]
        L = shp[-2] if x.dim() >= 2 else 1
        native = _GEMM_NATIVE == "native" and gemm_supported(M, Nn, K)
        r = 0 if lora_a is None else lora_a.shape[0]
        lora_fused = native and r in (16, 32, 64)
        h = None
        pre = None
        res2 = None if residual is None else _c(residual).view(-1, Nn)
        gate_v = None
        if gate is not None:
            gate_v, _ = _mod_view(gate, Nn)
        if native:
            need_pre = act is not None and any(ctx.needs_input_grad[:5])
            if need_pre:
                pre = torch.empty(M, Nn, dtype=x.dtype, device=x.device)
            if r and lora_fused:
                h = skinny_gemm(x2, lora_a, alpha=lora_scale)     # the launch right before the GEMM
            elif r:
                h = (x2 @ lora_a.t()) * lora_scale
            if r and not lora_fused:
                y = gemm_native(x2, w, bias=bias)
                y = y + h @ lora_b.t()
                if act is not None:
                    pre = y
                    y = R.gelu_tanh(y) if act == "gelu" else R.silu(y)
                if gate_v is not None or res2 is not None:
                    y = R.gate_residual(None if res2 is None else res2.view(-1, L, Nn),
                                        y.view(-1, L, Nn), gate_v).view(M, Nn)
            elif pre is not None and res2 is None and gate_v is None and _act_outside_epilogue(M, Nn, K):
                # training keeps the pre-activation anyway: the GEMM writes it as its output and the
                # activation is a pass of its own (cheaper than storing both from the epilogue)
                gemm_native(x2, w, bias=bias, lora_h=h, lora_b=lora_b if r else None, out=pre, pdl=_pdl_ok())
                y = torch.empty_like(pre)
                N.check(N.require().eri_act_fwd(pre.data_ptr(), y.data_ptr(), pre.numel(), 0 if act == "gelu" else 1,
                                                N.stream_ptr()), "act_fwd")
            else:
                y = gemm_native(x2, w, bias=bias, lora_h=h, lora_b=lora_b if r else None,
                                act=act, pre_out=pre, residual=res2, gate=gate_v,
                                rows_per_batch=L, pdl=_pdl_ok())
        else:
            y = torch.nn.functional.linear(x2, w, bias)
            if r:
                h = (x2 @ lora_a.t()) * lora_scale
                y = y + h @ lora_b.t()
            if act is not None:
                pre = y
                y = R.gelu_tanh(y) if act == "gelu" else R.silu(y)
            if gate_v is not None or res2 is not None:
                y = R.gate_residual(None if res2 is None else res2.view(-1, L, Nn),
                                    y.view(-1, L, Nn), gate_v).view(M, Nn)
        ctx.save_for_backward(x2, w, lora_a, lora_b, h, pre, gate_v, wt)
        ctx.meta = (shp, Nn, L, lora_scale, act, residual is not None, bias is not None)
        return y.view(*shp[:-1], Nn)

    @staticmethod
    def backward(ctx, dy):
        x2, w, lora_a, lora_b, h, pre, gate_v, wt = ctx.saved_tensors
        shp, Nn, L, s, act, has_res, has_bias = ctx.meta
        need = ctx.needs_input_grad
        M, K = x2.shape
        dy2 = _c(dy).view(M, Nn)
        d_res = dy.reshape(*shp[:-1], Nn) if has_res else None
        lib = N.require() if dy2.is_cuda and _BACKEND == "fused" else None
        # undo gate / activation on the incoming gradient
        dgate = None
        if gate_v is not None:
            if lib is not None:
                g = torch.empty_like(dy2)
                N.check(lib.eri_gate_residual(None, dy2.data_ptr(), gate_v.data_ptr(),
                                              g.data_ptr(), M, Nn, L, gate_v.stride(0),
                                              N.stream_ptr()), "gate_bwd")
            else:
                g = R.gate_residual(None, dy2.view(-1, L, Nn), gate_v).view(M, Nn)
            dy2 = g
        if act is not None:
            if lib is not None:
                g = torch.empty_like(dy2)
                N.check(lib.eri_act_bwd(dy2.data_ptr(), pre.data_ptr(), g.data_ptr(), dy2.numel(),
                                        0 if act == "gelu" else 1, N.stream_ptr()), "act_bwd")
                dy2 = g
            else:
                pf = pre.float().requires_grad_(True)
                with torch.enable_grad():
                    a = torch.nn.functional.gelu(pf, approximate="tanh") if act == "gelu" \
                        else torch.nn.functional.silu(pf)
                dy2 = torch.autograd.grad(a, pf, dy2.float())[0].to(dy2.dtype)
        dx, dw, dbias, da, db = _linear_grads(dy2, x2, w, lora_a, lora_b, h, s, wt, need, shp, has_bias, lib)
        return dx, dw, dbias, da, db, None, None, d_res, dgate, None


def linear(x, w, bias=None, lora=None, act=None, residual=None, gate=None, wt=None):
    """Fused linear. lora = (A [r,K], B [N,r], scale) or None; act in {None,"gelu","silu"};
    residual [.., N] and gate [B, N] give ``residual + gate * y``."""
    if _native_ok(x, w, bias) and x.shape[-1] % 8 == 0:
        a, b, s = lora if lora is not None else (None, None, 1.0)
        if gate is not None and gate.requires_grad:
            # trainable modulation: keep the gate outside so that its gradient is produced
            y = _FusedLinear.apply(x, w, bias, a, b, float(s), act, None, None, wt)
            return gate_residual(residual, y, gate)
        return _FusedLinear.apply(x, w, bias, a, b, float(s), act, residual, gate, wt)
    y = R.linear(x, w, bias, lora, act, None, None)
    if gate is not None or residual is not None:
        y = R.gate_residual(residual, y, gate)
    return y


class _FusedLinearPair(torch.autograd.Function):
    """Two fused linears with the same shape of weight (the image and the text stream of a dual-stream
    block): y_i = [residual_i + gate_i *] act(x_i W_i^T + b_i + s_i (x_i A_i^T) B_i^T). The two main GEMMs
    share one launch in the forward, and the two input-gradient GEMMs one in the backward
    (``gemm_native_pair``), as do the rank-r products of both streams (``skinny_gemm_pair``); everything
    else is what ``_FusedLinear`` does per stream. Only for the native path with rank-16/32/64 adapters
    (or none) on both streams; ``linear_pair`` checks that.

    Two more modes chain an MLP without a separate activation-gradient pass. ``emit_pre``: the outputs
    are (pre_0, pre_1, u_0, u_1) with u_i = act(pre_i) marked non-differentiable, i.e. the layer is the
    plain linear that produces the pre-activation and the activation is a by-product of its epilogue.
    ``act_in`` with ``xp_i``: x_i is act_in(xp_i) (such a by-product), the layer is linear-of-activation
    as a function of xp_i, and its input-gradient GEMM applies the activation's derivative at xp_i in its
    epilogue, so the gradient it returns is already the one of the pre-activation."""

    @staticmethod
    def forward(ctx, act, emit_pre, act_in, x0, xp0, w0, b0, la0, lb0, s0, res0, gate0,
                x1, xp1, w1, b1, la1, lb1, s1, res1, gate1):
        streams = ((x0, xp0, w0, b0, la0, lb0, s0, res0, gate0), (x1, xp1, w1, b1, la1, lb1, s1, res1, gate1))
        need = ctx.needs_input_grad
        need_any = (any(need[3:9]), any(need[12:18]))
        kws, saved, metas = [], [], []
        for i, (x, xp, w, b, la, lb, sc, res, gate) in enumerate(streams):
            shp = x.shape
            K, Nn = shp[-1], w.shape[0]
            x2 = _c(x).view(-1, K)
            M, L = x2.shape[0], shp[-2]
            r = 0 if la is None else la.shape[0]
            pre = None
            if act is not None and (need_any[i] or emit_pre):
                pre = torch.empty(M, Nn, dtype=x.dtype, device=x.device)
            res2 = None if res is None else _c(res).view(-1, Nn)
            gate_v = _mod_view(gate, Nn)[0] if gate is not None else None
            xp2 = None if xp is None else _c(xp).view(-1, K)
            kws.append(dict(a=x2, b=w, bias=b, lora_h=None, lora_b=lb if r else None, act=act, pre_out=pre,
                            residual=res2, gate=gate_v, rows_per_batch=L, pdl=_pdl_ok()))
            saved += [x2, w, la, lb, None, None if emit_pre else pre, gate_v, xp2]
            metas.append((shp, Nn, L, sc, res is not None, b is not None))
        if la0 is not None:
            # both rank-r products in one launch, right before the grouped GEMM that consumes them
            h0, h1 = skinny_gemm_pair(kws[0]["a"], la0, s0, kws[1]["a"], la1, s1)
            kws[0]["lora_h"], kws[1]["lora_h"] = h0, h1
            saved[4], saved[12] = h0, h1
        # Training keeps the pre-activation anyway: the GEMM then writes it as its output and the activation
        # is a pass of its own (storing both from the epilogue costs the GEMM more than that pass does).
        unfuse = (act is not None and all(k["pre_out"] is not None and k["residual"] is None and k["gate"] is None
                                          for k in kws)
                  and _act_outside_epilogue(kws[0]["a"].shape[0], kws[0]["b"].shape[0], kws[0]["a"].shape[1]))
        if unfuse:
            for k in kws:
                k.update(out=k["pre_out"], act=None, pre_out=None)
        y0, y1 = gemm_native_pair(kws[0], kws[1])
        if unfuse:
            pres = (y0, y1)
            y0, y1 = torch.empty_like(y0), torch.empty_like(y1)
            for pr, yy in zip(pres, (y0, y1)):
                N.check(N.require().eri_act_fwd(pr.data_ptr(), yy.data_ptr(), pr.numel(), 0 if act == "gelu" else 1,
                                                N.stream_ptr()), "act_fwd")
            for k, pr in zip(kws, pres):
                k["pre_out"] = pr
        ctx.save_for_backward(*saved)
        ctx.meta = (act, emit_pre, act_in, metas)
        ctx.set_materialize_grads(False)       # an unused output (None gradient) costs nothing in backward
        y0, y1 = y0.view(*metas[0][0][:-1], metas[0][1]), y1.view(*metas[1][0][:-1], metas[1][1])
        if emit_pre:
            ctx.mark_non_differentiable(y0, y1)
            return kws[0]["pre_out"].view_as(y0), kws[1]["pre_out"].view_as(y1), y0, y1
        return y0, y1

    @staticmethod
    def backward(ctx, *douts):
        act, emit_pre, act_in, metas = ctx.meta
        dy0, dy1 = douts[0], douts[1]      # emit_pre: the gradients of the pre-activations
        sv = ctx.saved_tensors
        lib = N.require()
        need = ctx.needs_input_grad
        base = (3, 12)                     # positions of x0 / x1 among the forward's arguments
        parts = []
        kws = []
        for i, dy in enumerate((dy0, dy1)):
            if dy is None:
                kws.append(None)
                parts.append(None)
                continue
            x2, w, la, lb, h, pre, gate_v, xp2 = sv[8 * i: 8 * i + 8]
            shp, Nn, L, sc, has_res, has_bias = metas[i]
            M, K = x2.shape
            dy2 = _c(dy).view(M, Nn)
            d_res = dy.reshape(*shp[:-1], Nn) if has_res else None
            if gate_v is not None:
                g = torch.empty_like(dy2)
                N.check(lib.eri_gate_residual(None, dy2.data_ptr(), gate_v.data_ptr(), g.data_ptr(), M, Nn, L,
                                              gate_v.stride(0), N.stream_ptr()), "gate_bwd")
                dy2 = g
            if act is not None and not emit_pre:
                g = torch.empty_like(dy2)
                N.check(lib.eri_act_bwd(dy2.data_ptr(), pre.data_ptr(), g.data_ptr(), dy2.numel(),
                                        0 if act == "gelu" else 1, N.stream_ptr()), "act_bwd")
                dy2 = g
            r = 0 if la is None else la.shape[0]
            lb_t = la_t = None
            if r:
                lb_t, la_t = _lora_transposed(lb), _lora_transposed(la)
            kw = dict(a=dy2, b=w, b_mn=True, lora_h=None, lora_b=la_t, pdl=_pdl_ok())
            if act_in is not None:
                kw.update(act=act_in + "_bwd", pre_in=xp2)     # the input's activation derivative in the epilogue
            kws.append(kw)
            parts.append([dy2, None, d_res, lb_t, sc])
        # Ts_i = s_i * dY_i B_i: one launch for both streams when both have a gradient, right before the
        # grouped input-gradient GEMM
        live = [i for i in range(2) if parts[i] is not None and parts[i][3] is not None]
        if len(live) == 2:
            t0, t1 = skinny_gemm_pair(parts[0][0], parts[0][3], parts[0][4], parts[1][0], parts[1][3], parts[1][4])
            parts[0][1], parts[1][1] = t0, t1
        else:
            for i in live:
                parts[i][1] = skinny_gemm(parts[i][0], parts[i][3], alpha=parts[i][4])
        for i in live:
            kws[i]["lora_h"] = parts[i][1]
        dxs = [None, None]
        xin = 1 if act_in is not None else 0          # the differentiable input: xp_i or x_i
        want = [need[base[0] + xin] and kws[0] is not None, need[base[1] + xin] and kws[1] is not None]
        if all(want):
            dxs = list(gemm_native_pair(kws[0], kws[1]))
        else:
            for i in range(2):
                if want[i]:
                    dxs[i] = gemm_native(**kws[i])
        grads = [None, None, None]
        for i in range(2):
            if parts[i] is None:
                grads += [None] * 9
                continue
            x2, w, la, lb, h, pre, gate_v, xp2 = sv[8 * i: 8 * i + 8]
            shp, Nn, L, sc, has_res, has_bias = metas[i]
            dy2, ts, d_res = parts[i][:3]
            nd = need[base[i] + 1: base[i] + 6]      # (xp,) w, bias, A, B at offsets 1..4 of this slice
            dw = dbias = da = db = None
            if nd[1]:
                if _ACCUM_INTO_GRAD and w.grad is not None and w.grad.dtype == x2.dtype and w.grad.is_contiguous():
                    wgrad(dy2, x2, accum=w.grad)
                else:
                    dw = wgrad(dy2, x2)
            if has_bias and nd[2]:
                dbias = dy2.sum(0)
            if la is not None and nd[3]:
                if _ACCUM_INTO_GRAD and la.grad is not None and la.grad.dtype == x2.dtype:
                    lora_wgrad(x2, ts, out=la.grad, transpose_out=True, accumulate=True)
                else:
                    da = lora_wgrad(x2, ts, transpose_out=True)
            if la is not None and nd[4]:
                if _ACCUM_INTO_GRAD and lb.grad is not None and lb.grad.dtype == h.dtype:
                    lora_wgrad(dy2, h, out=lb.grad, accumulate=True)
                else:
                    db = lora_wgrad(dy2, h)
            dx = None if dxs[i] is None else dxs[i].view(shp)
            grads += [None if xin else dx, dx if xin else None, dw, dbias, da, db, None, d_res, None]
        return tuple(grads)


def _linear_pair_ok(x0, lin0, x1, lin1) -> bool:
    (w0, b0, lo0, r0, g0), (w1, b1, lo1, r1, g1) = lin0, lin1

    def rank_ok(lo):
        return lo is None or lo[0].shape[0] in (16, 32, 64)
    return bool(_GEMM_GROUP and _GEMM_NATIVE == "native" and _native_ok(x0, w0, b0) and _native_ok(x1, w1, b1)
                and w0.shape == w1.shape and x0.shape[-1] % 8 == 0 and rank_ok(lo0) and rank_ok(lo1)
                and (lo0 is None) == (lo1 is None) and (lo0 is None or lo0[0].shape[0] == lo1[0].shape[0])
                and (b0 is None) == (b1 is None)
                and x0.numel() // x0.shape[-1] >= 256 and x1.numel() // x1.shape[-1] >= 256
                and gemm_supported(x0.numel() // x0.shape[-1], w0.shape[0], x0.shape[-1])
                and gemm_supported(x1.numel() // x1.shape[-1], w1.shape[0], x1.shape[-1]))


def linear_pair_ok(x0, lin0, x1, lin1) -> bool:
    """Whether ``linear_pair`` would run the two layers as grouped launches."""
    return _linear_pair_ok(x0, lin0, x1, lin1)


def linear_pair(x0, lin0, x1, lin1, act=None, emit_pre=False, act_in=None, x_pre=(None, None)):
    """``lin_i`` = (w, bias, lora or None, residual or None, gate or None). Returns (y0, y1) of two fused
    linears whose main GEMMs (and input-gradient GEMMs) share one launch when both run on the native path
    with matching shapes; otherwise exactly ``linear`` twice. ``emit_pre`` / ``act_in`` + ``x_pre`` (only
    when ``linear_pair_ok``): see ``_FusedLinearPair``; with ``emit_pre`` the result is
    (pre_0, pre_1, act(pre_0), act(pre_1))."""
    (w0, b0, lo0, r0, g0), (w1, b1, lo1, r1, g1) = lin0, lin1
    if emit_pre or act_in is not None:
        a0, bb0, s0 = lo0 if lo0 is not None else (None, None, 1.0)
        a1, bb1, s1 = lo1 if lo1 is not None else (None, None, 1.0)
        return _FusedLinearPair.apply(act, emit_pre, act_in, x0, x_pre[0], w0, b0, a0, bb0, float(s0), r0, g0,
                                      x1, x_pre[1], w1, b1, a1, bb1, float(s1), r1, g1)

    if not _linear_pair_ok(x0, lin0, x1, lin1):
        return (linear(x0, w0, b0, lora=lo0, act=act, residual=r0, gate=g0),
                linear(x1, w1, b1, lora=lo1, act=act, residual=r1, gate=g1))
    a0, bb0, s0 = lo0 if lo0 is not None else (None, None, 1.0)
    a1, bb1, s1 = lo1 if lo1 is not None else (None, None, 1.0)
    if (g0 is not None and g0.requires_grad) or (g1 is not None and g1.requires_grad):
        # trainable modulation: the gates stay outside the GEMM epilogue so that their gradients are produced
        y0, y1 = _FusedLinearPair.apply(act, False, None, x0, None, w0, b0, a0, bb0, float(s0), None, None,
                                        x1, None, w1, b1, a1, bb1, float(s1), None, None)
        return gate_residual(r0, y0, g0), gate_residual(r1, y1, g1)
    return _FusedLinearPair.apply(act, False, None, x0, None, w0, b0, a0, bb0, float(s0), r0, g0,
                                  x1, None, w1, b1, a1, bb1, float(s1), r1, g1)


_GLU_FUSED = os.environ.get("ERI_B200_GLU_FUSED", "1") == "1"
_GLU_CODE = {("gelu", False): 1, ("silu", False): 2, ("gelu", True): 3, ("silu", True): 4}


class _FusedLinearGlu(torch.autograd.Function):
    """out[M, hidden] = glu(x W^T + b + s (x A^T) B^T) with W an up-projection [2*hidden, K]: the
    gate is applied in the GEMM epilogue (each CTA pair holds the value columns next to their gate
    columns), so the [M, 2*hidden] projection is written once for backward and never re-read in
    forward. The reference fuses the same pair in its feed-forward kernel
    (crates/training/src/sdxl/runtime.rs:249-321, host side :698-799)."""

    @staticmethod
    def forward(ctx, x, w, bias, lora_a, lora_b, lora_scale, code, wt):
        shp = x.shape
        K = shp[-1]
        x2 = _c(x).view(-1, K)
        M, N2 = x2.shape[0], w.shape[0]
        r = 0 if lora_a is None else lora_a.shape[0]
        need_pre = any(ctx.needs_input_grad[:5])
        pre = torch.empty(M, N2, dtype=x.dtype, device=x.device) if need_pre else None
        h = skinny_gemm(x2, lora_a, alpha=lora_scale) if r else None
        out = gemm_native(x2, w, bias=bias, lora_h=h, lora_b=lora_b if r else None, glu=code,
                          pre_out=pre, pdl=_pdl_ok())
        ctx.save_for_backward(x2, w, lora_a, lora_b, h, pre, wt)
        ctx.meta = (shp, N2, lora_scale, code, bias is not None)
        return out.view(*shp[:-1], N2 // 2)

    @staticmethod
    def backward(ctx, dout):
        x2, w, lora_a, lora_b, h, pre, wt = ctx.saved_tensors
        shp, N2, s, code, has_bias = ctx.meta
        M = x2.shape[0]
        lib = N.require()
        d2 = _c(dout).view(M, N2 // 2)
        dh = torch.empty(M, N2, dtype=x2.dtype, device=x2.device)
        N.check(lib.eri_glu_bwd(d2.data_ptr(), pre.data_ptr(), dh.data_ptr(), M, N2 // 2,
                                0 if code in (1, 3) else 1, 1 if code >= 3 else 0, N.stream_ptr()), "glu_bwd")
        dx, dw, dbias, da, db = _linear_grads(dh, x2, w, lora_a, lora_b, h, s, wt, ctx.needs_input_grad,
                                              shp, has_bias, lib)
        return dx, dw, dbias, da, db, None, None, None


def linear_glu(x, lin, mode="gelu", act_first=True):
    """``glu(lin(x), mode, act_first)`` for an up-projection module ``lin`` ([2*hidden, K] weight).
    One GEMM launch with the gate in its epilogue when the shape fits the two-CTA kernel and the
    adapter (if any) is a plain LoRA; otherwise the projection and the gate run as separate ops."""
    ad = getattr(lin, "adapter", None)
    w, b = lin.weight, lin.bias
    rows = x.numel() // x.shape[-1]
    plain_lora = ad is not None and getattr(ad, "kind", "") == "lora" and ad.rank in (16, 32, 64) \
        and not (ad.dropout > 0 and ad.training)
    if _GLU_FUSED and _GEMM_NATIVE == "native" and _native_ok(x, w, b) and (ad is None or plain_lora) \
            and type(lin).__name__ == "Linear" and rows >= 256 and w.shape[0] >= 256 and w.shape[0] % 16 == 0 \
            and x.shape[-1] % 8 == 0 and x.shape[-1] >= 64:
        wt = lin.frozen_transpose() if torch.is_grad_enabled() else None
        a, bb, s = (ad.lora_A, ad.lora_B, float(ad.scale)) if ad is not None else (None, None, 1.0)
        return _FusedLinearGlu.apply(x, w, b, a, bb, s, _GLU_CODE[(mode, bool(act_first))], wt)
    return glu(lin(x), mode, act_first)


def _rows_ok(*ts):
    return all(t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0
               and t.data_ptr() % 16 == 0 for t in ts)


def small_wgrad(dy2, xin, scale: float = 1.0):
    """dW[N, K] = scale * dy2[T, N]^T @ xin[T, K] for a handful of rows (T <= 8): one pass that is
    bound by writing dW (native kernel); other shapes use ``torch``."""
    T, Nn = dy2.shape
    K = xin.shape[1]
    lib = N.lib() if dy2.is_cuda else None
    if lib is not None and _BACKEND == "fused" and hasattr(lib, "eri_rows_wgrad") and T <= 8 and K % 8 == 0 \
            and _rows_ok(xin) and dy2.dtype == torch.bfloat16 and dy2.stride(1) == 1:
        dw = torch.empty(Nn, K, dtype=torch.bfloat16, device=dy2.device)
        N.check(lib.eri_rows_wgrad(dy2.data_ptr(), dy2.stride(0), xin.data_ptr(), xin.stride(0), dw.data_ptr(), K,
                                   T, Nn, K, 0, float(scale), N.stream_ptr()), "rows_wgrad")
        return dw
    dw = dy2.t() @ xin
    return dw if scale == 1.0 else dw * scale


def small_dgrad(dy2, w):
    """dx[T, K] = dy2[T, N] @ w[N, K] for T <= 8: one pass over w split across CTAs by rows of w; the
    fp32 partial planes are added in split order (deterministic)."""
    T, Nn = dy2.shape
    K = w.shape[1]
    lib = N.lib() if dy2.is_cuda else None
    if lib is not None and _BACKEND == "fused" and hasattr(lib, "eri_rows_dgrad") and T <= 8 and K % 8 == 0 \
            and _rows_ok(w) and dy2.dtype == torch.bfloat16 and dy2.stride(1) == 1:
        max_splits = 1024
        part = torch.empty(max_splits, T, K, dtype=torch.float32, device=dy2.device)
        n = lib.eri_rows_dgrad(dy2.data_ptr(), dy2.stride(0), w.data_ptr(), w.stride(0), part.data_ptr(), T, Nn, K,
                               max_splits, N.stream_ptr())
        N.check(0 if n > 0 else (n or -1), "rows_dgrad")
        return part[:n].sum(0).to(torch.bfloat16)
    return dy2 @ w


class _SmallLinear(torch.autograd.Function):
    """Conditioning-vector linear (M <= 8 rows): y = f_out(silu_in?(x) W^T + b)."""

    @staticmethod
    def forward(ctx, x, w, bias, silu_in):
        x2 = _c(x).view(-1, x.shape[-1])
        M, K = x2.shape
        Nn = w.shape[0]
        y = torch.empty(M, Nn, dtype=x.dtype, device=x.device)
        N.check(N.require().eri_gemv_bf16(x2.data_ptr(), w.data_ptr(), N.ptr(bias), y.data_ptr(),
                                          M, Nn, K, x2.stride(0), w.stride(0), Nn,
                                          1 if silu_in else 0, 0, N.stream_ptr()), "gemv")
        ctx.save_for_backward(x2, w)
        ctx.meta = (x.shape, silu_in, bias is not None)
        return y.view(*x.shape[:-1], Nn)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        shp, silu_in, has_bias = ctx.meta
        dy2 = dy.reshape(-1, dy.shape[-1])
        xin = torch.nn.functional.silu(x2.float()).to(x2.dtype) if silu_in else x2
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = small_dgrad(dy2, w)
            if silu_in:
                xf = x2.float()
                sg = torch.sigmoid(xf)
                dx = (dx.float() * (sg * (1 + xf * (1 - sg)))).to(x2.dtype)
            dx = dx.view(shp)
        if ctx.needs_input_grad[1]:
            dw = small_wgrad(dy2, xin)
        if has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0)
        return dx, dw, db, None


def small_linear(x, w, bias=None, silu_in=False):
    """Linear on a handful of rows (adaLN modulation and embedders); SiLU on the input optional."""
    rows = x.numel() // x.shape[-1]
    if _native_ok(x, w, bias) and rows <= 8 and x.shape[-1] % 8 == 0 and x.shape[-1] * rows <= 50000:
        return _SmallLinear.apply(x, w, bias, silu_in)
    xin = torch.nn.functional.silu(x) if silu_in else x
    return torch.nn.functional.linear(xin, w, bias)


# ---------------------------------------------------------------------------- attention
# read once at import: the ATTN_* switches of the library attention path (utils/env_flags.py)
_ATTN_ENV_POLICY = any(os.environ.get(k) for k in ("ATTN_Q_CHUNK", "ATTN_KV_CHUNK", "ATTN_MAX_WS_MB", "ATTN_MIN_FREE_MB"))


_HEAD_PAD = os.environ.get("ERI_B200_ATTN_HEAD_PAD", "1") == "1"
ATTENTION_CALLS = {"native": 0, "library": 0}     # forward calls by path since import (benchmarks print it)


def attention(q, k, v, scale=None, mask=None, out=None):
    """Non-causal attention over token-major [B, L, H, Dh] tensors. ``out``: optional destination
    buffer for the native kernel (ignored by the library path, which returns its own tensor)."""
    if _ATTN_NATIVE == "native" and _native_ok(q, k, v):
        from . import flash_attn as FA
        # key-only masks (text padding, [B, 1, 1, T]) ride on the native kernel as a per-key bias
        if FA.supported(q, k, v) and (mask is None or FA.mask_is_key_only(mask, q.shape[0], k.shape[1])):
            ATTENTION_CALLS["native"] += 1
            return FA.flash_attention(q, k, v, scale, out, mask)
        # other head sizes below 128 (SD1.5: 40 and 80) ride on the 64 / 128 kernels with zero columns
        # appended: zero query / key columns leave the scores unchanged, zero value columns give zero
        # output columns that are cut off again (the pad and the slice are differentiable copies)
        D = q.shape[-1]
        if _HEAD_PAD and D not in (64, 128) and 16 <= D < 128 and D % 8 == 0 and \
                (mask is None or FA.mask_is_key_only(mask, q.shape[0], k.shape[1])):
            pad = (64 if D < 64 else 128) - D
            qp, kp, vp = (torch.nn.functional.pad(t, (0, pad)) for t in (q, k, v))
            if FA.supported(qp, kp, vp):
                ATTENTION_CALLS["native"] += 1
                sc = scale if scale is not None else 1.0 / math.sqrt(D)
                return FA.flash_attention(qp, kp, vp, sc, None, mask)[..., :D].contiguous()
    ATTENTION_CALLS["library"] += 1
    if mask is None and _ATTN_ENV_POLICY:
        from ..utils.env_flags import library_attention
        o = library_attention(q, k, v, scale)
        if o is not None:
            return o
    return R.attention(q, k, v, scale, mask)


# ---------------------------------------------------------------------------- losses / noise
class _MseLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pred, target, weight):
        pred, target = _c(pred), _c(target)
        n = pred.numel()
        npb = n // pred.shape[0]
        loss = torch.zeros((), dtype=torch.float32, device=pred.device)
        dpred = torch.empty_like(pred)
        w = None if weight is None else weight.float().contiguous()
        N.check(N.require().eri_mse_fwd_bwd(pred.data_ptr(), target.data_ptr(), N.ptr(w),
                                            loss.data_ptr(), dpred.data_ptr(), n, npb, 1.0,
                                            N.stream_ptr()), "mse")
        ctx.save_for_backward(dpred)
        return loss

    @staticmethod
    def backward(ctx, g):
        (dpred,) = ctx.saved_tensors
        return dpred * g.to(dpred.dtype), None, None


def mse_loss(pred, target, weight=None):
    """mean(weight[b] * (pred - target)^2) with the gradient produced in the same pass."""
    if _native_ok(pred, target) and pred.numel() % 8 == 0 and (pred.numel() // pred.shape[0]) % 8 == 0:
        return _MseLoss.apply(pred, target, weight)
    return R.mse(pred, target, weight)


def noise_mix(x0, coef, seed: int, offset: int = 0, eps=None, patch=2, want_eps=False):
    """Build x_t and the regression target from clean latents in one pass.

    x0 [B, C, H, W]; coef [4, B] fp32 rows (a, s, ca, cb): x_t = a*x0 + s*eps,
    target = ca*eps + cb*x0. Noise comes from a Philox counter stream (seed, offset) unless
    ``eps`` is given. Returns token-major (x_t, target[, eps]) of shape [B, HW/p^2, C*p*p].
    """
    B, C, H, W = x0.shape
    if _native_ok(x0, eps) and (B * C * H * W) % 4 == 0:
        x0 = _c(x0)
        L, D = (H // patch) * (W // patch), C * patch * patch
        xt = torch.empty(B, L, D, dtype=x0.dtype, device=x0.device)
        tg = torch.empty_like(xt)
        eo = torch.empty_like(xt) if want_eps else None
        cf = coef.float().contiguous()
        N.check(N.require().eri_noise_mix(x0.data_ptr(), N.ptr(_c(eps)), cf.data_ptr(),
                                          xt.data_ptr(), tg.data_ptr(), N.ptr(eo), B, C, H, W,
                                          patch, seed, offset, N.stream_ptr()), "noise_mix")
        return (xt, tg, eo) if want_eps else (xt, tg)
    if eps is None:
        gen = torch.Generator(device=x0.device).manual_seed(seed + offset)
        eps = torch.randn(x0.shape, generator=gen, device=x0.device, dtype=torch.float32).to(x0.dtype)
    xt, tg = R.noise_mix(x0, eps, coef, patch)
    return (xt, tg, R.patchify(eps, patch)) if want_eps else (xt, tg)


def randn_bf16(shape, seed: int, offset: int = 0, device="cuda", mean=0.0, std=1.0):
    out = torch.empty(shape, dtype=torch.bfloat16, device=device)
    if out.is_cuda and _BACKEND == "fused":
        N.check(N.require().eri_randn_bf16(out.data_ptr(), out.numel(), seed, offset, mean, std,
                                           N.stream_ptr()), "randn")
        return out
    gen = torch.Generator(device=out.device).manual_seed(seed + offset)
    return (torch.randn(shape, generator=gen, device=out.device) * std + mean).to(torch.bfloat16)


def sumsq(flat, out=None):
    """Sum of squares of a flat bf16 buffer into a device fp32 scalar (no host sync)."""
    if out is None:
        out = torch.zeros((), dtype=torch.float32, device=flat.device)
    else:
        out.zero_()
    if _native_ok(flat):
        N.check(N.require().eri_sumsq_bf16(flat.data_ptr(), flat.numel(), out.data_ptr(),
                                           N.stream_ptr()), "sumsq")
    else:
        out.add_(flat.float().pow(2).sum())
    return out


# ---------------------------------------------------------------------------- GroupNorm (+SiLU)
class _GroupNormSilu(torch.autograd.Function):
    """x [N, HW, C] (channels-last rows). Two bandwidth-bound passes each way (csrc/groupnorm.cu);
    the channel->group reductions between them run on the [N, C] statistics."""

    @staticmethod
    def forward(ctx, x, weight, bias, groups, eps, silu_flag):
        Nn, HW, C = x.shape
        x = _c(x)
        lib = N.require()
        stats = torch.zeros(Nn, C, 2, dtype=torch.float32, device=x.device)
        N.check(lib.eri_gn_stats_fwd(x.data_ptr(), stats.data_ptr(), Nn, HW, C, N.stream_ptr()), "gn_stats_fwd")
        m = HW * (C // groups)
        gs = stats.view(Nn, groups, C // groups, 2).sum(2)
        mean = gs[..., 0] / m
        var = (gs[..., 1] / m - mean * mean).clamp_min_(0.0)
        rstd = torch.rsqrt(var + eps)
        mean, rstd = mean.contiguous(), rstd.contiguous()
        y = torch.empty_like(x)
        N.check(lib.eri_gn_apply_fwd(x.data_ptr(), weight.data_ptr(), N.ptr(bias), mean.data_ptr(),
                                     rstd.data_ptr(), y.data_ptr(), Nn, HW, C, groups, int(silu_flag),
                                     N.stream_ptr()), "gn_apply_fwd")
        ctx.save_for_backward(x, weight, bias, mean, rstd)
        ctx.meta = (groups, silu_flag)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, bias, mean, rstd = ctx.saved_tensors
        groups, silu_flag = ctx.meta
        Nn, HW, C = x.shape
        dy = _c(dy)
        lib = N.require()
        stats = torch.zeros(Nn, C, 2, dtype=torch.float32, device=x.device)
        N.check(lib.eri_gn_stats_bwd(x.data_ptr(), dy.data_ptr(), weight.data_ptr(), N.ptr(bias),
                                     mean.data_ptr(), rstd.data_ptr(), stats.data_ptr(), Nn, HW, C, groups,
                                     int(silu_flag), N.stream_ptr()), "gn_stats_bwd")
        m = HW * (C // groups)
        wf = weight.float()
        ws = (stats * wf[None, :, None]).view(Nn, groups, C // groups, 2).sum(2) / m
        s1, s2 = ws[..., 0].contiguous(), ws[..., 1].contiguous()
        dx = torch.empty_like(x)
        N.check(lib.eri_gn_apply_bwd(x.data_ptr(), dy.data_ptr(), weight.data_ptr(), N.ptr(bias),
                                     mean.data_ptr(), rstd.data_ptr(), s1.data_ptr(), s2.data_ptr(),
                                     dx.data_ptr(), Nn, HW, C, groups, int(silu_flag), N.stream_ptr()),
                "gn_apply_bwd")
        dw = stats[..., 1].sum(0).to(weight.dtype) if ctx.needs_input_grad[1] else None
        db = stats[..., 0].sum(0).to(weight.dtype) if (bias is not None and ctx.needs_input_grad[2]) else None
        return dx, dw, db, None, None, None


def group_norm_silu(x, weight, bias=None, groups=32, eps=1e-5, silu=True):
    """GroupNorm followed by an optional SiLU on a channels-last activation. ``x`` is either
    [N, HW, C] or an [N, C, H, W] tensor in ``torch.channels_last`` memory format (returned in the
    same logical shape and format)."""
    nchw = x.dim() == 4
    if nchw:
        Nn, C, H, W = x.shape
        rows = x.permute(0, 2, 3, 1)
        if not rows.is_contiguous():
            rows = rows.contiguous()
        rows = rows.view(Nn, H * W, C)
    else:
        rows = x
    C = rows.shape[-1]
    if _native_ok(rows, weight, bias) and C % 8 == 0 and C % groups == 0 and C <= 8192:
        y = _GroupNormSilu.apply(rows, weight, bias, groups, eps, silu)
    else:
        y = R.group_norm_silu(rows, weight, bias, groups, eps, silu)
    if nchw:
        return y.view(Nn, H, W, C).permute(0, 3, 1, 2)
    return y


# ---------------------------------------------------------------------------- token routing
def token_scores(x):
    """L2 norm of every token row of x [B, L, D] -> fp32 [B, L]."""
    if _native_ok(x) and x.shape[-1] % 8 == 0:
        x = _c(x)
        out = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
        N.check(N.require().eri_row_l2norm(x.data_ptr(), out.data_ptr(), out.numel(), x.shape[-1],
                                           N.stream_ptr()), "row_l2norm")
        return out
    return x.float().norm(dim=-1)


def topk_indices(scores, k):
    """Indices [B, k] (int64) of the k largest non-negative scores per row, descending, ties by
    lower index; selection runs on the device (no host sort)."""
    B, L = scores.shape
    if scores.is_cuda and _BACKEND == "fused" and L <= 16384 and scores.dtype == torch.float32:
        idx = torch.empty(B, k, dtype=torch.int32, device=scores.device)
        N.check(N.require().eri_topk_desc(_c(scores).data_ptr(), idx.data_ptr(), B, L, k, N.stream_ptr()), "topk")
        return idx.long()
    return scores.topk(k, dim=1).indices


class _GatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, idx32):
        B, L, D = x.shape
        k = idx32.shape[1]
        x = _c(x)
        out = torch.empty(B, k, D, dtype=x.dtype, device=x.device)
        N.check(N.require().eri_gather_rows(x.data_ptr(), idx32.data_ptr(), out.data_ptr(), B, L, k, D,
                                            N.stream_ptr()), "gather_rows")
        ctx.save_for_backward(idx32)
        ctx.L = L
        return out

    @staticmethod
    def backward(ctx, dy):
        (idx32,) = ctx.saved_tensors
        B, k, D = dy.shape
        L = ctx.L
        dy = _c(dy)
        lib = N.require()
        inv = torch.full((B, L), -1, dtype=torch.int32, device=dy.device)
        N.check(lib.eri_build_inverse(idx32.data_ptr(), inv.data_ptr(), B, L, k, N.stream_ptr()), "build_inverse")
        dx = torch.empty(B, L, D, dtype=dy.dtype, device=dy.device)
        N.check(lib.eri_reinject_rows(None, dy.data_ptr(), inv.data_ptr(), dx.data_ptr(), B, L, k, D,
                                      N.stream_ptr()), "scatter_rows")
        return dx, None


class _ReinjectRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, full, routed, idx32):
        B, L, D = full.shape
        k = idx32.shape[1]
        full, routed = _c(full), _c(routed)
        lib = N.require()
        inv = torch.full((B, L), -1, dtype=torch.int32, device=full.device)
        N.check(lib.eri_build_inverse(idx32.data_ptr(), inv.data_ptr(), B, L, k, N.stream_ptr()), "build_inverse")
        out = torch.empty_like(full)
        N.check(lib.eri_reinject_rows(full.data_ptr(), routed.data_ptr(), inv.data_ptr(), out.data_ptr(),
                                      B, L, k, D, N.stream_ptr()), "reinject_rows")
        ctx.save_for_backward(idx32, inv)
        return out

    @staticmethod
    def backward(ctx, dy):
        idx32, inv = ctx.saved_tensors
        B, L, D = dy.shape
        k = idx32.shape[1]
        dy = _c(dy)
        lib = N.require()
        d_routed = torch.empty(B, k, D, dtype=dy.dtype, device=dy.device)
        N.check(lib.eri_gather_rows(dy.data_ptr(), idx32.data_ptr(), d_routed.data_ptr(), B, L, k, D,
                                    N.stream_ptr()), "gather_rows")
        d_full = dy * (inv < 0).unsqueeze(-1).to(dy.dtype)
        return d_full, d_routed, None


def gather_rows(x, idx):
    """x [B, L, D], idx [B, k] -> [B, k, D]."""
    if _native_ok(x) and x.shape[-1] % 8 == 0:
        return _GatherRows.apply(x, idx.to(torch.int32).contiguous())
    return torch.gather(x, 1, idx.long().unsqueeze(-1).expand(-1, -1, x.shape[-1]))


def reinject_rows(full, routed, idx):
    """Copy of ``full`` [B, L, D] whose rows ``idx`` [B, k] are replaced by ``routed`` [B, k, D]."""
    if _native_ok(full, routed) and full.shape[-1] % 8 == 0:
        return _ReinjectRows.apply(full, routed, idx.to(torch.int32).contiguous())
    return full.scatter(1, idx.long().unsqueeze(-1).expand(-1, -1, full.shape[-1]), routed)
