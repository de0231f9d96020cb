"""Python binding of the tcgen05 flash-attention kernels (``csrc/flash_attn.cu``).

Tensors are token-major ``[B, L, H, Dh]`` bf16. The forward returns the output and the
log-sum-exp per (batch, head, query); the backward kernels recompute the probabilities from it.
"""
from __future__ import annotations

import math

import torch

from . import _native as N

_P, _I, _F = N.C.c_void_p, N.C.c_int, N.C.c_float
N._SIGNATURES.update({
    "eri_flash_attn_fwd": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P],
    "eri_flash_attn_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P],
    "eri_fa_check_error": [],
    "eri_fa_bwd_check_error": [],
})


def _bind(lib):
    for name in ("eri_flash_attn_fwd", "eri_flash_attn_bwd", "eri_fa_check_error",
                 "eri_fa_bwd_check_error"):
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.argtypes = N._SIGNATURES[name]
            fn.restype = N.C.c_int


def has_forward() -> bool:
    lib = N.lib()
    return lib is not None and hasattr(lib, "eri_flash_attn_fwd")


def has_backward() -> bool:
    lib = N.lib()
    return lib is not None and hasattr(lib, "eri_flash_attn_bwd")


def supported(q, k, v) -> bool:
    if not has_forward():
        return False
    B, L, H, D = q.shape
    return (D in (64, 128) and q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
            and k.shape[1] >= 128 and L >= 128 and k.shape[2] == H and v.shape == k.shape)


def fwd(q, k, v, scale=None, out=None):
    """Returns (out [B, Lq, H, Dh] bf16, lse [B, H, Lq] fp32). ``out``: optional contiguous
    destination of q's shape (e.g. a buffer that peers can read)."""
    lib = N.require()
    _bind(lib)
    B, Lq, H, D = q.shape
    Lk = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty_like(q)
    elif out.shape != q.shape or out.dtype != q.dtype or not out.is_contiguous():
        raise ValueError("flash attention: out must be contiguous with q's shape and dtype")
    lse = torch.empty(B, H, Lq, dtype=torch.float32, device=q.device)
    N.check(lib.eri_flash_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                   lse.data_ptr(), B, H, Lq, Lk, D, scale, N.stream_ptr()),
            "flash_attn_fwd")
    return out, lse


def bwd(do, q, k, v, out, lse, scale=None):
    """Returns (dq, dk, dv)."""
    lib = N.require()
    _bind(lib)
    B, Lq, H, D = q.shape
    Lk = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    Lp = (Lq + 127) // 128 * 128
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    lse2 = torch.empty(B, H, Lp, dtype=torch.float32, device=q.device)
    delta = torch.empty_like(lse2)
    N.check(lib.eri_flash_attn_bwd(do.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                   out.data_ptr(), lse.data_ptr(), lse2.data_ptr(),
                                   delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                   B, H, Lq, Lk, D, scale, N.stream_ptr()), "flash_attn_bwd")
    return dq, dk, dv


def check_error() -> int:
    lib = N.require()
    _bind(lib)
    e = lib.eri_fa_check_error()
    if not e and hasattr(lib, "eri_fa_bwd_check_error"):
        e = lib.eri_fa_bwd_check_error()
    return e


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, out_buf=None):
        if out_buf is not None:
            ctx.mark_dirty(out_buf)          # an input that is written in place and returned
        out, lse = fwd(q, k, v, scale, out_buf)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse = ctx.saved_tensors
        do = do.contiguous()
        if has_backward():
            dq, dk, dv = bwd(do, q, k, v, out, lse, ctx.scale)
            return dq, dk, dv, None, None
        # Library recompute path, used only while the native backward is absent from the build.
        from . import reference as R
        with torch.enable_grad():
            qq, kk, vv = (t.detach().requires_grad_() for t in (q, k, v))
            o = R.attention(qq, kk, vv, ctx.scale)
        dq, dk, dv = torch.autograd.grad(o, (qq, kk, vv), do)
        return dq, dk, dv, None, None


def flash_attention(q, k, v, scale=None, out=None):
    return _FlashAttention.apply(q, k, v, scale, out)
