"""Python binding of the tcgen05 flash-attention kernels (``csrc/flash_attn.cu``).

Tensors are token-major ``[B, L, H, Dh]`` bf16. The forward returns the output and the
log-sum-exp per (batch, head, query); the backward kernels recompute the probabilities from it.

Key masks: a mask that depends on (batch, key) only — the text-padding mask ``[B, 1, 1, T]`` of
cached-embedding batches, boolean or additive — becomes a per-key bias row that the kernels add to
the scaled scores (``key_bias``). Fewer than 128 keys (SDXL cross-attention over 77 text tokens) run
as one key tile whose padding is blanked by the same bias.
"""
from __future__ import annotations

import math
import os

import torch

from . import _native as N

_P, _I, _F = N.C.c_void_p, N.C.c_int, N.C.c_float
N._SIGNATURES.update({
    "eri_flash_attn_fwd": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P],
    "eri_flash_attn_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P],
    "eri_flash_attn_fwd_ld": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, N.C.c_longlong, _P],
    "eri_flash_attn_bwd_ld": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, N.C.c_longlong, _P],
    "eri_flash_attn_fwd_masked": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P],
    "eri_flash_attn_bwd_masked": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P],
    "eri_flash_attn_fwd_pair": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P],
    "eri_fa_check_error": [],
    "eri_fa2_check_error": [],
    "eri_fa_bwd_check_error": [],
})

_LOG2E = 1.4426950408889634
_PAD_BIAS = {}
_MASKED = -1.0e30      # bias of a masked key: its probability is exactly zero, and the value stays finite


def _bind(lib):
    for name in ("eri_flash_attn_fwd", "eri_flash_attn_bwd", "eri_flash_attn_fwd_ld", "eri_flash_attn_bwd_ld",
                 "eri_flash_attn_fwd_masked",
                 "eri_flash_attn_bwd_masked", "eri_flash_attn_fwd_pair", "eri_fa_check_error",
                 "eri_fa2_check_error", "eri_fa_bwd_check_error"):
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


# The forward for head size 128 without a mask runs on CTA pairs (csrc/flash_attn2.cu) once a
# one-time self-check on the device has passed: the pair kernel's result on a small case must agree
# with the one-CTA kernel and leave its error word clear. ERI_B200_FA_PAIR=0 keeps the one-CTA kernel.
_PAIR_ENABLED = os.environ.get("ERI_B200_FA_PAIR", "0") == "1"
_PAIR_OK = {}


def _poly_pairs() -> int:
    v = os.environ.get("ERI_B200_FA_POLY", "4")
    return int(v) if v in ("0", "4", "8") else 4


def _pair_call(lib, q, k, v, out, lse, scale):
    B, Lq, H, D = q.shape
    return lib.eri_flash_attn_fwd_pair(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                       B, H, Lq, k.shape[1], D, scale, _poly_pairs(), N.stream_ptr())


def pair_forward_ok(device, force: bool = False) -> bool:
    """Whether the CTA-pair forward kernel may be used on ``device`` (checked once per device).
    ``force`` runs the self-check although ``ERI_B200_FA_PAIR`` leaves the kernel off (tests, benchmarks)."""
    if not (_PAIR_ENABLED or force):
        return False
    key = str(device)
    if key in _PAIR_OK:
        return _PAIR_OK[key]
    lib = N.require()
    _bind(lib)
    ok = False
    if hasattr(lib, "eri_flash_attn_fwd_pair"):
        g = torch.Generator(device=device).manual_seed(1234)
        q, k, v = (torch.randn(1, 384, 2, 128, device=device, generator=g).bfloat16() for _ in range(3))
        scale = 1.0 / math.sqrt(128)
        o1, o2 = torch.empty_like(q), torch.empty_like(q)
        l1 = torch.empty(1, 2, 384, dtype=torch.float32, device=device)
        l2 = torch.empty_like(l1)
        c1 = lib.eri_flash_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o1.data_ptr(), l1.data_ptr(), 1, 2, 384,
                                    384, 128, scale, N.stream_ptr())
        c2 = _pair_call(lib, q, k, v, o2, l2, scale)
        torch.cuda.synchronize(device)
        err = lib.eri_fa2_check_error()
        ok = (c1 == 0 and c2 == 0 and err == 0
              and (o1.float() - o2.float()).abs().max().item() < 2e-2 and (l1 - l2).abs().max().item() < 1e-2)
        if not ok:
            import warnings
            warnings.warn(f"CTA-pair attention forward failed its self-check on {device} (codes {c1}/{c2}, error word "
                          f"{err}); using the one-CTA kernel")
    _PAIR_OK[key] = ok
    return ok


def supported(q, k, v) -> bool:
    """Shapes the kernels take: head size 64 / 128, at least one key, at least 16 query rows
    (shorter query sets are conditioning-vector sized and stay on the library)."""
    if not has_forward():
        return False
    B, L, H, D = q.shape
    return (D in (64, 128) and q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
            and k.shape[1] >= 1 and L >= 16 and k.shape[2] == H and v.shape == k.shape and k.shape[0] == B)


def mask_is_key_only(mask, B, Lk) -> bool:
    """True for masks that depend on (batch, key) only: [B|1, Lk] or [B|1, 1, 1, Lk]."""
    if mask is None:
        return False
    shp = tuple(mask.shape)
    if len(shp) == 2:
        return shp[1] == Lk and shp[0] in (1, B)
    return len(shp) == 4 and shp[1] == 1 and shp[2] == 1 and shp[3] == Lk and shp[0] in (1, B)


def _with_tile_flags(kb):
    """[B, Lkb] bias rows -> one flat fp32 buffer: the rows, then one int32 per (batch, 128-key tile)
    that is 1 when any key of the tile carries a non-zero bias. The kernels run their unmasked fast
    path on the tiles whose flag is 0 (all but the text-padding tiles of a joint sequence)."""
    B, Lkb = kb.shape
    flags = (kb.view(B, Lkb // 128, 128) != 0).any(-1).to(torch.int32)
    return torch.cat([kb.reshape(-1), flags.reshape(-1).view(torch.float32)])


def key_bias(mask, B, Lk, device):
    """Additive key bias in log2 units for the masked kernels: a flat fp32 buffer holding
    [B, ceil(Lk/128)*128] rows followed by the per-tile flags (see ``_with_tile_flags``). ``mask``:
    None (only the padding beyond Lk is blanked), boolean (True = visible) or additive (natural-log
    units; -inf allowed), of a shape accepted by ``mask_is_key_only``."""
    Lkb = (Lk + 127) // 128 * 128
    if mask is None:
        # constant per (B, Lk, device): built once (70 cross-attention calls per SDXL step share it)
        key = (B, Lk, str(device))
        kb = _PAD_BIAS.get(key)
        if kb is None:
            rows = torch.full((B, Lkb), _MASKED, dtype=torch.float32, device=device)
            rows[:, :Lk] = 0.0
            kb = _with_tile_flags(rows)
            _PAD_BIAS[key] = kb
        return kb
    rows = torch.full((B, Lkb), _MASKED, dtype=torch.float32, device=device)
    m = mask.reshape(mask.shape[0], Lk).to(device)
    if m.dtype == torch.bool:
        row = torch.where(m, 0.0, _MASKED).float()
    else:
        row = (m.float() * _LOG2E).clamp_min(_MASKED)
    rows[:, :Lk] = row.expand(B, Lk)
    return _with_tile_flags(rows)


def _token_stride(t):
    """Elements between consecutive tokens of a [B, L, H, Dh] view whose heads are packed (a column block
    of a wider [B * L, ld] matrix); raises for any other layout."""
    B, L, H, D = t.shape
    ld = t.stride(1)
    if t.stride(3) != 1 or t.stride(2) != D or ld < H * D or ld % 8 or (B > 1 and t.stride(0) != L * ld):
        raise ValueError(f"flash attention: unsupported output strides {t.stride()} for shape {tuple(t.shape)}")
    return ld


def fwd(q, k, v, scale=None, out=None, kbias=None):
    """Returns (out [B, Lq, H, Dh] bf16, lse [B, H, Lq] fp32). ``out``: optional destination of q's shape,
    contiguous (e.g. a buffer that peers can read) or a column block of a wider row-major matrix. ``kbias``: key bias from
    ``key_bias`` (required when there are fewer than 128 keys)."""
    lib = N.require()
    _bind(lib)
    B, Lq, H, D = q.shape
    Lk = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    ld = 0
    if out is None:
        out = torch.empty_like(q)
    elif out.shape != q.shape or out.dtype != q.dtype:
        raise ValueError("flash attention: out must have q's shape and dtype")
    elif not out.is_contiguous():
        ld = _token_stride(out)
    lse = torch.empty(B, H, Lq, dtype=torch.float32, device=q.device)
    if kbias is None and Lk < 128:
        kbias = key_bias(None, B, Lk, q.device)
    if ld:
        if kbias is not None:
            raise ValueError("flash attention: a strided output is not supported together with a key bias")
        N.check(lib.eri_flash_attn_fwd_ld(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                          lse.data_ptr(), B, H, Lq, Lk, D, scale, ld, N.stream_ptr()),
                "flash_attn_fwd_ld")
        return out, lse
    if kbias is not None:
        N.check(lib.eri_flash_attn_fwd_masked(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                              lse.data_ptr(), kbias.data_ptr(), B, H, Lq, Lk, D, scale,
                                              N.stream_ptr()), "flash_attn_fwd_masked")
        return out, lse
    if D == 128 and Lq >= 256 and Lk >= 128 and pair_forward_ok(q.device):
        code = _pair_call(lib, q, k, v, out, lse, scale)
        if code != -100:
            N.check(code, "flash_attn_fwd_pair")
            return out, lse
    N.check(lib.eri_flash_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                   lse.data_ptr(), B, H, Lq, Lk, D, scale, N.stream_ptr()),
            "flash_attn_fwd")
    return out, lse


def bwd(do, q, k, v, out, lse, scale=None, kbias=None):
    """Returns (dq, dk, dv). ``kbias``: the key bias the forward ran with."""
    lib = N.require()
    _bind(lib)
    B, Lq, H, D = q.shape
    Lk = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    Lp = (Lq + 127) // 128 * 128
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    lse2 = torch.empty(B, H, Lp, dtype=torch.float32, device=q.device)
    delta = torch.empty_like(lse2)
    if kbias is None and Lk < 128:
        kbias = key_bias(None, B, Lk, q.device)
    if not out.is_contiguous():
        if kbias is not None:
            raise ValueError("flash attention: a strided forward output is not supported together with a key bias")
        N.check(lib.eri_flash_attn_bwd_ld(do.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                          out.data_ptr(), lse.data_ptr(), lse2.data_ptr(),
                                          delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                          B, H, Lq, Lk, D, scale, _token_stride(out), N.stream_ptr()),
                "flash_attn_bwd_ld")
        return dq, dk, dv
    if kbias is not None:
        N.check(lib.eri_flash_attn_bwd_masked(do.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                              out.data_ptr(), lse.data_ptr(), lse2.data_ptr(),
                                              delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                              kbias.data_ptr(), B, H, Lq, Lk, D, scale, N.stream_ptr()),
                "flash_attn_bwd_masked")
        return dq, dk, dv
    N.check(lib.eri_flash_attn_bwd(do.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                   out.data_ptr(), lse.data_ptr(), lse2.data_ptr(),
                                   delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                   B, H, Lq, Lk, D, scale, N.stream_ptr()), "flash_attn_bwd")
    return dq, dk, dv


def check_error() -> int:
    lib = N.require()
    _bind(lib)
    e = lib.eri_fa_check_error()
    if not e and hasattr(lib, "eri_fa2_check_error"):
        e = lib.eri_fa2_check_error()
    if not e and hasattr(lib, "eri_fa_bwd_check_error"):
        e = lib.eri_fa_bwd_check_error()
    return e


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, out_buf=None, kbias=None):
        if out_buf is not None:
            ctx.mark_dirty(out_buf)          # an input that is written in place and returned
        if kbias is None and k.shape[1] < 128:
            kbias = key_bias(None, k.shape[0], k.shape[1], q.device)
        out, lse = fwd(q, k, v, scale, out_buf, kbias)
        ctx.save_for_backward(q, k, v, out, lse, kbias)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse, kbias = ctx.saved_tensors
        do = do.contiguous()
        if has_backward():
            dq, dk, dv = bwd(do, q, k, v, out, lse, ctx.scale, kbias)
            return dq, dk, dv, None, None, None
        if kbias is not None:
            raise RuntimeError("masked flash attention needs the native backward kernels")
        # Library recompute path, used only while the native backward is absent from the build.
        from . import reference as R
        with torch.enable_grad():
            qq, kk, vv = (t.detach().requires_grad_() for t in (q, k, v))
            o = R.attention(qq, kk, vv, ctx.scale)
        dq, dk, dv = torch.autograd.grad(o, (qq, kk, vv), do)
        return dq, dk, dv, None, None, None


def flash_attention(q, k, v, scale=None, out=None, mask=None):
    """``mask``: None or a key-only mask (see ``mask_is_key_only``); the bias row is built here."""
    kbias = None if mask is None else key_bias(mask, q.shape[0], k.shape[1], q.device)
    return _FlashAttention.apply(q, k, v, scale, out, kbias)
