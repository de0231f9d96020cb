"""Block-level fusions: the FLUX single-stream block as one autograd node.

The block computes ``x + gate * linear2(cat(attn(qkv), gelu(mlp)))`` where ``qkv`` and ``mlp`` are
column ranges of one projection ``linear1``. Written with separate ops this needs a split, an
activation pass and a concatenation in forward and zero-fill / copy / add passes for the slice
gradients in backward. Here the column-split epilogue of the GEMM writes the qkv columns and
``gelu(mlp)`` straight to where the next op reads them (the activation output lands inside the
concatenated buffer), and backward produces the gradient of the wide projection output in place:
the attention-gradient columns come from the QK-norm/RoPE backward with a row stride, the MLP
columns from linear2's input-gradient GEMM with the GELU-derivative epilogue.

Reference block: single blocks of src/models/flux_model_complete.rs:830-956 (linear1
[3D+4D, D], linear2 [D, D+4D], QK-norm, 3-way modulation).
"""
from __future__ import annotations

import torch

from . import _native as N
from . import flash_attn as FA
from . import functional as F


# GELU of the MLP half in the first linear's epilogue (forward) / its derivative in the second linear's
# input-gradient epilogue (backward), or as row passes of their own. Measured with eight epilogue warps at
# [4608 x 12288 x 3072]: storing activation + pre-activation from the epilogue 296 us against 244 + 43 us, the
# derivative in the epilogue 280 us against 250 + 55 us: the forward pass stays separate, the backward is fused.
_ACT_FWD_IN_EPILOGUE = __import__("os").environ.get("ERI_B200_SS_ACT_EPILOGUE", "0") == "1"
_ACT_BWD_IN_EPILOGUE = __import__("os").environ.get("ERI_B200_SS_ACT_BWD_EPILOGUE", "1") == "1"


class _SingleStream(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xm, x, gate, w1, b1, w2, b2, a1, bb1, s1, a2, bb2, s2, qs, ks, cos, sin, heads):
        B, L, D = xm.shape
        M = B * L
        Fm = w1.shape[0] - 3 * D
        Dh = D // heads
        dev, dt = xm.device, xm.dtype
        lib = N.require()
        xm2 = xm.contiguous().view(M, D)
        x2 = x.contiguous().view(M, D)
        gate_v, _ = F._mod_view(gate, D)
        qkv = torch.empty(M, 3 * D, dtype=dt, device=dev)
        cat = torch.empty(M, D + Fm, dtype=dt, device=dev)
        pre = torch.empty(M, Fm, dtype=dt, device=dev)
        # each rank-r product is the launch right before the GEMM that consumes it, so that GEMM can
        # start while it still runs (programmatic dependent launch)
        h1 = F.skinny_gemm(xm2, a1, alpha=s1) if a1 is not None else None
        if _ACT_FWD_IN_EPILOGUE:
            F.gemm_native(xm2, w1, bias=b1, lora_h=h1, lora_b=bb1, out=qkv, n_split=3 * D,
                          out2=cat[:, D:], act="gelu", pre_out=pre, pdl=F._pdl_ok())
        else:
            # the MLP half's pre-activation goes straight to its buffer and GELU is a pass of its own into
            # the second linear's input: storing both from the epilogue costs the GEMM more than that pass
            F.gemm_native(xm2, w1, bias=b1, lora_h=h1, lora_b=bb1, out=qkv, n_split=3 * D, out2=pre,
                          pdl=F._pdl_ok())
            mlp_in = cat[:, D:]
            N.check(lib.eri_act_fwd_rows(pre.data_ptr(), pre.stride(0), mlp_in.data_ptr(), cat.stride(0), M, Fm, 0,
                                         N.stream_ptr()), "act_fwd_rows")
        q = torch.empty(B, L, heads, Dh, dtype=dt, device=dev)
        k, v = torch.empty_like(q), torch.empty_like(q)
        N.check(lib.eri_qknorm_rope_fwd(qkv.data_ptr(), N.ptr(qs), N.ptr(ks), N.ptr(cos), N.ptr(sin),
                                        q.data_ptr(), k.data_ptr(), v.data_ptr(), B, L, heads, Dh, L, 0,
                                        1e-6, 3 * D, D, N.stream_ptr()), "qknorm_rope_fwd")
        # the attention writes its output straight into the left column block of the second linear's input
        o, lse = FA.fwd(q, k, v, out=cat.view(B, L, D + Fm)[:, :, :D].unflatten(-1, (heads, Dh)))
        h2 = F.skinny_gemm(cat, a2, alpha=s2) if a2 is not None else None
        y = F.gemm_native(cat, w2, bias=b2, lora_h=h2, lora_b=bb2, residual=x2,
                          gate=gate_v, rows_per_batch=L, pdl=F._pdl_ok())
        ctx.save_for_backward(xm2, qkv, pre, cat, q, k, v, lse, h1, h2, gate_v, w1, w2, a1, bb1, a2,
                              bb2, qs, ks, cos, sin)
        ctx.meta = (B, L, D, Fm, heads, Dh, s1, s2)
        return y.view(B, L, D)

    @staticmethod
    def backward(ctx, dy):
        (xm2, qkv, pre, cat, q, k, v, lse, h1, h2, gate_v, w1, w2, a1, bb1, a2, bb2, qs, ks, cos,
         sin) = ctx.saved_tensors
        B, L, D, Fm, heads, Dh, s1, s2 = ctx.meta
        o = cat.view(B, L, D + Fm)[:, :, :D].unflatten(-1, (heads, Dh))    # the forward's attention output
        M = B * L
        dev, dt = dy.device, dy.dtype
        lib = N.require()
        need = ctx.needs_input_grad
        dy2 = dy.contiguous().view(M, D)
        g = torch.empty_like(dy2)
        N.check(lib.eri_gate_residual(None, dy2.data_ptr(), gate_v.data_ptr(), g.data_ptr(), M, D, L,
                                      gate_v.stride(0), N.stream_ptr()), "gate_bwd")
        lt = F._lora_transposed
        bb2_t, a2_t = (lt(bb2), lt(a2)) if a2 is not None else (None, None)
        bb1_t, a1_t = (lt(bb1), lt(a1)) if a1 is not None else (None, None)
        d_attn = torch.empty(M, D, dtype=dt, device=dev)
        d_h = torch.empty(M, 3 * D + Fm, dtype=dt, device=dev)
        ts2 = F.skinny_gemm(g, bb2_t, alpha=s2) if a2 is not None else None
        if _ACT_BWD_IN_EPILOGUE:
            F.gemm_native(g, w2, b_mn=True, lora_h=ts2, lora_b=a2_t,
                          out=d_attn, n_split=D, out2=d_h[:, 3 * D:], act="gelu_bwd", pre_in=pre, pdl=F._pdl_ok())
        else:
            # the GELU derivative as a pass of its own over the MLP half of d_h, in place: the epilogue's
            # row-strided reads of the pre-activation cost the GEMM more than this pass does
            F.gemm_native(g, w2, b_mn=True, lora_h=ts2, lora_b=a2_t,
                          out=d_attn, n_split=D, out2=d_h[:, 3 * D:], pdl=F._pdl_ok())
            mlp_g = d_h[:, 3 * D:]
            N.check(lib.eri_act_bwd_rows(mlp_g.data_ptr(), d_h.stride(0), pre.data_ptr(), pre.stride(0),
                                         mlp_g.data_ptr(), d_h.stride(0), M, Fm, 0, N.stream_ptr()), "act_bwd_rows")
        da2 = F.lora_wgrad(cat, ts2, transpose_out=True) if (a2 is not None and need[10]) else None
        db2 = F.lora_wgrad(g, h2) if (a2 is not None and need[11]) else None
        dq, dk, dv = FA.bwd(d_attn.view(B, L, heads, Dh), q, k, v, o, lse)
        f32 = dict(dtype=torch.float32, device=dev)
        dqs = torch.zeros(Dh, **f32) if (qs is not None and need[13]) else None
        dks = torch.zeros(Dh, **f32) if (ks is not None and need[14]) else None
        N.check(lib.eri_qknorm_rope_bwd(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), qkv.data_ptr(),
                                        N.ptr(qs), N.ptr(ks), N.ptr(cos), N.ptr(sin), d_h.data_ptr(),
                                        N.ptr(dqs), N.ptr(dks), B, L, heads, Dh, L, 0, 1e-6, 3 * D, D,
                                        3 * D + Fm, N.stream_ptr()), "qknorm_rope_bwd")
        ts1 = F.skinny_gemm(d_h, bb1_t, alpha=s1) if a1 is not None else None
        dxm = None
        if need[0]:
            dxm = F.gemm_native(d_h, w1, b_mn=True, lora_h=ts1, lora_b=a1_t, pdl=F._pdl_ok()).view(B, L, D)
        da1 = F.lora_wgrad(xm2, ts1, transpose_out=True) if (a1 is not None and need[7]) else None
        db1 = F.lora_wgrad(d_h, h1) if (a1 is not None and need[8]) else None
        dw1 = F.wgrad(d_h, xm2) if need[3] else None
        dw2 = F.wgrad(g, cat) if need[5] else None
        dgate = None
        if need[2]:
            raise NotImplementedError("trainable modulation uses the unfused single-stream path")
        cv = lambda t: None if t is None else t.to(dt)
        return (dxm, dy if need[1] else None, dgate, dw1, d_h.sum(0) if need[4] else None, dw2,
                g.sum(0) if need[6] else None, da1, db1, None, da2, db2, None, cv(dqs), cv(dks), None,
                None, None)


def single_stream_supported(xm, gate, lin1, lin2, heads) -> bool:
    if not (xm.is_cuda and xm.dtype == torch.bfloat16 and F.get_backend() == "fused"):
        return False
    if F._GEMM_NATIVE != "native" or F._ATTN_NATIVE != "native" or not FA.has_backward():
        return False
    B, L, D = xm.shape
    if B * L < 128 or L < 128 or D // heads not in (64, 128) or D % 256 or gate.requires_grad:
        return False
    for lin in (lin1, lin2):
        ad = getattr(lin, "adapter", None)
        if type(lin).__name__ != "Linear":
            return False
        if ad is not None and not (getattr(ad, "kind", "") == "lora" and ad.rank in (16, 32, 64)
                                   and not (ad.dropout > 0 and ad.training)):
            return False
    return True


def single_stream(xm, x, gate, lin1, lin2, q_scale, k_scale, cos, sin, heads):
    """xm: modulated/normalised input [B, L, D]; x: residual stream; gate [B, D]."""
    def lora(lin):
        ad = getattr(lin, "adapter", None)
        return (None, None, 1.0) if ad is None else (ad.lora_A, ad.lora_B, float(ad.scale))
    a1, bb1, s1 = lora(lin1)
    a2, bb2, s2 = lora(lin2)
    cosf = None if cos is None else cos.float().contiguous()
    sinf = None if sin is None else sin.float().contiguous()
    return _SingleStream.apply(xm, x, gate, lin1.weight, lin1.bias, lin2.weight, lin2.bias, a1, bb1, s1,
                               a2, bb2, s2, q_scale, k_scale, cosf, sinf, heads)
