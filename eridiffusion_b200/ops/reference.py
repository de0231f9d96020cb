"""Plain PyTorch fp32 statements of every fused op.

These are the numerics oracle for the CUDA kernels (tests compare kernel output against these
functions evaluated in fp32) and the execution path on CPU tensors. They are differentiable
through ordinary autograd.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _f32(t):
    return None if t is None else t.float()


def norm_modulate(x, scale=None, shift=None, weight=None, bias=None, eps=1e-6, rms=False):
    """``(xhat * weight + bias) * (1 + scale[:, None]) + shift[:, None]`` over the last dim.

    x: [B, L, D]; scale/shift: [B, D]; weight/bias: [D]. ``rms`` selects RMSNorm instead of
    LayerNorm. Matches the reference's norm + scale/shift sequence
    (crates/training/src/flux/runtime.rs:893-922).
    """
    xf = x.float()
    if rms:
        xh = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    else:
        mu = xf.mean(-1, keepdim=True)
        var = (xf - mu).pow(2).mean(-1, keepdim=True)
        xh = (xf - mu) * torch.rsqrt(var + eps)
    if weight is not None:
        xh = xh * weight.float()
    if bias is not None:
        xh = xh + bias.float()
    if scale is not None:
        xh = xh * (1.0 + scale.float().unsqueeze(1))
    if shift is not None:
        xh = xh + shift.float().unsqueeze(1)
    return xh.to(x.dtype)


def rope_rotate(x, cos, sin):
    """Rotate interleaved pairs: x [..., L, H, Dh], cos/sin [L, Dh/2]."""
    xf = x.float()
    x0, x1 = xf[..., 0::2], xf[..., 1::2]
    c = cos.float()[:, None, :]
    s = sin.float()[:, None, :]
    o0 = c * x0 - s * x1
    o1 = s * x0 + c * x1
    return torch.stack((o0, o1), dim=-1).flatten(-2)


def qknorm_rope(qkv, q_scale, k_scale, cos, sin, num_heads, eps=1e-6):
    """qkv [B, L, 3*H*Dh] ("b l (k h d)") -> q, k, v each [B, L, H, Dh].

    q and k get per-head RMSNorm times a learned scale (when given) and rotary embedding of
    interleaved pairs (when cos/sin given; tables cover exactly these L tokens).
    """
    B, L, _ = qkv.shape
    t = qkv.view(B, L, 3, num_heads, -1)
    q, k, v = t[:, :, 0], t[:, :, 1], t[:, :, 2]

    def nrm(a, s):
        if s is None:
            return a.float()
        af = a.float()
        return af * torch.rsqrt(af.pow(2).mean(-1, keepdim=True) + eps) * s.float()

    qf, kf = nrm(q, q_scale), nrm(k, k_scale)
    if cos is not None:
        qf, kf = rope_rotate(qf, cos, sin), rope_rotate(kf, cos, sin)
    return qf.to(qkv.dtype), kf.to(qkv.dtype), v.contiguous()


def gate_residual(x, y, gate=None):
    """x + gate[:, None] * y  (x optional; gate [B, D] optional)."""
    out = y.float()
    if gate is not None:
        out = out * gate.float().unsqueeze(1)
    if x is not None:
        out = out + x.float()
    return out.to(y.dtype)


def gelu_tanh(x):
    return F.gelu(x.float(), approximate="tanh").to(x.dtype)


def silu(x):
    return F.silu(x.float()).to(x.dtype)


def glu(h, mode="gelu", act_first=True):
    """Gated linear unit over the last dim split in halves (GEGLU / SwiGLU)."""
    a, g = h.float().chunk(2, dim=-1)
    if not act_first:
        a, g = g, a
    a = F.gelu(a, approximate="tanh") if mode == "gelu" else F.silu(a)
    return (a * g).to(h.dtype)


def attention(q, k, v, scale=None, mask=None):
    """Non-causal attention on token-major tensors [B, L, H, Dh] -> [B, L, H, Dh].

    ``mask``: optional additive or boolean mask broadcastable to [B, H, Lq, Lk].
    """
    qh, kh, vh = (t.transpose(1, 2) for t in (q, k, v))
    if q.is_cuda and torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        # The cuDNN attention backward of this torch build rejects the graph for these strided
        # layouts ("mha_graph.execute ... is_good()"), so training uses the flash / efficient
        # library kernels; cuDNN stays available for no-grad calls.
        from torch.nn.attention import SDPBackend, sdpa_kernel
        with sdpa_kernel([SDPBackend.FLASH_ATTENTION, SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH]):
            o = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask, scale=scale)
    else:
        o = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask, scale=scale)
    return o.transpose(1, 2).contiguous()


def attention_fp32(q, k, v, scale=None, mask=None):
    """Explicit softmax(QK^T)V in fp32 (test oracle)."""
    B, L, H, D = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    s = torch.einsum("blhd,bmhd->bhlm", q.float(), k.float()) * scale
    if mask is not None:
        s = s + (mask.float() if mask.dtype != torch.bool else
                 torch.zeros_like(s).masked_fill(~mask, float("-inf")))
    p = s.softmax(-1)
    return torch.einsum("bhlm,bmhd->blhd", p, v.float())


def attention_chunked(q, k, v, scale=None, q_chunk=1024, kv_chunk=1024):
    """Blockwise attention with an online softmax: queries in chunks of ``q_chunk``, keys / values
    in chunks of ``kv_chunk``, a running row maximum ``m``, row sum ``l`` and accumulator that is
    rescaled when the maximum moves. Peak memory is one [B, H, q_chunk, kv_chunk] score block
    instead of [B, H, Lq, Lk]. This is the reference's single-GPU long-sequence mechanism
    (``sdpa_chunked_bf16``, crates/training/src/sdxl/runtime.rs:2814-3025; running ``(m, l, acc)``
    at :2958-2997) and the recurrence the tcgen05 flash kernels implement; here it serves the
    eager path when the score matrix would not fit, and as an oracle for the kernels' recurrence.
    Differentiable through autograd. Token-major [B, L, H, Dh] in and out."""
    B, Lq, H, D = q.shape
    Lk = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qh, kh, vh = (t.transpose(1, 2).float() for t in (q, k, v))          # [B, H, L, D]
    outs = []
    for q0 in range(0, Lq, q_chunk):
        qc = qh[:, :, q0:q0 + q_chunk] * scale
        m = torch.full(qc.shape[:-1], float("-inf"), device=q.device)
        l = torch.zeros_like(m)
        acc = torch.zeros(*qc.shape[:-1], vh.shape[-1], device=q.device)
        for k0 in range(0, Lk, kv_chunk):
            s = qc @ kh[:, :, k0:k0 + kv_chunk].transpose(-1, -2)
            m_new = torch.maximum(m, s.amax(-1))
            alpha = torch.exp(m - m_new)                                  # exp(-inf) = 0 on the first chunk
            p = torch.exp(s - m_new.unsqueeze(-1))
            l = l * alpha + p.sum(-1)
            acc = acc * alpha.unsqueeze(-1) + p @ vh[:, :, k0:k0 + kv_chunk]
            m = m_new
        outs.append(acc / l.unsqueeze(-1))
    return torch.cat(outs, dim=2).transpose(1, 2).to(q.dtype).contiguous()


def linear(x, w, bias=None, lora=None, act=None, residual=None, gate=None):
    """y = act(x W^T + bias + s * (x A^T) B^T); then residual + gate[:, None] * y.

    lora = (A [r, K], B [N, r], s).
    """
    y = F.linear(x, w, bias)
    if lora is not None:
        A, Bm, s = lora
        y = y + F.linear(F.linear(x, A), Bm) * s
    if act == "gelu":
        y = F.gelu(y, approximate="tanh")
    elif act == "silu":
        y = F.silu(y)
    if gate is not None:
        y = y * gate.unsqueeze(1)
    if residual is not None:
        y = residual + y
    return y


def patchify(x, p=2):
    """[B, C, H, W] -> [B, (H/p)(W/p), C*p*p]  ("b c (h ph) (w pw) -> b (h w) (c ph pw)")."""
    B, C, H, W = x.shape
    x = x.view(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5)
    return x.reshape(B, (H // p) * (W // p), C * p * p)


def unpatchify(tok, C, H, W, p=2):
    B = tok.shape[0]
    x = tok.view(B, H // p, W // p, C, p, p).permute(0, 3, 1, 4, 2, 5)
    return x.reshape(B, C, H, W)


def noise_mix(x0, eps, coef, p=2):
    """x_t = a*x0 + s*eps, target = ca*eps + cb*x0 (coef [4, B]); returns patchified tensors."""
    a, s, ca, cb = (coef[i].float().view(-1, 1, 1, 1) for i in range(4))
    xt = a * x0.float() + s * eps.float()
    tg = ca * eps.float() + cb * x0.float()
    return patchify(xt.to(x0.dtype), p), patchify(tg.to(x0.dtype), p)


def mse(pred, target, weight=None):
    d = (pred.float() - target.float()).pow(2)
    if weight is not None:
        d = d * weight.float().view(-1, *([1] * (d.dim() - 1)))
    return d.mean()


def group_norm_silu(x, weight, bias=None, groups=32, eps=1e-5, silu=True):
    """x [N, HW, C] channels-last rows -> GroupNorm over (HW, C/groups) (+ SiLU), fp32 math."""
    Nn, HW, C = x.shape
    xf = _f32(x).transpose(1, 2)                                   # [N, C, HW]
    y = torch.nn.functional.group_norm(xf, groups, _f32(weight), None if bias is None else _f32(bias), eps)
    if silu:
        y = torch.nn.functional.silu(y)
    return y.transpose(1, 2).to(x.dtype)
