"""Small single-kernel workloads for profiler captures (inputs larger than L2, a few hundred MB on
the device, a handful of launches), one per hot kernel:

    python -m eridiffusion_b200.cli.profile_target gemm|gemm_lora|rank_stream|attn_fwd|attn_bwd|norm|qknorm|adamw|gemv|
        elementwise|groupnorm|token_route|dequant

Meant to be run as ``ncu --set full --clock-control none -k regex:<kernel> -s 2 -c 1 ... python -m
eridiffusion_b200.cli.profile_target <what>`` after the same command line exited 0 without ncu.
"""
from __future__ import annotations

import sys

import torch

from ..ops import flash_attn as FA
from ..ops import functional as F


def main():
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    iters = 4
    dev = "cuda"
    r = lambda *s: torch.randn(*s, device=dev).bfloat16()
    if what in ("gemm", "gemm_lora"):
        M, N, K = 4096, 9216, 3072
        a, b = r(M, K), r(N, K)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        h, lb = r(M, 16), r(N, 16)
        for _ in range(iters):
            F.gemm_native(a, b, out=out, lora_h=h if what == "gemm_lora" else None,
                          lora_b=lb if what == "gemm_lora" else None)
        assert F.gemm_error_check() == 0
    elif what == "rank_stream":
        # LoRA down-projection [M, K] x [16, K]^T; eight different activations so that every launch
        # reads from DRAM (226 MB in total, larger than L2)
        xs = [r(4608, 3072) for _ in range(8)]
        la = r(16, 3072)
        for x in xs:
            F.skinny_gemm(x, la, alpha=0.5)
        assert F.kernel_error_check() == {}
    elif what in ("attn_fwd", "attn_bwd"):
        B, L, H, D = 1, 4608, 24, 128
        q, k, v = r(B, L, H, D), r(B, L, H, D), r(B, L, H, D)
        for _ in range(iters):
            o, lse = FA.fwd(q, k, v)
        if what == "attn_bwd":
            do = torch.randn_like(o)
            for _ in range(iters):
                FA.bwd(do, q, k, v, o, lse)
        assert FA.check_error() == 0
    elif what == "norm":
        x, mod = r(8, 4608, 3072), r(8, 3 * 3072)
        sh, sc, _ = mod.split(3072, -1)
        x.requires_grad_()
        g = torch.randn_like(x)
        for _ in range(iters):
            y = F.norm_modulate(x, sc, sh)
            y.backward(g)
            x.grad = None
        assert F.kernel_error_check() == {}
    elif what == "qknorm":
        qkv = r(4, 4608, 9216)
        s = torch.ones(128, device=dev).bfloat16()
        cos, sin = torch.rand(4608, 64, device=dev), torch.rand(4608, 64, device=dev)
        for _ in range(iters):
            F.qknorm_rope_joint([(qkv, s, s)], cos, sin, 24)
    elif what == "adamw":
        from ..optim import AdamW8bit
        p = torch.nn.Parameter(r(112_000_000))
        opt = AdamW8bit([p])
        opt.arena.grad.normal_()
        ss = F.sumsq(opt.arena.grad)
        for _ in range(iters):
            opt.step(grad_sumsq=ss, max_grad_norm=1.0)
    elif what == "gemv":
        x, w, b = r(1, 3072), r(18432, 3072), r(18432)
        for _ in range(iters):
            F.small_linear(x, w, b, silu_in=True)
    elif what == "elementwise":
        # gate + residual, GELU forward / backward, GEGLU, weighted MSE, noise mix: 4 x 4608 x 3072
        # activations (113 MB each, larger than L2 together)
        x, y = r(4, 4608, 3072), r(4, 4608, 3072)
        gate = r(4, 3072)
        wide = r(4, 4608, 6144)
        lat = r(4, 16, 128, 128)
        coef = torch.tensor([[0.5] * 4, [0.5] * 4, [1.0] * 4, [-1.0] * 4], device=dev)   # rows a, s, ca, cb
        for _ in range(iters):
            F.gate_residual(x, y, gate)
            xg = x.detach().requires_grad_()
            F.gelu_tanh(xg).backward(y)
            F.glu(wide, "gelu")
            F.mse_loss(x, y)
            F.noise_mix(lat, coef, seed=1, patch=2)
    elif what == "groupnorm":
        x = r(2, 128, 128, 320).permute(0, 3, 1, 2)                # channels-last view of [2, 320, 128, 128]
        w, b = r(320), r(320)
        x.requires_grad_()
        for _ in range(iters):
            yv = F.group_norm_silu(x, w, b, 32)
            yv.backward(torch.ones_like(yv))
            x.grad = None
    elif what == "token_route":
        x = r(4, 4608, 3072)
        for _ in range(iters):
            sc = F.token_scores(x)
            idx = F.topk_indices(sc, 2304)
            F.gather_rows(x, idx)
    elif what == "dequant":
        from ..memory import dequantize, quantize
        w = r(12288, 3072)
        qs = [quantize(w, kind) for kind in ("int8", "int4", "nf4")]
        for _ in range(iters):
            for q in qs:
                dequantize(q)
    else:
        raise SystemExit(f"unknown target {what}")
    torch.cuda.synchronize()
    print("ok", what)


if __name__ == "__main__":
    main()
