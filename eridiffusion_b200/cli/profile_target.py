"""Small single-kernel workloads for profiler captures (inputs larger than L2, a few hundred MB on
the device, a handful of launches), one per hot kernel:

    python -m eridiffusion_b200.cli.profile_target gemm|gemm_lora|rank_stream|attn_fwd|attn_bwd|norm|qknorm|adamw|gemv|
        elementwise|groupnorm|token_route|dequant|attn_masked|small_linear_bwd|slot_reduce|gemm_small_m|gemm_group

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
    elif what == "attn_masked":
        # joint sequence with a text-padding mask (keys 300..511 of the text part hidden) and the SDXL
        # cross-attention shape (77 keys): the MASK variants of the forward and backward kernels
        from ..ops import functional as Fn
        B, L, H, D = 1, 4608, 24, 128
        q, k, v = (r(B, L, H, D).requires_grad_() for _ in range(3))
        vis = torch.ones(B, 1, 1, L, dtype=torch.bool, device=dev)
        vis[..., 300:512] = False
        for _ in range(iters):
            o = Fn.attention(q, k, v, mask=vis)
            o.backward(torch.ones_like(o))
        q2, k2, v2 = r(2, 4096, 10, 64).requires_grad_(), r(2, 77, 10, 64).requires_grad_(), r(2, 77, 10, 64).requires_grad_()
        for _ in range(iters):
            o = Fn.attention(q2, k2, v2)
            o.backward(torch.ones_like(o))
        assert FA.check_error() == 0
    elif what == "small_linear_bwd":
        # modulation linear [18432 x 3072] on one conditioning vector: dW (bound by writing 113 MB) and dx
        # (bound by reading it); three weights so that every launch goes to DRAM
        ws = [r(18432, 3072) for _ in range(3)]
        dy, x = r(1, 18432), r(1, 3072)
        for _ in range(iters):
            for w in ws:
                F.small_dgrad(dy, w)
                F.small_wgrad(dy, x)
    elif what == "slot_reduce":
        # owner-side sum of the 8 ranks' slots of a [1536 x 3072] weight-gradient slab (ZeRO-3 fused reduce-scatter)
        lib = F.N.require()
        world, n = 8, 1536 * 3072
        slots = [r(world * n) for _ in range(3)]
        out = torch.empty(n, device=dev, dtype=torch.bfloat16)
        for _ in range(iters):
            for s_ in slots:
                F.N.check(lib.eri_slot_reduce(s_.data_ptr(), out.data_ptr(), world, n, 1.0 / world, 0, F.N.stream_ptr()),
                          "slot_reduce")
    elif what == "gemm_small_m":
        # text-stream GEMMs (512 tokens) on the one-CTA kernel's 128-column tiles
        a1, a2 = r(512, 3072), r(512, 12288)
        b1, b2 = r(3072, 3072), r(3072, 12288)
        for _ in range(iters):
            F.gemm_native(a1, b1)
            F.gemm_native(a2, b2)
        assert F.gemm_error_check() == 0
    elif what == "gemm_group":
        # image (4096 tokens) and text (512 tokens) projection of a dual-stream block, 3072 -> 3072 with
        # rank-16 adapters: one grouped launch, then the two separate launches (pair kernel for the
        # image stream, one-CTA kernel for the text stream)
        kws = []
        for M in (4096, 512):
            x, w, hh, lb = r(M, 3072), r(3072, 3072), r(M, 16), r(3072, 16)
            kws.append(dict(a=x, b=w, bias=r(3072), lora_h=hh, lora_b=lb, residual=r(M, 3072), gate=r(1, 3072),
                            rows_per_batch=M))
        for _ in range(iters):
            F.gemm_native_pair(kws[0], kws[1])
        for _ in range(iters):
            F.gemm_native(**kws[0])
            F.gemm_native(**kws[1])
        assert F.gemm_error_check() == 0
    else:
        raise SystemExit(f"unknown target {what}")
    torch.cuda.synchronize()
    print("ok", what)


if __name__ == "__main__":
    main()
