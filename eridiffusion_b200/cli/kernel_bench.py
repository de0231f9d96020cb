"""Per-kernel timing against the library equivalents and the measured roofline.

    python -m eridiffusion_b200.cli.kernel_bench [--what gemm,skinny,attn,elementwise,optim,dequant,narrow,wgrad,small_m,gather_emul,epilogue] [--small]

Timing: CUDA events on the launching stream, >= 3 warm-up launches, L2 flushed between timed
launches by writing a 256 MB buffer, median of the timed launches. Roofline denominators come from
``MEASURED_PEAKS.json`` at the repository root when present (copy bandwidth and cuBLAS bf16
throughput measured on this pool), otherwise the documented fallback (6.65 TB/s, 1.59 PFLOP/s).
"""
from __future__ import annotations

import argparse
import json
import statistics
from pathlib import Path

import torch

from ..ops import functional as F
from ..ops import reference as R


def peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "of measured"
    return 6.65e12, 1.59e15, "of fallback"


_flush = None


def timeit(fn, iters=10, warm=3, flush=True):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(iters):
        if flush:
            _flush.zero_()
        # a device-side delay lets the host enqueue fn's launches before the start event fires, so
        # host launch overhead (tens of microseconds in Python) is not measured as kernel time
        torch.cuda._sleep(600_000)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e-3)
    return statistics.median(ts)


def bench_gemm(small):
    bw, fl, tag = peaks()
    shapes = [(4096, 9216, 3072), (4096, 3072, 3072), (4096, 12288, 3072), (4096, 3072, 12288),
              (512, 9216, 3072), (4608, 21504, 3072), (4608, 3072, 15360), (8192, 8192, 8192)]
    if small:
        shapes = [(1024, 2048, 1024), (4096, 3072, 3072)]
    print(f"{'M':>6} {'N':>6} {'K':>6} | {'ours us':>9} {'TF/s':>7} {'frac':>6} | {'cuBLAS us':>9} {'TF/s':>7} | lora16 us")
    for M, N, K in shapes:
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = torch.randn(N, K, device="cuda").bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        t_ours = timeit(lambda: F.gemm_native(a, b, out=out))
        t_lib = timeit(lambda: torch.matmul(a, b.t(), out=out))
        h = torch.randn(M, 16, device="cuda").bfloat16()
        lb = torch.randn(N, 16, device="cuda").bfloat16()
        la = torch.randn(16, K, device="cuda").bfloat16()
        t_lora = timeit(lambda: F.gemm_native(a, b, out=out, lora_h=F.gemm_native(a, la, alpha=0.5), lora_b=lb))
        fl_ = 2.0 * M * N * K
        bt = b.t().contiguous()
        t_mn = timeit(lambda: F.gemm_native(a, bt, out=out, b_mn=True))
        print(f"{M:6d} {N:6d} {K:6d} | {t_ours*1e6:9.1f} {fl_/t_ours/1e12:7.1f} {fl_/t_ours/fl:6.2f} | "
              f"{t_lib*1e6:9.1f} {fl_/t_lib/1e12:7.1f} | {t_lora*1e6:9.1f} | B[K,N]: {t_mn*1e6:9.1f}   ({tag})")
    assert F.gemm_error_check() == 0


def bench_small_m(small):
    """Text-stream GEMMs (512 tokens): few 256 x 256 pair tiles, so the tile width decides how many SMs
    work. Pair kernel (default route) against the one-CTA kernel at 128- and 64-column tiles and cuBLAS;
    second line: the same with B given as [K, N] (the dX product)."""
    bw, fl, tag = peaks()
    for M, N, K in ([(512, 3072, 3072), (512, 3072, 12288), (512, 3072, 9216), (512, 9216, 3072), (512, 12288, 3072)]
                    if not small else [(512, 1024, 1024)]):
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = torch.randn(N, K, device="cuda").bfloat16()
        bt = b.t().contiguous()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        fl_ = 2.0 * M * N * K
        for mn, bb in ((False, b), (True, bt)):
            ts = [timeit(lambda: F.gemm_native(a, bb, out=out, b_mn=mn, force_bn=f)) for f in (256, 128, 64)]
            t_auto = timeit(lambda: F.gemm_native(a, bb, out=out, b_mn=mn))
            t_lib = timeit(lambda: torch.matmul(a, b.t() if not mn else bt, out=out))
            print(f"{M}x{N}x{K} {'B[K,N]' if mn else 'B[N,K]'}: pair {ts[0]*1e6:6.1f} | one-CTA bn128 {ts[1]*1e6:6.1f} | bn64 {ts[2]*1e6:6.1f} | "
                  f"default route {t_auto*1e6:6.1f} us {fl_/t_auto/1e12:5.0f} TF/s | cuBLAS {t_lib*1e6:6.1f} us")
    assert F.gemm_error_check() == 0


def bench_gather_emul(small):
    """The ZeRO-3 gather-in-GEMM launch with its eight ranks' shards all on THIS GPU (peer pointers are
    local buffers): what the launch costs apart from NVLink - copy CTAs taking SMs, the extra pass of the
    gathered operand through HBM, counter waits - against the plain GEMM on an already gathered weight."""
    from ..parallel.gather_gemm import GatherPlan
    bw, fl, tag = peaks()
    W, M = 8, 4608 if not small else 512
    for n_out, k_in in ([(12288, 3072), (9216, 3072), (3072, 12288)] if not small else [(2048, 512)]):
        x = torch.randn(M, k_in, device="cuda").bfloat16()
        shards = [torch.randn(n_out // W, k_in, device="cuda").bfloat16() for _ in range(W)]
        full = torch.cat(shards, 0)
        out = torch.empty(M, n_out, device="cuda", dtype=torch.bfloat16)
        t_plain = timeit(lambda: F.gemm_native(x, full, out=out))
        row = []
        for n_copy in (8, 16, 32):
            landing = torch.empty(n_out, k_in, device="cuda", dtype=torch.bfloat16)
            plan = GatherPlan.rows(3, W, [s_.data_ptr() for s_ in shards], landing, n_copy=n_copy)
            stamps = torch.zeros(8, dtype=torch.int64, device="cuda")

            t = timeit(lambda: F.gemm_native(x, landing, out=out, gather=plan.launch_args()))
            # one more launch with the kernel's own phase record
            stamps.zero_()
            stamps[0] = -1
            F.gemm_native(x, landing, out=out, gather=dict(plan.launch_args(), stamps=stamps))
            torch.cuda.synchronize()
            s_ = stamps.tolist()
            row.append(f"{n_copy} copy CTAs {t*1e6:.1f} us (slabs landed at {(s_[1]-s_[0])/1e3:.0f} us, compute done at "
                       f"{(s_[2]-s_[0])/1e3:.0f} us, {s_[5]} producers waited, longest {s_[4]/1e3:.0f} us)")
        fl_ = 2.0 * M * n_out * k_in
        print(f"gather-in-GEMM, 8 emulated ranks on one GPU [{M}x{k_in}] x [{n_out}x{k_in}]^T: plain GEMM {t_plain*1e6:.1f} us "
              f"({fl_/t_plain/fl:.2f} {tag}) | " + " | ".join(row))
        # input gradient dX[M, k_in] = dY[M, n_out] W[n_out, k_in]: the gathered rows are the reduction dimension
        dy = torch.randn(M, n_out, device="cuda").bfloat16()
        dx = torch.empty(M, k_in, device="cuda", dtype=torch.bfloat16)
        t_plain = timeit(lambda: F.gemm_native(dy, full, out=dx, b_mn=True))
        row = []
        for n_copy in (16, 32):
            landing = torch.empty(n_out, k_in, device="cuda", dtype=torch.bfloat16)
            plan = GatherPlan.rows(3, W, [s_.data_ptr() for s_ in shards], landing, along_k=True, n_copy=n_copy)
            t = timeit(lambda: F.gemm_native(dy, landing, out=dx, b_mn=True, gather=plan.launch_args()))
            stamps = torch.zeros(8, dtype=torch.int64, device="cuda")
            stamps[0] = -1
            F.gemm_native(dy, landing, out=dx, b_mn=True, gather=dict(plan.launch_args(), stamps=stamps))
            torch.cuda.synchronize()
            s_ = stamps.tolist()
            row.append(f"{n_copy} copy CTAs {t*1e6:.1f} us (landed at {(s_[1]-s_[0])/1e3:.0f} us, compute done at "
                       f"{(s_[2]-s_[0])/1e3:.0f} us, longest wait {s_[4]/1e3:.0f} us)")
        print(f"   input gradient [{M}x{n_out}] x [{n_out}x{k_in}]: plain GEMM {t_plain*1e6:.1f} us | " + " | ".join(row))
    assert F.gemm_error_check() == 0


def bench_skinny(small):
    """LoRA down-projection shapes: [M, K] x [16, K]^T; bandwidth-bound on reading the activation."""
    bw, fl, tag = peaks()
    for M, K in ([(4608, 3072), (4608, 15360), (4608, 21504), (512, 3072)] if not small else [(1024, 2048)]):
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = torch.randn(16, K, device="cuda").bfloat16()
        t = timeit(lambda: F.skinny_gemm(a, b, alpha=0.5))
        t0 = timeit(lambda: F.gemm_native(a, b, alpha=0.5))
        t1 = timeit(lambda: torch.matmul(a, b.t()))
        nb = a.numel() * 2
        print(f"skinny [{M}x{K}]x[16x{K}]^T: split-K {t*1e6:.1f} us {nb/t/1e9:.0f} GB/s {nb/t/bw:.2f} {tag} | "
              f"128-row tiles only {t0*1e6:.1f} us | cuBLAS {t1*1e6:.1f} us")


def bench_wgrad(small):
    """Weight-gradient products: dW = dY^T X on the two-CTA kernel (both operands token-major) and the
    skinny token reductions of the LoRA gradients, against torch (cuBLAS)."""
    bw, fl, tag = peaks()
    T = 4608 if not small else 1024
    for Nn, K in ([(9216, 3072), (3072, 3072), (12288, 3072), (3072, 12288)] if not small else [(1024, 512)]):
        dy = torch.randn(T, Nn, device="cuda").bfloat16()
        x = torch.randn(T, K, device="cuda").bfloat16()
        g = torch.zeros(Nn, K, device="cuda", dtype=torch.bfloat16)
        t = timeit(lambda: F.wgrad(dy, x, accum=g))
        t_lib = timeit(lambda: g.addmm_(dy.t(), x))
        fl_ = 2.0 * T * Nn * K
        print(f"wgrad dW[{Nn}x{K}] += dY[{T}x{Nn}]^T X: ours {t*1e6:.1f} us {fl_/t/1e12:.0f} TF/s {fl_/t/fl:.2f} {tag} | "
              f"cuBLAS addmm {t_lib*1e6:.1f} us {fl_/t_lib/1e12:.0f} TF/s")
    lib = F.N.require()
    for Mg in ([3072, 9216, 12288, 15360, 21504] if not small else [2048]):
        a = torch.randn(T, Mg, device="cuda").bfloat16()
        b = torch.randn(T, 16, device="cuda").bfloat16()
        g = torch.zeros(Mg, 16, device="cuda", dtype=torch.bfloat16)
        gt = torch.zeros(16, Mg, device="cuda", dtype=torch.bfloat16)
        nb = a.numel() * 2
        row = []
        for target in (0, 74, 296):
            lib.eri_gemm_tokred_set_target(target)
            t = timeit(lambda: F.lora_wgrad(a, b, out=g, accumulate=True))
            t2 = timeit(lambda: F.lora_wgrad(a, b, out=gt, transpose_out=True, accumulate=True))
            row.append(f"target {target}: {t*1e6:.1f} / {t2*1e6:.1f} us ({nb/t/bw:.2f})")
        lib.eri_gemm_tokred_set_target(0)
        t_lib = timeit(lambda: g.addmm_(a.t(), b))
        t_lib2 = timeit(lambda: gt.addmm_(b.t(), a))
        print(f"token reduction [{T}x{Mg}]^T x [{T}x16] (plain / transposed out): " + "; ".join(row) +
              f" | cuBLAS addmm {t_lib*1e6:.1f} / {t_lib2*1e6:.1f} us   ({tag})")
    assert F.kernel_error_check() == {}


def bench_elementwise(small):
    bw, fl, tag = peaks()
    B, L, D = 1, 4608, 3072
    lib = F.N.require()
    # both row kernels (rows resident in shared memory / in registers) at the step's size and at eight times it
    for Bn in (1, 8):
        xb = torch.randn(Bn, L, D, device="cuda").bfloat16()
        modb = torch.randn(Bn, 2 * D, device="cuda").bfloat16()
        shb, scb = modb.split(D, -1)
        xg = xb.clone().requires_grad_()
        for variant, name in ((1, "shared-memory rows"), (0, "register rows")):
            if not hasattr(lib, "eri_norm_set_smem_variant"):
                continue
            prev = lib.eri_norm_set_smem_variant(variant)
            t = timeit(lambda: F.norm_modulate(xb, scb, shb))
            nb = 2 * xb.numel() * 2
            yg = F.norm_modulate(xg, scb, shb)
            go = torch.randn_like(yg)
            tb = timeit(lambda: torch.autograd.grad(yg, xg, go, retain_graph=True))
            nbb = 3 * xb.numel() * 2
            print(f"norm_modulate [{Bn * L}x{D}] {name}: fwd {t*1e6:.1f} us {nb/t/bw:.2f}, "
                  f"bwd (dx only) {tb*1e6:.1f} us {nbb/tb/bw:.2f} {tag}")
            lib.eri_norm_set_smem_variant(prev)
    x = torch.randn(B, L, D, device="cuda").bfloat16()
    mod = torch.randn(B, 3 * D, device="cuda").bfloat16()
    sh, sc, g = mod.split(D, -1)
    F.set_backend("eager")
    t2 = timeit(lambda: R.norm_modulate(x, sc, sh))
    F.set_backend("fused")
    print(f"   eager composition: {t2*1e6:.1f} us")
    y = torch.randn_like(x)
    t = timeit(lambda: F.gate_residual(x, y, g))
    print(f"gate_residual [{L}x{D}]: {t*1e6:.1f} us  {3*x.numel()*2/t/1e9:.0f} GB/s  {3*x.numel()*2/t/bw:.2f} {tag}")
    qkv = torch.randn(B, L, 3 * D, device="cuda").bfloat16()
    qs = torch.ones(128, device="cuda").bfloat16()
    cos = torch.rand(L, 64, device="cuda"); sin = torch.rand(L, 64, device="cuda")
    t = timeit(lambda: F.qknorm_rope_joint([(qkv, qs, qs)], cos, sin, 24))
    print(f"qknorm_rope [{L}x{3*D}]: {t*1e6:.1f} us  {2*qkv.numel()*2/t/1e9:.0f} GB/s  {2*qkv.numel()*2/t/bw:.2f} {tag}")
    h = torch.randn(L, 12288, device="cuda").bfloat16()
    t = timeit(lambda: F.gelu_tanh(h))
    print(f"gelu [{L}x12288]: {t*1e6:.1f} us  {2*h.numel()*2/t/1e9:.0f} GB/s  {2*h.numel()*2/t/bw:.2f} {tag}")


def bench_optim(small):
    from ..optim import AdamW8bit
    bw, fl, tag = peaks()
    n = 56_000_000 if not small else 4_000_000
    p = torch.nn.Parameter(torch.randn(n, device="cuda").bfloat16())
    opt = AdamW8bit([p])
    opt.arena.grad.normal_()
    ss = F.sumsq(opt.arena.grad)
    nb = opt.arena.numel * (2 + 2 + 2 + 1 + 1 + 1 + 1)
    lib = F.N.require()
    for variant, name in ((1, "packed pairs"), (0, "element-wise")):
        if not hasattr(lib, "eri_adamw8bit_set_pair_variant"):
            continue
        prev = lib.eri_adamw8bit_set_pair_variant(variant)
        for sr in (True, False):
            opt.stochastic_rounding = sr
            t = timeit(lambda: opt.step(grad_sumsq=ss, max_grad_norm=1.0))
            print(f"adamw8bit [{n/1e6:.0f}M params] {name}, stochastic rounding {'on' if sr else 'off'}: "
                  f"{t*1e6:.1f} us  {nb/t/1e9:.0f} GB/s  {nb/t/bw:.2f} {tag}")
        lib.eri_adamw8bit_set_pair_variant(prev)
    opt.stochastic_rounding = True
    t = timeit(lambda: F.sumsq(opt.arena.grad, ss))
    print(f"sumsq: {t*1e6:.1f} us  {opt.arena.numel*2/t/1e9:.0f} GB/s")


def bench_dequant(small):
    """Quantised base weight -> bf16 GEMM operand (codes read + bf16 written)."""
    from ..memory import dequantize, quantize
    bw, fl, tag = peaks()
    rows, cols = (12288, 3072) if not small else (2048, 1024)
    w = torch.randn(rows, cols, device="cuda").bfloat16()
    for kind, code_bytes in (("int8", 1.0), ("int4", 0.5), ("nf4", 0.5)):
        q = quantize(w, kind)
        out = torch.empty_like(w)
        t = timeit(lambda: dequantize(q, out=out))
        nb = rows * cols * (code_bytes + 2)
        print(f"dequant {kind} [{rows}x{cols}]: {t*1e6:.1f} us  {nb/t/1e9:.0f} GB/s  {nb/t/bw:.2f} {tag}")


def bench_narrow(small):
    """Slice gather and slice-gradient accumulation against the PyTorch statements
    (``narrow().contiguous()``, ``narrow().add_()``). Bytes: slice read + slice written for the copy;
    slice read twice + written once for the accumulation."""
    from ..ops.narrow import narrow_backward_add, narrow_copy_raw
    bw, fl, tag = peaks()
    B, L, D = (4, 4608, 21504) if not small else (2, 1024, 4096)
    x = torch.randn(B, L, D, device="cuda").bfloat16()
    for dim, start, length in ((2, 3 * 3072, 4 * 3072), (1, 512, L - 512)):
        nb = x.numel() // x.shape[dim] * length * 2
        t = timeit(lambda: narrow_copy_raw(x, dim, start, length))
        t_lib = timeit(lambda: x.narrow(dim, start, length).contiguous())
        print(f"narrow copy [{B}x{L}x{D}] dim {dim} len {length}: {t*1e6:.1f} us {2*nb/t/1e9:.0f} GB/s "
              f"{2*nb/t/bw:.2f} {tag}   torch {t_lib*1e6:.1f} us")
        g = torch.randn_like(x.narrow(dim, start, length).contiguous())
        gi = torch.zeros_like(x)
        t = timeit(lambda: narrow_backward_add(g, gi, dim, start))
        t_lib = timeit(lambda: gi.narrow(dim, start, length).add_(g))
        print(f"narrow grad add same slice: {t*1e6:.1f} us {3*nb/t/1e9:.0f} GB/s {3*nb/t/bw:.2f} {tag}   "
              f"torch {t_lib*1e6:.1f} us")


def bench_epilogue(small):
    """What the GEMM epilogue's extra operands cost at the training step's shapes, against the same work as a
    separate bandwidth-bound pass: residual + gate, GELU with a stored pre-activation, the GELU derivative read
    from a stored pre-activation."""
    r = lambda *s: torch.randn(*s, device="cuda").bfloat16()
    shapes = [("single-stream second linear", 4608, 3072, 15360), ("attention out-projection", 4096, 3072, 3072),
              ("MLP down-projection", 4096, 3072, 12288), ("MLP up-projection / its input gradient", 4096, 12288, 3072)]
    for tag, M, Nn, K in (shapes[1:2] if small else shapes):
        a, w, wt = r(M, K), r(Nn, K), r(K, Nn)
        h, lb = r(M, 16), r(Nn, 16)
        res, gate, bias = r(M, Nn), r(1, Nn), r(Nn)
        pre = torch.empty(M, Nn, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, Nn, device="cuda", dtype=torch.bfloat16)
        y = r(1, M, Nn)
        t = {
            "plain (bias + rank-16 K step)": timeit(lambda: F.gemm_native(a, w, out=out, bias=bias, lora_h=h, lora_b=lb)),
            "+ residual + gate": timeit(lambda: F.gemm_native(a, w, out=out, bias=bias, lora_h=h, lora_b=lb, residual=res,
                                                              gate=gate, rows_per_batch=M)),
            "+ GELU + stored pre-activation": timeit(lambda: F.gemm_native(a, w, out=out, bias=bias, lora_h=h, lora_b=lb,
                                                                           act="gelu", pre_out=pre)),
            "input gradient, plain": timeit(lambda: F.gemm_native(a, wt, b_mn=True, out=out, lora_h=h, lora_b=lb)),
            "input gradient + GELU derivative": timeit(lambda: F.gemm_native(a, wt, b_mn=True, out=out, lora_h=h, lora_b=lb,
                                                                             act="gelu_bwd", pre_in=pre)),
            "gate + residual as a pass": timeit(lambda: F.gate_residual(res.view(1, M, Nn), y, gate)),
            "GELU as a pass": timeit(lambda: F.gelu_tanh(y)),
        }
        print(f"epilogue extras, {tag} [{M} x {Nn} x {K}]: " + "; ".join(f"{k} {v*1e6:.1f} us" for k, v in t.items()))
    assert F.gemm_error_check() == 0


def bench_attn(small):
    bw, fl, tag = peaks()
    for (B, L, H, D) in ([(1, 4608, 24, 128)] if not small else [(1, 1024, 8, 128)]):
        q, k, v = (torch.randn(B, L, H, D, device="cuda").bfloat16() for _ in range(3))
        fl_ = 4.0 * B * H * L * L * D
        t_lib = timeit(lambda: R.attention(q, k, v))
        print(f"attention fwd B{B} L{L} H{H} D{D}: library SDPA {t_lib*1e6:.1f} us {fl_/t_lib/1e12:.0f} TF/s")
        from ..ops import flash_attn as FA
        if FA.supported(q, k, v):
            t = timeit(lambda: FA.flash_attention(q, k, v))
            which = "CTA-pair kernel" if (D == 128 and FA.pair_forward_ok(q.device)) else "one-CTA kernel"
            print(f"   ours ({which}) {t*1e6:.1f} us {fl_/t/1e12:.0f} TF/s  {fl_/t/fl:.2f} {tag}")
            if which == "CTA-pair kernel":
                lib = FA.N.require()
                o1 = torch.empty_like(q)
                l1 = torch.empty(B, H, L, dtype=torch.float32, device="cuda")
                t1 = timeit(lambda: lib.eri_flash_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o1.data_ptr(),
                                                           l1.data_ptr(), B, H, L, L, D, D ** -0.5, FA.N.stream_ptr()))
                print(f"   ours (one-CTA kernel) {t1*1e6:.1f} us {fl_/t1/1e12:.0f} TF/s  {fl_/t1/fl:.2f} {tag}")
        if FA.supported(q, k, v) and FA.has_backward():
            o_, lse_ = FA.fwd(q, k, v)
            go_ = torch.randn_like(o_)
            t = timeit(lambda: FA.bwd(go_, q, k, v, o_, lse_))
            print(f"   ours bwd {t*1e6:.1f} us {2.5*fl_/t/1e12:.0f} TF/s (algorithmic 2.5x fwd flops; "
                  f"3.5x executed)  {2.5*fl_/t/fl:.2f} {tag}")
            assert FA.check_error() == 0
        qg, kg, vg = (t_.clone().requires_grad_() for t_ in (q, k, v))
        o = R.attention(qg, kg, vg)
        go = torch.randn_like(o)
        t_b = timeit(lambda: torch.autograd.grad(o, (qg, kg, vg), go, retain_graph=True))
        print(f"   library SDPA bwd {t_b*1e6:.1f} us {2.5*fl_/t_b/1e12:.0f} TF/s")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="gemm,elementwise,optim,attn")
    ap.add_argument("--small", action="store_true")
    a = ap.parse_args()
    for w in a.what.split(","):
        {"gemm": bench_gemm, "skinny": bench_skinny, "elementwise": bench_elementwise, "optim": bench_optim,
         "epilogue": bench_epilogue,
         "attn": bench_attn, "dequant": bench_dequant, "narrow": bench_narrow, "wgrad": bench_wgrad, "small_m": bench_small_m, "gather_emul": bench_gather_emul}[w](a.small)


if __name__ == "__main__":
    main()
