"""Multi-GPU timing of the fused communication paths against their rooflines and against NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m eridiffusion_b200.cli.comm_bench [--what fused_dp,zero3,ulysses,link] [--params 56000000]

Times are CUDA-event device times, max over ranks, median of the timed launches after warm-up.
Rooflines (the slower of the two bounds is the target, as for any fused compute + collective):

* fused data-parallel step: bytes that must cross NVLink per direction, ``2 * (W-1)/W *
  arena_bytes``, over the measured 770 GB/s per direction (900 nominal);
* ZeRO-3 gather-in-GEMM (Qwen-Image shapes, weight rows sharded): max(GEMM FLOPs / measured cuBLAS
  peak, (W-1)/W * weight bytes / 770 GB/s);
* Ulysses QKV projection with scatter epilogue and out-projection with gathered A operand (LTX
  shapes, 19008 tokens over W ranks): max(GEMM FLOPs / peak, (W-1)/W * activation bytes / 770 GB/s).
"""
from __future__ import annotations

import argparse
import json
import statistics
from pathlib import Path

import torch
import torch.distributed as dist

from ..models.layers import Linear
from ..ops import _native as N_
from ..ops import functional as F
from ..optim import AdamW8bit, ParamArena
from ..parallel.dist import GradSync, ProcessGroup, init_from_env
from ..parallel.fused_dp import FusedDataParallel

LINK_GBS = 770.0


def gemm_peak():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text())["bf16_tflops"] * 1e12, "measured"
    return 1.59e15, "fallback"


def gemm_peak_sustained():
    """cuBLAS bf16 throughput in a seconds-long loop under the power cap (what a GEMM inside a long
    training step can reach); the burst figure of ``gemm_peak`` applies to a kernel timed alone."""
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d.get("bf16_tflops_sustained", d["bf16_tflops"]) * 1e12
    return 1.4e15


def roofline_fields(flops, link_bytes, t_ms, n_copy):
    """Both rooflines of a fused compute + collective launch: against the burst cuBLAS peak and
    against the sustained one, with the SMs that the launch gives to copy CTAs stated."""
    peak, _ = gemm_peak()
    sus = gemm_peak_sustained()
    link = link_bytes / (LINK_GBS * 1e9)
    roof, roof_s = max(flops / peak, link) * 1e3, max(flops / sus, link) * 1e3
    return {"roofline_ms": round(roof, 4), "fraction_of_roofline": round(roof / t_ms, 3),
            "roofline_sustained_ms": round(roof_s, 4), "fraction_of_roofline_sustained": round(roof_s / t_ms, 3),
            "copy_ctas_of_148_sms": n_copy}


def timed(fn, iters=10, warm=3):
    for i in range(warm):
        fn()
        if i == 0:
            # a bounded wait that ran out on any rank ends the benchmark on all ranks, instead of
            # repeating the same wait in every following launch
            bad = torch.tensor([1.0 if F.kernel_error_check() else 0.0], device="cuda")
            dist.all_reduce(bad, dist.ReduceOp.MAX)
            if bad.item():
                raise SystemExit("a kernel reported an error in the first launch; stopping")
    ts = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # a short device-side sleep lets the host queue the launches before the start event fires, so
        # the interval is device time and not the host's launch path (as inside a busy training step)
        torch.cuda._sleep(1_000_000)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    t = torch.tensor([statistics.median(ts)], device="cuda")
    dist.all_reduce(t, dist.ReduceOp.MAX)
    return t.item()


def bench_fused_dp(a, pg, rank, world, dev):
    n = a.params // (256 * world) * (256 * world)
    p = [torch.nn.Parameter(torch.randn(n, device=dev).bfloat16() * 0.02)]
    arena = ParamArena(p, shard_multiple=world)
    opt = AdamW8bit(arena, lr=1e-4, shard=(rank, world) if world > 1 else (0, 1))
    fdp = FusedDataParallel(pg, arena, opt)
    arena.grad.normal_()
    step = [0]

    def fused():
        step[0] += 1
        fdp.step(lr=1e-4, max_grad_norm=1.0, step=step[0])

    t_f = timed(fused)
    st = fdp.status()
    fdp.enable_phase_timing()
    dist.barrier()
    torch.cuda.synchronize()
    fused()
    torch.cuda.synchronize()
    phases = fdp.phase_times_us()
    fdp.stamps = None
    # NCCL + separate kernels: reduce-scatter, norm all-reduce, optimizer on shard, all-gather
    p2 = [torch.nn.Parameter(torch.randn(n, device=dev).bfloat16() * 0.02)]
    arena2 = ParamArena(p2, shard_multiple=world)
    opt2 = AdamW8bit(arena2, lr=1e-4, shard=(rank, world) if world > 1 else None)
    gs = GradSync("zero1")
    gs.attach(arena2, opt2)
    arena2.grad.normal_()

    def nccl():
        gs.reduce_grads()
        ss = gs.grad_sumsq()
        opt2.step(grad_sumsq=ss, max_grad_norm=1.0)
        gs.gather_params()

    t_n = timed(nccl)
    if rank == 0:
        nbytes = fdp.bytes_over_nvlink_per_direction()
        roof_ms = nbytes / (LINK_GBS * 1e9) * 1e3
        print(json.dumps({"what": "fused_dp_step (reduce-scatter + clip + adamw8bit + all-gather)",
                          "world": world, "params": n, "fused_ms": round(t_f, 4), "nccl_path_ms": round(t_n, 4),
                          "nvlink_bytes_per_direction": nbytes, "roofline_ms": round(roof_ms, 4),
                          "fraction_of_roofline": round(roof_ms / t_f, 3) if world > 1 else None,
                          "link_gbs_used": LINK_GBS, "status": st,
                          "phases_us_rank0": {k: round(v, 1) for k, v in phases.items()}}))


def bench_zero3(a, pg, rank, world, dev):
    """Forward of a row-sharded Linear (Qwen-Image MLP up-projection 3072 -> 12288, QKV
    3072 -> 9216 and MLP down-projection 12288 -> 3072 at 4096 + 512 tokens): the weight gather
    runs inside the GEMM launch."""
    from ..parallel.zero3 import Zero3Context, Zero3Linear
    peak, tag = gemm_peak()
    z3 = Zero3Context(pg, heap_bytes=512 << 20, max_weight_elems=48 << 20, n_copy=a.n_copy)
    M = 4608
    for n_out, k_in in ((12288, 3072), (9216, 3072), (3072, 12288)):
        torch.manual_seed(0)
        lin = Linear(k_in, n_out, bias=False, device=dev)
        zl = Zero3Linear(lin, z3)
        shard = z3.arena_alloc(zl.weight.numel(), torch.bfloat16, dev).view_as(zl.weight)
        shard.copy_(zl.weight.data)
        zl.weight.data = shard
        z3.barrier()
        x = torch.randn(1, M, k_in, device=dev).bfloat16()
        full = torch.empty(n_out, k_in, device=dev, dtype=torch.bfloat16)

        def fused():
            with torch.no_grad():
                zl(x)

        def nccl():
            with torch.no_grad():
                dist.all_gather_into_tensor(full, zl.weight.data)
                F.linear(x, full)

        t_f, t_n = timed(fused), timed(nccl)
        # one more launch with the kernel's own %globaltimer record
        z3.stamps = torch.zeros(8, dtype=torch.int64, device=dev)
        dist.barrier()
        fused()
        torch.cuda.synchronize()
        phases = z3.phase_times_us()
        z3.stamps = None
        flops = 2.0 * M * n_out * k_in
        link_bytes = (world - 1) / world * n_out * k_in * 2
        if rank == 0:
            print(json.dumps({"what": f"zero3 gather-in-GEMM forward [{M}x{k_in}] x [{n_out}x{k_in}]^T", "world": world,
                              "fused_ms": round(t_f, 4), "nccl_allgather_then_gemm_ms": round(t_n, 4),
                              "gemm_bound_ms": round(flops / peak * 1e3, 4),
                              "nvlink_bound_ms": round(link_bytes / (LINK_GBS * 1e9) * 1e3, 4),
                              **roofline_fields(flops, link_bytes, t_f, a.n_copy),
                              "n_copy": a.n_copy, "gemm_peak": tag, "status": z3.comm.status(), "gemm_err": F.gemm_error_check(),
                              "two_cta_gather_launches": N_.require().eri_gemm2_gather_count(),
                              "phases_us_rank0": {k: round(v, 1) for k, v in phases.items()}}))
        # forward + backward: two gathers inside GEMMs and the weight-gradient reduce-scatter inside the
        # dW GEMM's epilogue, against all-gather + three library GEMMs + NCCL reduce-scatter
        xg = x.clone().requires_grad_()
        dy = torch.randn(1, M, n_out, device=dev).bfloat16()
        zl.weight.requires_grad_(True)
        dws = torch.empty(n_out // world, k_in, device=dev, dtype=torch.bfloat16)
        dwf = torch.empty(n_out, k_in, device=dev, dtype=torch.bfloat16)

        def fused_fb():
            zl.weight.grad = None
            xg.grad = None
            zl(xg).backward(dy)

        def nccl_fb():
            with torch.no_grad():
                dist.all_gather_into_tensor(full, zl.weight.data)
                F.linear(x, full)
                dist.all_gather_into_tensor(full, zl.weight.data)       # ZeRO-3 re-gathers for backward
                torch.matmul(dy[0], full)
                torch.matmul(dy[0].t(), x[0], out=dwf)
                dist.reduce_scatter_tensor(dws, dwf, op=dist.ReduceOp.AVG)

        t_f, t_n = timed(fused_fb), timed(nccl_fb)
        if rank == 0:
            print(json.dumps({"what": f"zero3 forward + backward (gather, gather, dW reduce-scatter) [{M}x{k_in}] x [{n_out}x{k_in}]^T",
                              "world": world, "fused_ms": round(t_f, 4), "nccl_and_library_gemms_ms": round(t_n, 4),
                              **roofline_fields(3 * flops, 3 * link_bytes, t_f, a.n_copy),
                              "fused_reduce_scatter": bool(z3.fused_rs), "n_copy": a.n_copy, "gemm_peak": tag,
                              "status": z3.comm.status(), "gemm_err": F.gemm_error_check()}))
        zl.weight.requires_grad_(False)
    # A stack: three MLPs (3072 -> 12288 -> 3072) forward and backward as one step, with the next layer's slabs
    # pulled by the copy engines while the current GEMM runs (prefetch), and without.
    torch.manual_seed(1)
    layers = []
    for i in range(6):
        k_in, n_out = (3072, 12288) if i % 2 == 0 else (12288, 3072)
        zl = Zero3Linear(Linear(k_in, n_out, bias=False, device=dev), z3)
        shard = z3.arena_alloc(zl.weight.numel(), torch.bfloat16, dev).view_as(zl.weight)
        shard.copy_(zl.weight.data)
        zl.weight.data = shard
        zl.weight.requires_grad_(True)
        layers.append(zl)
    z3.barrier()
    x = torch.randn(1, M, 3072, device=dev).bfloat16()
    dy = torch.randn(1, M, 3072, device=dev).bfloat16()

    def step():
        z3.begin_step()
        h = x.clone().requires_grad_()
        y = h
        for zl in layers:
            zl.weight.grad = None
            y = zl(y)
        y.backward(dy)

    res = {}
    for on in (True, False):
        z3.prefetch = on and world > 1 and z3.prefetch_stream is not None
        step()                                    # records the order for the following steps
        n0 = z3.prefetched_launches
        res[on] = timed(step)
        res[(on, "n")] = z3.prefetched_launches - n0
    z3.begin_step()
    flops = 3 * 6 * 2.0 * M * 3072 * 12288
    link_bytes = 2 * 6 * (world - 1) / world * 3072 * 12288 * 2 + 6 * (world - 1) / world * 3072 * 12288 * 2
    if rank == 0:
        print(json.dumps({"what": "zero3 stack of six linears (3072 <-> 12288) forward + backward as one step", "world": world,
                          "prefetch_ms": round(res[True], 4), "no_prefetch_ms": round(res[False], 4),
                          "prefetched_launches_timed": res[(True, "n")],
                          **roofline_fields(flops, link_bytes, res[True], 0),
                          "status": z3.comm.status(), "gemm_err": F.gemm_error_check()}))


def bench_ulysses(a, pg, rank, world, dev):
    """LTX-shaped attention projections under sequence parallelism: hidden 4096, 32 heads, 19008
    tokens over W ranks. QKV projection with the head scatter in its epilogue, and out-projection
    whose A operand is gathered from the peers inside the launch."""
    from ..parallel.ulysses import UlyssesContext, ulysses_out_proj, ulysses_qkv
    peak, tag = gemm_peak()
    D, H = 4096, 32
    Ll = (19008 // world) // 128 * 128
    u = UlyssesContext(pg, batch=1, l_local=Ll, hidden=D, heads=H, n_copy=a.n_copy, attn_slots=2)
    torch.manual_seed(0)
    qkv = Linear(D, 3 * D, bias=False, device=dev)
    out = Linear(D, D, bias=False, device=dev)
    x = torch.randn(1, Ll, D, device=dev).bfloat16()
    attn = torch.randn(1, u.Lt, H // world, D // H, device=dev).bfloat16()
    send = torch.empty(world, Ll, 3 * D // world, device=dev, dtype=torch.bfloat16)
    recv = torch.empty_like(send)

    def fused_qkv():
        with torch.no_grad():
            ulysses_qkv(x, qkv, u)

    def nccl_qkv():
        with torch.no_grad():
            y = F.linear(x, qkv.weight)
            send.copy_(y.view(Ll, world, 3 * D // world).transpose(0, 1))
            dist.all_to_all_single(recv.view(-1), send.view(-1))

    # as in the model: the attention kernel writes its output into the layer's symmetric slot
    attn_slot = u.attn_buffer(1, H // world)
    attn_slot.copy_(attn)

    def fused_out():
        with torch.no_grad():
            ulysses_out_proj(attn_slot, out, u)

    def fused_out_publish():
        # attention output in ordinary memory: published with a barrier and a copy first
        with torch.no_grad():
            ulysses_out_proj(attn, out, u)

    send2 = torch.empty(world, Ll, D // world, device=dev, dtype=torch.bfloat16)
    recv2 = torch.empty_like(send2)

    def nccl_out():
        with torch.no_grad():
            send2.copy_(attn.view(world, Ll, D // world))
            dist.all_to_all_single(recv2.view(-1), send2.view(-1))
            F.linear(recv2.transpose(0, 1).reshape(1, Ll, D), out.weight)

    for name, f_f, f_n, n_out, act_cols in (("qkv projection + head scatter", fused_qkv, nccl_qkv, 3 * D, 3 * D),
                                             ("head gather + out projection", fused_out, nccl_out, D, D)):
        t_f, t_n = timed(f_f), timed(f_n)
        extra = {"fused_with_publish_copy_ms": round(timed(fused_out_publish), 4)} if f_f is fused_out else {}
        flops = 2.0 * Ll * n_out * D
        link_bytes = (world - 1) / world * Ll * act_cols * 2
        if rank == 0:
            print(json.dumps({"what": f"ulysses {name}, {Ll} local tokens, hidden {D}", "world": world,
                              "fused_ms": round(t_f, 4), "gemm_plus_nccl_all_to_all_ms": round(t_n, 4),
                              "gemm_bound_ms": round(flops / peak * 1e3, 4),
                              "nvlink_bound_ms": round(link_bytes / (LINK_GBS * 1e9) * 1e3, 4),
                              **roofline_fields(flops, link_bytes, t_f, a.n_copy if f_f is not fused_qkv else 0),
                              "n_copy": a.n_copy, "gemm_peak": tag, "status": u.comm.status(), "gemm_err": F.gemm_error_check(),
                              "two_cta_gather_launches": N_.require().eri_gemm2_gather_count(), **extra}))


def bench_link(a, pg, rank, world, dev):
    """Peer transfer rate by mechanism and CTA count: every rank moves 64 MiB between its own memory
    and the next rank's at the same time (all links busy in both directions, as in a gather)."""
    import ctypes as C
    from ..parallel.symm import SymmetricHeap
    lib = N_.require()
    lib.eri_link_probe.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_void_p, C.c_int,
                                   C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    lib.eri_link_probe.restype = C.c_int
    nbytes = 64 << 20
    heap = SymmetricHeap(2 * nbytes + (1 << 20), group=pg.group)
    src_sym = heap.tensor((nbytes,), torch.uint8)
    dst_sym = heap.tensor((nbytes,), torch.uint8)
    src_sym.local.random_(0, 255)
    local_dst = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    local_src = torch.empty(nbytes, dtype=torch.uint8, device=dev).random_(0, 255)
    peer = (rank + 1) % world
    torch.cuda.synchronize()
    dist.barrier()
    flags = torch.zeros(4096, dtype=torch.int32, device=dev)
    targets = torch.full((4096,), 1 << 30, dtype=torch.int32, device=dev)

    def jobs_for(src_ptr, dst_ptr, n_ctas):
        # one contiguous slab per job, several jobs per CTA so that the ring stays busy
        per = 1 << 20
        arr = (N_.GatherJob * (nbytes // per))()
        for i in range(nbytes // per):
            arr[i].src, arr[i].dst, arr[i].rows, arr[i].row_bytes = src_ptr + i * per, dst_ptr + i * per, 1, per
            arr[i].src_stride = arr[i].dst_stride = per
            arr[i].flag = i % 4096
        return torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).to(dev), nbytes // per

    rows = []
    for mode, name, s_ptr, d_ptr in ((0, "bulk pull (cp.async.bulk peer -> smem -> local)", src_sym.peer_ptrs[peer], local_dst.data_ptr()),
                                     (1, "load pull (16-byte peer loads)", src_sym.peer_ptrs[peer], local_dst.data_ptr()),
                                     (2, "store push (16-byte peer stores)", local_src.data_ptr(), dst_sym.peer_ptrs[peer]),
                                     (3, "bulk push (local -> smem -> cp.async.bulk to peer)", local_src.data_ptr(), dst_sym.peer_ptrs[peer])):
        for n_ctas in (8, 16, 32, 64, 132):
            jobs, nj = jobs_for(s_ptr, d_ptr, n_ctas) if mode in (0, 3) else (None, 0)
            stream = torch.cuda.current_stream().cuda_stream

            def run():
                code = lib.eri_link_probe(mode, s_ptr, d_ptr, nbytes, n_ctas, jobs.data_ptr() if jobs is not None else None,
                                          nj, flags.data_ptr(), targets.data_ptr(), 6, stream)
                if code:
                    raise RuntimeError(f"link probe mode {mode} failed with code {code}")
            t = timed(run, iters=5, warm=2)
            rows.append((name, n_ctas, t))
            if rank == 0:
                print(json.dumps({"what": f"link probe, {name}", "world": world, "ctas": n_ctas, "mib": nbytes >> 20,
                                  "ms": round(t, 4), "gbs_per_gpu_per_direction": round(nbytes / t / 1e6, 1),
                                  "probe_err": lib.eri_link_probe_check_error()}))
    # NCCL reference point: all-gather of the same 64 MiB per rank
    full = torch.empty(world * nbytes, dtype=torch.uint8, device=dev)
    t = timed(lambda: dist.all_gather_into_tensor(full, local_src), iters=5, warm=2)
    if rank == 0:
        print(json.dumps({"what": "NCCL all-gather of 64 MiB per rank", "world": world, "ms": round(t, 4),
                          "ingress_gbs_per_gpu": round((world - 1) * nbytes / t / 1e6, 1)}))


def bench_ring(a, pg, rank, world, dev):
    """Context parallelism at the headline attention shape (B1, 4608 tokens, 24 heads of 128): ring
    attention over NCCL send / recv (sequence sharded, keys and values travel) against Ulysses-style
    head sharding (NCCL all-to-all, then the flash kernel over the full sequence with H / W heads) and
    against one GPU doing the whole problem. Forward + backward; parity of the ring result against the
    one-GPU flash kernel is printed with the times."""
    from ..ops import flash_attn as FA
    from ..parallel.ring_attention import ring_attention
    B, L, H, D = 1, 4608, 24, 128
    Ll, Hl = L // world, H // world
    g = torch.Generator(device=dev).manual_seed(11)
    full = [torch.randn(B, L, H, D, device=dev, generator=g).bfloat16() for _ in range(4)]     # same on every rank
    q, k, v, do = (t[:, rank * Ll:(rank + 1) * Ll].contiguous() for t in full)

    def ring():
        ql, kl, vl = (t.clone().requires_grad_() for t in (q, k, v))
        o = ring_attention(ql, kl, vl)
        o.backward(do)
        return o, ql.grad, kl.grad, vl.grad

    def a2a(x, to_heads):
        # [B, Ll, H, D] -> [B, L, Hl, D] (to_heads) or back
        if to_heads:
            src = x.view(B, Ll, world, Hl, D).permute(2, 0, 1, 3, 4).contiguous()
            dst = torch.empty_like(src)
            dist.all_to_all_single(dst, src)
            return dst.permute(1, 0, 2, 3, 4).reshape(B, L, Hl, D)
        src = x.view(B, world, Ll, Hl, D).permute(1, 0, 2, 3, 4).contiguous()
        dst = torch.empty_like(src)
        dist.all_to_all_single(dst, src)
        return dst.permute(1, 2, 0, 3, 4).reshape(B, Ll, H, D)

    def ulysses():
        qh, kh, vh, doh = (a2a(t, True) for t in (q, k, v, do))
        o, lse = FA.fwd(qh, kh, vh)
        dq, dk, dv = FA.bwd(doh, qh, kh, vh, o, lse)
        return [a2a(t, False) for t in (o, dq, dk, dv)]

    def single():
        o, lse = FA.fwd(full[0], full[1], full[2])
        return (o,) + tuple(FA.bwd(full[3], full[0], full[1], full[2], o, lse))

    ref = single()
    got = ring()
    err = max(float((got[i].float() - ref[i][:, rank * Ll:(rank + 1) * Ll].float()).abs().max() /
                    ref[i].float().abs().max()) for i in range(4))
    e = torch.tensor([err], device=dev)
    dist.all_reduce(e, dist.ReduceOp.MAX)
    t_r, t_u, t_s = timed(ring), timed(ulysses), timed(single)
    if rank == 0:
        flops = 3.5 * 4.0 * L * L * D * H * B                                  # forward + 2.5x backward
        print(json.dumps({"what": f"context parallel attention fwd+bwd, B{B} L{L} H{H} Dh{D}", "world": world,
                          "ring_nccl_ms": round(t_r, 4), "ulysses_all_to_all_ms": round(t_u, 4),
                          "one_gpu_flash_ms": round(t_s, 4), "ideal_ms": round(t_s / world, 4),
                          "ring_vs_one_gpu_max_err_rel": round(float(e), 5),
                          "ring_tflops_per_gpu": round(flops / world / t_r / 1e9, 1),
                          "fa_err": FA.check_error()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--params", type=int, default=56_000_000)
    ap.add_argument("--what", default="fused_dp")
    ap.add_argument("--n-copy", default="16", help="copy CTAs of the gather-fused GEMM launches; a comma-separated "
                    "list repeats the zero3 / ulysses measurements for every value")
    a = ap.parse_args()
    rank, world, local = init_from_env()
    dev = torch.device("cuda", local)
    pg = ProcessGroup()
    sweep = [int(v) for v in str(a.n_copy).split(",")]
    for w in a.what.split(","):
        for nc in (sweep if w not in ("fused_dp", "link", "ring") else sweep[:1]):
            a.n_copy = nc
            {"fused_dp": bench_fused_dp, "zero3": bench_zero3, "ulysses": bench_ulysses, "link": bench_link, "ring": bench_ring}[w](
                a, pg, rank, world, dev)
            dist.barrier()
            torch.cuda.empty_cache()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
