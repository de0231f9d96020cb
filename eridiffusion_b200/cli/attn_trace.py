"""Print the device-side timeline of the attention-backward dQ kernel (CTA 0).

    python -m eridiffusion_b200.cli.attn_trace [--L 4608] [--H 24] [--tiles 6]

The kernel records ``clock64`` at every hand-off between its MMA-issuing thread and its softmax
warps when a trace buffer is set (``eri_fa_bwd_set_trace``); this prints the cycle deltas for the
first tiles so the pipeline's stalls can be read directly. Event codes of the dQ kernel, MMA
thread: 1 operands staged, 2 K/V tile landed, 3 S consumed by softmax, 4 next S issued, 7 next dP
issued, 5 dS ready, 6 dQ issued. Softmax warp 0: 10 loop top, 11 S complete, 12 S in registers,
13 P computed, 14 dP complete, 15 dP in registers, 16 dS store issued, 17 dS store complete.
dK/dV kernel, MMA thread: 2 P ready, 3 dV issued, 4 next Q/dO landed, 5 next S issued, 6 dS ready,
7 dK issued, 8 next dP issued; softmax warp 0: 10 loop top, 11 S complete, 13 P stored,
14 dP complete, 17 dS stored.
"""
from __future__ import annotations

import argparse
import ctypes as C

import torch

from ..ops import _native as N
from ..ops import flash_attn as FA


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--L", type=int, default=4608)
    ap.add_argument("--H", type=int, default=24)
    ap.add_argument("--D", type=int, default=128)
    ap.add_argument("--tiles", type=int, default=6)
    ap.add_argument("--kernel", choices=["dq", "dkdv"], default="dq")
    a = ap.parse_args()
    lib = N.require()
    lib.eri_fa_bwd_set_trace.argtypes = [C.c_void_p, C.c_int, C.c_int]
    lib.eri_fa_bwd_set_trace.restype = C.c_int
    q, k, v = (torch.randn(1, a.L, a.H, a.D, device="cuda").bfloat16() for _ in range(3))
    o, lse = FA.fwd(q, k, v)
    do = torch.randn_like(o)
    for _ in range(2):
        FA.bwd(do, q, k, v, o, lse)
    cap = 512
    buf = torch.zeros(2 * cap, dtype=torch.int64, device="cuda")
    lib.eri_fa_bwd_set_trace(buf.data_ptr(), cap, 0 if a.kernel == "dq" else 1)
    FA.bwd(do, q, k, v, o, lse)
    torch.cuda.synchronize()
    lib.eri_fa_bwd_set_trace(None, 0, 0)
    h = buf.cpu().tolist()
    t0 = min(x >> 8 for x in h if x)
    for rec, name in ((0, "MMA thread"), (1, "softmax warp 0")):
        ev = [(x >> 8, x & 0xFF) for x in h[rec * cap:(rec + 1) * cap] if x]
        print(f"--- {name}: {len(ev)} events; (cycles since start, +delta, code)")
        prev = None
        for t, code in ev[: a.tiles * 8 + 4]:
            print(f"{t - t0:9d} {'' if prev is None else f'+{t - prev:6d}':>8}  {code}")
            prev = t
        if len(ev) > 40:
            # steady state: mean cycles per tile over the middle of the loop
            marks = [t for t, code in ev if code == ((5 if a.kernel == "dq" else 6) if rec == 0 else 11)]
            if len(marks) > 8:
                mid = marks[4:-2]
                print(f"steady-state cycles per tile: {(mid[-1] - mid[0]) / (len(mid) - 1):.0f}")
    assert FA.check_error() == 0


if __name__ == "__main__":
    main()
