"""Check the RMS-norm kernels against an fp32 statement of the op.

    python -m eridiffusion_b200.cli.verify_rms_norm [--rows 4608] [--dim 3072] [--device cuda:0]

Counterpart of the reference's ``verify_rms_norm`` binary (src/bin/verify_rms_norm.rs, one of its
five default-built programs). Covers the plain row norm with a weight, the modulated form
``x_hat * (1 + scale) + shift`` and the per-head QK norm, forward and input gradient, and prints one
accuracy line per case; the exit code is the number of failed cases. On a machine without a GPU the
same cases run through the PyTorch path (the check is then of the op's definition, not of a kernel).
"""
from __future__ import annotations

import argparse
import sys

import torch

from ..ops import functional as F
from ..utils.accuracy import AccuracyTestSuite


def rms_ref(x, weight=None, scale=None, shift=None, eps=1e-6):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    if scale is not None:
        y = y * (1 + scale.float().unsqueeze(1)) + shift.float().unsqueeze(1)
    return y


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=4608)
    ap.add_argument("--dim", type=int, default=3072)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--tolerance", type=float, default=2e-2)
    a = ap.parse_args(argv)
    dev = torch.device(a.device)
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    tol = a.tolerance if dt == torch.bfloat16 else 1e-4
    g = torch.Generator().manual_seed(0)
    mk = lambda *s: torch.randn(*s, generator=g).to(dev, dt)
    suite = AccuracyTestSuite()
    x = mk(a.batch, a.rows, a.dim)
    w = (1 + 0.1 * mk(a.dim))
    sc, sh = 0.1 * mk(a.batch, a.dim), 0.1 * mk(a.batch, a.dim)
    cases = {"rms_norm(weight)": dict(weight=w), "rms_norm(modulated)": dict(scale=sc, shift=sh),
             "rms_norm(plain)": {}}
    for name, kw in cases.items():
        xi = x.clone().requires_grad_()
        if "scale" in kw:
            y = F.norm_modulate(xi, kw["scale"], kw["shift"], rms=True)
        else:
            y = F.norm_modulate(xi, weight=kw.get("weight"), rms=True)
        xr = x.detach().clone().requires_grad_()
        yr = rms_ref(xr, **kw)
        suite.add_comparison(f"{name} fwd", y, yr, tol)
        go = mk(*y.shape)
        y.backward(go)
        yr.backward(go.float())
        suite.add_comparison(f"{name} dx", xi.grad, xr.grad, tol)
    # per-head QK norm: [B, L, H, Dh] normalised over Dh
    H, Dh = 8, 128
    q = mk(a.batch, min(a.rows, 1024), H, Dh)
    qs = (1 + 0.1 * mk(Dh))
    yq = F.norm_modulate(q.view(-1, 1, Dh).contiguous(), weight=qs, rms=True).view_as(q)
    suite.add_comparison("qk_norm(per head) fwd", yq, rms_ref(q, weight=qs), tol)
    print(suite.generate_summary())
    return suite.num_failed()


if __name__ == "__main__":
    sys.exit(main())
