"""The reference's debugging / workspace environment switches.

* ``ATTN_Q_CHUNK``, ``ATTN_KV_CHUNK`` -- force the blockwise (online-softmax) attention of the
  library path with these block sizes; ``ATTN_MAX_WS_MB`` caps the score workspace
  ``B * H * q_chunk * kv_chunk * 4`` bytes and ``ATTN_MIN_FREE_MB`` keeps that much device memory
  free; ``ATTN_REUSE=1`` lets consecutive calls share one workspace and makes overlapping use an
  error (crates/training/src/sdxl/runtime.rs:375-463 reuse guard and workspace-cap errors; read by
  ``sdxl_10steps``, crates/training/src/bin/sdxl_10steps.rs).
* ``SDXL_TIMING=1`` -- per-stage timing breakdown (runtime.rs:323-361); here it turns on the
  trainer's device-timed phases.
* ``SDXL_LOAD_TRACE=1`` -- GiB/s of weight loads (crates/training/src/sdxl/trace.rs).
* ``BACKWARD_DEBUG=1`` -- verbose backward (crates/training/src/gradient_accumulator.rs:114-119);
  here autograd anomaly detection plus a per-parameter gradient report.
* ``ERID_PINNED_CHECKPOINT_CACHE_MB`` -- size of the pinned staging cache used when checkpoints are
  written from the GPU.

The native flash-attention kernels never materialise scores, so the ``ATTN_*`` switches only act on
the library path (masks, unsupported head sizes, CPU).
"""
from __future__ import annotations

import contextlib
import os
import time
from dataclasses import dataclass

import torch


def _int(name, default=None):
    v = os.environ.get(name)
    return int(v) if v not in (None, "") else default


def flag(name: str) -> bool:
    return os.environ.get(name, "") not in ("", "0", "false", "False")


class WorkspaceError(RuntimeError):
    pass


@dataclass
class AttentionWorkspacePolicy:
    q_chunk: int | None = None
    kv_chunk: int | None = None
    reuse: bool = False
    max_ws_mb: int | None = None
    min_free_mb: int | None = None

    @classmethod
    def from_env(cls):
        return cls(_int("ATTN_Q_CHUNK"), _int("ATTN_KV_CHUNK"), flag("ATTN_REUSE"), _int("ATTN_MAX_WS_MB"),
                   _int("ATTN_MIN_FREE_MB"))

    @property
    def active(self) -> bool:
        return any(v is not None for v in (self.q_chunk, self.kv_chunk, self.max_ws_mb, self.min_free_mb))

    def plan(self, B: int, H: int, Lq: int, Lk: int, free_bytes: int | None = None):
        """(q_chunk, kv_chunk) honouring the forced sizes and the caps; halves the larger block
        until the fp32 score block fits. Raises ``WorkspaceError`` when even 64 x 64 does not."""
        q = min(self.q_chunk or Lq, Lq)
        k = min(self.kv_chunk or Lk, Lk)
        cap = None
        if self.max_ws_mb is not None:
            cap = self.max_ws_mb << 20
        if self.min_free_mb is not None and free_bytes is not None:
            room = free_bytes - (self.min_free_mb << 20)
            cap = room if cap is None else min(cap, room)
        if cap is not None:
            while B * H * q * k * 4 > cap:
                if max(q, k) <= 64:
                    raise WorkspaceError(f"attention workspace cap {cap / 2 ** 20:.1f} MiB is below one 64 x 64 score "
                                         f"block for B={B}, H={H}")
                if q >= k:
                    q = max(64, q // 2)
                else:
                    k = max(64, k // 2)
        return q, k


class WorkspaceReuseGuard:
    """One shared workspace; entering it twice at the same time is a bug in the caller's stream /
    thread structure and raises instead of corrupting scores."""

    def __init__(self):
        self.busy = False
        self.buffer = None
        self.uses = 0

    @contextlib.contextmanager
    def acquire(self, nbytes: int, device):
        if self.busy:
            raise WorkspaceError("attention workspace is already in use (ATTN_REUSE=1 forbids overlapping calls)")
        if self.buffer is None or self.buffer.numel() < nbytes or self.buffer.device != torch.device(device):
            self.buffer = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.busy = True
        self.uses += 1
        try:
            yield self.buffer[:nbytes]
        finally:
            self.busy = False


_GUARD = WorkspaceReuseGuard()


def library_attention(q, k, v, scale=None, policy: AttentionWorkspacePolicy | None = None):
    """Blockwise attention under the ``ATTN_*`` policy, or None when no switch is set (the caller
    then uses its default path). Token-major ``[B, L, H, Dh]``."""
    policy = policy or AttentionWorkspacePolicy.from_env()
    if not policy.active:
        return None
    from ..ops import reference as R
    B, Lq, H, _ = q.shape
    free = torch.cuda.mem_get_info(q.device)[0] if q.is_cuda else None
    qc, kc = policy.plan(B, H, Lq, k.shape[1], free)
    if policy.reuse:
        with _GUARD.acquire(B * H * qc * kc * 4, q.device):
            return R.attention_chunked(q, k, v, scale, qc, kc)
    return R.attention_chunked(q, k, v, scale, qc, kc)


@contextlib.contextmanager
def load_trace(what: str, nbytes_fn=None, print_fn=print):
    """``with load_trace("unet", lambda: bytes_loaded): ...`` prints ``GiB/s`` when
    ``SDXL_LOAD_TRACE`` is set."""
    t0 = time.perf_counter()
    yield
    if flag("SDXL_LOAD_TRACE"):
        dt = max(time.perf_counter() - t0, 1e-9)
        nb = nbytes_fn() if nbytes_fn else 0
        print_fn(f"[load] {what}: {nb / 2 ** 30:.3f} GiB in {dt:.3f} s = {nb / 2 ** 30 / dt:.2f} GiB/s")


@contextlib.contextmanager
def backward_debug(named_params=None, print_fn=print):
    """Under ``BACKWARD_DEBUG=1``: autograd anomaly detection for the body, then one line per
    parameter with a gradient (norm, max, non-finite count)."""
    if not flag("BACKWARD_DEBUG"):
        yield
        return
    # gradient statistics are taken by tensor hooks at the moment each gradient is produced: a
    # trainer that steps and clears its gradients inside the body would leave nothing to read after
    stats, handles = {}, []
    for name, p in (named_params or []):
        if p.requires_grad:
            def hook(g, name=name):
                gf = g.detach().float()
                stats[name] = (gf.norm(), gf.abs().max(), (~torch.isfinite(gf)).sum())
            handles.append(p.register_hook(hook))
    try:
        with torch.autograd.set_detect_anomaly(True):
            yield
    finally:
        for h in handles:
            h.remove()
    for name, (n, m, bad) in stats.items():
        print_fn(f"[backward] {name}: norm {float(n):.4e} max {float(m):.4e} nonfinite {int(bad)}")


def pinned_checkpoint_cache_bytes(default_mb: int = 256) -> int:
    return (_int("ERID_PINNED_CHECKPOINT_CACHE_MB", default_mb)) << 20
