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

``apply_reference_env`` maps the switches that gate the reference's attention / fusion behaviour onto
this package's own switches (or refuses them by name when nothing here corresponds):

* ``FLUX_FORCE_DENSE_ATTENTION`` (crates/training/src/flux/runtime.rs:484-486) -> dense library
  attention instead of the flash kernels;
* ``STREAMING_SDPA_CHUNK_MAX`` / ``ATTN_CHUNK_SIZE`` (runtime.rs:210, 488-520; default cap 2048 keys)
  -> blockwise library attention with that key-block size; ``ATTN_MAX_WORKSPACE_MB`` and
  ``ATTN_CHUNK_REUSE`` are the reference's spellings of ``ATTN_MAX_WS_MB`` / ``ATTN_REUSE``;
* ``STREAM_ATTENTION_SELFTEST`` -> blockwise vs dense attention compared once at start-up;
* ``STREAM_ATTENTION_CAUSAL_TEXT`` -> refused: there is no causal text mask here;
* ``STREAM_ATTENTION_LOG_ALLOCS`` / ``STREAM_ATTENTION_DEBUG_WRITES`` / ``ATTN_LOG_MS`` -> noted as
  having no effect (no score workspace is ever allocated on the native path);
* ``ERID_FUSE`` (crates/core/src/layers/norms.rs:5-12, mlp.rs:45-56): ``0`` selects the unfused
  PyTorch statements (``ERI_B200_BACKEND=eager``), ``1`` the fused kernels (the default here);
* ``STRICT_BF16=1`` -> the strict-bf16 counters run around every training step and a violation
  count is reported with the log row (``=panic`` raises at the first event);
* ``GRADIENT_CHECKPOINT_POLICY`` = ``recompute | cpu_offload | adaptive``
  (src/trainers/gpu_gradient_checkpoint.rs:165-188) -> activation policy of the block runner, with
  ``GRADIENT_CHECKPOINT_MEMORY_THRESHOLD_MB`` / ``GRADIENT_CHECKPOINT_PREFER_RECOMPUTE`` for the
  adaptive choice;
* ``DISABLE_LAYER_STREAMING=1`` -> ``use_layer_streaming`` off; ``TREAD_*`` -> the ``tread`` block.
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


# ------------------------------------------------------------------------------- reference switches
_NO_EFFECT = ("STREAM_ATTENTION_LOG_ALLOCS", "STREAM_ATTENTION_DEBUG_WRITES", "ATTN_LOG_MS")
_REFUSED = {"STREAM_ATTENTION_CAUSAL_TEXT": "causal text masks are not implemented (attention here is non-causal; "
                                            "key-padding masks are supported)"}


class ReferenceEnvError(RuntimeError):
    """An environment switch of the reference asks for behaviour that does not exist here."""


def _truthy(v) -> bool:
    return str(v).lower() in ("1", "true", "on", "yes")


def adaptive_checkpoint_settings():
    """(memory threshold in bytes, prefer recompute) of ``GRADIENT_CHECKPOINT_POLICY=adaptive``."""
    mb = max(1, _int("GRADIENT_CHECKPOINT_MEMORY_THRESHOLD_MB", 8192))
    prefer = _truthy(os.environ.get("GRADIENT_CHECKPOINT_PREFER_RECOMPUTE", "1"))
    return mb << 20, prefer


def apply_reference_env(cfg=None, environ=None, print_fn=print) -> dict:
    """Apply the reference's behaviour switches found in ``environ`` (default ``os.environ``) to this
    package's module-level switches and, when given, to a loaded ``TrainCfg``. Returns what was
    applied as ``{variable: effect}``; raises ``ReferenceEnvError`` for a switch that cannot be
    honoured."""
    env = os.environ if environ is None else environ
    done = {}
    for name, why in _REFUSED.items():
        if _truthy(env.get(name, "")):
            raise ReferenceEnvError(f"{name}: {why}")
    for name in _NO_EFFECT:
        if env.get(name):
            done[name] = "no effect: the native attention allocates no score workspace"
            print_fn(f"[env] {name} is set but has no effect here ({done[name][11:]})")
    from ..ops import functional as F
    if _truthy(env.get("FLUX_FORCE_DENSE_ATTENTION", "")):
        F.set_attention_impl("library")
        done["FLUX_FORCE_DENSE_ATTENTION"] = "attention -> dense library path"
    chunk = env.get("STREAMING_SDPA_CHUNK_MAX") or env.get("ATTN_CHUNK_SIZE")
    if chunk:
        n = int(chunk)
        if n < 16:
            raise ReferenceEnvError(f"attention chunk size {n} is below 16 keys")
        os.environ.setdefault("ATTN_KV_CHUNK", str(n))
        F.set_attention_impl("library")
        F._ATTN_ENV_POLICY = True
        done["STREAMING_SDPA_CHUNK_MAX" if env.get("STREAMING_SDPA_CHUNK_MAX") else "ATTN_CHUNK_SIZE"] = \
            f"blockwise library attention, {n}-key blocks"
    for ref, ours in (("ATTN_MAX_WORKSPACE_MB", "ATTN_MAX_WS_MB"), ("ATTN_CHUNK_REUSE", "ATTN_REUSE")):
        if env.get(ref):
            os.environ.setdefault(ours, env[ref])
            F._ATTN_ENV_POLICY = True
            done[ref] = f"-> {ours}"
    if _truthy(env.get("STREAM_ATTENTION_SELFTEST", "")):
        from ..ops import reference as R
        g = torch.Generator().manual_seed(0)
        q, k, v = (torch.randn(1, 96, 2, 32, generator=g) for _ in range(3))
        err = (R.attention_chunked(q, k, v, None, 32, 32) - R.attention_fp32(q, k, v)).abs().max().item()
        if err > 1e-4:
            raise ReferenceEnvError(f"STREAM_ATTENTION_SELFTEST: blockwise attention differs from dense by {err:.2e}")
        done["STREAM_ATTENTION_SELFTEST"] = f"passed (max difference {err:.1e})"
    fuse = env.get("ERID_FUSE")
    if fuse is not None and fuse != "":
        F.set_backend("fused" if fuse == "1" else "eager")
        done["ERID_FUSE"] = f"backend -> {F.get_backend()}"
    strict = env.get("STRICT_BF16", "")
    if strict and strict != "0":
        done["STRICT_BF16"] = "panic" if strict.lower() == "panic" else "count"
    pol = env.get("GRADIENT_CHECKPOINT_POLICY", "").lower()
    if pol:
        policy = {"cpu": "cpu_offload", "cpu_offload": "cpu_offload", "cpu-offload": "cpu_offload",
                  "adaptive": "adaptive"}.get(pol, "recompute")
        if pol not in ("cpu", "cpu_offload", "cpu-offload", "adaptive", "recompute"):
            print_fn(f"[env] unknown GRADIENT_CHECKPOINT_POLICY={pol!r}: using recompute")
        done["GRADIENT_CHECKPOINT_POLICY"] = policy
        if cfg is not None:
            cfg.gradient_checkpointing = True
            cfg.meta["checkpoint_policy"] = policy
    if cfg is not None:
        if _truthy(env.get("DISABLE_LAYER_STREAMING", "")) and cfg.use_layer_streaming:
            cfg.use_layer_streaming = False
            done["DISABLE_LAYER_STREAMING"] = "use_layer_streaming -> false"
        if "STRICT_BF16" in done:
            cfg.meta["strict_bf16"] = done["STRICT_BF16"]
        t = cfg.tread
        if env.get("TREAD_ENABLED") is not None and env.get("TREAD_ENABLED") != "":
            t.enabled = _truthy(env["TREAD_ENABLED"])
            done["TREAD_ENABLED"] = str(t.enabled)
        for var, attr, cast in (("TREAD_MASK_TYPE", "mask_type", str), ("TREAD_K", "k", int), ("TREAD_K_FRAC", "k_frac", float),
                                ("TREAD_REINJECT_MODE", "reinject", str), ("TREAD_LAMBDA", "route_lambda", float)):
            if env.get(var):
                setattr(t, attr, cast(env[var]))
                done[var] = f"tread.{attr} = {getattr(t, attr)}"
        if env.get("TREAD_SCHEDULE"):
            # "out:in,out:in" pairs
            t.schedule = [{"out": int(a), "in": int(b)} for a, b in
                          (p.split(":") for p in env["TREAD_SCHEDULE"].split(",") if p)]
            done["TREAD_SCHEDULE"] = str(t.schedule)
    return done
