"""Environment switches of the library attention path and of the SDXL harness (CPU)."""
import os
import subprocess
import sys

import pytest
import torch

from eridiffusion_b200.utils.env_flags import (AttentionWorkspacePolicy, WorkspaceError, WorkspaceReuseGuard,
                                               backward_debug, library_attention, load_trace,
                                               pinned_checkpoint_cache_bytes)


def test_workspace_policy_plan_and_caps():
    assert not AttentionWorkspacePolicy().active
    p = AttentionWorkspacePolicy(q_chunk=512, kv_chunk=2048)
    assert p.active and p.plan(1, 8, 4096, 4096) == (512, 2048) and p.plan(1, 8, 100, 300) == (100, 300)
    capped = AttentionWorkspacePolicy(max_ws_mb=4)
    q, k = capped.plan(2, 8, 4096, 4096)
    assert 2 * 8 * q * k * 4 <= 4 << 20 and q >= 64 and k >= 64
    with pytest.raises(WorkspaceError):
        AttentionWorkspacePolicy(max_ws_mb=1).plan(64, 64, 4096, 4096)
    free = AttentionWorkspacePolicy(min_free_mb=10)
    q, k = free.plan(1, 1, 1024, 1024, free_bytes=11 << 20)
    assert q * k * 4 <= 1 << 20


def test_library_attention_under_policy_matches_full():
    from eridiffusion_b200.ops.reference import attention_fp32
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(2, 96, 2, 16, generator=g) for _ in range(3))
    assert library_attention(q, k, v, policy=AttentionWorkspacePolicy()) is None
    for pol in (AttentionWorkspacePolicy(q_chunk=32, kv_chunk=40), AttentionWorkspacePolicy(kv_chunk=17, reuse=True)):
        o = library_attention(q, k, v, policy=pol)
        assert torch.allclose(o, attention_fp32(q, k, v), atol=1e-5)
    guard = WorkspaceReuseGuard()
    with guard.acquire(128, "cpu") as buf:
        assert buf.numel() == 128
        with pytest.raises(WorkspaceError):
            with guard.acquire(64, "cpu"):
                pass
    with guard.acquire(64, "cpu"):
        pass
    assert guard.uses == 2 and guard.buffer.numel() == 128          # grown once, then shared


def test_traces_and_debug(monkeypatch):
    lines = []
    with load_trace("x", lambda: 1 << 30, lines.append):
        pass
    assert lines == []
    monkeypatch.setenv("SDXL_LOAD_TRACE", "1")
    with load_trace("x", lambda: 1 << 30, lines.append):
        pass
    assert "1.000 GiB" in lines[0] and "GiB/s" in lines[0]
    w = torch.nn.Parameter(torch.ones(3))
    monkeypatch.setenv("BACKWARD_DEBUG", "1")
    out = []
    with backward_debug([("w", w)], out.append):
        (w * 2).sum().backward()
    assert out and out[0].startswith("[backward] w: norm 3.4641e+00") and "nonfinite 0" in out[0]
    monkeypatch.setenv("ERID_PINNED_CHECKPOINT_CACHE_MB", "8")
    assert pinned_checkpoint_cache_bytes() == 8 << 20


def test_attention_env_switch_reaches_op_in_fresh_process():
    code = ("import torch; from eridiffusion_b200.ops import functional as F, reference as R;"
            "import eridiffusion_b200.utils.env_flags as E;"
            "calls=[];orig=R.attention_chunked;"
            "R.attention_chunked=lambda *a,**k:(calls.append(a[4:]),orig(*a,**k))[1];"
            "q=torch.randn(1,64,2,8);o=F.attention(q,q,q);"
            "assert torch.allclose(o,R.attention_fp32(q,q,q),atol=1e-5);print(calls)")
    env = {**os.environ, "ATTN_KV_CHUNK": "16", "ERI_B200_NO_BUILD": "1"}
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=120)
    assert r.returncode == 0, r.stderr[-400:]
    assert "(64, 16)" in r.stdout


def test_reference_behaviour_switches_map_onto_this_package(monkeypatch):
    """The reference's attention / fusion / checkpoint-policy switches change this package's
    switches, or are refused by name."""
    import eridiffusion_b200.config as C
    from eridiffusion_b200.ops import functional as F
    from eridiffusion_b200.utils.env_flags import ReferenceEnvError, apply_reference_env
    monkeypatch.setattr(F, "_ATTN_NATIVE", "native")
    monkeypatch.setattr(F, "_BACKEND", "fused")
    monkeypatch.setattr(F, "_ATTN_ENV_POLICY", False)
    for k in ("ATTN_KV_CHUNK", "ATTN_MAX_WS_MB", "ATTN_REUSE"):
        monkeypatch.delenv(k, raising=False)
    notes = []
    done = apply_reference_env(environ={"FLUX_FORCE_DENSE_ATTENTION": "1", "ERID_FUSE": "0", "ATTN_LOG_MS": "1",
                                        "STREAM_ATTENTION_SELFTEST": "1"}, print_fn=notes.append)
    assert F._ATTN_NATIVE == "library" and F.get_backend() == "eager"
    assert "passed" in done["STREAM_ATTENTION_SELFTEST"] and "no effect" in done["ATTN_LOG_MS"] and notes
    F.set_backend("fused"); F.set_attention_impl("native")
    done = apply_reference_env(environ={"STREAMING_SDPA_CHUNK_MAX": "2048", "ATTN_MAX_WORKSPACE_MB": "64",
                                        "ATTN_CHUNK_REUSE": "1"}, print_fn=notes.append)
    assert os.environ["ATTN_KV_CHUNK"] == "2048" and os.environ["ATTN_MAX_WS_MB"] == "64" and os.environ["ATTN_REUSE"] == "1"
    assert F._ATTN_ENV_POLICY and F._ATTN_NATIVE == "library"
    F.set_attention_impl("native")
    with pytest.raises(ReferenceEnvError, match="CAUSAL_TEXT"):
        apply_reference_env(environ={"STREAM_ATTENTION_CAUSAL_TEXT": "1"})
    # through the configuration loader: checkpoint policy, streaming off, TREAD_* and strict bf16
    for k, v in {"GRADIENT_CHECKPOINT_POLICY": "cpu", "DISABLE_LAYER_STREAMING": "1", "TREAD_ENABLED": "1",
                 "TREAD_K_FRAC": "0.25", "TREAD_SCHEDULE": "2:5,7:9", "STRICT_BF16": "1"}.items():
        monkeypatch.setenv(k, v)
    cfg = C.load_config({"model_kind": "flux", "use_layer_streaming": True})
    assert cfg.gradient_checkpointing and cfg.meta["checkpoint_policy"] == "cpu_offload" and not cfg.use_layer_streaming
    assert cfg.tread.enabled and cfg.tread.k_frac == 0.25 and cfg.tread.schedule == [{"out": 2, "in": 5}, {"out": 7, "in": 9}]
    assert cfg.meta["strict_bf16"] == "count" and "GRADIENT_CHECKPOINT_POLICY" in cfg.meta["reference_env"]
    monkeypatch.setenv("STREAM_ATTENTION_CAUSAL_TEXT", "on")
    with pytest.raises(C.ConfigError, match="CAUSAL_TEXT"):
        C.load_config({"model_kind": "flux"})


def test_strict_bf16_counts_events_of_a_training_step(monkeypatch):
    import eridiffusion_b200.config as C
    from eridiffusion_b200.train.factory import build_job
    monkeypatch.setenv("STRICT_BF16", "1")
    cfg = C.load_config({"model_kind": "tiny_mmdit", "device": "cpu", "datasets": [{"synthetic": True, "resolution": [256]}]})
    tr, batches, _ = build_job(cfg, device="cpu")
    assert tr.strict_bf16 == "count"
    tr.train_step(next(batches))
    assert set(tr.strict_events) == {"clone_allocs", "f32_graph_casts", "layout_fixes"}
