"""The reference's other checkpoint layouts, written and read key-for-key so that its files and
the tools around them keep working.

* Chroma LoRA (crates/training/src/chroma/train.rs:1773-1818): ``lora_step{NNNN}.safetensors`` with
  bf16 tensors keyed ``lora_param_{i}`` in parameter order (metadata ``step``, ``param_count``),
  ``lora_ema_step{NNNN}.safetensors`` and ``trainer_state.json`` (``global_step``,
  ``optimizer_state``, ``grad_scaler{scale, growth}``).
* Adapter checkpoint (crates/training/src/checkpoint_manager.rs:51-108):
  ``checkpoint-{step}/{adapter_model.safetensors, optimizer.safetensors, metadata.json}`` and a
  ``checkpoint-latest`` symlink; metadata ``format=eridiffusion, network_type, rank, alpha``.
* Strict checkpoint (crates/training/src/strict_checkpoint.rs:14-119): one safetensors file whose
  ``__metadata__`` carries ``format_version, trainer, model, lora_rank, lora_alpha, step``; the
  reader insists that the keys found are exactly the keys expected.
* EMA file (crates/common/ema/src/ema.rs:44-109): safetensors with a selectable storage dtype.
"""
from __future__ import annotations

import json
import re
from pathlib import Path

import torch

from ..adapters import adapter_parameters, adapter_state_dict, load_adapter_state_dict
from ..io import safetensors as st

STRICT_FORMAT_VERSION = "1"


# ------------------------------------------------------------------------------ Chroma layout
def save_chroma_lora(adapters, root, step, ema=None, optimizer=None, scaler=None):
    root = Path(root)
    root.mkdir(parents=True, exist_ok=True)
    params = adapter_parameters(adapters)
    sd = {f"lora_param_{i}": p.detach().to(torch.bfloat16) for i, p in enumerate(params)}
    st.save_file(sd, root / f"lora_step{step:04d}.safetensors", {"step": step, "param_count": len(params)})
    if ema is not None:
        esd = {f"lora_param_{i}": t.detach().to(torch.bfloat16) for i, t in enumerate(ema)}
        st.save_file(esd, root / f"lora_ema_step{step:04d}.safetensors", {"step": step, "param_count": len(params)})
    state = {"global_step": step,
             "optimizer_state": {k: v for k, v in (optimizer.state_dict().items() if optimizer is not None else [])
                                 if isinstance(v, (int, float, str, list, tuple))},
             "grad_scaler": {"scale": getattr(scaler, "scale", 1.0), "growth": getattr(scaler, "growth_tracker", 0)}}
    (root / "trainer_state.json").write_text(json.dumps(state, indent=1))
    return root / f"lora_step{step:04d}.safetensors"


def load_chroma_lora(adapters, root, step=None):
    """Loads ``lora_step{step}`` (the highest step when ``step`` is None). Returns the step."""
    root = Path(root)
    if step is None:
        steps = sorted(int(m.group(1)) for p in root.iterdir() if (m := re.match(r"lora_step(\d+)\.safetensors$", p.name)))
        if not steps:
            return None
        step = steps[-1]
    sd = st.load_file(root / f"lora_step{step:04d}.safetensors")
    params = adapter_parameters(adapters)
    if len(sd) != len(params):
        raise KeyError(f"checkpoint holds {len(sd)} tensors, the adapters have {len(params)}")
    with torch.no_grad():
        for i, p in enumerate(params):
            p.copy_(sd[f"lora_param_{i}"].to(p.dtype).view_as(p))
    return step


# ------------------------------------------------------------------------------ adapter checkpoint
def save_adapter_checkpoint(adapters, root, step, network_type="lora", rank=None, alpha=None, optimizer=None,
                            keep_last=None):
    root = Path(root)
    d = root / f"checkpoint-{step}"
    d.mkdir(parents=True, exist_ok=True)
    sd = adapter_state_dict(adapters, "peft")
    meta = {"format": "eridiffusion", "network_type": network_type, "rank": rank, "alpha": alpha, "step": step}
    st.save_file({k: v.to(torch.bfloat16) for k, v in sd.items()}, d / "adapter_model.safetensors",
                 {k: v for k, v in meta.items() if v is not None})
    if optimizer is not None and hasattr(optimizer, "state_dict"):
        tens = {f"optimizer.{k}": v for k, v in optimizer.state_dict().items() if torch.is_tensor(v)}
        if tens:
            st.save_file(tens, d / "optimizer.safetensors", {"step": step})
    (d / "metadata.json").write_text(json.dumps(meta, indent=1))
    latest = root / "checkpoint-latest"
    try:
        if latest.is_symlink() or latest.exists():
            latest.unlink()
        latest.symlink_to(d.name)
    except OSError:
        pass
    if keep_last:
        found = sorted((int(m.group(1)), p) for p in root.iterdir()
                       if (m := re.match(r"checkpoint-(\d+)$", p.name)) and p.is_dir())
        import shutil
        for _, p in found[:-keep_last]:
            shutil.rmtree(p, ignore_errors=True)
    return d


def load_adapter_checkpoint(adapters, root):
    """Follows ``checkpoint-latest`` (or takes the highest step). Returns the metadata dict."""
    root = Path(root)
    d = root / "checkpoint-latest"
    if not d.exists():
        found = sorted((int(m.group(1)), p) for p in root.iterdir()
                       if (m := re.match(r"checkpoint-(\d+)$", p.name)) and p.is_dir())
        if not found:
            return None
        d = found[-1][1]
    load_adapter_state_dict(adapters, st.load_file(d / "adapter_model.safetensors"), strict=True)
    return json.loads((d / "metadata.json").read_text())


# ------------------------------------------------------------------------------ strict checkpoint
def save_strict(tensors: dict, path, trainer="flux_lora", model="flux", lora_rank=0, lora_alpha=0.0, step=0):
    st.save_file(tensors, path, {"format_version": STRICT_FORMAT_VERSION, "trainer": trainer, "model": model,
                                 "lora_rank": lora_rank, "lora_alpha": lora_alpha, "step": step})


def load_strict(path, expected_keys, device=None):
    """Reads the file and fails unless its key set equals ``expected_keys`` (no missing, no extra)
    and the format version matches."""
    md = st.read_metadata(path)
    if str(md.get("format_version")) != STRICT_FORMAT_VERSION:
        raise KeyError(f"{path}: format_version {md.get('format_version')!r}, expected {STRICT_FORMAT_VERSION!r}")
    sd = st.load_file(path, device=device)
    exp, got = set(expected_keys), set(sd)
    if exp != got:
        raise KeyError(f"{path}: missing {sorted(exp - got)[:5]}, unexpected {sorted(got - exp)[:5]}")
    return sd, md


# ------------------------------------------------------------------------------ EMA file
def save_ema(shadow: dict, path, dtype=torch.float32, decay=None, step=None):
    md = {k: v for k, v in (("ema_decay", decay), ("step", step)) if v is not None}
    st.save_file({f"ema.{k}": v.detach().to(dtype) for k, v in shadow.items()}, path, md)


def load_ema(path, device=None):
    return {k[len("ema."):]: v.float() for k, v in st.load_file(path, device=device).items()}
