"""Generic named-checkpoint manager: save / load / list / latest / convert / merge / extract.

Reference: ``CheckpointManager{save_checkpoint, load_checkpoint, list_checkpoints,
get_latest_checkpoint, convert_checkpoint, merge_checkpoints, extract_component}``,
``CheckpointMetadata{name, step, epoch, loss, timestamp, model_architecture, network_type}``,
``Checkpoint{metadata, training_state, optimizer_state, scheduler_state, config}``,
``CheckpointFormat`` and ``CheckpointComponent`` (crates/training/src/checkpoint.rs:19-454).

The trainer's own resume path writes the reference's concrete layouts (``train/checkpoint.py``,
``train/checkpoint_formats.py``). This manager is the layout-agnostic tool beside them: a checkpoint
is a directory ``{output_dir}/{name}/`` with one safetensors file per component (``model``,
``network``, ``optimizer``) and a ``checkpoint.json`` holding metadata, training / scheduler state
and the job configuration. In the reference ``convert``, ``merge`` and ``extract`` are declared
and return "not implemented"; here conversion changes dtype and container (safetensors <-> a
``torch.save`` file), merging is a weighted average of the tensors several checkpoints share, and
extraction copies one component out.
"""
from __future__ import annotations

import json
import os
import shutil
import time
from dataclasses import asdict, dataclass, field

import torch

from ..io import safetensors as st

COMPONENTS = ("model", "network", "optimizer")
FORMATS = ("safetensors", "pytorch")
_DTYPES = {"fp32": torch.float32, "float32": torch.float32, "bf16": torch.bfloat16, "bfloat16": torch.bfloat16,
           "fp16": torch.float16, "float16": torch.float16}


@dataclass
class CheckpointMetadata:
    name: str
    step: int = 0
    epoch: int = 0
    loss: float = float("nan")
    timestamp: float = field(default_factory=time.time)
    model_architecture: str = ""
    network_type: str | None = None


@dataclass
class Checkpoint:
    metadata: CheckpointMetadata
    training_state: dict = field(default_factory=dict)
    optimizer_state: dict = field(default_factory=dict)      # scalars (step counts, lr ...); tensors go to the file
    scheduler_state: dict = field(default_factory=dict)
    config: dict = field(default_factory=dict)
    tensors: dict = field(default_factory=dict)              # component -> {name: tensor}


class CheckpointManager:
    def __init__(self, output_dir, keep_last: int = 0):
        self.output_dir = str(output_dir)
        self.keep_last = keep_last
        os.makedirs(self.output_dir, exist_ok=True)

    def _dir(self, name):
        return os.path.join(self.output_dir, name)

    # ------------------------------------------------------------------ save / load
    def save_checkpoint(self, ckpt: Checkpoint) -> str:
        """Written to a temporary directory and renamed, so a crash never leaves a half checkpoint
        under the final name."""
        unknown = set(ckpt.tensors) - set(COMPONENTS)
        if unknown:
            raise ValueError(f"unknown components {sorted(unknown)}; expected {COMPONENTS}")
        final, tmp = self._dir(ckpt.metadata.name), self._dir(f".tmp_{ckpt.metadata.name}_{os.getpid()}")
        if os.path.isdir(tmp):
            shutil.rmtree(tmp)
        os.makedirs(tmp)
        for comp, tensors in ckpt.tensors.items():
            if tensors:
                st.save_file({k: v.detach().contiguous().cpu() for k, v in sorted(tensors.items())},
                             os.path.join(tmp, f"{comp}.safetensors"),
                             metadata={"step": str(ckpt.metadata.step), "component": comp})
        doc = {"metadata": asdict(ckpt.metadata), "training_state": ckpt.training_state,
               "optimizer_state": ckpt.optimizer_state, "scheduler_state": ckpt.scheduler_state, "config": ckpt.config,
               "components": sorted(c for c, t in ckpt.tensors.items() if t)}
        with open(os.path.join(tmp, "checkpoint.json"), "w") as f:
            json.dump(doc, f, indent=1, default=str)
        if os.path.isdir(final):
            shutil.rmtree(final)
        os.replace(tmp, final)
        if self.keep_last > 0:
            for old in self.list_checkpoints()[:-self.keep_last]:
                shutil.rmtree(self._dir(old.name), ignore_errors=True)
        return final

    def load_checkpoint(self, name: str, components=COMPONENTS, device="cpu") -> Checkpoint:
        d = self._dir(name)
        with open(os.path.join(d, "checkpoint.json")) as f:
            doc = json.load(f)
        tensors = {}
        for comp in components:
            p = os.path.join(d, f"{comp}.safetensors")
            if os.path.exists(p):
                tensors[comp] = st.load_file(p, device=device)
        return Checkpoint(CheckpointMetadata(**doc["metadata"]), doc.get("training_state", {}),
                          doc.get("optimizer_state", {}), doc.get("scheduler_state", {}), doc.get("config", {}), tensors)

    def list_checkpoints(self) -> list[CheckpointMetadata]:
        """Complete checkpoints, oldest step first (ties by time)."""
        out = []
        for name in os.listdir(self.output_dir):
            p = os.path.join(self.output_dir, name, "checkpoint.json")
            if name.startswith(".tmp_") or not os.path.isfile(p):
                continue
            try:
                with open(p) as f:
                    out.append(CheckpointMetadata(**json.load(f)["metadata"]))
            except (OSError, ValueError, KeyError, TypeError):
                continue                                       # damaged: not listed, never chosen as latest
        return sorted(out, key=lambda m: (m.step, m.timestamp))

    def get_latest_checkpoint(self) -> str | None:
        lst = self.list_checkpoints()
        return lst[-1].name if lst else None

    def get_best_checkpoint(self) -> str | None:
        lst = [m for m in self.list_checkpoints() if m.loss == m.loss]
        return min(lst, key=lambda m: m.loss).name if lst else None

    # ------------------------------------------------------------------ tools
    def extract_component(self, name: str, component: str, out_path: str, fmt: str = "safetensors") -> str:
        if component not in COMPONENTS:
            raise ValueError(f"component {component!r} not in {COMPONENTS}")
        ck = self.load_checkpoint(name, (component,))
        if component not in ck.tensors:
            raise FileNotFoundError(f"checkpoint {name!r} has no {component} tensors")
        return _write(ck.tensors[component], out_path, fmt, {"source": name, "component": component})

    def convert_checkpoint(self, name: str, out_path: str, fmt: str = "safetensors", dtype: str | None = None,
                           component: str = "model") -> str:
        """One component re-written in another container and / or floating-point dtype."""
        ck = self.load_checkpoint(name, (component,))
        tensors = ck.tensors.get(component)
        if tensors is None:
            raise FileNotFoundError(f"checkpoint {name!r} has no {component} tensors")
        if dtype is not None:
            dt = _DTYPES[dtype]
            tensors = {k: v.to(dt) if v.is_floating_point() else v for k, v in tensors.items()}
        return _write(tensors, out_path, fmt, {"source": name, "component": component, "dtype": dtype or "as stored"})

    def merge_checkpoints(self, names, out_name: str, weights=None, component: str = "model") -> str:
        """Weighted average (fp32 accumulation) of ``component`` over several checkpoints. Tensors
        must exist with the same shape in every input; weights default to uniform and are
        normalised to sum to one."""
        names = list(names)
        if not names:
            raise ValueError("nothing to merge")
        w = [1.0] * len(names) if weights is None else [float(x) for x in weights]
        if len(w) != len(names) or sum(w) == 0:
            raise ValueError("one non-degenerate weight per checkpoint is needed")
        w = [x / sum(w) for x in w]
        first = self.load_checkpoint(names[0], (component,))
        acc = {k: v.float() * w[0] for k, v in first.tensors[component].items()}
        dtypes = {k: v.dtype for k, v in first.tensors[component].items()}
        for name, wi in zip(names[1:], w[1:]):
            other = self.load_checkpoint(name, (component,)).tensors[component]
            if set(other) != set(acc):
                raise ValueError(f"checkpoint {name!r} has different {component} keys")
            for k, v in other.items():
                if v.shape != acc[k].shape:
                    raise ValueError(f"shape mismatch for {k!r} in {name!r}")
                acc[k] += v.float() * wi
        merged = {k: (v.to(dtypes[k]) if dtypes[k].is_floating_point else v.round().to(dtypes[k])) for k, v in acc.items()}
        meta = CheckpointMetadata(out_name, step=max(m.step for m in self.list_checkpoints() if m.name in names),
                                  model_architecture=first.metadata.model_architecture,
                                  network_type=first.metadata.network_type)
        return self.save_checkpoint(Checkpoint(meta, training_state={"merged_from": names, "weights": w},
                                               config=first.config, tensors={component: merged}))


def _write(tensors, out_path, fmt, metadata):
    if fmt not in FORMATS:
        raise ValueError(f"format {fmt!r} not in {FORMATS} (ONNX / TensorFlow export is not provided)")
    os.makedirs(os.path.dirname(os.path.abspath(out_path)), exist_ok=True)
    if fmt == "safetensors":
        st.save_file({k: v.contiguous() for k, v in sorted(tensors.items())}, out_path,
                     metadata={k: str(v) for k, v in metadata.items()})
    else:
        torch.save({k: v.contiguous() for k, v in tensors.items()}, out_path)
    return out_path
