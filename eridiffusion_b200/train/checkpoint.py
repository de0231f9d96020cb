"""Checkpoint layouts (kept from the reference so that its files and tools keep working).

* LoRA, primary:  ``{root}/step_{step:06}/lora.safetensors`` — bf16 tensors keyed
  ``lora.{module}.lora.{A,B}``, metadata ``step``, ``seed``, ``dtype_policy``; optional
  ``ema.safetensors`` (keys ``ema.{name}``, metadata + ``ema_decay``); ``meta.json`` with
  ``step, seed, time, param_names, lora_file, ema_file``
  (crates/training/src/flux_trainer.rs:416-439, 633-666). Resume picks the highest ``step_*``.
* Full / generic: ``{root}/checkpoint-{step:06}/model.safetensors`` (keys ``model.{name}``),
  ``optimizer.safetensors`` (keys ``optimizer.{name}``), ``metadata.json``; keep-last-N cleanup
  (src/trainers/checkpoint_saver.rs:63-118, 329-371).
* Adapter: ``{root}/checkpoint-{step}/adapter_model.safetensors`` + ``checkpoint-latest`` symlink,
  metadata ``format, network_type, rank, alpha`` (crates/training/src/checkpoint_manager.rs:51-108).
* kohya / ComfyUI export: ``lora_unet_{module}.lora_down.weight`` etc.
* Sharded optimizer state: ``optimizer.rank{r}.safetensors`` with the 8-bit codes and block scales,
  and the world size / shard map in ``meta.json``.
"""
from __future__ import annotations

import json
import os
import re
import shutil
import struct
import time
from pathlib import Path

import torch

from ..adapters import adapter_state_dict, load_adapter_state_dict
from ..io import safetensors as st


def _rank_world(trainer):
    gs = trainer.grad_sync
    return (gs.rank, gs.world_size) if gs is not None else (0, 1)


def _dist_group(trainer):
    """(dist module, group) when this trainer runs among several ranks of an initialised process
    group, else (None, None)."""
    gs = trainer.grad_sync
    if gs is None or gs.world_size <= 1:
        return None, None
    import torch.distributed as dist
    if not dist.is_available() or not dist.is_initialized():
        return None, None
    return dist, getattr(getattr(gs, "pg", None), "group", None)


def _host_barrier(trainer):
    """All ranks have finished their part of the checkpoint (their optimizer shard is on disk)."""
    dist, group = _dist_group(trainer)
    if dist is not None:
        dist.barrier(group=group)


def _gather_objects(trainer, value):
    """Every rank's ``value``, in rank order (a one-element list in a single-process run)."""
    dist, group = _dist_group(trainer)
    if dist is None:
        return [value]
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, value, group=group)
    return out


def _generator_state(trainer):
    """The timestep generator's state as a list of bytes-as-ints (JSON-friendly), or None."""
    gen = getattr(trainer, "_gen", None)
    if gen is None:
        return None
    return {"device": str(gen.device), "state": gen.get_state().cpu().tolist()}


def _restore_generator(trainer, saved):
    """Continue the timestep stream where the saved run stopped: without this every resume replays
    the draws of step 0 (early timesteps oversampled under frequent preemption, and a resumed run
    is not reproducible against an uninterrupted one)."""
    if not saved:
        return
    try:
        gen = trainer._generator(torch.device(saved["device"]))
        gen.set_state(torch.tensor(saved["state"], dtype=torch.uint8))
    except (RuntimeError, KeyError, TypeError, ValueError):
        trainer._gen = None          # a state from another device type: fall back to reseeding


def _optimizer_tensors(opt):
    sd = opt.state_dict() if hasattr(opt, "state_dict") else {}
    tensors, scalars = {}, {}
    for k, v in sd.items():
        if torch.is_tensor(v):
            tensors[f"optimizer.{k}"] = v
        elif isinstance(v, (int, float, str)):
            scalars[k] = v
        elif isinstance(v, (tuple, list)) and all(isinstance(x, (int, float)) for x in v):
            scalars[k] = list(v)
    return tensors, scalars


def save_training_checkpoint(trainer, root):
    root = Path(root)
    rank, world = _rank_world(trainer)
    step, cfg = trainer.step, trainer.cfg
    if trainer.adapters is not None:
        d = root / f"step_{step:06d}"
        d.mkdir(parents=True, exist_ok=True)
        meta = {"step": step, "seed": cfg.seed, "time": time.time(),
                "param_names": trainer.param_names, "lora_file": "lora.safetensors",
                "ema_file": None, "world_size": world,
                "optimizer_files": [f"optimizer.rank{r}.safetensors" for r in range(world)]}
        if rank == 0:
            layout = getattr(cfg, "lora_layout", "eri") or "eri"
            sd = adapter_state_dict(trainer.adapters, layout, model=trainer.model)
            acfg = cfg.adapter
            st.save_file({k: v.to(torch.bfloat16) for k, v in sd.items()}, d / "lora.safetensors",
                         {"step": step, "seed": cfg.seed, "dtype_policy": "storage=bf16,compute=fp32",
                          "layout": layout, "rank": acfg.rank if acfg else "",
                          "alpha": (acfg.alpha if acfg and acfg.alpha else (acfg.rank if acfg else ""))})
            if trainer.ema is not None:
                st.save_file(trainer.ema.state_dict(trainer.param_names), d / "ema.safetensors",
                             {"step": step, "seed": cfg.seed, "ema_decay": trainer.ema.decay})
                meta["ema_file"] = "ema.safetensors"
        tensors, scalars = _optimizer_tensors(trainer.optimizer)
        if tensors:
            st.save_file(tensors, d / f"optimizer.rank{rank}.safetensors",
                         {"step": step, "rank": rank, "world_size": world, **{k: json.dumps(v) for k, v in scalars.items()}})
        # the timestep generator differs per rank (per sequence-parallel group): one small file each
        (d / f"rng.rank{rank}.json").write_text(json.dumps({"step": step, "timestep_generator": _generator_state(trainer)}))
        # meta.json marks the directory complete and older directories are deleted only after EVERY
        # rank's shard is on disk: a crash before this point leaves no directory that looks whole
        # and never removes the last good one
        _host_barrier(trainer)
        if rank == 0:
            (d / "meta.json").write_text(json.dumps(meta, indent=1))
            _cleanup(root, r"step_(\d+)$", cfg.keep_last)
        _host_barrier(trainer)
        return d
    d = root / f"checkpoint-{step:06d}"
    d.mkdir(parents=True, exist_ok=True)
    if rank == 0:
        sd = {f"model.{n}": p.detach() for n, p in trainer.model.named_parameters()}
        st.save_file(sd, d / "model.safetensors", {"format": "pt", "step": step})
    tensors, scalars = _optimizer_tensors(trainer.optimizer)
    name = "optimizer.safetensors" if world == 1 else f"optimizer.rank{rank}.safetensors"
    if tensors:
        st.save_file(tensors, d / name, {"step": step, "rank": rank, "world_size": world})
    (d / f"rng.rank{rank}.json").write_text(json.dumps({"step": step, "timestep_generator": _generator_state(trainer)}))
    _host_barrier(trainer)                  # every shard is written before the directory is marked complete
    if rank == 0:
        (d / "metadata.json").write_text(json.dumps(
            {"step": step, "seed": cfg.seed, "time": time.time(), "world_size": world,
             "optimizer": scalars, "lr": trainer.optimizer.param_groups[0]["lr"]}, indent=1))
        _cleanup(root, r"checkpoint-(\d+)$", cfg.keep_last)
        latest = root / "checkpoint-latest"
        try:
            if latest.is_symlink() or latest.exists():
                latest.unlink()
            latest.symlink_to(d.name)
        except OSError:
            pass
    _host_barrier(trainer)
    return d


def _cleanup(root, pattern, keep_last):
    if not keep_last:
        return
    found = sorted((int(m.group(1)), p) for p in Path(root).iterdir()
                   if (m := re.match(pattern, p.name)) and p.is_dir())
    for _, p in found[:-keep_last]:
        shutil.rmtree(p, ignore_errors=True)


def find_latest(root, pattern=r"(?:step_|checkpoint-)(\d+)$"):
    root = Path(root)
    if not root.is_dir():
        return None
    found = sorted((int(m.group(1)), p) for p in root.iterdir()
                   if (m := re.match(pattern, p.name)) and p.is_dir())
    return found[-1][1] if found else None


def find_checkpoints(root, pattern=r"(?:step_|checkpoint-)(\d+)$"):
    """Checkpoint directories under ``root``, newest first."""
    root = Path(root)
    if not root.is_dir():
        return []
    found = sorted(((int(m.group(1)), p) for p in root.iterdir()
                    if (m := re.match(pattern, p.name)) and p.is_dir()), reverse=True)
    return [p for _, p in found]


class _OptimizerStateMismatch(ValueError):
    """The ranks disagree on whether the optimizer state of a checkpoint could be restored."""


def load_latest_training_checkpoint(trainer, root, on_skip=None):
    """Restore parameters (+EMA, + optimizer state when its world size matches) from the newest
    checkpoint that loads ON EVERY RANK. A checkpoint that is truncated, unreadable or inconsistent
    (a crash during the write, a damaged shard of one rank) is skipped by all ranks together and the
    one before it is tried; ``on_skip(path, error)`` is told. All ranks walk rank 0's list of
    directories and exchange their result after each attempt, so they always return the same
    ``(step, seed)`` — or ``None`` when there is nothing to resume from."""
    cands = [str(p) for p in find_checkpoints(root)]
    cands = _gather_objects(trainer, cands)[0]            # one list for everybody: rank 0's
    for d in map(Path, cands):
        err, res = None, None
        try:
            res = _load_checkpoint_dir(trainer, d)
        except (OSError, ValueError, KeyError, RuntimeError, json.JSONDecodeError, struct.error) as e:
            err = e
        states = _gather_objects(trainer, None if err is not None else (res[0], res[1], res[2]))
        if all(s is not None for s in states):
            if len({s[2] for s in states}) > 1:
                # some ranks restored their moments and some could not: training would continue out
                # of step, so the directory counts as damaged for everyone
                err = _OptimizerStateMismatch(f"optimizer state restored on ranks "
                                              f"{[i for i, s in enumerate(states) if s[2]]} only")
            elif len({(s[0], s[1]) for s in states}) > 1:
                err = ValueError(f"ranks disagree on (step, seed): {sorted({(s[0], s[1]) for s in states})}")
            else:
                return res[0], res[1]
        if err is None:
            bad = [i for i, s in enumerate(states) if s is None]
            err = ValueError(f"checkpoint did not load on ranks {bad}")
        if on_skip is not None:
            on_skip(d, err)
    return None


def _load_checkpoint_dir(trainer, d):
    rank, world = _rank_world(trainer)
    dev = trainer.arena.data.device
    opt_restored = False
    if trainer.adapters is not None:
        meta = json.loads((d / "meta.json").read_text())
        sd = st.load_file(d / meta["lora_file"], device=dev)
        from ..adapters.reference_keys import detect_layout, fill_adapters_from_reference
        ref_layout = detect_layout(sd.keys())
        if ref_layout is not None:
            fill_adapters_from_reference(trainer.adapters, trainer.model, sd, ref_layout)
        else:
            load_adapter_state_dict(trainer.adapters, sd, strict=True)
        if trainer.ema is not None and meta.get("ema_file"):
            trainer.ema.load_state_dict(st.load_file(d / meta["ema_file"], device=dev), trainer.param_names)
        step, seed = int(meta["step"]), int(meta["seed"])
        saved_world = int(meta.get("world_size", 1))
    else:
        meta = json.loads((d / "metadata.json").read_text())
        sd = st.load_file(d / "model.safetensors", device=dev)
        own = dict(trainer.model.named_parameters())
        with torch.no_grad():
            for k, v in sd.items():
                own[k[len("model."):]].copy_(v)
        step, seed = int(meta["step"]), int(meta["seed"])
        saved_world = int(meta.get("world_size", 1))
    opt_file = d / (f"optimizer.rank{rank}.safetensors" if (saved_world > 1 or trainer.adapters is not None)
                    else "optimizer.safetensors")
    if saved_world == world and opt_file.exists() and hasattr(trainer.optimizer, "load_state_dict"):
        t = st.load_file(opt_file, device=dev)
        md = st.read_metadata(opt_file)
        sdict = {k[len("optimizer."):]: v for k, v in t.items()}
        sdict["step"] = int(md.get("step", step))
        sdict["lr"] = trainer.optimizer.param_groups[0]["lr"]
        try:
            trainer.optimizer.load_state_dict(sdict)
            opt_restored = True
        except (KeyError, RuntimeError):
            # different optimizer kind: moments restart, as in the reference's Flux path. The caller
            # compares this flag across ranks, so a restart on one rank alone is not accepted.
            opt_restored = False
    elif saved_world != world and hasattr(trainer.optimizer, "m_q"):
        # the job restarts on another number of ranks: rebuild this rank's slice of the 8-bit state
        files = [d / f"optimizer.rank{r}.safetensors" for r in range(saved_world)]
        if saved_world == 1 and not files[0].exists():
            files = [d / "optimizer.safetensors"]
        if all(f.exists() for f in files):
            part = reshard_8bit_state(files, rank, world, trainer.optimizer.m_q.numel())
            md = st.read_metadata(files[0])
            part["step"] = int(md.get("step", step))
            part["lr"] = trainer.optimizer.param_groups[0]["lr"]
            trainer.optimizer.load_state_dict(part)
            opt_restored = True
    trainer.step = step
    trainer.micro = step * trainer.cfg.grad_accum
    rng = d / f"rng.rank{rank}.json"
    if saved_world == world and rng.exists():
        _restore_generator(trainer, json.loads(rng.read_text()).get("timestep_generator"))
    else:
        trainer._gen = None
    return step, seed, opt_restored


def reshard_8bit_state(files, new_rank: int, new_world: int, shard_numel: int, block: int = 256):
    """Block-wise 8-bit optimizer state saved by ``len(files)`` ranks -> the slice that rank
    ``new_rank`` of ``new_world`` owns. Shards are contiguous ranges of the flat parameter arena
    and start on block boundaries in every layout, so the codes and the per-block maxima are
    concatenated and cut again without de-quantising (lossless); a longer new layout is padded with
    zero codes (value 0)."""
    parts = [st.load_file(f) for f in files]
    out = {}
    for key, per_elem in (("m_q", 1), ("v_q", 1), ("m_absmax", block), ("v_absmax", block)):
        full = torch.cat([p[f"optimizer.{key}"].reshape(-1).cpu() for p in parts])
        n = shard_numel // per_elem
        lo, hi = new_rank * n, (new_rank + 1) * n
        if hi > full.numel():
            full = torch.cat([full, torch.zeros(hi - full.numel(), dtype=full.dtype)])
        out[key] = full[lo:hi].clone()
    return out


def export_lora(trainer, path, layout="kohya", strict=True):
    """Single-file export for other tools: kohya / ComfyUI / PEFT key conventions, or the reference's
    per-site names (``phase4``: ``lora.block{NN}.attn.q.lora.A`` ..., ``stable``, ``sdxl``)."""
    sd = adapter_state_dict(trainer.adapters, layout, model=trainer.model, strict=strict)
    acfg = trainer.cfg.adapter
    st.save_file({k: v.to(torch.bfloat16) if v.dim() else v.float() for k, v in sd.items()}, path,
                 {"format": "eridiffusion", "network_type": acfg.kind if acfg else "lora",
                  "rank": acfg.rank if acfg else "", "alpha": (acfg.alpha if acfg and acfg.alpha else "")})
