"""SDXL UNet checkpoints in the original (``model.diffusion_model.*``) layout -> this package's
``SDXLUNet`` parameters, including the fusion of separate attention projections.

The reference carries several remappers for the same job (src/loaders/sdxl_weight_mapper.rs,
sdxl_weight_remapper.rs, sdxl_full_remapper.rs, src/inference/sdxl_weight_converter.rs) and a
per-transformer-block key table for its streaming runtime
(crates/training/src/sdxl/keymap.rs:5-143). Differences handled here:

* the UNet is a flat ``down`` / ``mid`` / ``up`` list: ``input_blocks.i`` -> ``down.{i-1}``,
  ``output_blocks.i`` -> ``up.{i + i // 3}`` (an upsampling convolution follows every third block);
* ResBlock members: ``in_layers.0/2`` -> ``norm1/conv1``, ``emb_layers.1`` -> ``temb``,
  ``out_layers.0/3`` -> ``norm2/conv2``, ``skip_connection`` -> ``skip``;
* self-attention ``to_q/to_k/to_v`` are stored as one ``to_qkv`` weight and cross-attention
  ``to_k/to_v`` as one ``to_kv`` (row concatenation), ``to_out.0`` -> ``to_out``,
  ``ff.net.0.proj`` -> ``ff_in``, ``ff.net.2`` -> ``ff_out``.
"""
from __future__ import annotations

import re

import torch

_PREFIX = "model.diffusion_model."
_RES = {"in_layers.0": "norm1", "in_layers.2": "conv1", "emb_layers.1": "temb", "out_layers.0": "norm2",
        "out_layers.3": "conv2", "skip_connection": "skip"}
_TB = {"attn1.to_out.0": "attn1.to_out", "attn2.to_out.0": "attn2.to_out", "attn2.to_q": "attn2.to_q",
       "ff.net.0.proj": "ff_in", "ff.net.2": "ff_out", "norm1": "norm1", "norm2": "norm2", "norm3": "norm3"}
# (source suffix, destination, position in the fused weight)
_FUSED = {"attn1.to_q": ("attn1.to_qkv", 0), "attn1.to_k": ("attn1.to_qkv", 1), "attn1.to_v": ("attn1.to_qkv", 2),
          "attn2.to_k": ("attn2.to_kv", 0), "attn2.to_v": ("attn2.to_kv", 1)}


def _inner(rest: str):
    """Key inside one input/middle/output entry -> (destination suffix, fused slot or None)."""
    m = re.match(r"(\d+)\.(.*)\.(weight|bias)$", rest)
    if not m:
        return None
    j, body, leaf = int(m.group(1)), m.group(2), m.group(3)
    if body in _RES:
        return f"{j}.{_RES[body]}.{leaf}", None
    if body in ("norm", "proj_in", "proj_out"):
        return f"{j}.{body}.{leaf}", None
    tb = re.match(r"transformer_blocks\.(\d+)\.(.*)$", body)
    if tb:
        b, sub = tb.group(1), tb.group(2)
        if sub in _TB:
            return f"{j}.blocks.{b}.{_TB[sub]}.{leaf}", None
        if sub in _FUSED:
            dst, slot = _FUSED[sub]
            return f"{j}.blocks.{b}.{dst}.{leaf}", slot
    return None


def map_sdxl_key(key: str):
    """Original-layout key -> (parameter name in ``SDXLUNet``, fused slot or None); ``None`` for keys
    that do not belong to the UNet (VAE, text encoders) or are not parameters."""
    if not key.startswith(_PREFIX):
        return None
    k = key[len(_PREFIX):]
    for src, dst in (("time_embed.", "time_embed."), ("label_emb.0.", "add_embed."), ("out.0.", "norm_out."),
                     ("out.2.", "conv_out.")):
        if k.startswith(src):
            return dst + k[len(src):], None
    m = re.match(r"input_blocks\.(\d+)\.(.*)$", k)
    if m:
        i, rest = int(m.group(1)), m.group(2)
        if i == 0:
            return "conv_in." + rest[len("0."):], None
        op = re.match(r"0\.op\.(weight|bias)$", rest)
        if op:
            return f"down.{i - 1}.{op.group(1)}", None
        r = _inner(rest)
        return None if r is None else (f"down.{i - 1}.{r[0]}", r[1])
    m = re.match(r"middle_block\.(.*)$", k)
    if m:
        r = _inner(m.group(1))
        return None if r is None else (f"mid.{r[0]}", r[1])
    m = re.match(r"output_blocks\.(\d+)\.(.*)$", k)
    if m:
        i, rest = int(m.group(1)), m.group(2)
        up = re.match(r"\d+\.conv\.(weight|bias)$", rest)
        if up:
            return f"up.{i + i // 3 + 1}.{up.group(1)}", None
        r = _inner(rest)
        return None if r is None else (f"up.{i + i // 3}.{r[0]}", r[1])
    return None


def remap_sdxl_state_dict(sd: dict, strict: bool = True) -> dict:
    """Original-layout tensors -> ``SDXLUNet.state_dict()`` layout. Fused projections are
    concatenated in q, k, v (or k, v) order; with ``strict`` a fused weight with a missing part or
    an unmapped ``model.diffusion_model.*`` key raises."""
    out, parts, unmapped = {}, {}, []
    for k, t in sd.items():
        r = map_sdxl_key(k)
        if r is None:
            if k.startswith(_PREFIX):
                unmapped.append(k)
            continue
        name, slot = r
        if slot is None:
            out[name] = t
        else:
            parts.setdefault(name, {})[slot] = t
    for name, p in parts.items():
        n = 3 if name.endswith("to_qkv.weight") or name.endswith("to_qkv.bias") else 2
        if sorted(p) != list(range(n)):
            if strict:
                raise KeyError(f"{name}: fused projection is missing parts {sorted(set(range(n)) - set(p))}")
            continue
        out[name] = torch.cat([p[i] for i in range(n)], dim=0)
    if strict and unmapped:
        raise KeyError(f"unmapped UNet keys: {unmapped[:5]}")
    return out


def export_sdxl_state_dict(sd: dict) -> dict:
    """The inverse: ``SDXLUNet.state_dict()`` -> original layout (fused projections split)."""
    out = {}
    for name, t in sd.items():
        for src in _expand(name, t):
            out[_PREFIX + src[0]] = src[1]
    return out


def _expand(name: str, t):
    inv_res = {v: k for k, v in _RES.items()}
    inv_tb = {v: k for k, v in _TB.items()}
    leaf = name.rsplit(".", 1)[1]
    for src, dst in (("time_embed.", "time_embed."), ("add_embed.", "label_emb.0."), ("norm_out.", "out.0."),
                     ("conv_out.", "out.2."), ("conv_in.", "input_blocks.0.0.")):
        if name.startswith(src):
            return [(dst + name[len(src):], t)]
    m = re.match(r"(down|mid|up)\.(.*)$", name)
    kind, rest = m.group(1), m.group(2)
    if kind == "mid":
        head, rest2 = "middle_block.", rest
    else:
        idx, rest2 = rest.split(".", 1)
        idx = int(idx)
        if kind == "down":
            if rest2 in ("weight", "bias"):
                return [(f"input_blocks.{idx + 1}.0.op.{rest2}", t)]
            head = f"input_blocks.{idx + 1}."
        else:
            if rest2 in ("weight", "bias"):                 # upsampling conv after blocks 2 and 5
                blk = idx - idx // 4 - 1
                return [(f"output_blocks.{blk}.2.conv.{rest2}", t)]   # after the block's transformer
            head = f"output_blocks.{idx - idx // 4}."
    j, body = rest2.split(".", 1)
    body = body[: -len(leaf) - 1]
    if body in inv_res:
        return [(f"{head}{j}.{inv_res[body]}.{leaf}", t)]
    if body in ("norm", "proj_in", "proj_out"):
        return [(f"{head}{j}.{body}.{leaf}", t)]
    tb = re.match(r"blocks\.(\d+)\.(.*)$", body)
    b, sub = tb.group(1), tb.group(2)
    base = f"{head}{j}.transformer_blocks.{b}."
    if sub in inv_tb:
        return [(f"{base}{inv_tb[sub]}.{leaf}", t)]
    if sub == "attn1.to_qkv":
        q, k, v = t.chunk(3, dim=0)
        return [(f"{base}attn1.to_q.{leaf}", q), (f"{base}attn1.to_k.{leaf}", k), (f"{base}attn1.to_v.{leaf}", v)]
    if sub == "attn2.to_kv":
        k, v = t.chunk(2, dim=0)
        return [(f"{base}attn2.to_k.{leaf}", k), (f"{base}attn2.to_v.{leaf}", v)]
    raise KeyError(name)
