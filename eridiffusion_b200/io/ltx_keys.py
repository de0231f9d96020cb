"""LTX-2 checkpoint keys (diffusers layout) -> the fused layout of ``models/ltx_video.py``.

The released transformer stores separate ``to_q`` / ``to_k`` / ``to_v`` projections
(``transformer_blocks.{i}.attn1.to_q.weight`` ...; key list in src/models/ltx2_model.rs:18-40, loader
at :1230-1420). Here the self-attention runs one QKV GEMM and the text cross-attention one K/V GEMM,
so the three (two) matrices are concatenated along the output axis; everything else is a rename.
Audio-stream and cross-modal tensors are left to the audio + video model and skipped for the
video-only one.
"""
from __future__ import annotations

import re

import torch

_TOP = [
    (r"^proj_in\.", "patchify_proj."),
    (r"^caption_projection\.linear_1\.", "caption_in."), (r"^caption_projection\.linear_2\.", "caption_out."),
    (r"^time_embed\.emb\.timestep_embedder\.linear_1\.", "time_embed.in_layer."),
    (r"^time_embed\.emb\.timestep_embedder\.linear_2\.", "time_embed.out_layer."),
    (r"^time_embed\.linear\.", "adaln_single."),
]
_BLOCK = [
    (r"^attn1\.norm_q\.weight$", "attn1_qnorm"), (r"^attn1\.norm_k\.weight$", "attn1_knorm"),
    (r"^attn2\.norm_q\.weight$", "attn2_qnorm"), (r"^attn2\.norm_k\.weight$", "attn2_knorm"),
    (r"^attn1\.to_out\.0\.", "attn1_out."), (r"^attn2\.to_out\.0\.", "attn2_out."), (r"^attn2\.to_q\.", "attn2_q."),
    (r"^ff\.net\.0\.proj\.", "ff_in."), (r"^ff\.net\.2\.", "ff_out."),
]
_AUDIO = re.compile(r"(^|\.)(audio_|av_cross_attn|audio_to_video|video_to_audio|video_a2v|audio_a2v)")
# normalisation layers without parameters in this implementation (RMS / layer norm, no affine)
_NO_AFFINE = re.compile(r"(^|\.)(norm1|norm2|norm3|norm_out)\.(weight|bias)$")


def remap_ltx_state_dict(raw: dict, strict: bool = True) -> dict:
    out, parts, leftover = {}, {}, []
    for k, t in raw.items():
        k = re.sub(r"^(model\.diffusion_model\.|transformer\.)", "", k)
        if _AUDIO.search(k) or _NO_AFFINE.search(k):
            continue
        m = re.match(r"^transformer_blocks\.(\d+)\.(.+)$", k)
        if m is None:
            nk = k
            for pat, rep in _TOP:
                nk = re.sub(pat, rep, nk)
            out[nk] = t
            continue
        i, rest = int(m.group(1)), m.group(2)
        f = re.match(r"^(attn1)\.to_([qkv])\.(weight|bias)$", rest) or re.match(r"^(attn2)\.to_([kv])\.(weight|bias)$", rest)
        if f:
            parts.setdefault((i, f.group(1), f.group(3)), {})[f.group(2)] = t
            continue
        nk = rest
        for pat, rep in _BLOCK:
            nk = re.sub(pat, rep, nk)
        if nk == rest and rest != "scale_shift_table":
            leftover.append(k)
        out[f"blocks.{i}.{nk}"] = t
    for (i, attn, leaf), d in parts.items():
        order = "qkv" if attn == "attn1" else "kv"
        if set(d) != set(order):
            raise KeyError(f"transformer_blocks.{i}.{attn}: projections {sorted(d)} present, expected {list(order)}")
        out[f"blocks.{i}.{attn}_{order}.{leaf}"] = torch.cat([d[c] for c in order], dim=0)
    if strict and leftover:
        raise KeyError(f"unrecognised LTX checkpoint keys: {leftover[:5]}")
    return out


def export_ltx_state_dict(sd: dict) -> dict:
    """Inverse of ``remap_ltx_state_dict`` (fused projections split back into ``to_q/k/v``)."""
    out = {}
    inv_top = {"patchify_proj.": "proj_in.", "caption_in.": "caption_projection.linear_1.",
               "caption_out.": "caption_projection.linear_2.", "time_embed.in_layer.": "time_embed.emb.timestep_embedder.linear_1.",
               "time_embed.out_layer.": "time_embed.emb.timestep_embedder.linear_2.", "adaln_single.": "time_embed.linear."}
    inv_blk = {"attn1_qnorm": "attn1.norm_q.weight", "attn1_knorm": "attn1.norm_k.weight", "attn2_qnorm": "attn2.norm_q.weight",
               "attn2_knorm": "attn2.norm_k.weight", "attn1_out.": "attn1.to_out.0.", "attn2_out.": "attn2.to_out.0.",
               "attn2_q.": "attn2.to_q.", "ff_in.": "ff.net.0.proj.", "ff_out.": "ff.net.2."}
    for k, t in sd.items():
        m = re.match(r"^blocks\.(\d+)\.(.+)$", k)
        if m is None:
            nk = k
            for a, b in inv_top.items():
                if nk.startswith(a):
                    nk = b + nk[len(a):]
                    break
            out[nk] = t
            continue
        i, rest = m.group(1), m.group(2)
        f = re.match(r"^(attn1)_qkv\.(weight|bias)$", rest) or re.match(r"^(attn2)_kv\.(weight|bias)$", rest)
        if f:
            names = "qkv" if f.group(1) == "attn1" else "kv"
            for c, part in zip(names, t.chunk(len(names), dim=0)):
                out[f"transformer_blocks.{i}.{f.group(1)}.to_{c}.{f.group(2)}"] = part.contiguous()
            continue
        nk = rest
        for a, b in inv_blk.items():
            if nk == a or (a.endswith(".") and nk.startswith(a)):
                nk = b + nk[len(a):] if a.endswith(".") else b
                break
        out[f"transformer_blocks.{i}.{nk}"] = t
    return out
