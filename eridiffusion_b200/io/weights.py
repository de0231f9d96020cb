"""Weight loading: safetensors checkpoints -> model parameters with strict key accounting, plus
the key canonicalisation the reference applies to FLUX / SDXL files
(crates/training/src/flux/registry.rs:102-161 canonical key map + strict audit;
crates/common/weights/src/strict_loader.rs:21-92; src/loaders/weight_loader.rs)."""
from __future__ import annotations

import re
from pathlib import Path

import torch

from . import safetensors as st

_FLUX_RENAMES = [
    (r"^model\.diffusion_model\.", ""),
    (r"\.img_mlp\.0\.", ".img_mlp_0."), (r"\.img_mlp\.2\.", ".img_mlp_2."),
    (r"\.txt_mlp\.0\.", ".txt_mlp_0."), (r"\.txt_mlp\.2\.", ".txt_mlp_2."),
    (r"\.norm\.query_norm\.scale$", ".q_norm.scale"), (r"\.norm\.key_norm\.scale$", ".k_norm.scale"),
    (r"^(single_blocks\.\d+)\.norm\.query_norm\.scale$", r"\1.q_norm.scale"),
    (r"\.adaLN_modulation\.1\.", ".adaLN.lin."),
]


# SD3 / SD3.5 original layout (``joint_blocks.N.{x_block, context_block}.{attn, attn2, mlp,
# adaLN_modulation}``; crates/models/src/sd35/keymap.rs:3-348, src/loaders/mmdit_weights.rs) -> the
# two-stream block's names. The adaLN chunk order (shift, scale, gate of attention; shift, scale, gate of
# the MLP; then the second attention's three) is the same on both sides, so tensors copy as they are.
_SD35_RENAMES = [
    (r"^model\.diffusion_model\.", ""),
    (r"\.x_block\.adaLN_modulation\.1\.", ".img_mod.lin."), (r"\.context_block\.adaLN_modulation\.1\.", ".txt_mod.lin."),
    (r"\.x_block\.attn2\.", ".img_attn2."), (r"\.x_block\.attn\.", ".img_attn."), (r"\.context_block\.attn\.", ".txt_attn."),
    (r"\.ln_q\.weight$", ".q_norm.scale"), (r"\.ln_k\.weight$", ".k_norm.scale"),
    (r"\.x_block\.mlp\.fc1\.", ".img_mlp_0."), (r"\.x_block\.mlp\.fc2\.", ".img_mlp_2."),
    (r"\.context_block\.mlp\.fc1\.", ".txt_mlp_0."), (r"\.context_block\.mlp\.fc2\.", ".txt_mlp_2."),
    (r"^x_embedder\.proj\.", "x_embedder."),
    (r"^(t_embedder|y_embedder)\.mlp\.0\.", r"\1.in_layer."), (r"^(t_embedder|y_embedder)\.mlp\.2\.", r"\1.out_layer."),
    (r"^final_layer\.adaLN_modulation\.1\.", "final_layer.adaLN.lin."),
]
# Flux-2 Klein checkpoints (src/models/klein_model.rs:348-529, 600-640): per-stream names under
# ``{img,txt}_attn`` / ``{img,txt}_mlp``, model-level modulation linears, no bias tensors anywhere.
_KLEIN_RENAMES = [
    (r"^model\.diffusion_model\.", ""),
    (r"\.(img|txt)_attn\.norm\.query_norm\.scale$", r".\1.q_norm.scale"),
    (r"\.(img|txt)_attn\.norm\.key_norm\.scale$", r".\1.k_norm.scale"),
    (r"\.(img|txt)_attn\.(qkv|proj)\.", r".\1.\2."),
    (r"\.(img|txt)_mlp\.0\.", r".\1.mlp_in."), (r"\.(img|txt)_mlp\.2\.", r".\1.mlp_out."),
    (r"^(single_blocks\.\d+)\.norm\.query_norm\.scale$", r"\1.q_norm.scale"),
    (r"^(single_blocks\.\d+)\.norm\.key_norm\.scale$", r"\1.k_norm.scale"),
    (r"^double_stream_modulation_(img|txt)\.", r"double_mod_\1."), (r"^single_stream_modulation\.", "single_mod."),
    (r"^final_layer\.adaLN_modulation\.1\.", "final_layer.adaLN.lin."),
]
# parameters a family's checkpoints never carry: zero-filled instead of reported missing
_ZERO_IF_MISSING = {"klein": re.compile(r"\.bias$")}
# tensors of a checkpoint that the model computes instead of storing (none at present: the SD3
# ``pos_embed`` table is loaded into the model's buffer when the model keeps one)
_COMPUTED_KEYS = {}


def sd3_final_rows_to_model(t, out_channels, patch=2):
    """SD3 files order the rows of ``final_layer.linear`` (and its bias) as (patch row, patch column,
    channel) — their unpatchify reshapes a token to [p, p, C] (src/models/mmdit_blocks.rs:2280-2288).
    This package packs and unpacks a token as (channel, patch row, patch column) everywhere, so the
    rows are permuted once on load."""
    pp = patch * patch
    c = out_channels // pp
    return t.reshape(pp, c, *t.shape[1:]).transpose(0, 1).reshape(t.shape).contiguous()


def sd3_final_rows_to_file(t, out_channels, patch=2):
    """Inverse of ``sd3_final_rows_to_model`` (for exports in the original layout)."""
    pp = patch * patch
    c = out_channels // pp
    return t.reshape(c, pp, *t.shape[1:]).transpose(0, 1).reshape(t.shape).contiguous()


def export_sd3_original(model) -> dict:
    """State dict of an SD3 / SD3.5 model under the ORIGINAL checkpoint names and conventions
    (``joint_blocks.N.x_block...``, patch-embedding convolution, (p, p, c) final rows, ``pos_embed``
    as [1, N, D]); the inverse of ``load_model_weights(..., kind="sd35")``."""
    inv = [
        (r"\.img_mod\.lin\.", ".x_block.adaLN_modulation.1."), (r"\.txt_mod\.lin\.", ".context_block.adaLN_modulation.1."),
        (r"\.img_attn2\.", ".x_block.attn2."), (r"\.img_attn\.", ".x_block.attn."), (r"\.txt_attn\.", ".context_block.attn."),
        (r"\.q_norm\.scale$", ".ln_q.weight"), (r"\.k_norm\.scale$", ".ln_k.weight"),
        (r"\.img_mlp_0\.", ".x_block.mlp.fc1."), (r"\.img_mlp_2\.", ".x_block.mlp.fc2."),
        (r"\.txt_mlp_0\.", ".context_block.mlp.fc1."), (r"\.txt_mlp_2\.", ".context_block.mlp.fc2."),
        (r"^x_embedder\.", "x_embedder.proj."),
        (r"^(t_embedder|y_embedder)\.in_layer\.", r"\1.mlp.0."), (r"^(t_embedder|y_embedder)\.out_layer\.", r"\1.mlp.2."),
        (r"^final_layer\.adaLN\.lin\.", "final_layer.adaLN_modulation.1."),
    ]
    out = {}
    oc = model.final_layer.linear.weight.shape[0]
    items = list(model.named_parameters()) + [(k, b) for k, b in model.named_buffers() if k == "pos_embed"]
    for k, t in items:
        t = t.detach()
        if k.startswith("final_layer.linear."):
            t = sd3_final_rows_to_file(t, oc)
        elif k == "x_embedder.weight":
            c = t.shape[1] // 4
            t = t.reshape(t.shape[0], c, 2, 2)
        elif k == "pos_embed":
            t = t.unsqueeze(0)
        fk = k
        for pat, rep in inv:
            fk = re.sub(pat, rep, fk)
        out[fk] = t.contiguous()
    return out


def canonical_key(key: str, kind: str) -> str:
    if kind in ("flux", "chroma"):
        for pat, rep in _FLUX_RENAMES:
            key = re.sub(pat, rep, key)
    elif kind in ("sd3", "sd35", "sd35_medium"):
        for pat, rep in _SD35_RENAMES:
            key = re.sub(pat, rep, key)
    elif kind == "klein":
        for pat, rep in _KLEIN_RENAMES:
            key = re.sub(pat, rep, key)
    return key


def infer_num_blocks(keys, prefix="double_blocks."):
    """Number of blocks present in a checkpoint (crates/training/src/flux/weights.rs:44-58)."""
    idx = {int(m.group(1)) for k in keys if (m := re.match(re.escape(prefix) + r"(\d+)\.", k))}
    return max(idx) + 1 if idx else 0


def load_model_weights(model, path, kind="flux", strict=True, device=None):
    """Copy tensors of a safetensors file (or a directory of shards) into ``model``. With ``strict``
    every model parameter must be found and every file key used."""
    path = Path(path)
    files = sorted(path.glob("*.safetensors")) if path.is_dir() else [path]
    own = dict(model.named_parameters())
    sd3 = kind in ("sd3", "sd35", "sd35_medium")
    if sd3 and isinstance(getattr(model, "pos_embed", None), torch.Tensor):
        own["pos_embed"] = model.pos_embed          # position table buffer: loaded, not recomputed
    used, seen = set(), set()
    if kind == "sdxl":
        # single-file checkpoints in the original layout: remap (and fuse q/k/v) instead of renaming
        from .sdxl_keys import remap_sdxl_state_dict
        raw = {}
        for f in files:
            with st.SafeFile(f) as sf:
                ks = [k for k in sf.keys() if k.startswith("model.diffusion_model.")]
                raw.update({k: sf.get(k, device=device or "cpu") for k in ks})
        if raw:
            sd = remap_sdxl_state_dict(raw, strict=strict)
            with torch.no_grad():
                for k, t in sd.items():
                    if k in own:
                        if tuple(t.shape) != tuple(own[k].shape):
                            raise ValueError(f"{k}: shape {tuple(t.shape)} != parameter {tuple(own[k].shape)}")
                        own[k].copy_(t.to(own[k].dtype))
                        used.add(k)
            if strict and (set(own) - used or set(sd) - used):
                raise KeyError(f"strict weight load: missing={sorted(set(own) - used)[:5]} "
                               f"unused={sorted(set(sd) - used)[:5]}")
            return used
    if kind in ("ltx", "ltx_video"):
        # diffusers layout with separate q / k / v projections: fused while loading
        from .ltx_keys import remap_ltx_state_dict
        raw = {}
        for f in files:
            with st.SafeFile(f) as sf:
                raw.update({k: sf.get(k, device=device or "cpu") for k in sf.keys()})
        sd = remap_ltx_state_dict(raw, strict=strict)
        with torch.no_grad():
            for k, t in sd.items():
                if k in own:
                    if tuple(t.shape) != tuple(own[k].shape):
                        raise ValueError(f"{k}: shape {tuple(t.shape)} != parameter {tuple(own[k].shape)}")
                    own[k].copy_(t.to(own[k].dtype))
                    used.add(k)
        if strict and (set(own) - used or set(sd) - used):
            raise KeyError(f"strict weight load: missing={sorted(set(own) - used)[:5]} "
                           f"unused={sorted(set(sd) - used)[:5]}")
        return used
    for f in files:
        with st.SafeFile(f) as sf:
            st.assert_not_text_encoder(sf.keys())
            for k in sf.keys():
                ck = canonical_key(k, kind)
                if ck in _COMPUTED_KEYS.get(kind, ()):
                    continue
                if sd3 and ck == "pos_embed" and ck not in own:
                    continue                        # a model without a table computes positions itself
                seen.add(ck)
                if ck in own:
                    p = own[ck]
                    t = sf.get(k, device=device or p.device, dtype=p.dtype)
                    if t.dim() == 4 and p.dim() == 2 and t.shape[0] == p.shape[0] and t.numel() == p.numel():
                        t = t.reshape(p.shape)      # patch-embedding convolution [D, C, p, p] -> linear [D, C*p*p]
                    if sd3 and ck == "pos_embed" and t.dim() == 3:
                        t = t.reshape(t.shape[1], t.shape[2])
                    if sd3 and ck.startswith("final_layer.linear."):
                        t = sd3_final_rows_to_model(t, t.shape[0])
                    if tuple(t.shape) != tuple(p.shape):
                        raise ValueError(f"{k}: shape {tuple(t.shape)} != parameter {tuple(p.shape)}")
                    with torch.no_grad():
                        p.copy_(t)
                    used.add(ck)
    zero = _ZERO_IF_MISSING.get(kind)
    if zero is not None:
        with torch.no_grad():
            for k in set(own) - used:
                if zero.search(k):
                    own[k].zero_()
                    used.add(k)
    if strict:
        missing, unused = set(own) - used, seen - used
        if missing or unused:
            raise KeyError(f"strict weight load: missing={sorted(missing)[:5]} unused={sorted(unused)[:5]}")
    return used
