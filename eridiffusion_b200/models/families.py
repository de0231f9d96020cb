"""Registry entries for the model kinds the reference lists but ships only as placeholders
(``ModelKind`` in crates/training/src/model_registry.rs:125-138; crates/models/{hunyuan, krea,
lumina, omnigen2, qwen_edit_image}/src/lib.rs register builders whose forward returns zeros;
HiDream has a loader stub in crates/training/src/model_registry/models). Each is mapped onto the
block family it belongs to, with the published layer counts and widths where they are public, so
that configs naming these kinds build a real, trainable network of the right shape:

* ``krea``             FLUX.1 Krea is a FLUX.1-dev checkpoint: identical architecture.
* ``hunyuan``          HunyuanVideo-style dual + single stream DiT (20 + 40 blocks, width 3072,
                       24 heads, 3-axis rotary embedding over (t, h, w)).
* ``hidream``          dual + single stream DiT (16 + 32 blocks, width 2560, 20 heads); the sparse
                       mixture-of-experts feed-forward of the original is a dense MLP here.
* ``lumina``           Lumina-Image 2.0 NextDiT (width 2304, 24 heads, 26 layers, Gemma-2 captions).
* ``omnigen2``         single-stream NextDiT-style stack (width 2520, 21 heads, 32 layers).
* ``qwen_edit_image``  Qwen-Image with the reference image's latent tokens appended to the
                       image stream (edit conditioning); same 60 dual-stream blocks.
"""
from __future__ import annotations

import torch

from .mmdit import FLUX_DEV, QWEN_IMAGE, MMDiT, MMDiTConfig
from .nextdit import NextDiT, NextDiTConfig
from .registry import register_model


@register_model("krea")
def build_krea(dtype=torch.bfloat16, device=None, **ov):
    return MMDiT(MMDiTConfig(**{**FLUX_DEV.__dict__, **ov}), dtype=dtype, device=device)


HUNYUAN = MMDiTConfig(in_channels=64, hidden=3072, num_heads=24, depth_double=20, depth_single=40,
                      context_dim=4096, vec_dim=768, guidance_embed=True, axes_dim=(16, 56, 56))


@register_model("hunyuan")
def build_hunyuan(dtype=torch.bfloat16, device=None, **ov):
    return MMDiT(MMDiTConfig(**{**HUNYUAN.__dict__, **ov}), dtype=dtype, device=device)


HIDREAM = MMDiTConfig(in_channels=64, hidden=2560, num_heads=20, depth_double=16, depth_single=32,
                      context_dim=4096, vec_dim=2048, guidance_embed=False, axes_dim=(32, 48, 48))


@register_model("hidream")
def build_hidream(dtype=torch.bfloat16, device=None, **ov):
    return MMDiT(MMDiTConfig(**{**HIDREAM.__dict__, **ov}), dtype=dtype, device=device)


LUMINA = dict(dim=2304, num_heads=24, depth=26, refiner_depth=2, mlp_hidden=9216, caption_dim=2304)


@register_model("lumina")
def build_lumina(dtype=torch.bfloat16, device=None, **ov):
    return NextDiT(NextDiTConfig(**{**NextDiTConfig().__dict__, **LUMINA, **ov}), dtype=dtype, device=device)


OMNIGEN2 = dict(dim=2520, num_heads=21, depth=32, refiner_depth=2, mlp_hidden=10240, caption_dim=2048)


@register_model("omnigen2")
def build_omnigen2(dtype=torch.bfloat16, device=None, **ov):
    return NextDiT(NextDiTConfig(**{**NextDiTConfig().__dict__, **OMNIGEN2, **ov}), dtype=dtype, device=device)


class QwenImageEdit(MMDiT):
    """Qwen-Image-Edit: the latent tokens of the reference image ride along the image stream (so
    attention sees them) and are dropped from the prediction."""

    def forward(self, img, txt, t, y=None, guidance=None, grid_hw=None, ref_tokens=None):
        if ref_tokens is None:
            return super().forward(img, txt, t, y, guidance, grid_hw)
        n = img.shape[1]
        if grid_hw is None:
            s = int(round(n ** 0.5))
            grid_hw = (s, n // s)
        if ref_tokens.shape[1] % grid_hw[1]:
            raise ValueError("reference tokens must form whole rows of the image token grid")
        # the reference image occupies the rows below the target image in the rotary grid
        grid = (grid_hw[0] + ref_tokens.shape[1] // grid_hw[1], grid_hw[1])
        out = super().forward(torch.cat([img, ref_tokens.to(img.dtype)], dim=1), txt, t, y, guidance, grid)
        return out[:, :n]


@register_model("qwen_edit_image")
def build_qwen_edit(dtype=torch.bfloat16, device=None, **ov):
    return QwenImageEdit(MMDiTConfig(**{**QWEN_IMAGE.__dict__, **ov}), dtype=dtype, device=device)
