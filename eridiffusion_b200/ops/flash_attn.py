"""Python binding of the tcgen05 flash-attention kernels (``csrc/flash_attn.cu``)."""
from __future__ import annotations

import math

import torch

from . import _native as N


def supported(q, k, v) -> bool:
    lib = N.lib()
    if lib is None or not hasattr(lib, "eri_flash_attn_fwd"):
        return False
    B, L, H, D = q.shape
    return D in (64, 128) and q.is_contiguous() and k.is_contiguous() and v.is_contiguous() \
        and k.shape[1] >= 128 and L >= 128


def flash_attention(q, k, v, scale=None):
    raise NotImplementedError
