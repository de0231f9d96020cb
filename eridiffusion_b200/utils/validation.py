"""Input validation helpers (crates/core/src/validation.rs and its tests
crates/core/tests/validation_tests.rs: shape, dtype, range and finiteness checks with typed
errors)."""
from __future__ import annotations

import torch

from .errors import ConfigurationError, ShapeError


def validate_shape(t: torch.Tensor, expected, name="tensor"):
    """``expected`` entries: int (exact), None (any), or a tuple of allowed ints."""
    if t.dim() != len(expected):
        raise ShapeError(f"{name}: expected {len(expected)} dims {tuple(expected)}, got {tuple(t.shape)}")
    for i, (got, want) in enumerate(zip(t.shape, expected)):
        if want is None:
            continue
        ok = got in want if isinstance(want, (tuple, list, set)) else got == want
        if not ok:
            raise ShapeError(f"{name}: dim {i} is {got}, expected {want} (shape {tuple(t.shape)})")
    return t


def validate_dtype(t: torch.Tensor, allowed, name="tensor"):
    allowed = allowed if isinstance(allowed, (tuple, list, set)) else (allowed,)
    if t.dtype not in allowed:
        raise ShapeError(f"{name}: dtype {t.dtype}, expected one of {[str(a) for a in allowed]}")
    return t


def validate_range(value, lo=None, hi=None, name="value", inclusive=True):
    bad = (lo is not None and (value < lo or (not inclusive and value == lo))) or \
          (hi is not None and (value > hi or (not inclusive and value == hi)))
    if bad:
        raise ConfigurationError(f"{name}={value} outside [{lo}, {hi}]")
    return value


def validate_divisible(value, by, name="value"):
    if value % by:
        raise ConfigurationError(f"{name}={value} must be a multiple of {by}")
    return value


def validate_finite(t: torch.Tensor, name="tensor"):
    if not bool(torch.isfinite(t).all()):
        n_nan = int(torch.isnan(t).sum())
        n_inf = int(torch.isinf(t).sum())
        raise ShapeError(f"{name}: {n_nan} NaN and {n_inf} Inf values")
    return t


def validate_train_inputs(latents, text, timesteps=None, patch=2):
    """The checks a trainer runs on a batch before the first step: latents [B, C, H, W] with H, W
    divisible by the patch size, text [B, T, D], matching batch sizes, finite values."""
    if latents.dim() != 4:
        raise ShapeError(f"latents must be [B, C, H, W], got {tuple(latents.shape)}")
    B, _, H, W = latents.shape
    validate_divisible(H, patch, "latent height")
    validate_divisible(W, patch, "latent width")
    if text.dim() != 3 or text.shape[0] != B:
        raise ShapeError(f"text must be [B={B}, T, D], got {tuple(text.shape)}")
    if timesteps is not None and timesteps.shape[0] != B:
        raise ShapeError(f"timesteps must have {B} entries, got {tuple(timesteps.shape)}")
    validate_finite(latents, "latents")
    validate_finite(text, "text")
