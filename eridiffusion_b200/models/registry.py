"""Decorator registry of model builders (the reference uses an `inventory`-based plug-in registry:
crates/common/model_registry/src/lib.rs:5-54 — ``ModelEntry{id, build}``, ``build_model``,
``known_models``)."""
from __future__ import annotations

_REGISTRY: dict = {}


def register_model(model_id: str):
    def deco(fn):
        if model_id in _REGISTRY:
            raise KeyError(f"model id {model_id!r} registered twice")
        _REGISTRY[model_id] = fn
        return fn
    return deco


def build_model(model_id: str, **kw):
    if model_id not in _REGISTRY:
        raise KeyError(f"unknown model {model_id!r}; known: {known_models()}")
    return _REGISTRY[model_id](**kw)


def known_models():
    return sorted(_REGISTRY)
