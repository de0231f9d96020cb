"""Plug-in registry (crates/core/src/plugin.rs: a ``libloading`` registry of named extension
points; crates/common/model_registry: ``inventory``-based model entries). Here a plug-in is a
Python module or a ``module:attr`` entry; extension points are named groups (``models``,
``optimizers``, ``objectives``, ``callbacks``, ``samplers``) of name -> factory."""
from __future__ import annotations

import importlib
import os
import threading

from .errors import ConfigurationError


class PluginRegistry:
    def __init__(self):
        self._groups: dict[str, dict[str, object]] = {}
        self._loaded: set[str] = set()
        self._lock = threading.Lock()

    def register(self, group: str, name: str, factory=None, *, override=False):
        """``registry.register("optimizers", "lion", Lion)`` or as a decorator."""
        def put(obj):
            with self._lock:
                g = self._groups.setdefault(group, {})
                if name in g and not override and g[name] is not obj:
                    raise ConfigurationError(f"{group}:{name} is already registered")
                g[name] = obj
            return obj
        return put(factory) if factory is not None else put

    def get(self, group: str, name: str):
        try:
            return self._groups[group][name]
        except KeyError:
            known = ", ".join(sorted(self._groups.get(group, {}))) or "none"
            raise ConfigurationError(f"unknown {group} plug-in {name!r} (known: {known})") from None

    def names(self, group: str):
        return sorted(self._groups.get(group, {}))

    def create(self, group: str, name: str, *args, **kw):
        return self.get(group, name)(*args, **kw)

    def load(self, spec: str):
        """Import ``pkg.module`` (its import registers things) or ``pkg.module:setup`` (called with
        this registry)."""
        if spec in self._loaded:
            return
        mod_name, _, attr = spec.partition(":")
        mod = importlib.import_module(mod_name)
        if attr:
            getattr(mod, attr)(self)
        self._loaded.add(spec)

    def load_from_env(self, var="ERI_B200_PLUGINS"):
        for spec in filter(None, os.environ.get(var, "").split(",")):
            self.load(spec.strip())


plugin_registry = PluginRegistry()
