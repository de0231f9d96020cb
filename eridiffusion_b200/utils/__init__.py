"""Core utilities: typed errors, device management, plug-in registry, input validation, the
strict-bf16 guard counters and small telemetry helpers.

Counterpart of the reference's ``eridiffusion-core`` crate (crates/core/src: ``error.rs``,
``device.rs``, ``plugin.rs`` (libloading registry), ``validation.rs``), of ``common-telemetry``
(``memory_mb``, ``now_millis``), ``common-stability`` (``allow_tf32``, ``sanitize_attn_mask``,
``compute_loss_fp32``) and of flame-core's ``strict`` scope with its ``clone_allocs`` /
``f32_graph_casts`` / ``layout_fixes`` counters (tests/strict_mmdit_block.rs:8-80).
"""
from .errors import (CheckpointError, CommTimeoutError, ConfigurationError, DataError, DeviceError,
                     EriError, KernelError, OutOfMemoryError, ShapeError, classify_cuda_error)
from .device import Device, DeviceManager, current_device, memory_mb, now_millis, set_seed
from .plugins import PluginRegistry, plugin_registry
from .validation import (validate_divisible, validate_dtype, validate_finite, validate_range,
                         validate_shape, validate_train_inputs)
from .strict import StrictScope, strict_counters, strict_scope
from .stability import allow_tf32, compute_loss_fp32, sanitize_attn_mask

__all__ = [n for n in dir() if not n.startswith("_")]
