"""Typed errors (crates/core/src/error.rs; CUDA out-of-memory strings mapped to a typed error in
crates/core/src/cuda/mod.rs:69-96)."""
from __future__ import annotations


class EriError(Exception):
    """Base class of every error this package raises on purpose."""


class ConfigurationError(EriError, ValueError):
    pass


class ShapeError(EriError, ValueError):
    pass


class DataError(EriError):
    pass


class CheckpointError(EriError):
    pass


class DeviceError(EriError, RuntimeError):
    pass


class OutOfMemoryError(DeviceError):
    pass


class KernelError(DeviceError):
    """A native kernel returned an error code or set its device status word."""

    def __init__(self, what, code):
        super().__init__(f"{what}: code {code}")
        self.what, self.code = what, code


class CommTimeoutError(DeviceError):
    """A bounded wait on a peer ran out: ``status = ((channel + 1) << 8) | peer``."""

    def __init__(self, status, rank=None):
        self.status, self.rank = status, rank
        self.channel, self.peer = (status >> 8) - 1, status & 0xFF
        super().__init__(f"rank {rank}: wait on channel {self.channel} for peer {self.peer} timed out")


_OOM_MARKERS = ("out of memory", "cuda_error_out_of_memory", "cudaerrormemoryallocation", "cublas_status_alloc_failed")


def classify_cuda_error(exc: BaseException) -> EriError:
    """Map a runtime exception raised by torch / CUDA to a typed error."""
    text = str(exc).lower()
    if any(m in text for m in _OOM_MARKERS):
        return OutOfMemoryError(str(exc))
    if "nccl" in text or "timed out" in text or "timeout" in text:
        return DeviceError(f"communication failure: {exc}")
    if "cuda" in text or "cudnn" in text or "cublas" in text:
        return DeviceError(str(exc))
    return EriError(str(exc))
